// Split-KV decode attention for grouped-query heads (head dimension 128, bf16 KV cache).
//
// One CTA handles one (sequence, KV head, KV split) and all G query heads that share the KV head,
// so every K/V byte is read from HBM exactly once per step. K and V chunks of 64 cache positions are
// brought into a 3-stage shared-memory ring by TMA (tiled 4-D tensor maps over the cache, 128-byte
// swizzle, no multicast), so the copies of later chunks overlap the arithmetic. Per chunk:
//   A  half a cache row per lane: G partial scores, the two halves joined by one shuffle per head;
//   B  chunk maximum and sum per head, online-softmax rescale;
//   C  16 lanes cover one V row (8 columns each) and accumulate P*V from shared-memory probabilities.
// Splits write (max, sum, unnormalised output) to a scratch buffer; a second small kernel merges
// them. Decode attention is bandwidth-bound (G FLOP per byte), so this path uses the SIMT pipes;
// the tensor cores are kept for the GEMMs.
//
// Not part of the reference (it has no attention); needed by the Llama-shaped decoder layers.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cfloat>
#include <mutex>
#include <set>
#include "tdx/comm.h"
#include "tdx/launch.h"
#include "tdx/ops.h"
#include "tdx/tc.cuh"
#include "tdx/tma_host.h"
#include "tdx/ptx.cuh"
#include "tdx/sync.cuh"
#include "tdx/vec.cuh"

namespace tdx {
namespace {

constexpr int kD = 128;
constexpr int kChunk = 64;            // cache positions per pipeline stage
constexpr int kStagesKV = 3;
constexpr int kAttnThreads = 128;
constexpr int kMaxG = 8;
constexpr int kHalfBytes = kChunk * 128;          // one 64-column half of a K or V chunk
constexpr int kStageBytesKV = 4 * kHalfBytes;     // K lo, K hi, V lo, V hi
constexpr int kAttnSmem = kStagesKV * kStageBytesKV + 1024 /*alignment*/ + 256 /*barriers*/;
constexpr uint32_t kAttnWaitLimit = 1u << 22;

constexpr int kAttnCounters = 4096;   // words at the start of the scratch buffer: one arrival counter per (b, kv head)

struct AttnArgs {
  const __nv_bfloat16* q;      // [B, Hq, D]
  const int32_t* seq_lens;     // [B] valid positions per sequence
  uint32_t* counters;          // [B * Hkv] zero on entry, left zero on exit (null: a separate kernel merges)
  float* partial;              // [B, Hq, nsplit, D + 2]
  __nv_bfloat16* out;          // [B, Hq, D]
  int B, Hq, Hkv, S_max, nsplit;
  int64_t q_stride_b;          // elements
  float scale;
  uint32_t* status;
};

// 16 bytes (8 bf16) of row `r`, logical 16-byte chunk `c` (0..7) of a 128-byte-swizzled half tile.
__device__ __forceinline__ uint4 ld_swizzled(const uint8_t* half_tile, int r, int c) {
  return *reinterpret_cast<const uint4*>(half_tile + r * 128 + ((c ^ (r & 7)) << 4));
}

// K and V chunks arrive by TMA (tiled 4-D maps over the cache, 128-byte swizzle) in a 3-stage ring,
// so the loads of later chunks overlap the arithmetic on the current one and no thread issues a
// global load for the cache. Thread mapping per 64-row chunk:
//   scores   lane l of warp w takes row 16*w + (l & 15) and the column half (l >> 4); the two halves
//            are added with one shuffle per query head;
//   P * V    16 lanes cover one V row (8 columns each), a warp takes two rows per step.
template <int kG>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_split_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                         const __grid_constant__ CUtensorMap map_v,
                                                                         const AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ float q_s[kG][kD];
  __shared__ float p_s[kG][kChunk];
  __shared__ float wred[2][kG][4];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + kStagesKV * kStageBytesKV);
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(full + kStagesKV);

  const int b = blockIdx.x, hkv = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  ptx::pdl_wait();                // q, the caches and seq_lens come from earlier kernels of the stream
  ptx::pdl_launch_dependents();
  const int len = a.seq_lens[b];
  const int per = (len + a.nsplit - 1) / a.nsplit;
  const int s0 = split * per, s1 = min(len, s0 + per);
  const int nchunks = s1 > s0 ? (s1 - s0 + kChunk - 1) / kChunk : 0;

  auto issue = [&](int i) {
    const int st = i % kStagesKV;
    uint8_t* base = ring + st * kStageBytesKV;
    tc::mbar_arrive_expect_tx(&full[st], kStageBytesKV);
    const int pos0 = s0 + i * kChunk;
    tc::tma_load_4d(base, &map_k, &full[st], 0, hkv, pos0, b);
    tc::tma_load_4d(base + kHalfBytes, &map_k, &full[st], 64, hkv, pos0, b);
    tc::tma_load_4d(base + 2 * kHalfBytes, &map_v, &full[st], 0, hkv, pos0, b);
    tc::tma_load_4d(base + 3 * kHalfBytes, &map_v, &full[st], 64, hkv, pos0, b);
  };
  if (tid == 0) {
    for (int st = 0; st < kStagesKV; ++st) tc::mbar_init(&full[st], 1);
    *abort_flag = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_desc(&map_k);
    tc::tma_prefetch_desc(&map_v);
  }
  for (int i = tid; i < kG * kD; i += kAttnThreads) {
    const int g = i / kD, d = i % kD;
    q_s[g][d] = __bfloat162float(a.q[(int64_t)b * a.q_stride_b + (int64_t)(hkv * kG + g) * kD + d]) * a.scale;
  }
  __syncthreads();
  if (tid == 0)
    for (int i = 0; i < nchunks && i < kStagesKV; ++i) issue(i);

  float m_run[kG], l_run[kG];
  const int arow = warp * 16 + (lane & 15);   // score phase: row inside the chunk
  const int ahalf = lane >> 4;                // score phase: column half
  const int vslice = lane & 15;               // P*V phase: 8-column slice of the row
  const int vsub = lane >> 4;
  float acc[kG][8];
#pragma unroll
  for (int g = 0; g < kG; ++g) {
    m_run[g] = -FLT_MAX;
    l_run[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }

  for (int i = 0; i < nchunks; ++i) {
    const int st = i % kStagesKV;
    const uint8_t* base = ring + st * kStageBytesKV;
    // The threads leave the loop together: a thread whose wait ran out while its neighbours' succeeded would
    // otherwise skip block-wide barriers that the others still execute.
    const bool arrived = tc::mbar_wait(&full[st], (i / kStagesKV) & 1, kAttnWaitLimit, abort_flag);
    if (__syncthreads_or(!arrived)) {
      if (!arrived) {
        *abort_flag = 1;
        if (a.status) atomicExch(a.status, (uint32_t)kTimeoutGemmPipeline);
      }
      break;
    }
    const int c0 = s0 + i * kChunk;
    const bool live = c0 + arow < s1;
    // ---- scores: half a row per lane ----
    float s[kG];
#pragma unroll
    for (int g = 0; g < kG; ++g) s[g] = 0.f;
    const uint8_t* khalf = base + ahalf * kHalfBytes;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float kf[8];
      unpack<__nv_bfloat16>(ld_swizzled(khalf, arow, c), kf);
#pragma unroll
      for (int g = 0; g < kG; ++g)
#pragma unroll
        for (int j = 0; j < 8; ++j) s[g] = fmaf(q_s[g][ahalf * 64 + c * 8 + j], kf[j], s[g]);
    }
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      s[g] += __shfl_xor_sync(0xffffffffu, s[g], 16);
      if (!live) s[g] = -FLT_MAX;
      float v = s[g];
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
      if (lane == 0) wred[0][g][warp] = v;
    }
    __syncthreads();
    float corr[kG];
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      const float cmax = fmaxf(fmaxf(wred[0][g][0], wred[0][g][1]), fmaxf(wred[0][g][2], wred[0][g][3]));
      const float m_new = fmaxf(m_run[g], cmax);
      corr[g] = __expf(m_run[g] - m_new);
      const float p = live ? __expf(s[g] - m_new) : 0.f;
      if (ahalf == 0) p_s[g][arow] = p;
      float ps = ahalf == 0 ? p : 0.f;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      if (lane == 0) wred[1][g][warp] = ps;
      m_run[g] = m_new;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      const float csum = wred[1][g][0] + wred[1][g][1] + wred[1][g][2] + wred[1][g][3];
      l_run[g] = l_run[g] * corr[g] + csum;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[g][j] *= corr[g];
    }
    // ---- P * V: warp w covers rows 16w .. 16w+15 of the chunk, two rows per step ----
    const uint8_t* vhalf = base + (2 + (vslice >> 3)) * kHalfBytes;
#pragma unroll
    for (int step = 0; step < 8; ++step) {
      const int r = warp * 16 + step * 2 + vsub;
      float vf[8];
      unpack<__nv_bfloat16>(ld_swizzled(vhalf, r, vslice & 7), vf);
#pragma unroll
      for (int g = 0; g < kG; ++g) {
        const float p = p_s[g][r];       // zero for rows beyond the sequence
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = fmaf(p, vf[j], acc[g][j]);
      }
    }
    __syncthreads();   // every thread is done with this stage, p_s and wred
    if (tid == 0 && i + kStagesKV < nchunks) issue(i + kStagesKV);
  }
  // merge the two half-warps, then the four warps
#pragma unroll
  for (int g = 0; g < kG; ++g)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[g][j] += __shfl_xor_sync(0xffffffffu, acc[g][j], 16);
  // all chunks have been consumed, so the ring is free: use it for the per-warp partial outputs
  float (*acc_s)[kG][kD] = reinterpret_cast<float (*)[kG][kD]>(ring);
  if (vsub == 0) {
#pragma unroll
    for (int g = 0; g < kG; ++g)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc_s[warp][g][vslice * 8 + j] = acc[g][j];
  }
  __syncthreads();
  if (a.nsplit == 1) {
    // a single split: normalise and write the output directly
    for (int i = tid; i < kG * kD; i += kAttnThreads) {
      const int g = i / kD, d = i % kD;
      const float o = acc_s[0][g][d] + acc_s[1][g][d] + acc_s[2][g][d] + acc_s[3][g][d];
      a.out[((int64_t)b * a.Hq + hkv * kG + g) * kD + d] = __float2bfloat16(l_run[g] > 0.f ? o / l_run[g] : 0.f);
    }
  } else {
    for (int i = tid; i < kG * kD; i += kAttnThreads) {
      const int g = i / kD, d = i % kD;
      const float o = acc_s[0][g][d] + acc_s[1][g][d] + acc_s[2][g][d] + acc_s[3][g][d];
      float* dst = a.partial + (((int64_t)b * a.Hq + hkv * kG + g) * a.nsplit + split) * (kD + 2);
      dst[d] = o;
      if (d == 0) {
        dst[kD] = m_run[g];      // identical in every thread
        dst[kD + 1] = l_run[g];
      }
    }
    if (a.counters != nullptr) {
      // the split that arrives last merges all of them (saves a launch per layer)
      __shared__ uint32_t s_last;
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const uint32_t prev = atomicAdd(&a.counters[b * a.Hkv + hkv], 1u);
        s_last = (prev == (uint32_t)a.nsplit - 1u) ? 1u : 0u;
        if (s_last) a.counters[b * a.Hkv + hkv] = 0;
      }
      __syncthreads();
      if (s_last) {
        __threadfence();
        const int d = tid;   // kAttnThreads == kD
#pragma unroll
        for (int g = 0; g < kG; ++g) {
          const float* src = a.partial + ((int64_t)b * a.Hq + hkv * kG + g) * a.nsplit * (kD + 2);
          float m = -FLT_MAX;
          for (int sp = 0; sp < a.nsplit; ++sp) m = fmaxf(m, __ldcg(src + sp * (kD + 2) + kD));
          float num = 0.f, den = 0.f;
          for (int sp = 0; sp < a.nsplit; ++sp) {
            const float wgt = __expf(__ldcg(src + sp * (kD + 2) + kD) - m);
            num = fmaf(wgt, __ldcg(src + sp * (kD + 2) + d), num);
            den = fmaf(wgt, __ldcg(src + sp * (kD + 2) + kD + 1), den);
          }
          a.out[((int64_t)b * a.Hq + hkv * kG + g) * kD + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
        }
      }
    }
  }
  if (*abort_flag) {
    // let copies that were already requested land before the shared memory goes away
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
}

// out[b, h, :] = sum_s exp(m_s - m) * acc_s / sum_s exp(m_s - m) * l_s
__global__ void __launch_bounds__(kD) attn_combine_kernel(const AttnArgs a) {
  ptx::pdl_wait();
  ptx::pdl_launch_dependents();
  const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const float* src = a.partial + ((int64_t)b * a.Hq + h) * a.nsplit * (kD + 2);
  float m = -FLT_MAX;
  for (int s = 0; s < a.nsplit; ++s) m = fmaxf(m, src[s * (kD + 2) + kD]);
  float num = 0.f, den = 0.f;
  for (int s = 0; s < a.nsplit; ++s) {
    const float w = __expf(src[s * (kD + 2) + kD] - m);
    num = fmaf(w, src[s * (kD + 2) + d], num);
    den = fmaf(w, src[s * (kD + 2) + kD + 1], den);
  }
  a.out[((int64_t)b * a.Hq + h) * kD + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
}

}  // namespace

namespace {

template <int kG>
std::string launch_attn(const CUtensorMap& mk, const CUtensorMap& mv, const AttnArgs& a, dim3 grid, cudaStream_t stream) {
  auto kern = attn_decode_split_kernel<kG>;
  const std::string smem_err = reserve_dynamic_smem(kern, kAttnSmem);
  if (!smem_err.empty()) return smem_err;
  const cudaError_t e = launch_chained(kern, grid, dim3(kAttnThreads), kAttnSmem, stream, mk, mv, a);
  return e == cudaSuccess ? "" : std::string("attention launch failed: ") + cudaGetErrorString(e);
}

}  // namespace

std::string attention_decode(const void* q, const void* k_cache, const void* v_cache, const int32_t* seq_lens,
                             float* partial, size_t partial_floats, void* out, int B, int Hq, int Hkv, int D, int S_max,
                             int64_t q_stride_b, int64_t kv_stride_b, int64_t kv_stride_s, int nsplit, float scale,
                             cudaStream_t stream, uint32_t* status) {
  if (D != kD) return "decode attention supports head dimension 128";
  if (Hkv <= 0 || Hq % Hkv) return "query heads must be a multiple of KV heads";
  const int G = Hq / Hkv;
  if (G > kMaxG || (G & (G - 1))) return "query heads per KV head must be 1, 2, 4 or 8";
  if (nsplit < 1) nsplit = 1;
  // scratch layout: kAttnCounters arrival counters (zero on entry, zeroed again by the kernel), then the partials
  // A buffer longer than the counter block always carries it: the partial rows start behind it even when the
  // separate combine kernel is used, so that a cached scratch buffer never has its counters overwritten.
  const bool has_counters = partial_floats > (size_t)kAttnCounters;
  const bool in_kernel_merge = has_counters && (size_t)B * Hkv <= (size_t)kAttnCounters;
  const size_t head = has_counters ? (size_t)kAttnCounters : 0;
  if (head + (size_t)B * Hq * nsplit * (kD + 2) > partial_floats) return "attention scratch buffer is too small";
  if ((kv_stride_s * 2) % 16 || (kv_stride_b * 2) % 16 || reinterpret_cast<uintptr_t>(k_cache) % 16 ||
      reinterpret_cast<uintptr_t>(v_cache) % 16)
    return "KV cache rows must be 16-byte aligned";
  if (B == 0) return "";
  AttnArgs a{};
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.seq_lens = seq_lens;
  a.counters = in_kernel_merge ? reinterpret_cast<uint32_t*>(partial) : nullptr;
  a.partial = partial + head;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.S_max = S_max; a.nsplit = nsplit;
  a.q_stride_b = q_stride_b;
  a.scale = scale;
  a.status = status;
  CUtensorMap mk, mv;
  std::string err = tma::kv_cache_4d(&mk, k_cache, B, S_max, Hkv, kv_stride_b, kv_stride_s, kChunk);
  if (!err.empty()) return err;
  err = tma::kv_cache_4d(&mv, v_cache, B, S_max, Hkv, kv_stride_b, kv_stride_s, kChunk);
  if (!err.empty()) return err;
  const dim3 grid(B, Hkv, nsplit);
  switch (G) {
    case 1: err = launch_attn<1>(mk, mv, a, grid, stream); break;
    case 2: err = launch_attn<2>(mk, mv, a, grid, stream); break;
    case 4: err = launch_attn<4>(mk, mv, a, grid, stream); break;
    case 8: err = launch_attn<8>(mk, mv, a, grid, stream); break;
  }
  if (!err.empty()) return err;
  if (nsplit > 1 && !in_kernel_merge) launch_chained(attn_combine_kernel, dim3(B, Hq), dim3(kD), 0, stream, a);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? "" : cudaGetErrorString(e);
}

}  // namespace tdx
