// Split-KV decode attention on the tensor cores (tcgen05 / TMEM), head dimension 128, bf16 KV cache.
//
// Same interface and split/merge format as attention_decode.cu, whose arithmetic runs on the SIMT
// pipes and is issue-bound well below the HBM roofline. Here both products of a 128-position chunk
// are tcgen05 MMAs, with the cache positions (or the head dimension) on the 128-row side of the
// instruction and the few query heads that share the KV head padded to the narrowest N (16):
//
//   S^T[keys 128, heads 16] = K[keys, d] * Q[heads, d]^T     A = K chunk as TMA delivers it (K-major over d)
//   O^T[d 128,   heads 16] = V[keys, d]^T * P[heads, keys]^T  A = V chunk read MN-major (d contiguous), K = keys
//
// so neither K nor V is transposed or touched by a thread: TMA -> shared memory -> tensor core.
// Per chunk the four softmax warps read S^T from tensor memory (one cache position per thread),
// do the online-softmax bookkeeping and write the probabilities as a bf16 [heads, keys] tile (128-byte
// swizzle, the B operand of the second product). O^T accumulates in tensor memory over all chunks of a
// split; a head's column of it is rescaled there only when its running maximum has to be raised.
// Three more warps hold one single-thread role each - the TMA copies (3-stage ring), the score MMAs, the P*V MMAs -
// so that none of them queues behind the others' asynchronous instructions; S^T is double-buffered in TMEM and P
// in shared memory, so that the scores of chunk i+1 and the P*V product of chunk i-1 run while the softmax
// warps work on chunk i.
//
// Every wait is bounded; a wait that runs out records a status word, raises the CTA's abort flag
// (which ends every other wait early) and all threads still reach the common exit, where copies in
// flight are given time to land and the tensor memory is freed.
//
// The default decode-attention kernel (ops/attention.py; TDX_ATTN_TC=0 selects the SIMT kernel).
// Not part of the reference (it has no attention).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cfloat>
#include <mutex>
#include <set>
#include <string>
#include "tdx/comm.h"
#include "tdx/launch.h"
#include "tdx/ops.h"
#include "tdx/sync.cuh"
#include "tdx/tc.cuh"
#include "tdx/tma_host.h"

namespace tdx {
namespace {

constexpr int kD = 128;
constexpr int kKeys = 128;                        // cache positions per chunk = MMA M of the score product
constexpr int kNq = 16;                           // MMA N: query heads of one KV head, padded
constexpr int kStages = 3;
constexpr int kSoftmaxThreads = 128;
constexpr int kThreads = kSoftmaxThreads + 3 * 32;   // + three single-thread roles: copies (warp 4), score MMAs (5), P*V MMAs (6)
constexpr int kMaxG = 8;
constexpr int kHalfBytes = kKeys * 128;           // one 64-column half of a K or V chunk
constexpr int kStageBytes = 4 * kHalfBytes;       // K lo, K hi, V lo, V hi
constexpr int kSmallTileBytes = 2 * kNq * 128;    // Q or P: two 64-wide K blocks of 16 rows x 128 bytes
constexpr int kSmem = kStages * kStageBytes + 3 * kSmallTileBytes /*Q, two P tiles*/ + 256 /*barriers*/ + 1024 /*alignment*/;
constexpr uint32_t kTmemCols = 64;                // S^T buffers at columns 0 and 16, O^T chunk at 32
constexpr uint32_t kColO = 32;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr float kRescaleThreshold = 5.f;          // natural-log units
constexpr int kCounterWords = 4096;               // head of the scratch buffer reserved by the other kernel

struct TcAttnArgs {
  const __nv_bfloat16* q;      // [B, Hq, D]
  const int32_t* seq_lens;     // [B]
  float* partial;              // [B, Hq, nsplit, D + 2]
  uint32_t* counters;          // [B * Hkv] arrival counters (zero on entry, zeroed again by the kernel), or null
  __nv_bfloat16* out;          // [B, Hq, D]
  int B, Hq, Hkv, nsplit;
  int64_t q_stride_b;
  float scale;
  uint32_t idesc_s, idesc_pv;
  uint32_t* status;
};

// Byte offset of element (row, col) of a [16 rows x 128 columns] bf16 tile stored as two 64-column
// K blocks of [16 rows x 128 bytes] with the 128-byte swizzle (what tcgen05.mma reads as a K-major B operand).
__device__ __forceinline__ int small_tile_offset(int row, int col) {
  const int kb = col >> 6, c = (col & 63) >> 3;
  return kb * (kNq * 128) + row * 128 + ((c ^ (row & 7)) << 4) + (col & 7) * 2;
}

template <int kG>
__global__ void __launch_bounds__(kThreads, 1)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const TcAttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ float wred[2][kG][4];
  __shared__ uint32_t s_last, s_stop;
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_tile = ring + kStages * kStageBytes;
  uint8_t* p_tile = q_tile + kSmallTileBytes;
  // two P tiles, alternating by chunk: the probabilities of chunk i are written while P*V of chunk i - 1 may still run
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(p_tile + 2 * kSmallTileBytes);
  uint64_t* kv_free = kv_full + kStages;
  uint64_t* s_full = kv_free + kStages;     // [2]
  uint64_t* s_free = s_full + 2;            // [2]
  uint64_t* p_full = s_free + 2;            // [2]: the probabilities of chunk c are in P tile c & 1
  uint64_t* o_full = p_full + 2;            // [2]: P*V of chunk c completes o_full[c & 1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int b = blockIdx.x, hkv = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  ptx::pdl_wait();                // q, the caches and seq_lens come from earlier kernels of the stream
  ptx::pdl_launch_dependents();
  const int len = a.seq_lens[b];
  const int per = (len + a.nsplit - 1) / a.nsplit;
  const int s0 = split * per, s1 = min(len, s0 + per);
  const int nchunks = s1 > s0 ? (s1 - s0 + kKeys - 1) / kKeys : 0;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(&kv_full[s], 1);
      tc::mbar_init(&kv_free[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&s_full[i], 1);
      tc::mbar_init(&s_free[i], kSoftmaxThreads);
    }
    tc::mbar_init(&p_full[0], kSoftmaxThreads);
    tc::mbar_init(&p_full[1], kSoftmaxThreads);
    tc::mbar_init(&o_full[0], 1);
    tc::mbar_init(&o_full[1], 1);
    *abort_flag = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_desc(&map_k);
    tc::tma_prefetch_desc(&map_v);
  }
  // Q and P tiles: zero everything (rows beyond the G real heads stay zero), then the query rows
  for (int i = tid; i < 3 * kSmallTileBytes / 16; i += kThreads) reinterpret_cast<uint4*>(q_tile)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  for (int i = tid; i < kG * kD; i += kThreads) {
    const int g = i / kD, d = i % kD;
    *reinterpret_cast<__nv_bfloat16*>(q_tile + small_tile_offset(g, d)) =
        a.q[(int64_t)b * a.q_stride_b + (int64_t)(hkv * kG + g) * kD + d];
  }
  tc::fence_proxy_async();   // the tiles were written by threads and are read by the tensor core
  if (warp == 4) {
    tc::tmem_alloc(tmem_slot, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::fence_before_thread_sync();
  __syncthreads();
  tc::fence_after_thread_sync();
  const uint32_t tmem_base = *tmem_slot;

  auto fail = [&]() {
    *abort_flag = 1;
    if (a.status) atomicExch(a.status, (uint32_t)kTimeoutGemmPipeline);
  };

  float m_run[kG], l_run[kG], o[kG];
#pragma unroll
  for (int g = 0; g < kG; ++g) {
    m_run[g] = -FLT_MAX;
    l_run[g] = 0.f;
    o[g] = 0.f;
  }

  // Three single-thread roles, each with its own chain of waits: one thread needs 70-90 cycles per asynchronous
  // instruction (four copies, eight score MMAs, eight P*V MMAs and three commits per chunk), which done one after the
  // other took as long as HBM needs to deliver the chunk.
  if (warp == 4) {
    if (lane == 0 && nchunks > 0) {
      // ---- copies: a stage is refilled when the P*V product that read its V tile has completed ----
      auto issue_copy = [&](int c) {
        const int st = c % kStages;
        uint8_t* base = ring + st * kStageBytes;
        tc::mbar_arrive_expect_tx(&kv_full[st], kStageBytes);
        const int pos0 = s0 + c * kKeys;
        tc::tma_load_4d(base, &map_k, &kv_full[st], 0, hkv, pos0, b);
        tc::tma_load_4d(base + kHalfBytes, &map_k, &kv_full[st], 64, hkv, pos0, b);
        tc::tma_load_4d(base + 2 * kHalfBytes, &map_v, &kv_full[st], 0, hkv, pos0, b);
        tc::tma_load_4d(base + 3 * kHalfBytes, &map_v, &kv_full[st], 64, hkv, pos0, b);
      };
      bool ok = true;
      for (int c = 0; c < nchunks && c < kStages; ++c) issue_copy(c);
      for (int i = 0; i + kStages < nchunks && ok; ++i) {
        ok = tc::mbar_wait(&kv_free[i % kStages], (i / kStages) & 1, kWaitLimit, abort_flag);
        if (ok) issue_copy(i + kStages);
      }
      if (!ok) fail();
    }
  } else if (warp == 5) {
    if (lane == 0 && nchunks > 0) {
      // ---- scores: S^T[buf c & 1] = K chunk * Q^T, as soon as the chunk has landed and the buffer is free ----
      const uint32_t qbase = tc::smem_u32(q_tile);
      bool ok = true;
      for (int c = 0; c < nchunks && ok; ++c) {
        ok = tc::mbar_wait(&kv_full[c % kStages], (c / kStages) & 1, kWaitLimit, abort_flag) &&
             (c < 2 || tc::mbar_wait(&s_free[c & 1], ((c >> 1) - 1) & 1, kWaitLimit, abort_flag));
        if (!ok) break;
        tc::fence_after_thread_sync();
        const uint32_t kbase = tc::smem_u32(ring + (c % kStages) * kStageBytes);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            tc::umma<false>(tmem_base + (uint32_t)(c & 1) * kNq, tc::make_smem_desc_sw128(kbase + kb * kHalfBytes) + (uint64_t)(ks * 2),
                            tc::make_smem_desc_sw128(qbase + kb * (kNq * 128)) + (uint64_t)(ks * 2), a.idesc_s, (kb | ks) ? 1u : 0u);
        tc::umma_commit(&s_full[c & 1]);
      }
      if (!ok) fail();
    }
  } else if (warp == 6) {
    if (lane == 0 && nchunks > 0) {
      // ---- O^T (+)= V chunk^T * P^T, 16 cache positions per instruction, once the probabilities are written ----
      bool ok = true;
      for (int c = 0; c < nchunks && ok; ++c) {
        ok = tc::mbar_wait(&p_full[c & 1], (c >> 1) & 1, kWaitLimit, abort_flag) &&
             tc::mbar_wait(&kv_full[c % kStages], (c / kStages) & 1, kWaitLimit, abort_flag);
        if (!ok) break;
        tc::fence_after_thread_sync();
        const uint32_t vbase = tc::smem_u32(ring + (c % kStages) * kStageBytes + 2 * kHalfBytes);
        const uint32_t pbase = tc::smem_u32(p_tile + (c & 1) * kSmallTileBytes);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          tc::umma<false>(tmem_base + kColO, tc::make_smem_desc_mn_sw128(vbase + j * 2048, kHalfBytes),
                          tc::make_smem_desc_sw128(pbase + (j >> 2) * (kNq * 128)) + (uint64_t)((j & 3) * 2), a.idesc_pv,
                          (c | j) ? 1u : 0u);
        tc::umma_commit(&o_full[c & 1]);
        tc::umma_commit(&kv_free[c % kStages]);
      }
      if (!ok) fail();
    }
  } else {
    // ---- softmax warps: thread t owns cache position t of the chunk and head-dimension index t of the output ----
    // O^T accumulates in tensor memory over all chunks of the split (the P*V MMAs add to it), so a chunk costs the
    // softmax warps one read of the scores and one write of the probabilities. A head's running maximum is raised
    // - and its column of O^T rescaled in tensor memory - only when the new maximum exceeds it by more than
    // kRescaleThreshold; until then the probabilities are taken against the older maximum (at most e^5, exact in
    // the final O / l). The maxima are block-wide values, so every thread takes the same decision.
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    for (int i = 0; i < nchunks; ++i) {
      const int buf = i & 1;
      float sv[16];
      bool ok = tc::mbar_wait(&s_full[buf], (i >> 1) & 1, kWaitLimit, abort_flag);
      if (ok) {
        tc::fence_after_thread_sync();
        tc::tmem_ld_16(lane_addr + (uint32_t)buf * kNq, sv);
        tc::fence_before_thread_sync();
        tc::mbar_arrive(&s_free[buf]);
      } else {
        fail();
#pragma unroll
        for (int j = 0; j < 16; ++j) sv[j] = 0.f;
      }
      const bool live = s0 + i * kKeys + tid < s1;
      float s[kG];
#pragma unroll
      for (int g = 0; g < kG; ++g) {
        s[g] = live ? sv[g] * a.scale : -FLT_MAX;
        const float v = warp_max(s[g]);
        if (lane == 0) wred[0][g][warp] = v;
      }
      tc::named_barrier_sync(1, kSoftmaxThreads);
      float cmax[kG];
      bool grow = false;
#pragma unroll
      for (int g = 0; g < kG; ++g) {
        cmax[g] = fmaxf(fmaxf(wred[0][g][0], wred[0][g][1]), fmaxf(wred[0][g][2], wred[0][g][3]));
        grow = grow || (cmax[g] - m_run[g] > kRescaleThreshold);
      }
      if (i == 0) {
#pragma unroll
        for (int g = 0; g < kG; ++g) m_run[g] = cmax[g];
      } else {
        // this chunk's P tile was last read by P*V of chunk i - 2
        if (i >= 2 && !tc::mbar_wait(&o_full[i & 1], ((i - 2) >> 1) & 1, kWaitLimit, abort_flag)) fail();
        if (grow) {
          // O^T must be stable while it is rescaled: P*V of chunk i - 1 (and with it every earlier one) is complete
          if (!tc::mbar_wait(&o_full[(i - 1) & 1], ((i - 1) >> 1) & 1, kWaitLimit, abort_flag)) fail();
          tc::fence_after_thread_sync();
          float ov[16];
          tc::tmem_ld_16(lane_addr + kColO, ov);
#pragma unroll
          for (int g = 0; g < kG; ++g) {
            if (cmax[g] - m_run[g] > kRescaleThreshold) {
              const float f = __expf(m_run[g] - cmax[g]);
              ov[g] *= f;
              l_run[g] *= f;
              m_run[g] = cmax[g];
            }
          }
          tc::tmem_st_16(lane_addr + kColO, ov);
        }
      }
#pragma unroll
      for (int g = 0; g < kG; ++g) {
        const float p = live ? __expf(s[g] - m_run[g]) : 0.f;
        *reinterpret_cast<__nv_bfloat16*>(p_tile + buf * kSmallTileBytes + small_tile_offset(g, tid)) = __float2bfloat16(p);
        const float ps = warp_sum(p);
        if (lane == 0) wred[1][g][warp] = ps;
      }
      tc::fence_proxy_async();          // P was written by threads and is read by the tensor core
      tc::fence_before_thread_sync();   // orders the rescaled O^T (tcgen05.st) before the MMA that the arrival releases
      tc::mbar_arrive(&p_full[buf]);
      if (tid == 0) s_stop = *abort_flag;   // one thread samples the flag, so that all threads leave the loop together
      tc::named_barrier_sync(1, kSoftmaxThreads);
#pragma unroll
      for (int g = 0; g < kG; ++g) l_run[g] += wred[1][g][0] + wred[1][g][1] + wred[1][g][2] + wred[1][g][3];
      if (s_stop) break;
    }
    if (nchunks > 0) {
      float ov[16];
      if (!*abort_flag && tc::mbar_wait(&o_full[(nchunks - 1) & 1], ((nchunks - 1) >> 1) & 1, kWaitLimit, abort_flag)) {
        tc::fence_after_thread_sync();
        tc::tmem_ld_16(lane_addr + kColO, ov);
        tc::fence_before_thread_sync();
#pragma unroll
        for (int g = 0; g < kG; ++g) o[g] = ov[g];
      } else {
        fail();
      }
    }
    // ---- result: thread t holds output column t of the G heads ----
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      const int h = hkv * kG + g;
      if (a.nsplit == 1) {
        a.out[((int64_t)b * a.Hq + h) * kD + tid] = __float2bfloat16(l_run[g] > 0.f ? o[g] / l_run[g] : 0.f);
      } else {
        float* dst = a.partial + (((int64_t)b * a.Hq + h) * a.nsplit + split) * (kD + 2);
        dst[tid] = o[g];
        if (tid == 0) {
          dst[kD] = m_run[g];
          dst[kD + 1] = l_run[g];
        }
      }
    }
    if (a.nsplit > 1 && a.counters != nullptr) {
      // the split that arrives last merges all of them (saves a launch per layer)
      __threadfence();
      tc::named_barrier_sync(1, kSoftmaxThreads);
      if (tid == 0) {
        const uint32_t prev = atomicAdd(&a.counters[b * a.Hkv + hkv], 1u);
        s_last = (prev == (uint32_t)a.nsplit - 1u) ? 1u : 0u;
        if (s_last) a.counters[b * a.Hkv + hkv] = 0;
      }
      tc::named_barrier_sync(1, kSoftmaxThreads);
      if (s_last) {
        __threadfence();
        // Loads first, arithmetic after: a load whose value is needed by the next instruction costs a round trip to
        // L2 each, and written naively the merge is two dependent chains of nsplit loads per head. Eight splits at a
        // time: all their maxima (of every head) in one round trip, then per head their sums and partial outputs.
        const float* src0 = a.partial + ((int64_t)b * a.Hq + hkv * kG) * a.nsplit * (kD + 2);
        const int64_t head_stride = (int64_t)a.nsplit * (kD + 2);
        float m[kG];
#pragma unroll
        for (int g = 0; g < kG; ++g) m[g] = -FLT_MAX;
        for (int sp0 = 0; sp0 < a.nsplit; sp0 += 8) {
          float mv[kG][8];
#pragma unroll
          for (int g = 0; g < kG; ++g)
#pragma unroll
            for (int u = 0; u < 8; ++u)
              mv[g][u] = sp0 + u < a.nsplit ? __ldcg(src0 + g * head_stride + (sp0 + u) * (kD + 2) + kD) : -FLT_MAX;
#pragma unroll
          for (int g = 0; g < kG; ++g)
#pragma unroll
            for (int u = 0; u < 8; ++u) m[g] = fmaxf(m[g], mv[g][u]);
        }
#pragma unroll
        for (int g = 0; g < kG; ++g) {
          const float* src = src0 + g * head_stride;
          float num = 0.f, den = 0.f;
          for (int sp0 = 0; sp0 < a.nsplit; sp0 += 8) {
            float mm[8], ll[8], vv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const bool on = sp0 + u < a.nsplit;
              const float* row = src + (sp0 + u) * (kD + 2);
              mm[u] = on ? __ldcg(row + kD) : -FLT_MAX;
              ll[u] = on ? __ldcg(row + kD + 1) : 0.f;
              vv[u] = on ? __ldcg(row + tid) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const float wgt = sp0 + u < a.nsplit ? __expf(mm[u] - m[g]) : 0.f;
              num = fmaf(wgt, vv[u], num);
              den = fmaf(wgt, ll[u], den);
            }
          }
          a.out[((int64_t)b * a.Hq + hkv * kG + g) * kD + tid] = __float2bfloat16(den > 0.f ? num / den : 0.f);
        }
      }
    }
  }

  tc::fence_before_thread_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);   // copies already issued land before shared memory goes away
  }
  if (warp == 4) {
    tc::fence_after_thread_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// out[b, h, :] = sum_s exp(m_s - m) * acc_s / sum_s exp(m_s - m) * l_s
__global__ void __launch_bounds__(kD) attn_tc_combine_kernel(const TcAttnArgs a) {
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

template <int kG>
std::string launch(const CUtensorMap& mk, const CUtensorMap& mv, const TcAttnArgs& a, dim3 grid, cudaStream_t stream) {
  auto kern = attn_decode_tc_kernel<kG>;
  const std::string smem_err = reserve_dynamic_smem(kern, kSmem);
  if (!smem_err.empty()) return smem_err;
  const cudaError_t e = launch_chained(kern, grid, dim3(kThreads), kSmem, stream, mk, mv, a);
  return e == cudaSuccess ? "" : std::string("attention launch failed: ") + cudaGetErrorString(e);
}

}  // namespace

std::string attention_decode_tc(const void* q, const void* k_cache, const void* v_cache, const int32_t* seq_lens,
                                float* partial, size_t partial_floats, void* out, int B, int Hq, int Hkv, int D, int S_max,
                                int64_t q_stride_b, int64_t kv_stride_b, int64_t kv_stride_s, int nsplit, float scale,
                                cudaStream_t stream, uint32_t* status) {
  if (D != kD) return "decode attention supports head dimension 128";
  if (Hkv <= 0 || Hq % Hkv) return "query heads must be a multiple of KV heads";
  const int G = Hq / Hkv;
  if (G > kMaxG || (G & (G - 1))) return "query heads per KV head must be 1, 2, 4 or 8";
  if (nsplit < 1) nsplit = 1;
  // scratch layout as in attention_decode.cu: kCounterWords arrival counters (zero on entry, left zero), then the partials
  const size_t head = partial_floats > (size_t)kCounterWords ? (size_t)kCounterWords : 0;
  const bool in_kernel_merge = head != 0 && (size_t)B * Hkv <= (size_t)kCounterWords;
  if (head + (size_t)B * Hq * nsplit * (kD + 2) > partial_floats) return "attention scratch buffer is too small";
  if ((kv_stride_s * 2) % 16 || (kv_stride_b * 2) % 16 || reinterpret_cast<uintptr_t>(k_cache) % 16 ||
      reinterpret_cast<uintptr_t>(v_cache) % 16)
    return "KV cache rows must be 16-byte aligned";
  if (B == 0) return "";
  TcAttnArgs a{};
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.seq_lens = seq_lens;
  a.partial = partial + head;
  a.counters = in_kernel_merge ? reinterpret_cast<uint32_t*>(partial) : nullptr;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.nsplit = nsplit;
  a.q_stride_b = q_stride_b;
  a.scale = scale;
  a.idesc_s = tc::make_idesc(kKeys, kNq, 1, 1);                    // both operands K-major bf16
  a.idesc_pv = tc::make_idesc(kD, kNq, 1, 1) | tc::kIdescAMnMajor;         // A (the V chunk) is read MN-major
  a.status = status;
  CUtensorMap mk, mv;
  std::string err = tma::kv_cache_4d(&mk, k_cache, B, S_max, Hkv, kv_stride_b, kv_stride_s, kKeys);
  if (!err.empty()) return err;
  err = tma::kv_cache_4d(&mv, v_cache, B, S_max, Hkv, kv_stride_b, kv_stride_s, kKeys);
  if (!err.empty()) return err;
  const dim3 grid(B, Hkv, nsplit);
  switch (G) {
    case 1: err = launch<1>(mk, mv, a, grid, stream); break;
    case 2: err = launch<2>(mk, mv, a, grid, stream); break;
    case 4: err = launch<4>(mk, mv, a, grid, stream); break;
    case 8: err = launch<8>(mk, mv, a, grid, stream); break;
  }
  if (!err.empty()) return err;
  if (nsplit > 1 && !in_kernel_merge) launch_chained(attn_tc_combine_kernel, dim3(B, Hq), dim3(kD), 0, stream, a);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? "" : cudaGetErrorString(e);
}

}  // namespace tdx
