// Split-KV decode attention for grouped-query heads (head dimension 128, bf16 KV cache).
//
// One CTA handles one (sequence, KV head, KV split) and all G query heads that share the KV head,
// so every K/V byte is read from HBM exactly once per step. Per chunk of 128 cache positions:
//   A  each thread takes ONE position and forms its G scores (q is broadcast from shared memory,
//      the K row is read with 16-byte loads) - no cross-lane reduction per position;
//   B  chunk maximum and sum per head (one block reduction per chunk), online-softmax rescale;
//   C  threads re-map to (position group, 8-column slice) and accumulate P*V from shared-memory
//      probabilities, V rows read coalesced.
// Splits write (max, sum, unnormalised output) to a scratch buffer; a second small kernel merges
// them. Decode attention is bandwidth-bound (G FLOP per byte), so this path uses the SIMT pipes;
// the tensor cores are kept for the GEMMs.
//
// Not part of the reference (it has no attention); needed by the Llama-shaped decoder layers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cfloat>
#include "tdx/ops.h"
#include "tdx/ptx.cuh"
#include "tdx/sync.cuh"
#include "tdx/vec.cuh"

namespace tdx {
namespace {

constexpr int kD = 128;
constexpr int kChunk = 128;
constexpr int kAttnThreads = 128;
constexpr int kMaxG = 8;

struct AttnArgs {
  const __nv_bfloat16* q;      // [B, Hq, D]
  const __nv_bfloat16* k;      // [B, S_max, Hkv, D]
  const __nv_bfloat16* v;
  const int32_t* seq_lens;     // [B] valid positions per sequence
  float* partial;              // [B, Hq, nsplit, D + 2]
  __nv_bfloat16* out;          // [B, Hq, D]
  int B, Hq, Hkv, S_max, nsplit;
  int64_t q_stride_b, kv_stride_b, kv_stride_s;   // elements
  float scale;
};

template <int kG>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_split_kernel(const AttnArgs a) {
  __shared__ float q_s[kG][kD];
  __shared__ float p_s[kG][kChunk];
  __shared__ float acc_s[4][kG][kD];      // per-warp partial outputs, merged at the end
  const int b = blockIdx.x, hkv = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int len = a.seq_lens[b];
  const int per = (len + a.nsplit - 1) / a.nsplit;
  const int s0 = split * per, s1 = min(len, s0 + per);

  for (int i = tid; i < kG * kD; i += kAttnThreads) {
    const int g = i / kD, d = i % kD;
    q_s[g][d] = __bfloat162float(a.q[(int64_t)b * a.q_stride_b + (int64_t)(hkv * kG + g) * kD + d]) * a.scale;
  }
  __syncthreads();

  float m_run[kG], l_run[kG];
  // phase C mapping: 16 threads cover one V row (8 columns each); a warp handles 2 rows per step
  const int vslice = (lane & 15) * 8;
  const int vsub = lane >> 4;
  float acc[kG][8];
#pragma unroll
  for (int g = 0; g < kG; ++g) {
    m_run[g] = -FLT_MAX;
    l_run[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }
  const __nv_bfloat16* kbase = a.k + (int64_t)b * a.kv_stride_b + (int64_t)hkv * kD;
  const __nv_bfloat16* vbase = a.v + (int64_t)b * a.kv_stride_b + (int64_t)hkv * kD;

  for (int c0 = s0; c0 < s1; c0 += kChunk) {
    const int pos = c0 + tid;
    // ---- A: one position per thread ----
    float s[kG];
#pragma unroll
    for (int g = 0; g < kG; ++g) s[g] = 0.f;
    if (pos < s1) {
      const char* krow = reinterpret_cast<const char*>(kbase + (int64_t)pos * a.kv_stride_s);
#pragma unroll 4
      for (int d = 0; d < kD; d += 8) {
        float kf[8];
        unpack<__nv_bfloat16>(ptx::ld_v4(krow + d * 2), kf);
#pragma unroll
        for (int g = 0; g < kG; ++g)
#pragma unroll
          for (int i = 0; i < 8; ++i) s[g] = fmaf(q_s[g][d + i], kf[i], s[g]);
      }
    } else {
#pragma unroll
      for (int g = 0; g < kG; ++g) s[g] = -FLT_MAX;
    }
    // ---- B: chunk statistics, rescale ----
    // chunk maximum per head (scores can be negative: the identity is -FLT_MAX)
    float cmaxv[kG];
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      float v = s[g];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
      if (lane == 0) acc_s[0][g][warp] = v;   // scratch use before the final merge
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < kG; ++g)
      cmaxv[g] = fmaxf(fmaxf(acc_s[0][g][0], acc_s[0][g][1]), fmaxf(acc_s[0][g][2], acc_s[0][g][3]));
    float corr[kG];
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      const float m_new = fmaxf(m_run[g], cmaxv[g]);
      corr[g] = __expf(m_run[g] - m_new);
      const float p = (pos < s1) ? __expf(s[g] - m_new) : 0.f;
      p_s[g][tid] = p;
      float ps = p;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      if (lane == 0) acc_s[1][g][warp] = ps;
      m_run[g] = m_new;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      const float csum = acc_s[1][g][0] + acc_s[1][g][1] + acc_s[1][g][2] + acc_s[1][g][3];
      l_run[g] = l_run[g] * corr[g] + csum;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[g][i] *= corr[g];
    }
    // ---- C: P * V; warp w covers chunk rows w*32 .. w*32+31, two rows per step ----
    const int rows = min(kChunk, s1 - c0);
    for (int r = warp * 32 + vsub; r < min(rows, warp * 32 + 32); r += 2) {
      float vf[8];
      unpack<__nv_bfloat16>(ptx::ld_v4(reinterpret_cast<const char*>(vbase + (int64_t)(c0 + r) * a.kv_stride_s) + vslice * 2), vf);
#pragma unroll
      for (int g = 0; g < kG; ++g) {
        const float p = p_s[g][r];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(p, vf[i], acc[g][i]);
      }
    }
    __syncthreads();   // p_s / scratch reused by the next chunk
  }
  // merge the two half-warps, then the four warps
#pragma unroll
  for (int g = 0; g < kG; ++g)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] += __shfl_xor_sync(0xffffffffu, acc[g][i], 16);
  if (vsub == 0) {
#pragma unroll
    for (int g = 0; g < kG; ++g)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc_s[warp][g][vslice + i] = acc[g][i];
  }
  __syncthreads();
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
}

// out[b, h, :] = sum_s exp(m_s - m) * acc_s / sum_s exp(m_s - m) * l_s
__global__ void __launch_bounds__(kD) attn_combine_kernel(const AttnArgs a) {
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

std::string attention_decode(const void* q, const void* k_cache, const void* v_cache, const int32_t* seq_lens,
                             float* partial, size_t partial_floats, void* out, int B, int Hq, int Hkv, int D, int S_max,
                             int64_t q_stride_b, int64_t kv_stride_b, int64_t kv_stride_s, int nsplit, float scale,
                             cudaStream_t stream) {
  if (D != kD) return "decode attention supports head dimension 128";
  if (Hkv <= 0 || Hq % Hkv) return "query heads must be a multiple of KV heads";
  const int G = Hq / Hkv;
  if (G > kMaxG || (G & (G - 1))) return "query heads per KV head must be 1, 2, 4 or 8";
  if (nsplit < 1) nsplit = 1;
  if ((size_t)B * Hq * nsplit * (kD + 2) > partial_floats) return "attention scratch buffer is too small";
  if ((kv_stride_s * 2) % 16 || (kv_stride_b * 2) % 16 || reinterpret_cast<uintptr_t>(k_cache) % 16 ||
      reinterpret_cast<uintptr_t>(v_cache) % 16)
    return "KV cache rows must be 16-byte aligned";
  if (B == 0) return "";
  AttnArgs a{};
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.k = static_cast<const __nv_bfloat16*>(k_cache);
  a.v = static_cast<const __nv_bfloat16*>(v_cache);
  a.seq_lens = seq_lens;
  a.partial = partial;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.S_max = S_max; a.nsplit = nsplit;
  a.q_stride_b = q_stride_b; a.kv_stride_b = kv_stride_b; a.kv_stride_s = kv_stride_s;
  a.scale = scale;
  const dim3 grid(B, Hkv, nsplit);
  switch (G) {
    case 1: attn_decode_split_kernel<1><<<grid, kAttnThreads, 0, stream>>>(a); break;
    case 2: attn_decode_split_kernel<2><<<grid, kAttnThreads, 0, stream>>>(a); break;
    case 4: attn_decode_split_kernel<4><<<grid, kAttnThreads, 0, stream>>>(a); break;
    case 8: attn_decode_split_kernel<8><<<grid, kAttnThreads, 0, stream>>>(a); break;
  }
  attn_combine_kernel<<<dim3(B, Hq), kD, 0, stream>>>(a);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? "" : cudaGetErrorString(e);
}

}  // namespace tdx
