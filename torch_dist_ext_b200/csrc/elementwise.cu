// Standalone memory-bound ops of a decoder layer, written as 16-byte-vector sm_100a kernels:
// fp8 e4m3 quantisation (per-token and 1x128 block scales), SiLU(gate) * up (optionally
// quantising its output for an fp8 GEMM), and rotary position embedding (rotate-half layout).
//
// The reference contains none of these (its only device code is the fused all-reduce,
// src/common/all_reduce_fusion_impl.h); they are the remaining hot ops of the Llama-shaped
// tensor-parallel layers built on top of it.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "tdx/launch.h"
#include "tdx/ops.h"
#include "tdx/ptx.cuh"
#include "tdx/sync.cuh"
#include "tdx/vec.cuh"

namespace tdx {
namespace {

constexpr float kFp8MaxQ = 448.f;
constexpr float kAmaxFloorQ = 1e-10f;

template <int kVec>
__device__ __forceinline__ void store_fp8_vec(void* dst, const float (&q)[kVec]) {
  if constexpr (kVec == 8) {
    uint2 o;
    o.x = ptx::cvt_e4m3x4(q[0], q[1], q[2], q[3]);
    o.y = ptx::cvt_e4m3x4(q[4], q[5], q[6], q[7]);
    *reinterpret_cast<uint2*>(dst) = o;
  } else {
    *reinterpret_cast<uint32_t*>(dst) = ptx::cvt_e4m3x4(q[0], q[1], q[2], q[3]);
  }
}

// ---- fp8 quantisation ---------------------------------------------------------------------
// One CTA per row (grid-stride). kBlock: one scale per 128 columns; else one scale per row,
// found in a first pass over the row (the second pass re-reads it from L1/L2).
template <typename T, bool kBlock>
__global__ void __launch_bounds__(512) quant_fp8_kernel(const T* __restrict__ x, uint8_t* __restrict__ q,
                                                        float* __restrict__ scales, int rows, int cols) {
  constexpr int kVec = VecTraits<T>::kVec;
  __shared__ float red[32];
  ptx::pdl_wait();                // inputs come from earlier kernels of the stream
  ptx::pdl_launch_dependents();
  const int nvec = cols / kVec;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const char* src = reinterpret_cast<const char*>(x + (size_t)row * cols);
    uint8_t* dst = q + (size_t)row * cols;
    if constexpr (kBlock) {
      constexpr int kLanes = 128 / kVec;
      // nvec is a multiple of kLanes, so whole lane groups are active or inactive together
      for (int base = 0; base < nvec; base += blockDim.x) {
        const int i = base + threadIdx.x;
        float f[kVec];
        float amax = 0.f;
        if (i < nvec) {
          unpack<T>(ptx::ld_stream_v4(src + (size_t)i * 16), f);
#pragma unroll
          for (int k = 0; k < kVec; ++k) amax = fmaxf(amax, fabsf(f[k]));
        }
        amax = group_max<kLanes>(amax);
        const float scale = fmaxf(amax, kAmaxFloorQ) / kFp8MaxQ;
        const float inv = 1.f / scale;
        if (i < nvec) {
#pragma unroll
          for (int k = 0; k < kVec; ++k) f[k] *= inv;
          store_fp8_vec<kVec>(dst + (size_t)i * kVec, f);
          if ((threadIdx.x & (kLanes - 1)) == 0) scales[(size_t)row * (cols / 128) + (size_t)i * kVec / 128] = scale;
        }
      }
    } else {
      float amax = 0.f;
      for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float f[kVec];
        unpack<T>(ptx::ld_v4(src + (size_t)i * 16), f);
#pragma unroll
        for (int k = 0; k < kVec; ++k) amax = fmaxf(amax, fabsf(f[k]));
      }
      amax = block_allreduce<true>(amax, red);
      const float scale = fmaxf(amax, kAmaxFloorQ) / kFp8MaxQ;
      const float inv = 1.f / scale;
      if (threadIdx.x == 0) scales[row] = scale;
      for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float f[kVec];
        unpack<T>(ptx::ld_v4(src + (size_t)i * 16), f);
#pragma unroll
        for (int k = 0; k < kVec; ++k) f[k] *= inv;
        store_fp8_vec<kVec>(dst + (size_t)i * kVec, f);
      }
      __syncthreads();  // `red` is reused by the next row
    }
  }
}

// ---- SiLU(gate) * up --------------------------------------------------------------------------
// in: [rows, 2*inter] with the gate in the first half of each row; out: [rows, inter].
// kQuant: out is e4m3 with 1x128 block scales (input of an fp8 block-scaled down projection).
template <typename T, bool kQuant>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* __restrict__ in, void* __restrict__ out,
                                                       float* __restrict__ scales, int rows, int inter) {
  constexpr int kVec = VecTraits<T>::kVec;
  ptx::pdl_wait();                // inputs come from earlier kernels of the stream
  ptx::pdl_launch_dependents();
  const int nvec = inter / kVec;
  const size_t total = (size_t)rows * nvec;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  // Warp-uniform trip count: the quantising variant shuffles inside the loop.
  for (size_t base = (size_t)blockIdx.x * blockDim.x + (threadIdx.x & ~31u); base < total; base += stride) {
    const size_t idx = base + (threadIdx.x & 31u);
    const bool live = idx < total;
    const size_t row = live ? idx / nvec : 0;
    const int i = live ? int(idx % nvec) : 0;
    float g[kVec], u[kVec], y[kVec];
    if (live) {
      const char* base = reinterpret_cast<const char*>(in + row * 2 * (size_t)inter);
      unpack<T>(ptx::ld_stream_v4(base + (size_t)i * 16), g);
      unpack<T>(ptx::ld_stream_v4(base + (size_t)inter * sizeof(T) + (size_t)i * 16), u);
#pragma unroll
      for (int k = 0; k < kVec; ++k) y[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
    } else {
#pragma unroll
      for (int k = 0; k < kVec; ++k) y[k] = 0.f;
    }
    if constexpr (kQuant) {
      constexpr int kLanes = 128 / kVec;
      round_through<T>(y);  // quantise what a separate kernel would have stored in T
      float amax = 0.f;
#pragma unroll
      for (int k = 0; k < kVec; ++k) amax = fmaxf(amax, fabsf(y[k]));
      // lanes of one 128-column block are adjacent: nvec % kLanes == 0 and idx is linear in i
      amax = group_max<kLanes>(amax);
      const float scale = fmaxf(amax, kAmaxFloorQ) / kFp8MaxQ;
      const float inv = 1.f / scale;
      if (live) {
#pragma unroll
        for (int k = 0; k < kVec; ++k) y[k] *= inv;
        store_fp8_vec<kVec>(static_cast<uint8_t*>(out) + row * inter + (size_t)i * kVec, y);
        if ((i & (kLanes - 1)) == 0) scales[row * (inter / 128) + (size_t)i * kVec / 128] = scale;
      }
    } else {
      if (live) ptx::st_stream_v4(static_cast<char*>(out) + (row * inter + (size_t)i * kVec) * sizeof(T), pack<T>(y));
    }
  }
}

// ---- rotary embedding (rotate-half / "neox" layout), in place ------------------------------------
// x: [tokens, heads, dim]; cache: [max_pos, dim] fp32 = {cos[0..dim/2), sin[0..dim/2)} per position.
template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(T* __restrict__ q, T* __restrict__ k,
                                                   const int64_t* __restrict__ positions,
                                                   const float* __restrict__ cache, int tokens, int q_heads,
                                                   int k_heads, int dim, int64_t q_stride, int64_t k_stride,
                                                   const T* __restrict__ v, int64_t v_stride, T* __restrict__ k_cache,
                                                   T* __restrict__ v_cache, int64_t cache_stride_b,
                                                   int64_t cache_stride_s) {
  constexpr int kVec = VecTraits<T>::kVec;
  ptx::pdl_wait();                // inputs come from earlier kernels of the stream
  ptx::pdl_launch_dependents();
  const int half = dim / 2;
  const int per_head = half / kVec;
  const int items = (q_heads + k_heads) * per_head;
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    const int64_t pos = positions[t];
    const float* cs = cache + pos * dim;
    // decode: sequence t appends its new key/value row at position pos of its cache
    T* kc = k_cache ? k_cache + t * cache_stride_b + pos * cache_stride_s : nullptr;
    if (v_cache) {
      T* vc = v_cache + t * cache_stride_b + pos * cache_stride_s;
      const T* vsrc = v + (size_t)t * v_stride;
      for (int it = threadIdx.x; it < k_heads * dim / kVec; it += blockDim.x)
        *reinterpret_cast<uint4*>(vc + it * kVec) = ptx::ld_v4(vsrc + it * kVec);
    }
    for (int it = threadIdx.x; it < items; it += blockDim.x) {
      const int head = it / per_head;
      const int off = (it % per_head) * kVec;
      T* base = head < q_heads ? q + (size_t)t * q_stride + (size_t)head * dim
                               : k + (size_t)t * k_stride + (size_t)(head - q_heads) * dim;
      float a[kVec], b[kVec];
      unpack<T>(ptx::ld_v4(base + off), a);
      unpack<T>(ptx::ld_v4(base + half + off), b);
      float ra[kVec], rb[kVec];
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        const float c = cs[off + i], s = cs[half + off + i];
        ra[i] = a[i] * c - b[i] * s;
        rb[i] = b[i] * c + a[i] * s;
      }
      *reinterpret_cast<uint4*>(base + off) = pack<T>(ra);
      *reinterpret_cast<uint4*>(base + half + off) = pack<T>(rb);
      if (kc && head >= q_heads) {
        T* dst = kc + (size_t)(head - q_heads) * dim;
        *reinterpret_cast<uint4*>(dst + off) = pack<T>(ra);
        *reinterpret_cast<uint4*>(dst + half + off) = pack<T>(rb);
      }
    }
  }
}

int grid_for(size_t work_items, int threads, int max_blocks = 148 * 8) {
  size_t b = (work_items + threads - 1) / threads;
  if (b > (size_t)max_blocks) b = max_blocks;
  return b == 0 ? 1 : int(b);
}

}  // namespace

#define TDX_DISPATCH_DTYPE(dtype, ...)                                    \
  switch (dtype) {                                                        \
    case kF32: { using T = float; __VA_ARGS__; break; }                   \
    case kF16: { using T = __half; __VA_ARGS__; break; }                  \
    case kBF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }          \
    default: return "unsupported dtype";                                  \
  }

// Greedy sampling over a vocabulary that is sharded across ranks. One block per token: the largest logit of this
// rank's slice and its index in the whole vocabulary go into slot `rank` of the token's row of `pack`
// [tokens, 4 * nranks] fp32 as {value, index, 0, 0}; the other ranks' slots of the row are set to zero, so that the
// SUM of `pack` over the ranks (one call of the fused all-reduce) is the gather of every rank's candidate. Indices
// stay exact in fp32 up to 2^24. Of equal logits the lowest index wins; a NaN never wins.
__global__ void __launch_bounds__(1024) argmax_pack_kernel(const float* __restrict__ logits, int64_t ld, int vocab,
                                                           int index_base, int rank, int nranks, float* __restrict__ pack) {
  ptx::pdl_wait();
  ptx::pdl_launch_dependents();
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  const int t = blockIdx.x;
  const float* row = logits + (int64_t)t * ld;
  float best = -INFINITY;
  int at = 0x7fffffff;
  auto take = [&](float v, int i) {
    if (v > best) { best = v; at = i; }      // a thread walks its indices upwards, so the first of equal values stays
  };
  // 16-byte loads, four of them in flight per thread, when the row allows it; single elements otherwise and at the end
  const bool vec = ((reinterpret_cast<uintptr_t>(row) & 15u) == 0);
  const int nvec = vec ? vocab / 4 : 0;
  const float4* row4 = reinterpret_cast<const float4*>(row);
  int i = threadIdx.x;
  for (; i + 3 * (int)blockDim.x < nvec; i += 4 * blockDim.x) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldcs(row4 + i + u * blockDim.x);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = 4 * (i + u * (int)blockDim.x);
      take(v[u].x, e);
      take(v[u].y, e + 1);
      take(v[u].z, e + 2);
      take(v[u].w, e + 3);
    }
  }
  for (; i < nvec; i += blockDim.x) {
    const float4 v = __ldcs(row4 + i);
    take(v.x, 4 * i);
    take(v.y, 4 * i + 1);
    take(v.z, 4 * i + 2);
    take(v.w, 4 * i + 3);
  }
  for (int e = 4 * nvec + threadIdx.x; e < vocab; e += blockDim.x) take(row[e], e);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, off);
    const int oi = __shfl_xor_sync(0xffffffffu, at, off);
    if (ov > best || (ov == best && oi < at)) { best = ov; at = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = at; }
  __syncthreads();
  if (threadIdx.x < 4 * nranks) {
    float out = 0.f;
    const int slot = threadIdx.x >> 2, word = threadIdx.x & 3;
    if (slot == rank && word < 2) {
      best = s_val[0];
      at = s_idx[0];
      for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
        if (s_val[w] > best || (s_val[w] == best && s_idx[w] < at)) { best = s_val[w]; at = s_idx[w]; }
      if (at == 0x7fffffff) at = 0;   // a row of NaN or -inf: a valid index all the same
      out = word == 0 ? best : float(index_base + at);
    }
    pack[(int64_t)t * 4 * nranks + threadIdx.x] = out;
  }
}

// The winner among the ranks' candidates: gathered [tokens, 4 * nranks] fp32 -> token ids int64 [tokens].
__global__ void __launch_bounds__(128) select_token_kernel(const float* __restrict__ gathered, int tokens, int nranks,
                                                           int64_t* __restrict__ out) {
  ptx::pdl_wait();
  ptx::pdl_launch_dependents();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const float4* row = reinterpret_cast<const float4*>(gathered) + (int64_t)t * nranks;
  float best = row[0].x;
  float at = row[0].y;
  for (int r = 1; r < nranks; ++r) {
    const float4 c = row[r];
    if (c.x > best || (c.x == best && c.y < at)) { best = c.x; at = c.y; }
  }
  out[t] = (int64_t)at;
}

std::string argmax_pack(const float* logits, int64_t ld, int tokens, int vocab, int index_base, int rank, int nranks,
                        float* pack, cudaStream_t stream) {
  if (nranks < 1 || nranks > kMaxRanks || rank < 0 || rank >= nranks) return "rank / nranks out of range";
  if (vocab < 1 || (int64_t)index_base + vocab > (1 << 24)) return "vocabulary indices must stay below 2^24";
  if (tokens == 0) return "";
  launch_chained(argmax_pack_kernel, dim3(tokens), dim3(vocab >= 8192 ? 1024 : 256), 0, stream, logits, ld, vocab, index_base, rank, nranks, pack);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? "" : cudaGetErrorString(e);
}

std::string select_token(const float* gathered, int tokens, int nranks, int64_t* out, cudaStream_t stream) {
  if (nranks < 1 || nranks > kMaxRanks) return "nranks out of range";
  if (reinterpret_cast<uintptr_t>(gathered) & 15u) return "candidates must be 16-byte aligned";
  if (tokens == 0) return "";
  launch_chained(select_token_kernel, dim3((tokens + 127) / 128), dim3(128), 0, stream, gathered, tokens, nranks, out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? "" : cudaGetErrorString(e);
}

std::string quant_fp8(const void* x, void* q, float* scales, int rows, int cols, int dtype, bool block128,
                      cudaStream_t stream) {
  const int vec = dtype == kF32 ? 4 : 8;
  if (cols % vec) return "columns must be a multiple of 16 bytes";
  if (block128 && cols % 128) return "1x128 block scaling needs columns % 128 == 0";
  if (rows == 0) return "";
  const int nvec = cols / vec;
  int threads = (nvec + 31) / 32 * 32;
  if (threads > 512) threads = 512;
  const int grid = rows < 148 * 4 ? rows : 148 * 4;
  TDX_DISPATCH_DTYPE(dtype, {
    if (block128)
      launch_chained(quant_fp8_kernel<T, true>, dim3(grid), dim3(threads), 0, stream, static_cast<const T*>(x), static_cast<uint8_t*>(q), scales, rows, cols);
    else
      launch_chained(quant_fp8_kernel<T, false>, dim3(grid), dim3(threads), 0, stream, static_cast<const T*>(x), static_cast<uint8_t*>(q), scales, rows, cols);
  });
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? "" : cudaGetErrorString(e);
}

std::string silu_mul(const void* in, void* out, float* scales, int rows, int inter, int dtype, bool quant_block128,
                     cudaStream_t stream) {
  const int vec = dtype == kF32 ? 4 : 8;
  if (inter % vec) return "intermediate size must be a multiple of 16 bytes";
  if (quant_block128 && inter % 128) return "1x128 block scaling needs intermediate size % 128 == 0";
  if (rows == 0) return "";
  const size_t total = (size_t)rows * (inter / vec);
  const int grid = grid_for(total, 256);
  TDX_DISPATCH_DTYPE(dtype, {
    if (quant_block128)
      launch_chained(silu_mul_kernel<T, true>, dim3(grid), dim3(256), 0, stream, static_cast<const T*>(in), out, scales, rows, inter);
    else
      launch_chained(silu_mul_kernel<T, false>, dim3(grid), dim3(256), 0, stream, static_cast<const T*>(in), out, scales, rows, inter);
  });
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? "" : cudaGetErrorString(e);
}

std::string rope_inplace(void* q, void* k, const int64_t* positions, const float* cos_sin_cache, int tokens,
                         int q_heads, int k_heads, int dim, int64_t q_stride, int64_t k_stride, int dtype,
                         cudaStream_t stream, const void* v, int64_t v_stride, void* k_cache, void* v_cache,
                         int64_t cache_stride_b, int64_t cache_stride_s) {
  const int vec = dtype == kF32 ? 4 : 8;
  if (dim % (2 * vec)) return "head dimension must be a multiple of 2 x 16 bytes";
  if (tokens == 0) return "";
  const int grid = tokens < 148 * 8 ? tokens : 148 * 8;
  TDX_DISPATCH_DTYPE(dtype, {
    launch_chained(rope_kernel<T>, dim3(grid), dim3(256), 0, stream, static_cast<T*>(q), static_cast<T*>(k), positions, cos_sin_cache, tokens,
                                             q_heads, k_heads, dim, q_stride, k_stride, static_cast<const T*>(v), v_stride,
                                             static_cast<T*>(k_cache), static_cast<T*>(v_cache), cache_stride_b,
                                             cache_stride_s);
  });
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? "" : cudaGetErrorString(e);
}

}  // namespace tdx
