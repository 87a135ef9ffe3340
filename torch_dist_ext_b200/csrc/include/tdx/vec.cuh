// 16-byte vector helpers: unpack to fp32, pack with one round-to-nearest-even, and the
// sentinel tests used by the Lamport protocols.
//
// Covers what the reference does with vec_t / vec_add_ / vec_add_r_
// (src/common/all_reduce_fusion_impl.h:208-298) and with its per-dtype negative-zero
// helpers (src/common/negzero.h:3-66). The sentinel here is ONE 32-bit pattern for every
// dtype (fp32 -0.0, which for 16-bit types is the pair {+0.0, -0.0}); because 32-bit
// aligned accesses are single-copy atomic, readiness is tested per 32-bit lane and a
// change of dtype between calls needs no re-initialisation of the buffers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include "tdx/comm.h"

namespace tdx {

template <typename T>
struct VecTraits;
template <>
struct VecTraits<float> {
  static constexpr int kVec = 4;
  static constexpr int kDType = kF32;
};
template <>
struct VecTraits<__half> {
  static constexpr int kVec = 8;
  static constexpr int kDType = kF16;
};
template <>
struct VecTraits<__nv_bfloat16> {
  static constexpr int kVec = 8;
  static constexpr int kDType = kBF16;
};

template <typename T>
__device__ __forceinline__ void unpack(const uint4& v, float (&f)[VecTraits<T>::kVec]);

template <>
__device__ __forceinline__ void unpack<float>(const uint4& v, float (&f)[4]) {
  f[0] = __uint_as_float(v.x);
  f[1] = __uint_as_float(v.y);
  f[2] = __uint_as_float(v.z);
  f[3] = __uint_as_float(v.w);
}
template <>
__device__ __forceinline__ void unpack<__half>(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <>
__device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // bf16 -> fp32 is a 16-bit shift; cheaper than the cvt path
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <typename T>
__device__ __forceinline__ uint4 pack(const float (&f)[VecTraits<T>::kVec]);

template <>
__device__ __forceinline__ uint4 pack<float>(const float (&f)[4]) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                    __float_as_uint(f[3]));
}
template <>
__device__ __forceinline__ uint4 pack<__half>(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ uint4 pack<__nv_bfloat16>(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Round a vector of fp32 to T and back, in place: the value that a store-then-load in T gives.
template <typename T>
__device__ __forceinline__ void round_through(float (&f)[VecTraits<T>::kVec]) {
  if constexpr (sizeof(T) == 4) {
    return;
  } else {
    uint4 v = pack<T>(f);
    unpack<T>(v, f);
  }
}

// ---- sentinel ------------------------------------------------------------------

__device__ __forceinline__ bool all_arrived(const uint4& v) {
  return (v.x != kSentinel) & (v.y != kSentinel) & (v.z != kSentinel) & (v.w != kSentinel);
}

// Payload lanes that happen to equal the sentinel become +0.0 (numerically the same value).
__device__ __forceinline__ uint4 scrub(uint4 v) {
  v.x = (v.x == kSentinel) ? 0u : v.x;
  v.y = (v.y == kSentinel) ? 0u : v.y;
  v.z = (v.z == kSentinel) ? 0u : v.z;
  v.w = (v.w == kSentinel) ? 0u : v.w;
  return v;
}

__device__ __forceinline__ uint4 sentinel_vec() {
  return make_uint4(kSentinel, kSentinel, kSentinel, kSentinel);
}

}  // namespace tdx
