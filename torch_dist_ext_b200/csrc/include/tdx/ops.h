// Host-side launchers of the standalone ops (elementwise.cu), the GEMMs and attention.
// Every function returns an empty string on success, else the reason.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <string>
#include "tdx/comm.h"

namespace tdx {

// x [rows, cols] (dtype code) -> q e4m3 [rows, cols], scales fp32 [rows] or [rows, cols/128].
std::string quant_fp8(const void* x, void* q, float* scales, int rows, int cols, int dtype, bool block128,
                      cudaStream_t stream);

// in [rows, 2*inter] = {gate | up} -> out [rows, inter] = silu(gate) * up, in `dtype` or (quant_block128)
// e4m3 with fp32 scales [rows, inter/128].
std::string silu_mul(const void* in, void* out, float* scales, int rows, int inter, int dtype, bool quant_block128,
                     cudaStream_t stream);

// Rotary embedding in place on q [tokens, q_heads, dim] and k [tokens, k_heads, dim] (row strides in
// elements), rotate-half layout; cos_sin_cache [max_pos, dim] fp32 = {cos | sin}.
std::string rope_inplace(void* q, void* k, const int64_t* positions, const float* cos_sin_cache, int tokens,
                         int q_heads, int k_heads, int dim, int64_t q_stride, int64_t k_stride, int dtype,
                         cudaStream_t stream);

}  // namespace tdx
