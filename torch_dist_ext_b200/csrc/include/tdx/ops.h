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
// With caches given (decode: token t is the new token of sequence t) the rotated key row and the
// value row are also written to k_cache / v_cache [B, S, k_heads, dim] at [t, positions[t]].
std::string rope_inplace(void* q, void* k, const int64_t* positions, const float* cos_sin_cache, int tokens,
                         int q_heads, int k_heads, int dim, int64_t q_stride, int64_t k_stride, int dtype,
                         cudaStream_t stream, const void* v = nullptr, int64_t v_stride = 0, void* k_cache = nullptr,
                         void* v_cache = nullptr, int64_t cache_stride_b = 0, int64_t cache_stride_s = 0);

// Greedy sampling over a vocabulary sharded across ranks, in two launches around one fused all-reduce:
// argmax_pack writes {largest logit, its index + index_base, 0, 0} of every row of logits [tokens, vocab] fp32 (rows
// `ld` elements apart) into slot `rank` of pack [tokens, 4 * nranks] fp32 and zeroes the other slots, so that the
// sum of `pack` over the ranks holds every rank's candidate; select_token picks the winner per row (the lowest
// index among equal logits) into out [tokens] int64.
std::string argmax_pack(const float* logits, int64_t ld, int tokens, int vocab, int index_base, int rank, int nranks,
                        float* pack, cudaStream_t stream);
std::string select_token(const float* gathered, int tokens, int nranks, int64_t* out, cudaStream_t stream);

// Decode attention over a contiguous bf16 KV cache [B, S_max, Hkv, 128] for one new token per
// sequence: q [B, Hq, 128] -> out [B, Hq, 128]. `partial` is scratch of at least
// 4096 + B * Hq * nsplit * 130 floats whose first 4096 words must be ZERO on entry (arrival counters;
// the kernel leaves them zero again). Strides are in elements.
std::string attention_decode(const void* q, const void* k_cache, const void* v_cache, const int32_t* seq_lens,
                             float* partial, size_t partial_floats, void* out, int B, int Hq, int Hkv, int D, int S_max,
                             int64_t q_stride_b, int64_t kv_stride_b, int64_t kv_stride_s, int nsplit, float scale,
                             cudaStream_t stream, uint32_t* status = nullptr);
// The same computation with both products of a chunk on the tensor cores (attention_decode_tc.cu); same
// arguments and scratch layout.
std::string attention_decode_tc(const void* q, const void* k_cache, const void* v_cache, const int32_t* seq_lens,
                                float* partial, size_t partial_floats, void* out, int B, int Hq, int Hkv, int D, int S_max,
                                int64_t q_stride_b, int64_t kv_stride_b, int64_t kv_stride_s, int nsplit, float scale,
                                cudaStream_t stream, uint32_t* status = nullptr);

// Causal self-attention over one prompt on the tensor cores (attention_prefill_tc.cu): q [S, Hq, 128],
// k / v [S, Hkv, 128] bf16 with unit stride inside a head, heads 128 elements apart and rows `*_stride_s`
// elements apart (views into a fused qkv projection are fine); out [S, Hq, 128] contiguous. Query i
// attends to keys 0 .. i.
std::string attention_prefill_tc(const void* q, const void* k, const void* v, void* out, int S, int Hq, int Hkv, int D,
                                 int64_t q_stride_s, int64_t k_stride_s, int64_t v_stride_s, float scale, cudaStream_t stream,
                                 uint32_t* status = nullptr);

// Clock stamps of the last prompt attention launch (tracing flavour only): 3 roles x 64 chunks x 8 slots, see
// attention_prefill_tc.cu.
std::string attention_prefill_probe(unsigned long long* dst, size_t count);

}  // namespace tdx
