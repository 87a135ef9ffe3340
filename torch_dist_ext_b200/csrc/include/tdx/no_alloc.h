// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (xytpai/torch_dist_ext has no attention and no
// allocation-free interface); it is an addition of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits - inside a CUDA-graph capture region of
// an engine that forbids allocation while capturing, in a serving loop whose memory pool is owned and
// fully handed out by another component, or in a plug-in that is only given input and output pointers
// and may not touch the allocator. The regular entry (tdx::attention_decode, reached from Python through
// torch.ops.torch_dist_ext.attention_decode) asks its caller for a scratch buffer that holds the
// per-split partial results (maximum, sum and unnormalised output per query head and KV split), which
// in practice means somebody allocates it. Here that scratch is a fixed array that lives inside the
// library image on the device.
//
// Limits and rules:
//  * batch * query_heads * kv_splits must not exceed TDX_NOALLOC_ATTN_MAX_ROWS (16384); larger
//    requests are rejected with a message, nothing is launched. The array takes
//    16384 * 130 * 4 bytes (about 8.1 MiB) on EVERY GPU that loads the library, until the process ends.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and opts the
//    kernels in to their shared-memory size. Make that first call before any stream capture.
//  * All calls share the one array and it keeps the previous call's contents. The partial rows are
//    written before they are read, so they need no clearing; the 4096 arrival counters in front of
//    them must start at zero, which holds when the library is loaded and is restored by every call
//    that runs to its end (the partial rows always start behind the counters, also when batch * kv_heads
//    exceeds 4096 and a separate kernel merges the splits). Two calls that overlap on the GPU (two streams, two host threads) race on
//    both. Issue calls on one stream, or serialise them yourself.
//  * No cudaMalloc, cudaFree, or allocating library routine is called; inputs and outputs are the caller's.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define TDX_NOALLOC_ATTN_MAX_ROWS 16384

#ifdef __cplusplus
extern "C" {
#endif

// q        [batch, q_heads, 128] bf16, row pitch q_stride_b elements, heads densely packed
// k_cache  [batch, s_max, kv_heads, 128] bf16 (v_cache alike); strides in elements
// seq_lens [batch] int32 valid positions per sequence (device memory)
// out      [batch, q_heads, 128] bf16, contiguous
// Returns 0 on success. On failure returns non-zero and, if `err` is not null, writes a
// NUL-terminated reason of at most err_len bytes.
int tdx_attention_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, const int32_t* seq_lens,
                                 void* out, int batch, int q_heads, int kv_heads, int s_max, int64_t q_stride_b,
                                 int64_t kv_stride_b, int64_t kv_stride_s, int kv_splits, float scale,
                                 cudaStream_t stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
