// Host interface of the tcgen05 GEMM (gemm_tcgen05.cu).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <string>
#include "tdx/comm.h"

namespace tdx {

// D[x, y] = sum_k X[x, k] * Y[y, k];  D[x, y] is written to out[x * sx + y * sy].
// What the split-K finalizer of gemm_tn does with the summed tile instead of a plain store. Both kinds combine row r
// of a 128-row tile with row r + 64, so they need X on the 128-row side (the weights: decode orientation), at least
// two K splits (the finalizer is the CTA that arrives last at a tile) and a 16-bit or fp32 output.
enum PairEpilogueKind { kEpiNone = 0, kEpiRopeKv = 1, kEpiSiluMul = 2 };
struct PairEpilogue {
  int kind;
  // kEpiRopeKv: X rows are [q_heads | kv_heads keys | kv_heads values] x 128 (a fused qkv projection), y = token.
  // Query and key heads are rotated (rotate-half: element i pairs with i + 64) by the angle of positions[y] and written
  // to `out`; key and value heads are also written to k_cache / v_cache [batch, cache_seq, kv_heads, 128] (bf16) at
  // [y, positions[y]].
  int q_heads, kv_heads;
  const int64_t* positions;   // [y_rows]
  const float* cos_sin;       // [max_pos, 128]: the 64 cosines, then the 64 sines
  int max_pos, cache_seq;
  void* k_cache;
  void* v_cache;
  int64_t cache_batch_stride, cache_pos_stride;   // elements
  // kEpiSiluMul: X is [2 * ffn, k], gate rows then up rows (ffn a multiple of 64). Tile t holds gate rows
  // [64 t, 64 t + 64) in its rows 0-63 and the up rows of the same features in rows 64-127;
  // out[y * sy + (64 t + r) * sx] = silu(gate) * up.
  int ffn;
};

struct GemmProblem {
  const void* x;       // [x_rows, k], row pitch ldx elements; fills the 128-row side of the tile
  const void* y;       // [y_rows, k], row pitch ldy elements; the tile's narrow side (16..256)
  int x_rows, y_rows, k;
  int64_t ldx, ldy;
  int elem_size;       // 2 (bf16 / fp16) or 1 (e4m3)
  int elem_kind;       // kBF16 / kF16 for 2-byte operands (ignored for e4m3)
  void* out;
  int64_t sx, sy;
  int out_dtype;       // kF32 / kF16 / kBF16
  int block_n;         // 0 = choose from y_rows
  int splits;          // K splits (>= 1); > 1 needs the workspace below
  float* ws;           // zero-initialised fp32 scratch, left zeroed again by the kernel
  size_t ws_bytes;
  uint32_t* counters;  // zero-initialised, one per output tile
  size_t counter_count;
  uint32_t* status;    // optional device word, set non-zero when a pipeline wait ran out
  // fp8 block scaling (both or neither): fp32 [rows or ceil(rows/128), k/128]
  const float* x_scale;
  const float* y_scale;
  int x_scale_per_row, y_scale_per_row;
  // X holds data that no kernel writes (weights): with programmatic dependent launch its first tiles are requested
  // before the previous kernel of the stream has completed.
  int x_static;
  PairEpilogue epi;    // kind == kEpiNone: plain store
};

std::string gemm_tn(const GemmProblem& g, cudaStream_t stream);
// Same product on 256 x 256 tiles computed by CTA pairs (tcgen05.mma.cta_group::2, gemm_pair.cu). Unscaled
// operands, no split-K; block_n, splits and the scratch fields are ignored.
std::string gemm_tn_pair(const GemmProblem& g, cudaStream_t stream);
// Same product by a persistent grid (one CTA per SM walks the 128 x 256 tiles, the accumulator double-buffered in
// tensor memory so that the epilogue of a tile overlaps the main loop of the next; gemm_persist.cu). Unscaled
// operands, no split-K; block_n, splits and the scratch fields are ignored.
std::string gemm_tn_persistent(const GemmProblem& g, cudaStream_t stream);

// Row-parallel linear fused with reduce(-scatter) + residual + RMSNorm (gemm_fused.cu).
// `ar` carries the communication state (Workspace::fill_params) and describes the tail: tokens,
// hidden, residual_in, gamma, residual_out, norm_out, scale_out, eps, out_mode (bf16 or e4m3 with
// 1x128 scales), scatter_only. `ar.in` is unused: the partial rows come from the GEMM.
struct FusedGemmProblem {
  ArParams ar;
  const void* a;      // [tokens, k] bf16 or e4m3, this rank's K shard of the activations
  const void* w;      // [hidden, k] bf16 or e4m3, this rank's K shard of the weight
  int elem_size;      // 2: bf16 operands; 1: e4m3 operands with the block scales below (0 is read as 2)
  const float* a_scale;   // e4m3: [tokens, k / 128] fp32, one scale per token and 128-wide K block
  const float* w_scale;   // e4m3: [hidden / 128, k / 128] fp32, one scale per 128 x 128 block
  int k;
  int64_t lda, ldw;
  uint32_t* status;
  int splits;          // K splits (0 = fill the SMs); > 1 needs the scratch below
  float* ws;           // zero-initialised fp32 scratch, left zeroed by the kernel
  size_t ws_bytes;
  uint32_t* counters;  // zero-initialised, one per output tile
  size_t counter_count;
  bool one_hop = false;   // replicated output: tiles pushed to every rank, each rank reduces all rows (one NVSwitch hop)
};
std::string gemm_ar_rmsnorm(const FusedGemmProblem& g, cudaStream_t stream);
std::string gemm_ar_rmsnorm_n0(const FusedGemmProblem& g, cudaStream_t stream);
std::string gemm_ar_rmsnorm_n2(const FusedGemmProblem& g, cudaStream_t stream);
std::string gemm_ar_rmsnorm_n4(const FusedGemmProblem& g, cudaStream_t stream);
std::string gemm_ar_rmsnorm_n8(const FusedGemmProblem& g, cudaStream_t stream);
// The same step for token counts whose tiles outnumber the SMs (gemm_fused_persist.cu): one CTA per SM walks the
// tiles and joins the reduce / normalise tail after its last one; bf16 operands. gemm_ar_rmsnorm hands over to it
// by itself.
std::string gemm_ar_rmsnorm_persist(const FusedGemmProblem& g, cudaStream_t stream);

// All-gather of sequence-parallel activations fused with a column-parallel linear (gemm_fused.cu).
struct AgGemmProblem {
  void* peer[kMaxRanks];
  Layout layout;
  int rank, nranks;
  int tokens, k;
  const void* x_shard;   // [ceil((tokens - rank) / nranks), k] bf16: rows rank, rank + nranks, ...
  const void* w;         // [out_rows, k] bf16
  int64_t ldw;
  int out_rows;
  void* out;             // [tokens, out_rows] bf16
  int64_t ldo;
  uint32_t* status;
  uint64_t timeout_ns;
  uint32_t* host_status;
};
std::string ag_gemm(const AgGemmProblem& g, cudaStream_t stream);
int gemm_pick_block_n(int y_rows, bool scaled);

}  // namespace tdx
