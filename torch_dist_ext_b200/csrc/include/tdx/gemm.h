// Host interface of the tcgen05 GEMM (gemm_tcgen05.cu).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <string>

namespace tdx {

// D[x, y] = sum_k X[x, k] * Y[y, k];  D[x, y] is written to out[x * sx + y * sy].
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
};

std::string gemm_tn(const GemmProblem& g, cudaStream_t stream);
int gemm_pick_block_n(int y_rows, bool scaled);

}  // namespace tdx
