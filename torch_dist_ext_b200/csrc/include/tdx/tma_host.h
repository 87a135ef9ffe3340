// Host-side launch helpers: the opt-in to large dynamic shared memory, and construction of TMA tensor maps
// (cuTensorMapEncodeTiled through the runtime's driver entry point, so that nothing links against libcuda). Every map of this library is bf16 / fp16 / 8-bit data
// with the innermost box equal to one 128-byte swizzle span, L2 promotion to 256 bytes and zero fill
// outside the tensor. The reference has no TMA code.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <mutex>
#include <set>
#include <string>
#include <utility>
#include "tdx/comm.h"

namespace tdx {

// Opt in to a dynamic shared-memory size above the 48 KB default, once per kernel and device (the
// attribute belongs to the device's copy of the kernel). Returns an empty string or the reason.
template <typename Kernel>
std::string reserve_dynamic_smem(Kernel kernel, int bytes) {
  static std::mutex mu;
  static std::set<std::pair<const void*, int>> done;
  int dev = 0;
  cudaGetDevice(&dev);
  const auto key = std::make_pair(reinterpret_cast<const void*>(kernel), dev);
  std::lock_guard<std::mutex> lock(mu);
  if (done.count(key)) return "";
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return std::string("cannot reserve shared memory: ") + cudaGetErrorString(e);
  done.insert(key);
  return "";
}

namespace tma {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encoder() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// Tiled map of `rank` dimensions (innermost first) with 128-byte swizzle. `dims` in elements, `strides` in
// bytes for dimensions 1 .. rank-1, `box` in elements; box[0] * element size must be 128 bytes.
inline std::string encode_sw128(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* ptr, const cuuint64_t* dims,
                                const cuuint64_t* strides, const cuuint32_t* box, const char* what) {
  EncodeFn enc = encoder();
  if (!enc) return "cuTensorMapEncodeTiled is not available from this driver";
  if (reinterpret_cast<uintptr_t>(ptr) % 16) return std::string(what) + " must be 16-byte aligned";
  for (int i = 0; i + 1 < rank; ++i)
    if (strides[i] % 16) return std::string(what) + ": every pitch must be a multiple of 16 bytes";
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUresult r = enc(map, dt, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return std::string("cuTensorMapEncodeTiled failed for ") + what + " (CUresult " + std::to_string((int)r) + ")";
  return "";
}

// GEMM operand: row-major [rows, k] with row pitch ld (elements); box = one 128-byte span of K x box_rows rows.
inline std::string kmajor_2d(CUtensorMap* map, const void* ptr, int rows, int k, int64_t ld, int elem_size, int elem_kind,
                             int box_rows) {
  const CUtensorMapDataType dt = elem_size == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : elem_kind == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)(ld * elem_size)};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / elem_size), (cuuint32_t)box_rows};
  return encode_sw128(map, dt, 2, ptr, dims, strides, box, "GEMM operand");
}

// KV cache [B, S, Hkv, 128] bf16 (strides in elements) -> 4-D map (128, Hkv, S, B); box = 64 columns x box_rows
// positions of one head.
inline std::string kv_cache_4d(CUtensorMap* map, const void* ptr, int B, int S, int Hkv, int64_t stride_b, int64_t stride_s,
                               int box_rows) {
  const cuuint64_t dims[4] = {128, (cuuint64_t)Hkv, (cuuint64_t)S, (cuuint64_t)B};
  const cuuint64_t strides[3] = {128 * 2, (cuuint64_t)stride_s * 2, (cuuint64_t)stride_b * 2};
  const cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  return encode_sw128(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, ptr, dims, strides, box, "the KV cache");
}

// [S, heads, 128] bf16 with row pitch stride_s (elements) -> 3-D map (128, heads, S); box = 64 columns x box_rows
// rows of one head.
inline std::string head_rows_3d(CUtensorMap* map, const void* ptr, int S, int heads, int64_t stride_s, int box_rows,
                                const char* what) {
  const cuuint64_t dims[3] = {128, (cuuint64_t)heads, (cuuint64_t)S};
  const cuuint64_t strides[2] = {128 * 2, (cuuint64_t)stride_s * 2};
  const cuuint32_t box[3] = {64, 1, (cuuint32_t)box_rows};
  return encode_sw128(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, ptr, dims, strides, box, what);
}

}  // namespace tma
}  // namespace tdx
