// Allocation-free decode attention: the split-KV scratch is a fixed device array inside this library
// instead of a buffer that the caller has to provide (see tdx/no_alloc.h for who needs this and the
// rules that come with it).
#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include "tdx/no_alloc.h"
#include "tdx/ops.h"

namespace {

constexpr int kRowFloats = 130;   // 128 output columns + running maximum + running sum

// Lives on every GPU that loads the library. In host code this name is only a handle for
// cudaGetSymbolAddress - it is NOT a device address and must never be passed to a kernel.
// Layout: 4096 arrival counters (zero when the library is loaded; every call leaves them zero again),
// then the per-split partial rows.
constexpr size_t kCounterWords = 4096;
static __device__ __align__(256) float g_attn_scratch[kCounterWords + (size_t)TDX_NOALLOC_ATTN_MAX_ROWS * kRowFloats];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float* g_scratch_ptr[kMaxDevices] = {};

int fail(char* err, int err_len, const std::string& why) {
  if (err && err_len > 0) {
    std::strncpy(err, why.c_str(), (size_t)err_len - 1);
    err[err_len - 1] = '\0';
  }
  return 1;
}

}  // namespace

extern "C" int tdx_attention_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, const int32_t* seq_lens,
                                            void* out, int batch, int q_heads, int kv_heads, int s_max, int64_t q_stride_b,
                                            int64_t kv_stride_b, int64_t kv_stride_s, int kv_splits, float scale,
                                            cudaStream_t stream, char* err, int err_len) {
  if (kv_splits < 1) kv_splits = 1;
  if (batch < 0 || q_heads <= 0 || kv_heads <= 0) return fail(err, err_len, "batch, q_heads and kv_heads must be positive");
  const long long rows = (long long)batch * q_heads * kv_splits;
  if (rows > TDX_NOALLOC_ATTN_MAX_ROWS) {
    char buf[192];
    std::snprintf(buf, sizeof(buf), "batch * q_heads * kv_splits = %lld exceeds the built-in scratch of %d rows; "
                  "use fewer KV splits or the entry point that takes a caller-provided scratch buffer", rows,
                  TDX_NOALLOC_ATTN_MAX_ROWS);
    return fail(err, err_len, buf);
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(err, err_len, "no current CUDA device");
  float* scratch = nullptr;
  {
    // first call on this device: resolve the array's address on the CURRENT device
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_scratch_ptr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_attn_scratch);
      if (e != cudaSuccess || p == nullptr)
        return fail(err, err_len, std::string("cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
      g_scratch_ptr[dev] = static_cast<float*>(p);
    }
    scratch = g_scratch_ptr[dev];
  }
  const std::string why = tdx::attention_decode(q, k_cache, v_cache, seq_lens, scratch,
                                                kCounterWords + (size_t)TDX_NOALLOC_ATTN_MAX_ROWS * kRowFloats, out, batch, q_heads, kv_heads,
                                                128, s_max, q_stride_b, kv_stride_b, kv_stride_s, kv_splits, scale, stream,
                                                nullptr);
  if (!why.empty()) return fail(err, err_len, why);
  return 0;
}
