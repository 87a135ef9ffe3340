// Persistent tcgen05 GEMM for prefill-sized problems:  D[x, y] = sum_k X[x, k] * Y[y, k], both K-major.
//
// One CTA per SM walks the 128 x 256 output tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... The
// operand ring (TMA -> 128-byte-swizzled shared memory) keeps streaming across tile boundaries, and
// the accumulator is double-buffered in tensor memory (2 x 256 columns): while the epilogue warps read
// tile n back with tcgen05.ld and store it, the MMA thread is already accumulating tile n + 1. The
// one-tile-per-CTA kernel (gemm_tcgen05.cu) pays a pipeline fill, a drain and a serial epilogue per
// tile; here they are paid once per CTA.
//
//   warp 0     TMA producer (one thread): K blocks of all tiles of this CTA, back to back
//   warp 1     tensor-memory owner and MMA issue (one thread)
//   warps 2-5  epilogue: TMEM lane quarter = warp % 4
//
// Barriers: full[s] / empty[s] per ring stage (phases counted over ALL K blocks this CTA processes),
// acc_full[b] / acc_empty[b] per accumulator buffer (phases counted over the tiles that use it).
// Every wait is bounded; a wait that runs out records a status word, raises the CTA's abort flag and
// all roles fall through to the common exit (copies in flight land, tensor memory is freed).
//
// The default for prefill-sized problems (ops/gemm.py; TDX_GEMM_PERSIST=0 turns it off), bf16 / fp16 / unscaled
// e4m3 operands, no split-K. The reference (xytpai/torch_dist_ext) has no GEMM.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <string>
#include "tdx/comm.h"
#include "tdx/gemm.h"
#include "tdx/gemm_core.cuh"
#include "tdx/launch.h"
#include "tdx/ptx.cuh"
#include "tdx/tc.cuh"
#include "tdx/tma_host.h"

namespace tdx {
namespace {

using gemm_core::store_chunk;

constexpr int kThreads = 192;
constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kStages = 4;
constexpr int kXBytes = kBM * 128;
constexpr int kYBytes = kBN * 128;
constexpr int kStageBytes = kXBytes + kYBytes;          // 48 KB
constexpr int kBarrierOffset = kStages * kStageBytes;
constexpr int kSmemTotal = kBarrierOffset + 1024 /* barriers */ + 1024 /* alignment slack */;
constexpr uint32_t kTmemCols = 2 * kBN;                 // two accumulator buffers
constexpr uint32_t kWaitLimit = 1u << 22;

struct PersistArgs {
  int x_rows, y_rows, kblocks;
  int tiles_x, tiles_y;
  void* out;
  int64_t sx, sy;
  int out_dtype;
  uint32_t idesc;
  uint32_t* status;
};

template <bool kFp8>
__global__ void __launch_bounds__(kThreads, 1)
gemm_persist_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y, const PersistArgs a) {
  constexpr int kElemsPerBlock = kFp8 ? 128 : 64;   // K elements in one 128-byte span

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kBarrierOffset);
  uint64_t* empty = full + kStages;
  uint64_t* acc_full = empty + kStages;     // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = a.tiles_x * a.tiles_y;
  const int nkb = a.kblocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(&full[s], 1);
      tc::mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&acc_full[i], 1);
      tc::mbar_init(&acc_empty[i], 128);
    }
    *abort_flag = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_desc(&map_x);
    tc::tma_prefetch_desc(&map_y);
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::fence_before_thread_sync();
  __syncthreads();
  tc::fence_after_thread_sync();
  const uint32_t tmem_base = *tmem_slot;
  ptx::pdl_wait();                // prefill shapes: both operands may come from earlier kernels of the stream
  ptx::pdl_launch_dependents();

  auto fail = [&]() {
    *abort_flag = 1;
    if (a.status) atomicExch(a.status, (uint32_t)kTimeoutGemmPipeline);
  };

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: the x tile index runs fastest, so CTAs that work side by side share the Y (weight) tile in L2 ----
      uint32_t it = 0;                                   // K blocks issued so far by this CTA
      for (int t = blockIdx.x; t < ntiles && !*abort_flag; t += gridDim.x) {
        const int x_row0 = (t % a.tiles_x) * kBM, y_row0 = (t / a.tiles_x) * kBN;
        bool ok = true;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t s = it % kStages;
          if (it >= (uint32_t)kStages && !tc::mbar_wait(&empty[s], ((it / kStages) - 1) & 1, kWaitLimit, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* dst = smem + s * kStageBytes;
          tc::mbar_arrive_expect_tx(&full[s], kStageBytes);
          tc::tma_load_2d(dst, &map_x, &full[s], kb * kElemsPerBlock, x_row0);
          tc::tma_load_2d(dst + kXBytes, &map_y, &full[s], kb * kElemsPerBlock, y_row0);
        }
        if (!ok) {
          fail();
          break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issue ----
      uint32_t it = 0;
      int n = 0;                                         // tiles started so far by this CTA
      bool ok = true;
      for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++n) {
        const uint32_t buf = n & 1;
        if (n >= 2 && !tc::mbar_wait(&acc_empty[buf], ((n >> 1) - 1) & 1, kWaitLimit, abort_flag)) {
          ok = false;
          break;
        }
        tc::fence_after_thread_sync();
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t s = it % kStages;
          if (!tc::mbar_wait(&full[s], (it / kStages) & 1, kWaitLimit, abort_flag)) {
            ok = false;
            break;
          }
          tc::fence_after_thread_sync();
          const uint32_t xa = tc::smem_u32(smem + s * kStageBytes);
          const uint64_t dx = tc::make_smem_desc_sw128(xa);
          const uint64_t dy = tc::make_smem_desc_sw128(xa + kXBytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)   // 32 bytes of K per instruction, stepped inside the swizzle span
            tc::umma<kFp8>(tmem_base + buf * kBN, dx + (uint64_t)(k * 2), dy + (uint64_t)(k * 2), a.idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc::umma_commit(&empty[s]);   // the stage is reusable once these MMAs have read it
        }
        if (ok) tc::umma_commit(&acc_full[buf]);
      }
      if (!ok) fail();
    }
  } else {
    // ---- epilogue (warps 2..5): TMEM lane quarter = warp % 4 ----
    const int q = warp & 3;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    int n = 0;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++n) {
      const uint32_t buf = n & 1;
      const int x = (t % a.tiles_x) * kBM + q * 32 + lane;
      const int y_base = (t / a.tiles_x) * kBN;
      if (nkb <= 0 || !tc::mbar_wait(&acc_full[buf], (n >> 1) & 1, kWaitLimit, abort_flag)) {
        if (nkb > 0 && lane == 0 && q == 0) fail();
        break;
      }
      tc::fence_after_thread_sync();
#pragma unroll 4
      for (int c = 0; c < kBN; c += 16) {
        float v[16];
        tc::tmem_ld_16(lane_addr + buf * kBN + c, v);
        if (y_base + c < a.y_rows) store_chunk(a, x, y_base + c, v);
      }
      tc::fence_before_thread_sync();
      tc::mbar_arrive(&acc_empty[buf]);   // this thread has read its part of the buffer
    }
  }

  // ---- common exit ----
  tc::fence_before_thread_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);   // copies already issued land before shared memory goes away
  }
  if (warp == 1) {
    tc::fence_after_thread_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <bool kFp8>
std::string launch(const CUtensorMap& mx, const CUtensorMap& my, const PersistArgs& a, int grid, cudaStream_t stream) {
  auto kern = gemm_persist_kernel<kFp8>;
  const std::string err = reserve_dynamic_smem(kern, kSmemTotal);
  if (!err.empty()) return err;
  const cudaError_t e = launch_chained(kern, dim3(grid), dim3(kThreads), kSmemTotal, stream, mx, my, a);
  return e == cudaSuccess ? "" : std::string("GEMM launch failed: ") + cudaGetErrorString(e);
}

}  // namespace

std::string gemm_tn_persistent(const GemmProblem& g, cudaStream_t stream) {
  const bool fp8 = g.elem_size == 1;
  if (g.x_scale != nullptr || g.y_scale != nullptr) return "the persistent kernel takes unscaled operands";
  const int epb = 128 / g.elem_size;
  if (g.k <= 0 || g.k % epb) return "K must be a positive multiple of " + std::to_string(epb);
  if (g.x_rows <= 0 || g.y_rows <= 0) return "";
  PersistArgs a{};
  a.x_rows = g.x_rows;
  a.y_rows = g.y_rows;
  a.kblocks = g.k / epb;
  a.tiles_x = (g.x_rows + kBM - 1) / kBM;
  a.tiles_y = (g.y_rows + kBN - 1) / kBN;
  a.out = g.out;
  a.sx = g.sx;
  a.sy = g.sy;
  a.out_dtype = g.out_dtype;
  a.idesc = fp8 ? tc::make_idesc(kBM, kBN, 0, 0) : tc::make_idesc(kBM, kBN, g.elem_kind == kBF16 ? 1 : 0, g.elem_kind == kBF16 ? 1 : 0);
  a.status = g.status;
  CUtensorMap mx, my;
  std::string err = tma::kmajor_2d(&mx, g.x, g.x_rows, g.k, g.ldx, g.elem_size, g.elem_kind, kBM);
  if (!err.empty()) return err;
  err = tma::kmajor_2d(&my, g.y, g.y_rows, g.k, g.ldy, g.elem_size, g.elem_kind, kBN);
  if (!err.empty()) return err;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long ntiles = (long long)a.tiles_x * a.tiles_y;
  const int grid = (int)(ntiles < sms ? ntiles : sms);
  return fp8 ? launch<true>(mx, my, a, grid, stream) : launch<false>(mx, my, a, grid, stream);
}

}  // namespace tdx
