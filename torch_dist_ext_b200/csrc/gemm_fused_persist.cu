// Row-parallel linear + all-reduce (or reduce-scatter) + residual + RMSNorm for prompt-sized token counts: the
// persistent form of gemm_ar_rmsnorm_kernel (gemm_fused.cu).
//
// The decode kernel gives every output tile its own CTA, and because the CTAs later wait for each other's pushes the
// whole grid has to be resident: at hidden 4096 that caps it at 256 tokens. Here one CTA per SM walks the
// 128 (hidden columns) x 128 (tokens) tiles t = blockIdx.x, blockIdx.x + gridDim.x, ...: the TMA ring streams across
// tile boundaries, the accumulator is double-buffered in tensor memory, and the epilogue warps push every finished
// tile - 16 tokens at a time, transposed through shared memory into 256-byte row pieces - straight into the gather
// slots of the rows' OWNER ranks while the tensor core already works on the next tile. When a CTA has pushed its
// last tile it turns into a reducer of the two-shot Lamport flow (sum the N partial rows, residual, RMSNorm,
// optional 1x128 e4m3 quantisation, push back or keep scattered), exactly as the decode kernel does. A CTA waits for
// other CTAs only in that tail, after all of its own tiles; the grid never exceeds the SM count, so every CTA is
// resident and no wait can depend on a CTA that has not started.
//
//   warp 0     TMA producer (one thread)        warp 1     tensor-memory owner, MMA issue (one thread)
//   warps 2-5  epilogue / pushes                warps 6-7  idle until the tail
//
// bf16 operands. Every wait is bounded (mbarrier waits by a poll count, peer waits by the workspace time limit).
// The reference has no GEMM; its all-reduce kernel starts from a finished activation tensor
// (src/common/all_reduce_fusion_impl.h:342-474).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <string>
#include "tdx/ar_fusion_kernels.cuh"
#include "tdx/gemm.h"
#include "tdx/launch.h"
#include "tdx/tc.cuh"
#include "tdx/tma_host.h"

namespace tdx {
namespace {

using T = __nv_bfloat16;
constexpr int kThreads = 256;
constexpr int kBM = 128;                                 // hidden columns (weight rows) per tile
constexpr int kBN = 128;                                 // tokens per tile
constexpr int kStages = 5;
constexpr int kXBytes = kBM * 128;
constexpr int kYBytes = kBN * 128;
constexpr int kStageBytes = kXBytes + kYBytes;           // 32 KB: 64 K elements of both operands
constexpr int kChunk = 16;                               // tokens per push step
constexpr int kPushOffset = kStages * kStageBytes;
constexpr int kPushBytes = 2 * kChunk * kBM * 2;         // two transposition buffers [16 tokens][128 columns] bf16
constexpr int kBarrierOffset = kPushOffset + kPushBytes;
constexpr int kSmemTotal = kBarrierOffset + 1024 /* barriers */ + 1024 /* alignment slack */;
constexpr uint32_t kTmemCols = 2 * kBN;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr int kNumBarriers = 2 * kStages + 4;
static_assert(kNumBarriers * 8 + 8 <= 1024, "barrier area");

struct PersistFusedArgs {
  ArParams ar;
  int kblocks;
  int tiles_x, tiles_y;
  uint32_t idesc;
  uint32_t* status;
};

// Named barrier over `count` threads that also ORs a predicate over them.
__device__ __forceinline__ bool named_barrier_or(uint32_t id, uint32_t count, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, %2, %3, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"((uint32_t)pred), "r"(id), "r"(count)
      : "memory");
  return out != 0;
}

template <int kVpt, int kOut>
__global__ void __launch_bounds__(kThreads, 1)
gemm_ar_rmsnorm_persist_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                               const PersistFusedArgs f) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ float red[4][32];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kBarrierOffset);
  uint64_t* empty = full + kStages;
  uint64_t* acc_full = empty + kStages;     // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const ArParams& p = f.ar;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, nctas = gridDim.x;
  const int ntiles = f.tiles_x * f.tiles_y;
  const int nkb = f.kblocks;

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
    tc::tma_prefetch_desc(&map_w);
    tc::tma_prefetch_desc(&map_a);
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::fence_before_thread_sync();
  __syncthreads();
  tc::fence_after_thread_sync();
  const uint32_t tmem_base = *tmem_slot;
  ptx::pdl_wait();                 // the activations come from the previous kernel of the stream
  ptx::pdl_launch_dependents();

  char* self = static_cast<char*>(p.peer[p.rank]);
  Control* ctl = reinterpret_cast<Control*>(self + p.layout.off_control);
  const int groups = (p.tokens + p.nranks - 1) / p.nranks;
  const uint32_t epoch = ctl->lamport_epoch;
  const uint64_t dirty_prev = ctl->lamport_dirty[(epoch + 2u) % 3u];
  const size_t buf_off = p.layout.off_lamport + (size_t)(epoch % 3u) * p.layout.lamport_bytes;

  auto fail = [&]() {
    *abort_flag = 1;
    if (f.status) atomicExch(f.status, (uint32_t)kTimeoutGemmPipeline);
  };

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: the hidden-column tile index runs fastest, so CTAs working side by side share the token tile ----
      uint32_t it = 0;
      for (int t = cta; t < ntiles && !*abort_flag; t += nctas) {
        const int x_row0 = (t % f.tiles_x) * kBM, y_row0 = (t / f.tiles_x) * kBN;
        bool ok = true;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t s = it % kStages;
          if (it >= (uint32_t)kStages && !tc::mbar_wait(&empty[s], ((it / kStages) - 1) & 1, kWaitLimit, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* dst = smem + s * kStageBytes;
          tc::mbar_arrive_expect_tx(&full[s], kStageBytes);
          tc::tma_load_2d(dst, &map_w, &full[s], kb * 64, x_row0);
          tc::tma_load_2d(dst + kXBytes, &map_a, &full[s], kb * 64, y_row0);
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
      int n = 0;
      bool ok = true;
      for (int t = cta; t < ntiles && ok; t += nctas, ++n) {
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
          for (int k = 0; k < 4; ++k)
            tc::umma<false>(tmem_base + buf * kBN, dx + (uint64_t)(k * 2), dy + (uint64_t)(k * 2), f.idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc::umma_commit(&empty[s]);
        }
        if (ok) tc::umma_commit(&acc_full[buf]);
      }
      if (!ok) fail();
    }
  } else if (warp < 6) {
    // ---- epilogue (warps 2..5): TMEM lane quarter = warp % 4; the four warps push a tile together ----
    const int q = warp & 3;
    const int te = threadIdx.x - 64;                     // 0..127
    const int xl = q * 32 + lane;                        // hidden column of this thread inside the tile
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const size_t row_bytes = (size_t)p.hidden * sizeof(T);
    uint32_t chunk = 0;
    int n = 0;
    for (int t = cta; t < ntiles; t += nctas, ++n) {
      const uint32_t buf = n & 1;
      const int tile_x = t % f.tiles_x;
      const int y_base = (t / f.tiles_x) * kBN;
      // one verdict for all four warps: they meet at named barriers below
      const bool lost = nkb <= 0 || !tc::mbar_wait(&acc_full[buf], (n >> 1) & 1, kWaitLimit, abort_flag);
      if (named_barrier_or(1, 128, lost)) {
        if (nkb > 0 && te == 0) fail();
        break;
      }
      tc::fence_after_thread_sync();
      for (int c = 0; c < kBN && y_base + c < p.tokens; c += kChunk, ++chunk) {
        float v[16];
        tc::tmem_ld_16(lane_addr + buf * kBN + c, v);
        uint8_t* stage = smem + kPushOffset + (chunk & 1u) * (kChunk * kBM * 2);
        __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(stage);
#pragma unroll
        for (int j = 0; j < kChunk; ++j) st[j * kBM + xl] = __float2bfloat16(v[j]);
        // Readers of this buffer two steps ago passed the previous step's barrier before anyone got here, so one
        // barrier per step is enough with two buffers.
        tc::named_barrier_sync(1, 128);
#pragma unroll
        for (int i = te; i < kChunk * 16; i += 128) {
          const int tl = i >> 4, part = i & 15;
          const int tok = y_base + c + tl;
          if (tok < p.tokens) {
            const int owner = tok % p.nranks, j = tok / p.nranks;
            const uint4 val = scrub(*reinterpret_cast<const uint4*>(stage + (size_t)tl * (kBM * 2) + part * 16));
            char* dst = static_cast<char*>(p.peer[owner]) + buf_off + ((size_t)p.rank * groups + j) * row_bytes +
                        ((size_t)tile_x * kBM + part * 8) * sizeof(T);
            ptx::st_v4(dst, val);
          }
        }
      }
      tc::fence_before_thread_sync();
      tc::mbar_arrive(&acc_empty[buf]);
    }
  }

  // ---- every tile of this CTA is on its way: free tensor memory, then reduce and normalise the owned rows ----
  tc::fence_before_thread_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);   // copies already issued land before shared memory goes away
  }
  if (warp == 1) {
    tc::fence_after_thread_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
  clear_previous(lamport_buf(self, p.layout, (epoch + 2u) % 3u), dirty_prev, cta, nctas);
  const uint64_t dirty = twoshot_lamport_tail<T, 0, kVpt, kOut, true>(p, cta, nctas, epoch, red);
  finish_launch(ctl, true, epoch, dirty, 0, nctas);
}

template <int kVpt, int kOut>
std::string launch(const CUtensorMap& mw, const CUtensorMap& ma, const PersistFusedArgs& f, int grid, cudaStream_t s) {
  auto kern = gemm_ar_rmsnorm_persist_kernel<kVpt, kOut>;
  const std::string err = reserve_dynamic_smem(kern, kSmemTotal);
  if (!err.empty()) return err;
  const cudaError_t e = launch_chained(kern, dim3(grid), dim3(kThreads), kSmemTotal, s, mw, ma, f);
  return e == cudaSuccess ? "" : std::string("fused GEMM launch failed: ") + cudaGetErrorString(e);
}

}  // namespace

std::string gemm_ar_rmsnorm_persist(const FusedGemmProblem& g, cudaStream_t stream) {
  const ArParams& p = g.ar;
  if (p.dtype != kBF16 || g.elem_size != 2) return "the persistent fused GEMM takes bfloat16 operands";
  if (p.hidden % 128) return "hidden must be a multiple of 128";
  if (g.k <= 0 || g.k % 64) return "K must be a positive multiple of 64";
  if (p.out_mode != kOutSame && p.out_mode != kOutFp8Block128) return "fused GEMM output is bf16 or e4m3 with 1x128 scales";
  if (p.tokens <= 0) return "";
  const int nvec = p.hidden / 8;
  const int vpt = nvec <= kThreads ? 1 : nvec <= 2 * kThreads ? 2 : nvec <= 4 * kThreads ? 4 : 0;
  const uint64_t row_bytes = (uint64_t)p.hidden * 2;
  const uint64_t groups = ((uint64_t)p.tokens + p.nranks - 1) / p.nranks;
  const uint64_t need = (uint64_t)p.nranks * groups * row_bytes + (p.scatter_only ? 0 : (uint64_t)p.tokens * (row_bytes + 16));
  if (need > p.layout.lamport_bytes) return "message exceeds the Lamport buffer capacity";
  for (int r = 0; r < p.nranks; ++r)
    if (p.peer[r] == nullptr) return "workspace is not registered with all peers";
  PersistFusedArgs f{};
  f.ar = p;
  f.kblocks = g.k / 64;
  f.tiles_x = p.hidden / kBM;
  f.tiles_y = (p.tokens + kBN - 1) / kBN;
  f.idesc = tc::make_idesc(kBM, kBN, 1, 1);
  f.status = g.status;
  CUtensorMap mw, ma;
  std::string err = tma::kmajor_2d(&mw, g.w, p.hidden, g.k, g.ldw, 2, kBF16, kBM);
  if (!err.empty()) return err;
  err = tma::kmajor_2d(&ma, g.a, p.tokens, g.k, g.lda, 2, kBF16, kBN);
  if (!err.empty()) return err;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long ntiles = (long long)f.tiles_x * f.tiles_y;
  const int grid = (int)(ntiles < sms ? ntiles : sms);
  const bool q = p.out_mode == kOutFp8Block128;
  switch (vpt) {
    case 1: return q ? launch<1, kOutFp8Block128>(mw, ma, f, grid, stream) : launch<1, kOutSame>(mw, ma, f, grid, stream);
    case 2: return q ? launch<2, kOutFp8Block128>(mw, ma, f, grid, stream) : launch<2, kOutSame>(mw, ma, f, grid, stream);
    case 4: return q ? launch<4, kOutFp8Block128>(mw, ma, f, grid, stream) : launch<4, kOutSame>(mw, ma, f, grid, stream);
  }
  return "unsupported hidden size for the fused GEMM";
}

}  // namespace tdx
