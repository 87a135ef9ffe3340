// Two-SM persistent tcgen05 GEMM for prefill-sized problems:  D[x, y] = sum_k X[x, k] * Y[y, k], both K-major.
//
// A cluster of two CTAs (a "pair") computes 256 x 256 tiles with tcgen05.mma.cta_group::2:
// CTA r of the pair loads rows [128 r, 128 r + 128) of the X tile and rows [128 r, 128 r + 128) of the
// 256-row Y tile - each CTA fetches only its own half, with ordinary TMA copies - and the leader
// (r = 0) issues the MMAs, which read both CTAs' shared memory. Compared with two independent
// 128 x 256 tiles, every SM stages half as much of Y per K block (32 KB instead of 48 KB per stage),
// so the operand ring is deeper and the shared-memory traffic per FLOP lower. The accumulator is
// split by rows: rows 0-127 in the leader's tensor memory, rows 128-255 in the peer's.
//
// The grid is persistent: pair p walks the tiles p, p + pairs, ... (the x tile index runs fastest, so pairs that
// work side by side share the Y tile in L2). When the last round would be partly filled, its tiles are cut along K
// into 2-4 pieces, one piece per pair; every piece stores its fp32 partial tile in a scratch slice of its own and the
// CTA that arrives last at its half of the tile adds the slices up - the idle pairs of the last round then share its
// work. The operand ring keeps streaming across tile boundaries and the
// accumulator is double-buffered in tensor memory (2 x 256 columns in each CTA): while the epilogue warps of both
// CTAs read tile n back with tcgen05.ld and store it, the leader is already accumulating tile n + 1.
//
// Synchronisation (all waits bounded):
//  * full[s]       leader only: armed by the leader's producer for the bytes of BOTH CTAs; the peer's
//                  copies credit the leader's barrier (address translated with mapa).
//  * empty[s]      one per CTA: the leader's MMA thread commits to its own and (through the cluster's
//                  shared window) to the peer's.
//  * acc_full[b]   one per CTA and accumulator buffer, committed the same way after a tile's last K block.
//  * acc_empty[b]  leader only: one arrival per epilogue warp of BOTH CTAs (8) once the warp has read its part
//                  of buffer b; the leader waits for it before it reuses the buffer two tiles later.
//  * cluster barriers after barrier initialisation (no remote arrival before the target exists)
//    and before tensor memory is freed (no CTA leaves while its peer may still read its shared
//    memory or write its barriers).
// A wait that runs out records a status word, raises the abort flag of both CTAs and falls through
// to the common exit, where in-flight copies are given time to land and tensor memory is freed.
//
// Selected by ops/gemm.py (linear(..., cta_pair=True) or TDX_GEMM_PAIR=1) for bf16 / fp16 / unscaled e4m3
// operands. The reference (xytpai/torch_dist_ext) has no GEMM.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <mutex>
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
constexpr int kRowsPerCta = 128;                 // X rows and Y rows staged by one CTA
constexpr int kTileM = 2 * kRowsPerCta;          // rows of the pair's output tile
constexpr int kTileN = 2 * kRowsPerCta;          // columns of the pair's output tile (MMA N)
constexpr int kStages = 6;
constexpr int kOperandBytes = kRowsPerCta * 128; // 128 rows x one 128-byte swizzle span
constexpr int kStageBytes = 2 * kOperandBytes;   // X half + Y half
constexpr int kBarrierOffset = kStages * kStageBytes;
constexpr int kSmemTotal = kBarrierOffset + 1024 /* barriers */ + 1024 /* alignment slack */;
constexpr uint32_t kTmemCols = 2 * kTileN;       // two fp32 accumulator buffers
constexpr uint32_t kWaitLimit = 1u << 22;

struct PairArgs {
  int x_rows, y_rows, kblocks;
  int tiles_x, tiles_y;
  // Tail split: the tiles of the last, partly filled round (tail_first ...) are cut along K into tail_parts pieces of
  // tail_kb K blocks each, one piece per pair; every piece leaves its fp32 partial tile in its own slice of a scratch
  // buffer and the piece that arrives last adds them up (0 parts: no split).
  int tail_first, tail_parts, tail_kb;
  float* ws;               // [tail tiles][parts][256 columns][256 rows] fp32; contents undefined before and after
  uint32_t* counters;      // [tail tiles][2 CTAs of the pair], zero on entry and on exit
  void* out;
  int64_t sx, sy;
  int out_dtype;
  uint32_t idesc;
  uint32_t* status;
};

// The n-th piece of work of pair `pair`: a whole tile (full rounds: tiles pair, pair + pairs, ...) or, in the split
// tail, one K range of a tail tile. Every role of both CTAs walks the same sequence.
struct WorkItem {
  int tile, kb0, kb1;
  bool partial;
  int part;
};
__device__ __forceinline__ bool work_item(const PairArgs& a, int pair, int npairs, int n, WorkItem* w) {
  const int ntiles = a.tiles_x * a.tiles_y;
  const int full_rounds = a.tail_parts > 1 ? a.tail_first / npairs : 0x7fffffff;   // tail_first is a multiple of npairs
  if (n < full_rounds) {
    const int t = pair + n * npairs;
    if (t >= ntiles) return false;
    *w = WorkItem{t, 0, a.kblocks, false, 0};
    return true;
  }
  // split tail: unit u covers part u % parts of tail tile u / parts; a pair may get several units
  const int u = pair + (n - full_rounds) * npairs;
  const int tile = a.tail_first + u / a.tail_parts, part = u % a.tail_parts;
  if (tile >= ntiles) return false;
  const int kb0 = part * a.tail_kb, kb1 = min(a.kblocks, kb0 + a.tail_kb);
  *w = WorkItem{tile, kb0, kb1, true, part};
  return true;
}

template <bool kFp8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y, const PairArgs a) {
  constexpr int kElemsPerBlock = kFp8 ? 128 : 64;   // K elements in one 128-byte span

  // identical carve-up in both CTAs: descriptors, barriers and the TMEM slot sit at the same offsets
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kBarrierOffset);
  uint64_t* empty = full + kStages;
  uint64_t* acc_full = empty + kStages;      // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2], used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint32_t* last_flag = tmem_slot + 2;       // tail split: "this CTA arrived last at its half of the tile"

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tc::cluster_ctarank();      // 0: leader, 1: peer
  const uint32_t leader = rank & ~1u, other = rank ^ 1u;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int nkb = a.kblocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(&full[s], 1);
      tc::mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&acc_full[i], 1);
      tc::mbar_init(&acc_empty[i], 8);         // four epilogue warps in each of the two CTAs
    }
    *abort_flag = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_desc(&map_x);
    tc::tma_prefetch_desc(&map_y);
  }
  __syncthreads();
  tc::cluster_arrive();
  tc::cluster_wait();          // both CTAs' barriers exist before anyone arrives on them remotely
  if (warp == 1) {
    tc::tmem_alloc_pair(tmem_slot, kTmemCols);
    tc::tmem_relinquish_pair();
  }
  tc::fence_before_thread_sync();
  __syncthreads();
  tc::fence_after_thread_sync();
  const uint32_t tmem_base = *tmem_slot;
  ptx::pdl_wait();             // prefill shapes: both operands may come from earlier kernels of the stream
  ptx::pdl_launch_dependents();

  // a role that gives up tells the whole pair, so that the other roles stop early too
  auto fail = [&]() {
    *abort_flag = 1;
    tc::st_cluster_u32(tc::map_to_cta(tc::smem_u32(const_cast<uint32_t*>(abort_flag)), other), 1u);
    if (a.status) atomicExch(a.status, (uint32_t)kTimeoutGemmPipeline);
  };

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer (both CTAs): own halves of X and Y, bytes credited to the leader's barrier ----
      const uint32_t leader_full = tc::map_to_cta(tc::smem_u32(&full[0]), leader);
      uint32_t it = 0;                                   // K blocks issued so far by this CTA
      bool ok = true;
      WorkItem w;
      for (int n = 0; work_item(a, pair, npairs, n, &w) && ok && !*abort_flag; ++n) {
        const int t = w.tile;
        const int x_row0 = (t % a.tiles_x) * kTileM + (int)(rank & 1u) * kRowsPerCta;
        const int y_row0 = (t / a.tiles_x) * kTileN + (int)(rank & 1u) * kRowsPerCta;
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const uint32_t s = it % kStages;
          if (it >= (uint32_t)kStages && !tc::mbar_wait(&empty[s], ((it / kStages) - 1) & 1, kWaitLimit, abort_flag)) {
            ok = false;
            break;
          }
          if (rank == leader) tc::mbar_arrive_expect_tx(&full[s], 2 * kStageBytes);
          const uint32_t dst = tc::smem_u32(smem + s * kStageBytes);
          const uint32_t bar = leader_full + s * 8u;
          tc::tma_load_2d_pair(dst, &map_x, bar, kb * kElemsPerBlock, x_row0);
          tc::tma_load_2d_pair(dst + kOperandBytes, &map_y, bar, kb * kElemsPerBlock, y_row0);
        }
      }
      if (!ok) fail();
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == leader) {
      // ---- MMA issue (leader only) ----
      uint32_t it = 0;
      int n = 0;                                         // tiles started so far by this pair
      bool ok = true;
      WorkItem w;
      for (; work_item(a, pair, npairs, n, &w) && ok; ++n) {
        const uint32_t buf = n & 1;
        if (n >= 2 && !tc::mbar_wait(&acc_empty[buf], ((n >> 1) - 1) & 1, kWaitLimit, abort_flag)) {
          ok = false;
          break;
        }
        tc::fence_after_thread_sync();
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const uint32_t s = it % kStages;
          if (!tc::mbar_wait(&full[s], (it / kStages) & 1, kWaitLimit, abort_flag)) {
            ok = false;
            break;
          }
          tc::fence_after_thread_sync();
          const uint32_t xa = tc::smem_u32(smem + s * kStageBytes);
          const uint64_t dx = tc::make_smem_desc_sw128(xa);
          const uint64_t dy = tc::make_smem_desc_sw128(xa + kOperandBytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)   // 32 bytes of K per instruction, stepped inside the swizzle span
            tc::umma_pair<kFp8>(tmem_base + buf * kTileN, dx + (uint64_t)(k * 2), dy + (uint64_t)(k * 2), a.idesc,
                                (kb > w.kb0 || k > 0) ? 1u : 0u);
          tc::umma_commit_pair(&empty[s], other);   // the stage is free again in both CTAs
        }
        if (ok) tc::umma_commit_pair(&acc_full[buf], other);
      }
      if (!ok) fail();
    }
  } else {
    // ---- epilogue (warps 2..5 of both CTAs): TMEM lane quarter = warp % 4 ----
    const int q = warp & 3;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t leader_acc_empty = tc::map_to_cta(tc::smem_u32(&acc_empty[0]), leader);
    int n = 0;
    WorkItem w;
    for (; work_item(a, pair, npairs, n, &w); ++n) {
      const int t = w.tile;
      const uint32_t buf = n & 1;
      const int x = (t % a.tiles_x) * kTileM + (int)(rank & 1u) * kRowsPerCta + q * 32 + lane;
      const int y_base = (t / a.tiles_x) * kTileN;
      // the warp leaves the loop as a whole (tcgen05.ld is a warp-wide instruction)
      if (nkb <= 0 || !__all_sync(0xffffffffu, tc::mbar_wait(&acc_full[buf], (n >> 1) & 1, kWaitLimit, abort_flag))) {
        if (nkb > 0 && lane == 0 && q == 0) fail();
        break;
      }
      tc::fence_after_thread_sync();
      if (!w.partial) {
#pragma unroll 4
        for (int c = 0; c < kTileN; c += 16) {
          float v[16];
          tc::tmem_ld_16(lane_addr + buf * kTileN + c, v);
          if (y_base + c < a.y_rows) store_chunk(a, x, y_base + c, v);
        }
        tc::fence_before_thread_sync();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive_cluster(leader_acc_empty + buf * 8u);   // this warp has read its part of the buffer
      } else {
        // A K range of a tail tile: this CTA's 128 x 256 partial sums go to the piece's own slice of the scratch
        // (column-major, so that a warp's lanes write 32 consecutive floats; plain stores - fp32 atomics on a
        // shared tile cost several times the tile's own MMA time). The CTA that arrives last at its half of the
        // tile adds the slices up, writes the output and re-zeroes the counter.
        const int rem = t - a.tail_first, half = (int)(rank & 1u);
        const size_t slice = (size_t)kTileM * kTileN;
        float* tile_ws = a.ws + (size_t)rem * a.tail_parts * slice + half * kRowsPerCta + q * 32 + lane;
        float* mine = tile_ws + (size_t)w.part * slice;
#pragma unroll 4
        for (int c = 0; c < kTileN; c += 16) {
          float v[16];
          tc::tmem_ld_16(lane_addr + buf * kTileN + c, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) __stcg(mine + (size_t)(c + j) * kTileM, v[j]);
        }
        tc::fence_before_thread_sync();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive_cluster(leader_acc_empty + buf * 8u);
        __threadfence();
        tc::named_barrier_sync(1, 128);
        if (threadIdx.x == 64) {
          const uint32_t prev = atomicAdd(&a.counters[rem * 2 + half], 1u);
          *last_flag = (prev == (uint32_t)a.tail_parts - 1u) ? 1u : 0u;        // every piece is non-empty (host)
        }
        tc::named_barrier_sync(1, 128);
        if (*last_flag) {
          __threadfence();
          // 64 columns at a time: all loads of a piece are issued before the first add waits for one, and before the
          // stores of the group (which the compiler must assume to alias the scratch) - the pass is bound by how many
          // loads are in flight, not by bytes
#pragma unroll 1
          for (int c = 0; c < kTileN; c += 64) {
            float v[64];
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = 0.f;
            for (int pp = 0; pp < a.tail_parts; ++pp) {     // in the order of the pieces: the sum does not depend on who is last
              const float* src = tile_ws + (size_t)pp * slice + (size_t)c * kTileM;
              float in[64];
#pragma unroll
              for (int j = 0; j < 64; ++j) in[j] = __ldcg(src + (size_t)j * kTileM);
#pragma unroll
              for (int j = 0; j < 64; ++j) v[j] += in[j];
            }
#pragma unroll
            for (int cc = 0; cc < 64; cc += 16) {
              float o[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) o[j] = v[cc + j];
              if (y_base + c + cc < a.y_rows) store_chunk(a, x, y_base + c + cc, o);
            }
          }
          if (threadIdx.x == 64) a.counters[rem * 2 + half] = 0;
        }
      }
    }
  }

  // ---- common exit ----
  tc::fence_before_thread_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);   // copies already issued land before shared memory goes away
  }
  tc::cluster_arrive();
  tc::cluster_wait();
  if (warp == 1) {
    tc::fence_after_thread_sync();
    tc::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <bool kFp8>
std::string launch(const CUtensorMap& mx, const CUtensorMap& my, const PairArgs& a, dim3 grid, cudaStream_t stream) {
  auto kern = gemm_pair_kernel<kFp8>;
  const std::string err = reserve_dynamic_smem(kern, kSmemTotal);
  if (!err.empty()) return err;
  const cudaError_t e = launch_chained(kern, grid, dim3(kThreads), kSmemTotal, stream, mx, my, a);
  return e == cudaSuccess ? "" : std::string("GEMM launch failed: ") + cudaGetErrorString(e);
}

}  // namespace

std::string gemm_tn_pair(const GemmProblem& g, cudaStream_t stream) {
  const bool fp8 = g.elem_size == 1;
  if (g.x_scale != nullptr || g.y_scale != nullptr) return "the two-CTA kernel takes unscaled operands";
  const int epb = 128 / g.elem_size;
  if (g.k <= 0 || g.k % epb) return "K must be a positive multiple of " + std::to_string(epb);
  if (g.x_rows <= 0 || g.y_rows <= 0) return "";
  PairArgs a{};
  a.x_rows = g.x_rows;
  a.y_rows = g.y_rows;
  a.kblocks = g.k / epb;
  a.out = g.out;
  a.sx = g.sx;
  a.sy = g.sy;
  a.out_dtype = g.out_dtype;
  a.idesc = fp8 ? tc::make_idesc(kTileM, kTileN, 0, 0)
                : tc::make_idesc(kTileM, kTileN, g.elem_kind == kBF16 ? 1 : 0, g.elem_kind == kBF16 ? 1 : 0);
  a.status = g.status;
  CUtensorMap mx, my;
  std::string err = tma::kmajor_2d(&mx, g.x, g.x_rows, g.k, g.ldx, g.elem_size, g.elem_kind, kRowsPerCta);
  if (!err.empty()) return err;
  err = tma::kmajor_2d(&my, g.y, g.y_rows, g.k, g.ldy, g.elem_size, g.elem_kind, kRowsPerCta);
  if (!err.empty()) return err;
  a.tiles_x = (g.x_rows + kTileM - 1) / kTileM;
  a.tiles_y = (g.y_rows + kTileN - 1) / kTileN;
  // one pair per two SMs, fewer when there are fewer tiles; pairs that cannot be resident at once simply start later
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long ntiles = (long long)a.tiles_x * a.tiles_y;
  const int pairs = (int)(ntiles < sms / 2 ? ntiles : sms / 2);
  const dim3 grid(2 * pairs, 1, 1);
  // Tail split: when the last round is partly filled, its tiles are cut along K into `parts` pieces so that the idle
  // pairs share the work; the pieces meet in fp32 scratch slices. parts minimises the time of the tail in tile-times,
  // ceil(tail * parts / pairs) / parts, plus what the pieces pay for meeting in the scratch (128 KB written per CTA,
  // a memory fence and a counter per piece, parts x 128 KB read by the one that adds up: measured about
  // 6 + 3 x parts microseconds, against 8.6 ns of tile time per unit of K).
  a.tail_first = (int)ntiles;
  a.tail_parts = 0;
  const int tail = (int)(ntiles % pairs);
  if (tail > 0 && ntiles > pairs && g.ws != nullptr && g.counters != nullptr && (size_t)tail * 2 <= g.counter_count) {
    const double tile_us = 8.6e-3 * (double)g.k;
    int best = 1;
    // the unsplit tail costs one tile time; a split has to win by a margin (measured against cuBLAS on the same
    // box: 2048 x 8192 x 8192 went from 1.14 x to 1.04 x its time with two pieces, 2048 x 4096 x 14336 from 1.17 x to
    // 1.24 x with four pieces at a predicted 0.90)
    double best_cost = 0.89;
    for (int parts = 2; parts <= 4 && a.kblocks / parts >= 4; ++parts) {
      if ((size_t)tail * parts * kTileM * kTileN * sizeof(float) > g.ws_bytes) break;
      const double cost = (double)((tail * parts + pairs - 1) / pairs) / parts + (6.0 + 3.0 * parts) / tile_us;
      if (cost < best_cost - 1e-9) {
        best_cost = cost;
        best = parts;
      }
    }
    if (best > 1) {
      a.tail_kb = (a.kblocks + best - 1) / best;
      if ((best - 1) * a.tail_kb < a.kblocks) {      // every piece non-empty
        a.tail_first = (int)(ntiles - tail);
        a.tail_parts = best;
        a.ws = g.ws;
        a.counters = g.counters;
      }
    }
  }
  return fp8 ? launch<true>(mx, my, a, grid, stream) : launch<false>(mx, my, a, grid, stream);
}

}  // namespace tdx
