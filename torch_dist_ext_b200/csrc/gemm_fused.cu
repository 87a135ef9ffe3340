// GEMMs fused with their collectives over peer memory (NVLink / NVSwitch), one kernel each:
//
//  gemm_ar_rmsnorm   row-parallel linear (o_proj / down_proj of a tensor-parallel layer):
//                    every rank multiplies its K shard on the tensor cores (tcgen05, accumulator in
//                    TMEM); the epilogue pushes each finished 128-column x tokens tile straight into
//                    the gather slots of the rows' OWNER ranks (reduce-scatter by peer stores, tile
//                    by tile, while other CTAs are still multiplying); the same CTAs then turn into
//                    the reducers of the two-shot Lamport flow: sum the N partial rows, add the
//                    residual, RMS-normalise (optionally quantise to e4m3 with 1x128 scales), and
//                    either keep the scattered rows (sequence-parallel) or push them back to all
//                    peers (replicated output).
//  ag_gemm           column-parallel linear on sequence-parallel input: every rank pushes its row
//                    shard of the activations into all peers' staging buffers and raises a flag; the
//                    TMA producer prefetches the first ring of weight tiles, waits (bounded) for the
//                    N flags, then streams the gathered activations from LOCAL memory. No TMA load
//                    ever reads a peer's memory, and none uses cluster multicast.
//
// Both need all CTAs of the grid to be resident at once (CTAs wait for data produced by others), so
// the host refuses grids larger than the SM count; for gemm_ar_rmsnorm with bf16 operands the persistent kernel
// of gemm_fused_persist.cu takes over there.
//
// The reference has neither (its only kernel is the standalone all-reduce+RMSNorm,
// src/common/all_reduce_fusion_impl.h:342-474); these are the two paths that a tensor-parallel
// decoder layer built on that op needs next to it.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <mutex>
#include <set>
#include <utility>
#include "tdx/ar_fusion_kernels.cuh"
#include "tdx/gemm.h"
#include "tdx/gemm_core.cuh"
#include "tdx/launch.h"
#include "tdx/tc.cuh"
#include "tdx/tma_host.h"

#ifndef TDX_FUSED_N
#define TDX_FUSED_N 0
#endif

namespace tdx {
namespace {

using gemm_core::kBM;
using gemm_core::SmemLayout;
using T = __nv_bfloat16;
constexpr int kThreads = 256;
constexpr int kElemsPerBlock = 64;

struct FusedArgs {
  ArParams ar;        // communication state and the description of the reduce/normalise tail
  int kblocks;
  int kblocks_per_split;
  uint32_t idesc;
  uint32_t* status;
  float* ws;          // split-K scratch, zero on entry and on exit
  uint32_t* counters;
  // e4m3 operands with block scales (kScaled kernels): weights one scale per 128 x 128 block, activations one per
  // token and 128-wide K block; fp32, row length scale_kb = K / 128
  const float* w_scale;
  const float* a_scale;
  int scale_kb;
  int one_hop;        // replicated output at decode sizes: tiles go to EVERY rank and each rank reduces all rows itself
};

// D tile (TMEM) -> bf16 rows in shared memory -> 16-byte pushes into the owners' gather slots, or (one_hop) into this
// rank's slot of EVERY rank's buffer - one multimem.st per vector where NVSwitch multicast is mapped, else one peer
// store per rank - for the one-hop tail below.
// With K split over gridDim.z the partial tiles are first summed in an fp32 scratch tile with
// red.global.add; the CTA that arrives last at the tile converts and pushes it (and leaves the
// scratch tile and its counter zeroed for the next call).
// kFromRegs: the tile's values come from `acc` (this thread's row of the tile, promoted block by block from the
// scaled fp8 partial products) instead of tensor memory.
template <int kBN, bool kFromRegs>
__device__ __forceinline__ void push_tile_to_owners(const ArParams& p, const FusedArgs& f, uint8_t* stage,
                                                    uint32_t* shared_flag, uint32_t tmem_base, int tile_x, int tile_y,
                                                    size_t buf_off, int groups, const float* acc, bool one_hop) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = warp & 3;
  const int te = threadIdx.x - 64;                 // 0..127 among the epilogue threads
  const int xl = q * 32 + lane;                    // column of this thread inside the tile
  const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
  __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(stage);
  bool push = true;
  if (gridDim.z > 1) {
    // column-major scratch tile: a warp's 32 lanes add to one 128-byte line per instruction
    float* tile = f.ws + (size_t)(tile_y * gridDim.x + tile_x) * (kBM * kBN) + xl;
#pragma unroll
    for (int c = 0; c < kBN; c += 16) {
      float v[16];
      if constexpr (kFromRegs) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = acc[c + j];
      } else {
        tc::tmem_ld_16(lane_addr + c, v);
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) atomicAdd(tile + (size_t)(c + j) * kBM, v[j]);
    }
    __threadfence();
    tc::named_barrier_sync(1, 128);
    if (te == 0) {
      const uint32_t prev = atomicAdd(&f.counters[tile_y * gridDim.x + tile_x], 1u);
      *shared_flag = (prev == gridDim.z - 1) ? 1u : 0u;
    }
    tc::named_barrier_sync(1, 128);
    push = *shared_flag != 0;
    if (push) {
      __threadfence();
#pragma unroll
      for (int c = 0; c < kBN; ++c) {
        st[c * kBM + xl] = __float2bfloat16(__ldcg(tile + (size_t)c * kBM));
        __stcg(tile + (size_t)c * kBM, 0.f);
      }
      if (te == 0) f.counters[tile_y * gridDim.x + tile_x] = 0;
    }
  } else {
#pragma unroll
    for (int c = 0; c < kBN; c += 16) {
      float v[16];
      if constexpr (kFromRegs) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = acc[c + j];
      } else {
        tc::tmem_ld_16(lane_addr + c, v);
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) st[(c + j) * kBM + xl] = __float2bfloat16(v[j]);
    }
  }
  if (!push) return;
  tc::named_barrier_sync(1, 128);
  const int y_base = tile_y * kBN;
  const int valid = min(kBN, p.tokens - y_base);
  const size_t row_bytes = (size_t)p.hidden * sizeof(T);
  for (int i = te; i < valid * 16; i += 128) {
    const int tl = i >> 4, part = i & 15;
    const int t = y_base + tl;
    const int owner = t % p.nranks, j = t / p.nranks;
    const uint4 val = scrub(*reinterpret_cast<const uint4*>(stage + (size_t)tl * (kBM * 2) + part * 16));
    if (one_hop) {
      // slot `rank` of the one-shot layout [source rank][token][hidden], the same offset in every rank's buffer
      const size_t off = buf_off + ((size_t)p.rank * p.tokens + t) * row_bytes + ((size_t)tile_x * kBM + part * 8) * sizeof(T);
      if (p.mc_base != nullptr) {
        ptx::multimem_st_v4(symm_mc(p, off), val);
      } else {
        for (int r = 0; r < p.nranks; ++r) ptx::st_v4(static_cast<char*>(p.peer[r]) + off, val);
      }
    } else {
      char* dst = static_cast<char*>(p.peer[owner]) + buf_off + ((size_t)p.rank * groups + j) * row_bytes +
                  ((size_t)tile_x * kBM + part * 8) * sizeof(T);
      ptx::st_v4(dst, val);
    }
  }
}

// One-hop tail: every rank holds every rank's partial rows (slot r of the current Lamport buffer, this rank's own
// included), so each CTA takes rows cta, cta + nctas, ..., waits for the N vectors of a row, adds them and the
// residual, normalises and writes the outputs - the all-reduce is complete after ONE trip through NVSwitch. The
// reduction is done N times over (once per rank), which at decode sizes costs less than the second hop of the
// reduce-scatter + gather flow. Returns the bytes of the buffer that were written.
template <int kN, int kVpt, int kOut>
__device__ __forceinline__ uint64_t onehop_tail(const ArParams& p, int cta, int nctas, uint32_t epoch, float (*red)[32]) {
  constexpr int kVec = VecTraits<T>::kVec;
  const int nranks = kN > 0 ? kN : p.nranks;
  const RowView<T, kVpt> rv(p.hidden);
  char* self = static_cast<char*>(p.peer[p.rank]);
  Control* ctl = reinterpret_cast<Control*>(self + p.layout.off_control);
  const size_t msg_bytes = rv.row_bytes * p.tokens;
  const char* mine = lamport_buf(self, p.layout, epoch % 3u);
  uint4 gamma[kVpt];
  load_gamma<T, kVpt>(p, rv, gamma);
  Waiter w(p.timeout_ns);
  int parity = 0;
  for (int row = cta; row < p.tokens; row += nctas, parity ^= 1) {
    float x[kVpt][kVec];
    uint4 res[kVpt];
    request_residual<T, kVpt>(p, rv, row, res);
#pragma unroll
    for (int v = 0; v < kVpt; ++v) {
#pragma unroll
      for (int i = 0; i < kVec; ++i) x[v][i] = 0.f;
      if (!rv.active(v)) continue;
      const size_t off = (size_t)row * rv.row_bytes + (size_t)rv.vec_index(v) * 16;
      if constexpr (kN > 0) {
        uint4 vals[kN];
#pragma unroll
        for (int r = 0; r < kN; ++r) vals[r] = ptx::ld_volatile_v4(mine + (size_t)r * msg_bytes + off);   // all polls in flight together
#pragma unroll
        for (int r = 0; r < kN; ++r)
          if (!all_arrived(vals[r])) vals[r] = poll_vec(mine + (size_t)r * msg_bytes + off, w, p, ctl, kTimeoutLamportGather, r, 1, row);
#pragma unroll
        for (int r = 0; r < kN; ++r) {
          float f[kVec];
          unpack<T>(vals[r], f);
#pragma unroll
          for (int i = 0; i < kVec; ++i) x[v][i] += f[i];
        }
      } else {
        for (int r = 0; r < nranks; ++r) {
          const uint4 val = poll_vec(mine + (size_t)r * msg_bytes + off, w, p, ctl, kTimeoutLamportGather, r, 1, row);
          float f[kVec];
          unpack<T>(val, f);
#pragma unroll
          for (int i = 0; i < kVec; ++i) x[v][i] += f[i];
        }
      }
      add_residual_loaded<T>(x[v], p.residual_in != nullptr, res[v]);
      if (p.residual_out) ptx::st_stream_v4(static_cast<char*>(p.residual_out) + off, pack<T>(x[v]));
    }
    float rstd, sc;
    finish_row<T, kVpt, kOut>(p, rv, row, x, gamma, red, parity, rstd, sc);
  }
  return (uint64_t)nranks * msg_bytes;
}

template <int kBN, int kStages, int kN, int kVpt, int kOut, bool kScaled>
__global__ void __launch_bounds__(kThreads, 1)
gemm_ar_rmsnorm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, const FusedArgs f) {
  // kScaled: e4m3 operands with block scales; every 128-wide K block is multiplied into its own TMEM buffer (two,
  // alternating) and promoted in fp32 by the epilogue warps while the next block's MMAs run.
  constexpr uint32_t kTmemCols = kScaled ? (2 * kBN < 32 ? 32 : 2 * kBN) : (kBN < 32 ? 32 : kBN);
  constexpr int kEpb = kScaled ? 128 : kElemsPerBlock;   // K elements per 128-byte block
  extern __shared__ uint8_t smem_raw[];
  __shared__ float red[4][32];
  gemm_core::Pipeline<kBN, kStages> pipe;
  pipe.init(smem_raw, kTmemCols, &map_w, &map_a);
  const ArParams& p = f.ar;
  char* self = static_cast<char*>(p.peer[p.rank]);
  Control* ctl = reinterpret_cast<Control*>(self + p.layout.off_control);
  const int groups = (p.tokens + p.nranks - 1) / p.nranks;
  const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  const int nctas = gridDim.x * gridDim.y * gridDim.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb0 = blockIdx.z * f.kblocks_per_split;
  const int nkb = min(f.kblocks, kb0 + f.kblocks_per_split) - kb0;

  // The producer thread requests the first ring of WEIGHT tiles (never written by a kernel) before it waits for
  // the previous kernel of the stream; everything else - activations, the communication state - comes after.
  if (warp == 0 && lane == 0)
    pipe.template produce<kEpb>(&map_w, &map_a, blockIdx.x * kBM, blockIdx.y * kBN, kb0, nkb, f.status, [] {
      ptx::pdl_wait();
      return true;
    });
  ptx::pdl_wait();
  ptx::pdl_launch_dependents();
  const uint32_t epoch = ctl->lamport_epoch;
  const uint64_t dirty_prev = ctl->lamport_dirty[(epoch + 2u) % 3u];
  const size_t buf_off = p.layout.off_lamport + (size_t)(epoch % 3u) * p.layout.lamport_bytes;

  if (warp == 0) {
  } else if (warp == 1) {
    if (lane == 0) pipe.template issue<kScaled, kScaled>(nkb, f.idesc, f.status);
  } else if (warp < 6) {
    bool ok = true;
    float acc[kScaled ? kBN : 1];
    if constexpr (kScaled) {
      const int q = warp & 3;
      const int x = blockIdx.x * kBM + q * 32 + lane;          // weight row (output column) of this thread
      const uint32_t lane_addr = pipe.tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll
      for (int i = 0; i < kBN; ++i) acc[i] = 0.f;
      // Scales of a K block: the weight scale of this thread's row block, and the kBN (<= 64) token scales held two
      // per lane and handed round with shuffles; those of block i + 1 are requested before the wait for block i.
      static_assert(kBN <= 64, "the promoting epilogue keeps the token scales of a K block in two registers per lane");
      const float* ws_ptr = f.w_scale + (size_t)(x < p.hidden ? x / 128 : 0) * f.scale_kb;
      const float* as_lo_ptr = f.a_scale + (size_t)min((int)blockIdx.y * kBN + lane, p.tokens - 1) * f.scale_kb;
      const float* as_hi_ptr = f.a_scale + (size_t)min((int)blockIdx.y * kBN + 32 + lane, p.tokens - 1) * f.scale_kb;
      float ws_next = nkb > 0 ? ws_ptr[kb0] : 0.f;
      float lo_next = nkb > 0 ? as_lo_ptr[kb0] : 0.f;
      float hi_next = (nkb > 0 && kBN > 32) ? as_hi_ptr[kb0] : 0.f;
      for (int i = 0; i < nkb && ok; ++i) {
        const int buf = i & 1;
        const float ws = ws_next, as_lo = lo_next, as_hi = hi_next;
        if (i + 1 < nkb) {
          ws_next = ws_ptr[kb0 + i + 1];
          lo_next = as_lo_ptr[kb0 + i + 1];
          if (kBN > 32) hi_next = as_hi_ptr[kb0 + i + 1];
        }
        ok = __all_sync(0xffffffffu, tc::mbar_wait(&pipe.acc_full[buf], (i >> 1) & 1, gemm_core::kWaitLimit, pipe.abort_flag));
        if (!ok) break;
        tc::fence_after_thread_sync();
        gemm_core::promote_block<kBN>(lane_addr + buf * kBN, ws, as_lo, as_hi, acc);
        tc::fence_before_thread_sync();
        tc::mbar_arrive(&pipe.acc_empty[buf]);
      }
    } else {
      ok = tc::mbar_wait(&pipe.acc_full[0], 0, gemm_core::kWaitLimit, pipe.abort_flag);
      tc::fence_after_thread_sync();
    }
    if (!ok) pipe.fail(f.status);
    // every MMA has completed, so the operand ring is free: stage the tile there
    if (ok)
      push_tile_to_owners<kBN, kScaled>(p, f, pipe.smem, pipe.scratch, pipe.tmem_base, blockIdx.x, blockIdx.y, buf_off, groups,
                                        acc, f.one_hop != 0);
  }
  __syncthreads();
  clear_previous(lamport_buf(self, p.layout, (epoch + 2u) % 3u), dirty_prev, cta, nctas);
  const uint64_t dirty = f.one_hop ? onehop_tail<kN, kVpt, kOut>(p, cta, nctas, epoch, red)
                                   : twoshot_lamport_tail<T, kN, kVpt, kOut, true>(p, cta, nctas, epoch, red);
  finish_launch(ctl, true, epoch, dirty, 0, nctas);
  pipe.finish(kTmemCols);
}

// ---- all-gather -> GEMM --------------------------------------------------------------------------

struct AgArgs {
  void* peer[kMaxRanks];
  Layout layout;
  int rank, nranks;
  int tokens, k;            // gathered activation matrix [tokens, k]
  const void* x_shard;      // this rank's rows (token t with t % nranks == rank, in order), [ceil, k]
  int out_rows;             // weight rows of this rank (output columns)
  void* out;                // [tokens, out_rows] row-major
  int64_t ldo;
  int kblocks;
  uint32_t idesc;
  uint32_t* status;
  uint64_t timeout_ns;
  uint32_t* host_status;
};

__device__ __forceinline__ uint32_t* ag_flag(void* base, const Layout& l, int src) {
  return reinterpret_cast<uint32_t*>(static_cast<char*>(base) + l.off_ag_flags) + src;
}

template <int kBN, int kStages>
__global__ void __launch_bounds__(kThreads, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_g0,
               const __grid_constant__ CUtensorMap map_g1, const AgArgs a) {
  constexpr uint32_t kTmemCols = kBN < 32 ? 32 : kBN;
  extern __shared__ uint8_t smem_raw[];
  // 0 while the producer still waits for the peers' rows, then 1 (arrived) or 2 (gave up). The MMA thread and the
  // epilogue warps watch it with the workspace's TIME budget before they start their poll-counted pipeline waits,
  // so a peer that is late but within budget cannot make them give up first.
  __shared__ volatile uint32_t gate_state;
  if (threadIdx.x == 0) gate_state = 0;
  gemm_core::Pipeline<kBN, kStages> pipe;
  pipe.init(smem_raw, kTmemCols, &map_w, &map_g0);
  char* self = static_cast<char*>(a.peer[a.rank]);
  Control* ctl = reinterpret_cast<Control*>(self + a.layout.off_control);
  const int cta = blockIdx.x + gridDim.x * blockIdx.y, nctas = gridDim.x * gridDim.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t row_bytes = (size_t)a.k * sizeof(T);
  const int my_rows = (a.tokens - a.rank + a.nranks - 1) / a.nranks;
  // Only the producer thread runs ahead of the previous kernel of the stream, and only to request weight tiles
  // (its gate begins with the same wait); the epoch is read after the wait on every path.
  if (!(warp == 0 && lane == 0)) {
    ptx::pdl_wait();
    ptx::pdl_launch_dependents();
  }

  auto gate_passed = [&]() -> bool {
    Waiter w(a.timeout_ns * (uint64_t)(a.nranks + 1));   // the producer waits for the ranks one after the other
    w.begin();
    while (gate_state == 0) {
      if (!w.keep_waiting()) return false;
      __nanosleep(64);
    }
    return true;   // on 2 the producer has raised the abort flag already: the pipeline waits return at once
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t epoch_p = 0;
      auto gate = [&]() -> bool {
        ptx::pdl_wait();
        epoch_p = ctl->ag_epoch;
        const uint32_t target = epoch_p + 1u;
        // all N shards must have landed in THIS rank's staging buffer
        Waiter w(a.timeout_ns);
        for (int r = 0; r < a.nranks; ++r) {
          const uint32_t* fl = ag_flag(self, a.layout, r);
          w.begin();
          while ((int32_t)(ptx::ld_acquire_sys(fl) - target) < 0) {
            if (!w.keep_waiting()) {
              report_error(ctl, a.host_status, kTimeoutTileFlag, a.rank, r, 1, -1);
              gate_state = 2;
              return false;
            }
          }
        }
        // the rows were written through the generic proxy (peer stores); TMA reads through the async proxy
        asm volatile("fence.proxy.async.global;" ::: "memory");
        gate_state = 1;
        return true;
      };
      pipe.template produce_late_y<kElemsPerBlock>(&map_w, &map_g0, &map_g1, &epoch_p, blockIdx.x * kBM, blockIdx.y * kBN, 0,
                                                   a.kblocks, a.status, gate);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      if (gate_passed()) pipe.template issue<false, false>(a.kblocks, a.idesc, a.status);
      else pipe.fail(a.status);
    }
  } else {
    // warps 2..7: destination `d` of the all-gather is served by CTA d % nctas
    const uint32_t epoch = ctl->ag_epoch;
    const uint32_t target = epoch + 1u;
    const size_t gbuf_off = a.layout.off_ag + (size_t)(epoch & 1u) * a.layout.ag_buf_bytes;
    const int tp = threadIdx.x - 64;   // 0..191
    for (int d = cta; d < a.nranks; d += nctas) {
      char* dst_base = static_cast<char*>(a.peer[d]) + gbuf_off;
      const size_t vec_per_row = row_bytes / 16;
      const size_t total = (size_t)my_rows * vec_per_row;
      for (size_t i = tp; i < total; i += 192) {
        const size_t j = i / vec_per_row, part = i % vec_per_row;
        const uint4 val = ptx::ld_stream_v4(static_cast<const char*>(a.x_shard) + j * row_bytes + part * 16);
        ptx::st_v4(dst_base + (j * a.nranks + a.rank) * row_bytes + part * 16, val);
      }
      tc::named_barrier_sync(2, 192);
      if (tp == 0) ptx::st_release_sys(ag_flag(a.peer[d], a.layout, a.rank), target);
    }
    if (warp < 6) {
      // epilogue: D[x = weight row, y = token] -> out[token, weight row]
      const int q = warp & 3;
      const bool ok = gate_passed() && tc::mbar_wait(&pipe.acc_full[0], 0, gemm_core::kWaitLimit, pipe.abort_flag);
      tc::fence_after_thread_sync();
      if (!ok) pipe.fail(a.status);
      const int x = blockIdx.x * kBM + q * 32 + lane;
      const uint32_t lane_addr = pipe.tmem_base + ((uint32_t)(q * 32) << 16);
      if (ok) {
#pragma unroll
        for (int c = 0; c < kBN; c += 16) {
          float v[16];
          tc::tmem_ld_16(lane_addr + c, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = blockIdx.y * kBN + c + j;
            if (t < a.tokens && x < a.out_rows) static_cast<T*>(a.out)[(int64_t)t * a.ldo + x] = __float2bfloat16(v[j]);
          }
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(&ctl->arrive, 1u);
    if (done == (uint32_t)nctas - 1) {
      ctl->ag_epoch = ctl->ag_epoch + 1u;
      ctl->arrive = 0;
      __threadfence();
    }
  }
  pipe.finish(kTmemCols);
}

// ---- host side ---------------------------------------------------------------------------------------

std::string bf16_map(CUtensorMap* map, const void* ptr, int rows, int k, int64_t ld, int box_rows) {
  return tma::kmajor_2d(map, ptr, rows, k, ld, 2, kBF16, box_rows);
}

int sm_count() {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

template <int kBN, int kStages, int kVpt, int kOut, bool kScaled>
std::string launch_ar(const CUtensorMap& mw, const CUtensorMap& ma, const FusedArgs& f, dim3 grid, cudaStream_t s) {
  auto kern = gemm_ar_rmsnorm_kernel<kBN, kStages, TDX_FUSED_N, kVpt, kOut, kScaled>;
  std::string err = reserve_dynamic_smem(kern, SmemLayout<kBN, kStages>::kTotal);
  if (!err.empty()) return err;
  const cudaError_t e = launch_chained(kern, grid, dim3(kThreads), SmemLayout<kBN, kStages>::kTotal, s, mw, ma, f);
  return e == cudaSuccess ? "" : std::string("fused GEMM launch failed: ") + cudaGetErrorString(e);
}

template <int kBN, int kStages, bool kScaled>
std::string launch_ar_vpt(int vpt, int out_mode, const CUtensorMap& mw, const CUtensorMap& ma, const FusedArgs& f, dim3 grid,
                          cudaStream_t s) {
  const bool q = out_mode == kOutFp8Block128;
  switch (vpt) {
    case 1: return q ? launch_ar<kBN, kStages, 1, kOutFp8Block128, kScaled>(mw, ma, f, grid, s) : launch_ar<kBN, kStages, 1, kOutSame, kScaled>(mw, ma, f, grid, s);
    case 2: return q ? launch_ar<kBN, kStages, 2, kOutFp8Block128, kScaled>(mw, ma, f, grid, s) : launch_ar<kBN, kStages, 2, kOutSame, kScaled>(mw, ma, f, grid, s);
    case 4: return q ? launch_ar<kBN, kStages, 4, kOutFp8Block128, kScaled>(mw, ma, f, grid, s) : launch_ar<kBN, kStages, 4, kOutSame, kScaled>(mw, ma, f, grid, s);
  }
  return "unsupported hidden size for the fused GEMM";
}

}  // namespace

#define TDX_CAT2(a, b) a##b
#define TDX_CAT(a, b) TDX_CAT2(a, b)

// Row-parallel linear + reduce(-scatter) + residual + RMSNorm; one function per rank-count
// specialisation (0 = any rank count, runtime loop).
std::string TDX_CAT(gemm_ar_rmsnorm_n, TDX_FUSED_N)(const FusedGemmProblem& g, cudaStream_t stream) {
  const ArParams& p = g.ar;
  if (p.dtype != kBF16) return "the fused GEMM paths produce bfloat16 partial sums (bf16 or block-scaled e4m3 operands)";
  if (p.hidden % 128) return "hidden must be a multiple of 128";
  const bool scaled = g.elem_size == 1;
  if (scaled && (g.a_scale == nullptr || g.w_scale == nullptr)) return "e4m3 operands need block scales for both of them";
  const int epb = scaled ? 128 : 64;
  if (g.k <= 0 || g.k % epb) return "K must be a positive multiple of " + std::to_string(epb);
  if (p.out_mode != kOutSame && p.out_mode != kOutFp8Block128) return "fused GEMM output is bf16 or e4m3 with 1x128 scales";
  if (p.tokens <= 0) return "";
  const int bn = p.tokens <= 16 ? 16 : 64;
  dim3 grid(p.hidden / 128, (p.tokens + bn - 1) / bn, 1);
  const int sms = sm_count();
  if ((int)(grid.x * grid.y) > sms)
    return "too many tokens for the fused GEMM (all CTAs must be resident): use the GEMM followed by the all-reduce op";
  // split K until the grid covers the SMs (every CTA must stay resident, so never beyond them)
  const int kblocks = g.k / epb;
  int splits = g.splits > 0 ? g.splits : sms / (int)(grid.x * grid.y);
  if (splits > kblocks / 2) splits = kblocks / 2;
  if (splits < 1 || g.ws == nullptr || g.counters == nullptr) splits = 1;
  while (splits > 1 && (int)(grid.x * grid.y) * splits > sms) --splits;
  int per_split = (kblocks + splits - 1) / splits;
  splits = (kblocks + per_split - 1) / per_split;
  if (splits > 1 && ((size_t)grid.x * grid.y * kBM * bn * sizeof(float) > g.ws_bytes || (size_t)grid.x * grid.y > g.counter_count))
    return "split-K workspace is too small";
  grid.z = splits;
  const int nvec = p.hidden / 8;
  const int vpt = nvec <= kThreads ? 1 : nvec <= 2 * kThreads ? 2 : nvec <= 4 * kThreads ? 4 : 0;
  const uint64_t row_bytes = (uint64_t)p.hidden * 2;
  const uint64_t groups = ((uint64_t)p.tokens + p.nranks - 1) / p.nranks;
  if (g.one_hop && p.scatter_only) return "the one-hop tail produces replicated output";
  const uint64_t need = g.one_hop ? (uint64_t)p.nranks * p.tokens * row_bytes
                                  : (uint64_t)p.nranks * groups * row_bytes + (p.scatter_only ? 0 : (uint64_t)p.tokens * (row_bytes + 16));
  if (need > p.layout.lamport_bytes) return "message exceeds the Lamport buffer capacity";
  for (int r = 0; r < p.nranks; ++r)
    if (p.peer[r] == nullptr) return "workspace is not registered with all peers";
  FusedArgs f{};
  f.ar = p;
  f.one_hop = g.one_hop ? 1 : 0;
  f.kblocks = kblocks;
  f.kblocks_per_split = per_split;
  f.idesc = scaled ? tc::make_idesc(kBM, bn, 0, 0) : tc::make_idesc(kBM, bn, 1, 1);
  f.status = g.status;
  f.ws = g.ws;
  f.counters = g.counters;
  f.w_scale = g.w_scale;
  f.a_scale = g.a_scale;
  f.scale_kb = g.k / 128;
  CUtensorMap mw, ma;
  std::string err = tma::kmajor_2d(&mw, g.w, p.hidden, g.k, g.ldw, g.elem_size == 1 ? 1 : 2, kBF16, kBM);
  if (!err.empty()) return err;
  err = tma::kmajor_2d(&ma, g.a, p.tokens, g.k, g.lda, g.elem_size == 1 ? 1 : 2, kBF16, bn);
  if (!err.empty()) return err;
  if (scaled)
    return bn == 16 ? launch_ar_vpt<16, 10, true>(vpt, p.out_mode, mw, ma, f, grid, stream)
                    : launch_ar_vpt<64, 8, true>(vpt, p.out_mode, mw, ma, f, grid, stream);
  return bn == 16 ? launch_ar_vpt<16, 10, false>(vpt, p.out_mode, mw, ma, f, grid, stream)
                  : launch_ar_vpt<64, 8, false>(vpt, p.out_mode, mw, ma, f, grid, stream);
}

#if TDX_FUSED_N == 0
std::string ag_gemm(const AgGemmProblem& g, cudaStream_t stream) {
  if (g.k <= 0 || g.k % 64) return "K must be a positive multiple of 64";
  if (g.tokens <= 0 || g.out_rows <= 0) return "";
  if ((uint64_t)g.tokens * g.k * 2 > g.layout.ag_buf_bytes) return "gathered activations exceed the staging buffer";
  for (int r = 0; r < g.nranks; ++r)
    if (g.peer[r] == nullptr) return "workspace is not registered with all peers";
  const int bn = g.tokens <= 16 ? 16 : 64;
  const dim3 grid((g.out_rows + kBM - 1) / kBM, (g.tokens + bn - 1) / bn, 1);
  if ((int)(grid.x * grid.y) > sm_count())
    return "too many tiles for the fused all-gather GEMM (all CTAs must be resident)";
  AgArgs a{};
  for (int r = 0; r < kMaxRanks; ++r) a.peer[r] = g.peer[r];
  a.layout = g.layout;
  a.rank = g.rank;
  a.nranks = g.nranks;
  a.tokens = g.tokens;
  a.k = g.k;
  a.x_shard = g.x_shard;
  a.out_rows = g.out_rows;
  a.out = g.out;
  a.ldo = g.ldo;
  a.kblocks = g.k / 64;
  a.idesc = tc::make_idesc(kBM, bn, 1, 1);
  a.status = g.status;
  a.timeout_ns = g.timeout_ns;
  a.host_status = g.host_status;
  CUtensorMap mw, m0, m1;
  std::string err = bf16_map(&mw, g.w, g.out_rows, g.k, g.ldw, kBM);
  if (!err.empty()) return err;
  char* own = static_cast<char*>(g.peer[g.rank]) + g.layout.off_ag;
  err = bf16_map(&m0, own, g.tokens, g.k, g.k, bn);
  if (!err.empty()) return err;
  err = bf16_map(&m1, own + g.layout.ag_buf_bytes, g.tokens, g.k, g.k, bn);
  if (!err.empty()) return err;
  if (bn == 16) {
    auto kern = ag_gemm_kernel<16, 10>;
    err = reserve_dynamic_smem(kern, SmemLayout<16, 10>::kTotal);
    if (!err.empty()) return err;
    launch_chained(kern, grid, dim3(kThreads), SmemLayout<16, 10>::kTotal, stream, mw, m0, m1, a);
  } else {
    auto kern = ag_gemm_kernel<64, 8>;
    err = reserve_dynamic_smem(kern, SmemLayout<64, 8>::kTotal);
    if (!err.empty()) return err;
    launch_chained(kern, grid, dim3(kThreads), SmemLayout<64, 8>::kTotal, stream, mw, m0, m1, a);
  }
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? "" : std::string("all-gather GEMM launch failed: ") + cudaGetErrorString(e);
}

std::string gemm_ar_rmsnorm(const FusedGemmProblem& g, cudaStream_t stream) {
  // one CTA per tile only while all of them are resident; beyond that the persistent kernel walks the tiles
  const int bn = g.ar.tokens <= 16 ? 16 : 64;
  if (g.elem_size == 2 && (long long)(g.ar.hidden / 128) * ((g.ar.tokens + bn - 1) / bn) > sm_count())
    return gemm_ar_rmsnorm_persist(g, stream);
  switch (g.ar.nranks) {
    case 2: return gemm_ar_rmsnorm_n2(g, stream);
    case 4: return gemm_ar_rmsnorm_n4(g, stream);
    case 8: return gemm_ar_rmsnorm_n8(g, stream);
    default: return gemm_ar_rmsnorm_n0(g, stream);
  }
}
#endif

}  // namespace tdx
