// Warp/block reductions, bounded waits, error reporting, the cross-GPU flag barrier and
// the end-of-launch phase update.
//
// Counterparts in the reference: block_utils::warp_reduce / block_reduce
// (src/common/all_reduce_fusion_impl.h:32-57), comm::SyncComm (:63-93), comm::Barrier
// (:95-164) and comm::LamportComm (:166-204). Differences by design:
//  * every wait has a time budget; when it runs out the block records
//    {code, rank, peer, phase, block, row} once, stops waiting and runs to a normal exit;
//  * barrier flags carry a monotonically increasing epoch compared with a signed
//    difference, so flag rows that an earlier, smaller launch never touched need no
//    back-filling;
//  * phase state is advanced by whichever block finishes LAST (arrival counter), not by
//    block 0 spinning until every block has started.
#pragma once
#include "tdx/comm.h"
#include "tdx/ptx.cuh"

namespace tdx {

// ---- reductions ------------------------------------------------------------------

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Reduction over aligned groups of `kLanes` lanes (power of two <= 32).
template <int kLanes>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
  for (int o = kLanes / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide all-reduce; every thread gets the result. `slot` is 32 floats of shared
// memory; callers alternate between two slots so that no trailing barrier is needed.
template <bool kMax>
__device__ __forceinline__ float block_allreduce(float v, float* slot) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = kMax ? warp_max(v) : warp_sum(v);
  if (nwarps == 1) return v;
  if (lane == 0) slot[warp] = v;
  __syncthreads();
  float w = (lane < nwarps) ? slot[lane] : (kMax ? 0.f : 0.f);
  return kMax ? warp_max(w) : warp_sum(w);
}

// ---- bounded waiting ---------------------------------------------------------------

struct Waiter {
  uint64_t budget_ns;
  uint64_t deadline;   // 0 until the slow path is first entered
  uint32_t spins;
  bool failed;         // once a wait of this thread ran out, later waits give up at once

  __device__ __forceinline__ explicit Waiter(uint64_t budget)
      : budget_ns(budget), deadline(0), spins(0), failed(false) {}

  // Call once per unsuccessful poll. Returns false when the caller must stop waiting.
  __device__ __forceinline__ bool keep_waiting() {
    if (failed) return false;
    if ((++spins & 0xffu) != 0) return true;
    const uint64_t now = ptx::globaltimer_ns();
    if (deadline == 0) {
      deadline = now + budget_ns;
      return true;
    }
    if (now > deadline) {
      failed = true;
      return false;
    }
    return true;
  }
  __device__ __forceinline__ void begin() {
    deadline = 0;
    spins = 0;
  }
};

__device__ __forceinline__ void report_error(Control* ctl, uint32_t* host_status, uint32_t code,
                                             int rank, int peer, int phase, int row) {
  const uint32_t prior = atomicAdd(&ctl->error_count, 1u);
  if (prior == 0) {
    const uint32_t rec[8] = {code, (uint32_t)rank, (uint32_t)peer, (uint32_t)phase,
                             blockIdx.x, (uint32_t)row, 0u, 0u};
#pragma unroll
    for (int i = 7; i >= 0; --i) {
      ctl->status[i] = rec[i];
      if (host_status) reinterpret_cast<volatile uint32_t*>(host_status)[i] = rec[i];
    }
    __threadfence_system();
  }
}

// ---- addresses inside a symmetric allocation -----------------------------------------
// symm(p, r, off): address of the 16-byte vector at byte offset `off` of rank r's allocation; every
// store into a peer's memory takes its address from here. Built with -DTDX_BOUNDS (the checked build,
// which stands in for a memory checker that cannot see peer mappings), the range is first compared with
// the allocation's extent: a range that leaves it is recorded once as {kBoundsViolation, rank, r, 0,
// block, off / 1024} and the access goes to a scratch slot in the upper half of this rank's own control
// block instead, so that a wrong offset shows up as a status code and invalid outputs, never as a
// write into memory it does not own. The release build compiles to the pointer arithmetic alone.
constexpr size_t kBoundsScratchOffset = 2048;
static_assert(sizeof(Control) <= kBoundsScratchOffset, "scratch slots overlap the control fields");

__device__ __forceinline__ char* symm(const ArParams& p, int r, size_t off) {
#ifdef TDX_BOUNDS
  constexpr size_t bytes = 16;   // every access through here is one 16-byte vector (or a 4-byte flag)
  const uint64_t extent = p.debug_extent ? p.debug_extent : p.layout.total_bytes;
  if ((uint64_t)off + bytes > extent || r < 0 || r >= p.nranks) {
    char* self = static_cast<char*>(p.peer[p.rank]);
    report_error(reinterpret_cast<Control*>(self + p.layout.off_control), p.host_status, kBoundsViolation, p.rank, r, 0,
                 (int)(off >> 10));
    return self + p.layout.off_control + kBoundsScratchOffset + (size_t)(threadIdx.x & 63) * 16;
  }
#endif
  return static_cast<char*>(p.peer[r]) + off;
}

// Address of the same 16-byte vector in the NVSwitch multicast mapping: one multimem.st to it lands in EVERY
// rank's allocation (this rank's included).
__device__ __forceinline__ char* symm_mc(const ArParams& p, size_t off) {
#ifdef TDX_BOUNDS
  const uint64_t extent = p.debug_extent ? p.debug_extent : p.layout.total_bytes;
  if ((uint64_t)off + 16 > extent) {
    char* self = static_cast<char*>(p.peer[p.rank]);
    report_error(reinterpret_cast<Control*>(self + p.layout.off_control), p.host_status, kBoundsViolation, p.rank, -1, 0,
                 (int)(off >> 10));
    off = p.layout.off_control + kBoundsScratchOffset + (size_t)(threadIdx.x & 63) * 16;
  }
#endif
  return static_cast<char*>(p.mc_base) + off;
}

// ---- phase time stamps (tracing build only) ---------------------------------------------------
// Compiled with -DTDX_TRACE, thread 0 of every block records when it passed each phase of the protocol
// (see TraceSlot); the release build compiles these calls to nothing.
__device__ __forceinline__ void trace_mark(const ArParams& p, int slot) {
#ifdef TDX_TRACE
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[(size_t)blockIdx.x * kTraceSlots + slot] = (uint64_t)clock64();
#endif
}
__device__ __forceinline__ void trace_mark_ns(const ArParams& p, int slot) {
#ifdef TDX_TRACE
  if (p.trace != nullptr && threadIdx.x == 0) {
    p.trace[(size_t)blockIdx.x * kTraceSlots + slot] = ptx::globaltimer_ns();
    if (slot == kTraceStartNs) {
      uint32_t sm;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
      p.trace[(size_t)blockIdx.x * kTraceSlots + kTraceSm] = sm;
    }
  }
#endif
}

// ---- cross-GPU flag barrier ---------------------------------------------------------
// flags[block][src_rank] on every rank. Thread t < nranks of block b publishes `target`
// into rank t's flags[b][my_rank], then waits for its own flags[b][t] to reach `target`.
// Block b only ever synchronises with block b of the peers.

// Two planes of flags: plane 0 carries "scatter done" / general barriers, plane 1 "results done".
__device__ __forceinline__ uint32_t* flag_ptr(void* base, const Layout& l, int plane, int block, int src) {
  return reinterpret_cast<uint32_t*>(static_cast<char*>(base) + l.off_flags) +
         ((size_t)plane * kMaxBarrierBlocks + block) * kMaxRanks + src;
}

// Publish `target` to every peer (release: everything this block wrote before is visible first).
__device__ __forceinline__ void flag_signal(const ArParams& p, int plane, uint32_t target) {
  __syncthreads();
  if ((int)threadIdx.x < p.nranks)
    ptx::st_release_sys(reinterpret_cast<uint32_t*>(symm(
                            p, threadIdx.x,
                            p.layout.off_flags + (((size_t)plane * kMaxBarrierBlocks + blockIdx.x) * kMaxRanks + p.rank) * sizeof(uint32_t))),
                        target);
}

// Wait (bounded) until every peer has published at least `target` for this block index.
__device__ __forceinline__ void flag_wait(const ArParams& p, Control* ctl, int plane, uint32_t target,
                                          Waiter& w, int phase) {
  if ((int)threadIdx.x < p.nranks) {
    const int peer = threadIdx.x;
    const uint32_t* mine = flag_ptr(p.peer[p.rank], p.layout, plane, blockIdx.x, peer);
    w.begin();
    while ((int32_t)(ptx::ld_acquire_sys(mine) - target) < 0) {
      if (!w.keep_waiting()) {
        report_error(ctl, p.host_status, kTimeoutBarrier, p.rank, peer, phase, -1);
        break;
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void flag_barrier(const ArParams& p, Control* ctl, uint32_t target,
                                             Waiter& w, int phase) {
  flag_signal(p, 0, target);
  flag_wait(p, ctl, 0, target, w, phase);
}

// ---- end of launch -------------------------------------------------------------------
// The last block to finish advances the epochs. Launches on one stream are ordered, so the
// next launch reads the new values.
__device__ __forceinline__ void finish_launch(Control* ctl, bool used_lamport, uint32_t epoch,
                                              uint64_t dirty_bytes, uint32_t barriers_used,
                                              uint32_t nctas = 0) {
  if (nctas == 0) nctas = gridDim.x;   // blocks of THIS rank (an emulated launch holds several ranks)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(&ctl->arrive, 1u);
    if (done == nctas - 1) {
      if (used_lamport) {
        ctl->lamport_dirty[epoch % 3u] = dirty_bytes;
        ctl->lamport_epoch = epoch + 1u;
      }
      if (barriers_used) ctl->barrier_epoch += barriers_used;
      ctl->arrive = 0;
      __threadfence();
    }
  }
}

}  // namespace tdx
