// Layout of the per-rank symmetric communication buffer, the device-resident pointer
// table, kernel parameter blocks and status codes. Shared by host and device code.
//
// Counterpart of the reference's workspace layout and pointer table
// (src/ops/all_reduce_fusion.cpp:63-96, :135-141, :159-169) and of its kernel argument
// struct (src/common/all_reduce_fusion_impl.h:300-314). Differences by design:
//  * one contiguous allocation per rank with fixed offsets, so a kernel needs only the
//    peers' base pointers (passed by value, no dependent pointer-table load on the hot path);
//  * phase state (epochs, dirty extents) lives in a control block at the start of the
//    allocation and is advanced by the last block of every launch, so CUDA-graph replays
//    need no host-side state;
//  * every size is 64-bit and checked against the capacity before a launch.
#pragma once
#include <cstddef>
#include <cstdint>

namespace tdx {

constexpr int kMaxRanks = 8;            // one NVSwitch domain (HGX B200 board)
constexpr int kMaxBarrierBlocks = 1024; // barrier flag rows per rank
constexpr uint32_t kSentinel = 0x80000000u;  // fp32 -0.0 / (bf16 -0.0, +0.0) pair

// ---- region offsets inside one rank's symmetric allocation --------------------
constexpr size_t kControlBytes = 4096;
constexpr size_t kFlagBytes = 2 * size_t(kMaxBarrierBlocks) * kMaxRanks * sizeof(uint32_t);  // two planes
constexpr size_t kAgFlagBytes = 256;    // all-gather->GEMM: one arrival word per source rank

struct Layout {
  uint64_t off_control;   // Control block (touched by the owning rank only)
  uint64_t off_flags;     // uint32 flags[2 planes][kMaxBarrierBlocks][kMaxRanks], written by peers
  uint64_t off_lamport;   // 3 x lamport_bytes, sentinel-initialised
  uint64_t lamport_bytes; // capacity of ONE of the three Lamport buffers
  uint64_t off_stage;     // flag-synchronised staging of the peer-to-peer two-shot path
  uint64_t stage_bytes;
  uint64_t off_ag_flags;  // uint32 ag_flags[kMaxRanks], written by peers (all-gather->GEMM)
  uint64_t off_ag;        // all-gather->GEMM: two gathered-activation buffers (by epoch parity)
  uint64_t ag_buf_bytes;  // capacity of one of them
  uint64_t off_nvls;      // NVLS: two input staging buffers (by barrier-epoch parity) + result area
  uint64_t nvls_in_bytes; // capacity of one NVLS input buffer (0: no NVLS region)
  uint64_t nvls_bytes;
  uint64_t total_bytes;
};

inline Layout make_layout(uint64_t max_message_bytes, uint64_t lamport_bytes, bool with_nvls = false) {
  auto align_up = [](uint64_t v, uint64_t a) { return (v + a - 1) / a * a; };
  Layout l{};
  l.off_control = 0;
  l.off_flags = kControlBytes;
  l.off_ag_flags = l.off_flags + kFlagBytes;
  l.off_lamport = align_up(l.off_ag_flags + kAgFlagBytes, 1 << 16);
  l.lamport_bytes = align_up(lamport_bytes, 1 << 16);
  l.off_stage = l.off_lamport + 3 * l.lamport_bytes;
  // gather area + result area + per-row trailers and row padding
  l.stage_bytes = align_up(2 * max_message_bytes + max_message_bytes / 8 + (1 << 20), 1 << 16);
  l.off_ag = l.off_stage + l.stage_bytes;
  l.ag_buf_bytes = align_up(max_message_bytes < (32ull << 20) ? max_message_bytes : (32ull << 20), 1 << 16);
  l.off_nvls = l.off_ag + 2 * l.ag_buf_bytes;
  l.nvls_in_bytes = with_nvls ? align_up(max_message_bytes, 1 << 16) : 0;
  l.nvls_bytes = with_nvls ? 2 * l.nvls_in_bytes + align_up(max_message_bytes + max_message_bytes / 8 + (1 << 20), 1 << 16) : 0;
  l.total_bytes = align_up(l.off_nvls + l.nvls_bytes, 1 << 21);
  return l;
}

// Per-rank phase state. Only the owning rank reads or writes it.
struct Control {
  uint32_t lamport_epoch;      // Lamport calls completed; buffer in use = epoch % 3
  uint32_t barrier_epoch;      // flag barriers completed
  uint32_t arrive;             // blocks of the running launch that have finished
  uint32_t error_count;        // waits that ran out since the last reset
  uint32_t ag_epoch;           // all-gather->GEMM calls completed; buffer in use = epoch & 1
  uint32_t reserved0;
  uint64_t lamport_dirty[3];   // bytes (from buffer start) that hold non-sentinel data
  uint32_t status[8];          // first error: {code, rank, peer, phase, block, row, 0, 0}
};
static_assert(sizeof(Control) <= kControlBytes, "control block overflow");

// What the uint8 tensor returned by get_workspace() holds, in device memory.
struct CommTable {
  uint64_t magic;
  int32_t rank;
  int32_t nranks;
  void* peer[kMaxRanks];  // base of every rank's symmetric allocation (own entry = local)
  void* mc_base;          // NVSwitch multicast mapping of the same allocation, or null
  Layout layout;
  uint64_t reserved[5];
};
constexpr uint64_t kTableMagic = 0x7464785f62323030ull;  // "tdx_b200"

// ---- status codes ------------------------------------------------------------
enum Status : uint32_t {
  kOk = 0,
  kTimeoutLamportGather = 1,   // one-shot / two-shot: partial sums from a peer never arrived
  kTimeoutLamportResult = 2,   // two-shot: reduced row from its owner never arrived
  kTimeoutBarrier = 3,         // flag barrier: a peer never arrived
  kTimeoutNvls = 4,
  kTimeoutGemmPipeline = 5,    // an mbarrier of a GEMM pipeline never completed
  kTimeoutTileFlag = 6,        // all-gather->GEMM: a peer tile never became ready
  kBoundsViolation = 7,        // checked build: an address left the symmetric allocation (access redirected)
};

// ---- op description ------------------------------------------------------------
enum DType : int32_t { kF32 = 0, kF16 = 1, kBF16 = 2 };
enum OutMode : int32_t {
  kOutSame = 0,        // norm_out has the input dtype (what the reference produces)
  kOutFp8Token = 1,    // norm_out e4m3, one fp32 scale per token   [tokens, 1]
  kOutFp8Block128 = 2, // norm_out e4m3, one fp32 scale per 128 cols [tokens, hidden/128]
};
enum Algo : int32_t {
  kAlgoAuto = 0,
  kAlgoLocal = 1,            // nranks == 1: residual + RMSNorm (+quant) only
  kAlgoOneShotLamport = 2,   // push everything to everyone, sentinel polling, no barrier
  kAlgoTwoShotLamport = 3,   // push-scatter -> owner reduce -> push-gather, sentinel polling
  kAlgoTwoShotBarrier = 4,   // same data flow, flag barriers, any size up to the capacity
  kAlgoNvlsOneShot = 5,      // multimem.ld_reduce of every row by every rank
  kAlgoNvlsTwoShot = 6,      // multimem.ld_reduce own rows -> epilogue -> multimem.st
  kAlgoOneShotMc = 7,        // one-shot Lamport whose push is ONE multimem.st per vector (the switch replicates it)
  kAlgoTwoShotMc = 8,        // two-shot Lamport whose result hop is one multimem.st per vector and trailer
};

struct ArParams {
  void* peer[kMaxRanks];
  void* mc_base;
  Layout layout;
  int32_t rank;
  int32_t nranks;
  int32_t tokens;
  int32_t hidden;
  const void* in;           // [tokens, hidden] this rank's partial sums
  const void* residual_in;  // [tokens, hidden] or null (treated as zeros)
  const void* gamma;        // [hidden]
  void* residual_out;       // [tokens, hidden] or null (not written)
  void* norm_out;           // [tokens, hidden] input dtype or e4m3
  float* scale_out;         // fp8 modes only
  float eps;
  int32_t dtype;
  int32_t out_mode;
  int32_t algo;
  // Reduce-scatter variant: only the rows this rank owns (row % nranks == rank) are
  // produced; outputs are then [ceil(tokens/nranks), hidden] and nothing is gathered.
  int32_t scatter_only;
  int32_t waves;            // flag-synchronised two-shot paths: pipeline depth (1..4), 0 = 1
  int32_t nvls_batch;       // NVLS two-shot: rows whose switch-side sums are requested together (1..4), 0 = 1
  uint64_t timeout_ns;      // budget of every device-side wait
  uint32_t* host_status;    // pinned, host-mapped mirror of Control::status (or null)
  uint64_t debug_extent;    // checked build (-DTDX_BOUNDS): extent to check against; 0 = layout.total_bytes
  uint64_t* trace;          // tracing build (-DTDX_TRACE): kTraceSlots time stamps per block, or null
};

// Tracing build: what block b writes to trace[b * kTraceSlots + slot] (thread 0's view).
constexpr int kTraceSlots = 16;
enum TraceSlot : int32_t {
  kTraceStartNs = 0,      // %globaltimer when the block starts working (after the dependency wait)
  kTraceStartClk = 1,     // clock64 at the same point; the slots below are clock64 values
  kTracePushed = 2,       // own rows pushed (one-shot: to every peer; two-shot: to their owners)
  kTraceCleared = 3,      // previous Lamport buffer re-filled with sentinels
  kTraceGathered = 4,     // owner / one-shot: every peer's vector of the (last) row has arrived
  kTraceOwnerDone = 5,    // two-shot owner: reduced row and trailer pushed
  kTraceTrailer = 6,      // two-shot receiver: trailer of the (last) received row has arrived
  kTraceReceived = 7,     // two-shot receiver: data of that row has arrived
  kTraceEndClk = 8,       // before the end-of-launch bookkeeping
  kTraceEndNs = 9,        // %globaltimer at the same point
  kTraceSm = 10,          // SM the block ran on
};

}  // namespace tdx
