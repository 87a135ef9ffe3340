// Host-side C++ interface of the native runtime: launch planning for the fused all-reduce
// kernels and the symmetric-workspace manager. Nothing here depends on PyTorch; the torch
// bindings (register.cpp) and the standalone C++ test harness both sit on top of it.
//
// Reference counterparts: allreduce_fusion_kernel_launcher / allreduce_rms_fusion_impl
// (src/common/all_reduce_fusion_impl.h:476-535) and class CommWorkspace
// (src/ops/all_reduce_fusion.h:10-40, src/ops/all_reduce_fusion.cpp:63-174).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <string>
#include <vector>
#include "tdx/comm.h"

namespace tdx {

struct LaunchPlan {
  int algo;      // Algo actually used
  int n_tmpl;    // rank-count template argument (0 = runtime loop)
  int vpt;       // 16-byte vectors per thread
  int threads;
  int grid;      // blocks per rank
  int emu_ranks; // 0 for a real launch
};

// Crossover sizes (bytes of one rank's message) used by kAlgoAuto, per rank count.
struct Policy {
  uint64_t oneshot_max_bytes[kMaxRanks + 1];
  uint64_t lamport_max_bytes[kMaxRanks + 1];   // above: flag-barrier two-shot
  int prefer_nvls;                             // use NVLS paths when a multicast mapping exists
  uint64_t nvls_min_bytes[kMaxRanks + 1];      // per rank count; NVLS two-shot at or above this size
  // With a multicast mapping: push through multimem.st (the switch replicates) instead of one store per peer.
  uint8_t mc_oneshot[kMaxRanks + 1];
  uint8_t mc_twoshot[kMaxRanks + 1];
};
Policy& policy();

// True in the library flavour compiled with -DTDX_BOUNDS (range-checked stores into symmetric memory).
bool bounds_checked_build();
// True in the flavour compiled with -DTDX_TRACE (the kernels record phase time stamps, see TraceSlot).
bool tracing_build();
// Programmatic dependent launch of the fused all-reduce kernels (on unless TDX_PDL=0).
bool pdl_enabled();

// Validates shapes, alignment and capacity, resolves kAlgoAuto and sizes the launch.
// Returns an empty string on success, else the reason.
std::string plan_allreduce(const ArParams& p, int emu_ranks, LaunchPlan* plan);

// Launches one rank's kernel on `stream` (real multi-GPU / multi-process use).
std::string launch_allreduce(const ArParams& p, cudaStream_t stream, LaunchPlan* used = nullptr);

// Launches ALL ranks as one cooperative kernel on the current device. `host_ranks` holds the
// per-rank parameters, `dev_ranks` is a device copy of the same array.
std::string launch_allreduce_emulated(const ArParams* host_ranks, const ArParams* dev_ranks,
                                      int nranks, cudaStream_t stream, LaunchPlan* used = nullptr);

// Per-dtype back ends (one translation unit per dtype, so that they compile in parallel).
cudaError_t launch_ar_f32(const LaunchPlan&, int out_mode, const ArParams&, const ArParams* dev_ranks, cudaStream_t);
cudaError_t launch_ar_f16(const LaunchPlan&, int out_mode, const ArParams&, const ArParams* dev_ranks, cudaStream_t);
cudaError_t launch_ar_bf16(const LaunchPlan&, int out_mode, const ArParams&, const ArParams* dev_ranks, cudaStream_t);
cudaError_t launch_ar_f32_emu(const LaunchPlan&, int out_mode, const ArParams&, const ArParams* dev_ranks, cudaStream_t);
cudaError_t launch_ar_f16_emu(const LaunchPlan&, int out_mode, const ArParams&, const ArParams* dev_ranks, cudaStream_t);
cudaError_t launch_ar_bf16_emu(const LaunchPlan&, int out_mode, const ArParams&, const ArParams* dev_ranks, cudaStream_t);
// blocks of `plan.threads` threads that one SM holds for the kernel the plan selects
int occupancy_ar_f32(const LaunchPlan&, int out_mode);
int occupancy_ar_f16(const LaunchPlan&, int out_mode);
int occupancy_ar_bf16(const LaunchPlan&, int out_mode);
int occupancy_ar_f32_emu(const LaunchPlan&, int out_mode);
int occupancy_ar_f16_emu(const LaunchPlan&, int out_mode);
int occupancy_ar_bf16_emu(const LaunchPlan&, int out_mode);

// ---- symmetric workspace -----------------------------------------------------------------

constexpr int kHandleBytes = 128;  // opaque blob exchanged between ranks

struct WorkspaceStats {
  uint64_t total_bytes;
  uint64_t lamport_bytes;
  uint64_t stage_bytes;
  uint32_t error_count;
  uint32_t status[8];
  uint32_t lamport_epoch;
  uint32_t barrier_epoch;
  int has_multicast;
};

class Workspace {
 public:
  // `device` < 0 keeps the current device. `max_message_bytes` bounds one rank's message on
  // the flag-barrier path; `lamport_bytes` is the capacity of each of the three Lamport buffers
  // (0 = default). `multicast`: 1 = allocate through the virtual-memory API, share by POSIX file
  // descriptor and bind to an NVSwitch multicast object (needed by the NVLS kernels; falls back
  // to plain cudaIpc sharing when the device or the container does not allow it), 0 = cudaMalloc
  // + cudaIpc, -1 = decide from the TDX_NVLS environment variable (default on) and world size.
  Workspace(int rank, int world_size, int nblocks, uint64_t max_message_bytes,
            uint64_t lamport_bytes = 0, int device = -1, int multicast = -1);
  ~Workspace();
  Workspace(const Workspace&) = delete;
  Workspace& operator=(const Workspace&) = delete;

  // Cross-process registration: export this rank's handle, then open everyone's.
  void export_handle(uint8_t out[kHandleBytes]) const;
  void open_handles(const std::vector<const uint8_t*>& handles);
  // Single-process registration (one process drives several GPUs, or emulated ranks on one
  // GPU): peers are given directly. Enables peer access where the devices differ.
  static void connect_local(const std::vector<Workspace*>& all);

  // Device-resident table; valid after registration. Never re-uploaded.
  const CommTable* device_table() const { return table_dev_; }
  const CommTable& host_table() const { return table_host_; }
  // Fills the communication part of a parameter block.
  void fill_params(ArParams* p) const;
  uint32_t* host_status_device_ptr() const { return host_status_dev_; }
  const Layout& layout() const { return layout_; }
  void* peer_base(int r) const { return peer_[r]; }

  // Re-initialise flags, epochs, sentinels and the status record. Collective: all ranks must
  // be idle and must call it between two host barriers.
  void reset();
  WorkspaceStats stats() const;       // synchronises the device
  uint32_t errors_seen() const;       // non-blocking: reads the host-mapped status mirror
  // Drop the multicast mapping from the table (all ranks must agree; used when some rank could
  // not join the multicast object). The NVLS algorithms are then refused by the planner.
  void disable_multicast();
  bool has_multicast() const { return table_host_.mc_base != nullptr; }
  const std::string& multicast_note() const { return mc_note_; }
  void set_timeout_ns(uint64_t t) { timeout_ns_ = t; }
  // Checked build only: pretend the allocation ends after `bytes` (0 = its real size), so that a test can
  // watch a store that leaves the extent being recorded and redirected.
  void set_debug_extent(uint64_t bytes) { debug_extent_ = bytes; }
  // Tracing build only: device buffer of kTraceSlots 64-bit words per block that the kernels fill with phase
  // time stamps (null = off). The release build ignores it.
  void set_trace(uint64_t* dev_buffer) { trace_ = dev_buffer; }
  uint64_t timeout_ns() const { return timeout_ns_; }
  int rank() const { return rank_; }
  int world_size() const { return world_; }
  int device() const { return device_; }
  bool registered() const { return registered_; }

  // Looks up the workspace that owns a device table pointer (what the op receives).
  static Workspace* from_table(const void* table_dev);
  // Makes from_table() also recognise a device copy of the table (what a traced op returns, since an
  // op's output must not alias memory that the library owns). Forgotten when the workspace is destroyed.
  void adopt_table_copy(const void* copy_dev);

 private:
  void init_device_state();
  int rank_, world_, device_, nblocks_;
  Layout layout_;
  void* base_ = nullptr;
  void* peer_[kMaxRanks] = {};
  bool opened_[kMaxRanks] = {};
  CommTable table_host_{};
  CommTable* table_dev_ = nullptr;
  uint32_t* host_status_ = nullptr;   // pinned + mapped
  uint32_t* host_status_dev_ = nullptr;
  uint64_t timeout_ns_;
  uint64_t debug_extent_ = 0;
  uint64_t* trace_ = nullptr;
  bool registered_ = false;
  struct Vmm;                // virtual-memory / multicast state (workspace.cu)
  Vmm* vmm_ = nullptr;
  std::string mc_note_;      // why multicast is off, when it is
  void release_vmm();
  void upload_table();
};

// Run-time override of the pipeline depth of the flag-synchronised two-shot paths (TDX_WAVES) and of the number of
// rows whose switch-side sums the NVLS two-shot requests together (TDX_NVLS_BATCH); negative = keep the environment's.
void set_tuning(int waves, int nvls_batch);

// Every (device, peer) pair of this process: check and enable peer access. Returns the number
// of visible devices. Used by single-process multi-GPU harnesses.
int enable_all_peer_access();

}  // namespace tdx
