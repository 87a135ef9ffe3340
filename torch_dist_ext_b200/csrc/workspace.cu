// Symmetric-workspace manager: allocates one peer-mappable buffer per rank, exports and
// opens cudaIpc handles, keeps the pointer table resident on the device, initialises flags
// and sentinels with a kernel, mirrors the error record into host-mapped memory and closes
// what it opened.
//
// Reference counterpart: class CommWorkspace (src/ops/all_reduce_fusion.cpp:63-174) and
// enable_p2p (src/common/collectives.h:5-19). Differences by design: the table is uploaded
// once at registration (the reference rebuilds and copies it on every get_workspace call,
// :159-173); flags are zeroed and sentinels written by a device kernel at construction and by
// reset() (the reference never zeroes its barrier flags and re-fills sentinels with a blocking
// host copy whenever the dtype changes, :143-158); IPC mappings are closed in the destructor;
// sizes are 64-bit; the CUDA device is explicit instead of being equal to the rank.
#include <unistd.h>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include "tdx/api.h"
#include "tdx/ptx.cuh"
#include "tdx/vec.cuh"

namespace tdx {

namespace {

#define TDX_CUDA_CHECK(expr)                                                                     \
  do {                                                                                           \
    cudaError_t e__ = (expr);                                                                    \
    if (e__ != cudaSuccess)                                                                      \
      throw std::runtime_error(std::string(#expr) + " failed: " + cudaGetErrorString(e__));     \
  } while (0)

struct HandleBlob {
  uint64_t magic;
  int32_t rank;
  int32_t device;
  int64_t pid;
  uint64_t total_bytes;
  uint64_t local_ptr;  // for same-process registration
  cudaIpcMemHandle_t ipc;
  uint8_t pad[kHandleBytes - 8 - 4 - 4 - 8 - 8 - 8 - sizeof(cudaIpcMemHandle_t)];
};
static_assert(sizeof(HandleBlob) == kHandleBytes, "handle blob size");

// Zero the control block and flags, write the sentinel over the three Lamport buffers.
__global__ void init_workspace_kernel(char* base, Layout l) {
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t nthreads = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t zero_vecs = l.off_lamport / 16;
  for (uint64_t i = tid; i < zero_vecs; i += nthreads)
    reinterpret_cast<uint4*>(base)[i] = make_uint4(0, 0, 0, 0);
  const uint64_t lam_vecs = 3 * l.lamport_bytes / 16;
  uint4* lam = reinterpret_cast<uint4*>(base + l.off_lamport);
  const uint4 s = make_uint4(kSentinel, kSentinel, kSentinel, kSentinel);
  for (uint64_t i = tid; i < lam_vecs; i += nthreads) lam[i] = s;
}

std::mutex g_registry_mu;
std::map<const void*, Workspace*>& registry() {
  static std::map<const void*, Workspace*> r;
  return r;
}

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (dev != prev) cudaSetDevice(dev);
  }
  ~DeviceGuard() {
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != prev && prev >= 0) cudaSetDevice(prev);
  }
};

}  // namespace

Workspace::Workspace(int rank, int world_size, int nblocks, uint64_t max_message_bytes,
                     uint64_t lamport_bytes, int device)
    : rank_(rank), world_(world_size), device_(device), nblocks_(nblocks), timeout_ns_(5000000000ull) {
  if (world_size < 1 || world_size > kMaxRanks)
    throw std::invalid_argument("world_size must be between 1 and 8");
  if (rank < 0 || rank >= world_size) throw std::invalid_argument("rank out of range");
  if (device_ < 0) TDX_CUDA_CHECK(cudaGetDevice(&device_));
  DeviceGuard guard(device_);
  if (lamport_bytes == 0) lamport_bytes = 32ull << 20;
  layout_ = make_layout(max_message_bytes, lamport_bytes);
  TDX_CUDA_CHECK(cudaMalloc(&base_, layout_.total_bytes));
  TDX_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&host_status_), 64, cudaHostAllocMapped));
  std::memset(host_status_, 0, 64);
  TDX_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&host_status_dev_), host_status_, 0));
  TDX_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&table_dev_), sizeof(CommTable)));
  init_device_state();
  peer_[rank_] = base_;
  if (world_ == 1) {
    std::vector<Workspace*> self{this};
    connect_local(self);
  }
}

void Workspace::init_device_state() {
  DeviceGuard guard(device_);
  init_workspace_kernel<<<296, 512>>>(static_cast<char*>(base_), layout_);
  TDX_CUDA_CHECK(cudaGetLastError());
  TDX_CUDA_CHECK(cudaDeviceSynchronize());
  std::memset(host_status_, 0, 64);
}

Workspace::~Workspace() {
  {
    std::lock_guard<std::mutex> lock(g_registry_mu);
    registry().erase(table_dev_);
  }
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  for (int r = 0; r < world_; ++r)
    if (opened_[r] && peer_[r]) cudaIpcCloseMemHandle(peer_[r]);
  if (table_dev_) cudaFree(table_dev_);
  if (base_) cudaFree(base_);
  if (host_status_) cudaFreeHost(host_status_);
  if (prev >= 0) cudaSetDevice(prev);
}

void Workspace::export_handle(uint8_t out[kHandleBytes]) const {
  DeviceGuard guard(device_);
  HandleBlob h{};
  h.magic = kTableMagic;
  h.rank = rank_;
  h.device = device_;
  h.pid = (int64_t)getpid();
  h.total_bytes = layout_.total_bytes;
  h.local_ptr = reinterpret_cast<uint64_t>(base_);
  TDX_CUDA_CHECK(cudaIpcGetMemHandle(&h.ipc, base_));
  std::memcpy(out, &h, sizeof(h));
}

void Workspace::open_handles(const std::vector<const uint8_t*>& handles) {
  if ((int)handles.size() != world_)
    throw std::invalid_argument("open_handles expects one handle per rank (" + std::to_string(world_) +
                                "), got " + std::to_string(handles.size()));
  if (registered_) throw std::runtime_error("workspace is already registered");
  DeviceGuard guard(device_);
  for (int r = 0; r < world_; ++r) {
    if (handles[r] == nullptr) throw std::invalid_argument("missing handle for rank " + std::to_string(r));
    HandleBlob h;
    std::memcpy(&h, handles[r], sizeof(h));
    if (h.magic != kTableMagic) throw std::invalid_argument("handle " + std::to_string(r) + " is not a workspace handle");
    if (h.rank != r) throw std::invalid_argument("handle at position " + std::to_string(r) + " belongs to rank " + std::to_string(h.rank));
    if (h.total_bytes != layout_.total_bytes)
      throw std::invalid_argument("rank " + std::to_string(r) + " allocated a workspace of a different size");
    if (r == rank_) {
      peer_[r] = base_;
    } else if (h.pid == (int64_t)getpid()) {
      // Same process (several ranks driven by one host process): the pointer is already valid
      // here; an IPC handle cannot be opened by the process that exported it.
      int can = 0;
      if (h.device != device_) {
        TDX_CUDA_CHECK(cudaDeviceCanAccessPeer(&can, device_, h.device));
        if (!can) throw std::runtime_error("no peer access between devices " + std::to_string(device_) + " and " + std::to_string(h.device));
        cudaError_t e = cudaDeviceEnablePeerAccess(h.device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) TDX_CUDA_CHECK(e);
        cudaGetLastError();
      }
      peer_[r] = reinterpret_cast<void*>(h.local_ptr);
    } else {
      TDX_CUDA_CHECK(cudaIpcOpenMemHandle(&peer_[r], h.ipc, cudaIpcMemLazyEnablePeerAccess));
      opened_[r] = true;
    }
  }
  table_host_ = CommTable{};
  table_host_.magic = kTableMagic;
  table_host_.rank = rank_;
  table_host_.nranks = world_;
  for (int r = 0; r < world_; ++r) table_host_.peer[r] = peer_[r];
  table_host_.mc_base = nullptr;
  table_host_.layout = layout_;
  TDX_CUDA_CHECK(cudaMemcpy(table_dev_, &table_host_, sizeof(CommTable), cudaMemcpyHostToDevice));
  registered_ = true;
  std::lock_guard<std::mutex> lock(g_registry_mu);
  registry()[table_dev_] = this;
}

void Workspace::connect_local(const std::vector<Workspace*>& all) {
  std::vector<std::vector<uint8_t>> blobs(all.size(), std::vector<uint8_t>(kHandleBytes));
  for (size_t r = 0; r < all.size(); ++r) all[r]->export_handle(blobs[r].data());
  std::vector<const uint8_t*> ptrs;
  for (auto& b : blobs) ptrs.push_back(b.data());
  for (auto* w : all) w->open_handles(ptrs);
}

void Workspace::fill_params(ArParams* p) const {
  for (int r = 0; r < kMaxRanks; ++r) p->peer[r] = r < world_ ? peer_[r] : nullptr;
  p->mc_base = table_host_.mc_base;
  p->layout = layout_;
  p->rank = rank_;
  p->nranks = world_;
  p->timeout_ns = timeout_ns_;
  p->host_status = host_status_dev_;
}

void Workspace::reset() { init_device_state(); }

WorkspaceStats Workspace::stats() const {
  DeviceGuard guard(device_);
  WorkspaceStats s{};
  Control c;
  TDX_CUDA_CHECK(cudaDeviceSynchronize());
  TDX_CUDA_CHECK(cudaMemcpy(&c, static_cast<char*>(base_) + layout_.off_control, sizeof(c), cudaMemcpyDeviceToHost));
  s.total_bytes = layout_.total_bytes;
  s.lamport_bytes = layout_.lamport_bytes;
  s.stage_bytes = layout_.stage_bytes;
  s.error_count = c.error_count;
  std::memcpy(s.status, c.status, sizeof(s.status));
  s.lamport_epoch = c.lamport_epoch;
  s.barrier_epoch = c.barrier_epoch;
  s.has_multicast = table_host_.mc_base != nullptr;
  return s;
}

uint32_t Workspace::errors_seen() const {
  return reinterpret_cast<volatile uint32_t*>(host_status_)[0];
}

Workspace* Workspace::from_table(const void* table_dev) {
  std::lock_guard<std::mutex> lock(g_registry_mu);
  auto it = registry().find(table_dev);
  return it == registry().end() ? nullptr : it->second;
}

int enable_all_peer_access() {
  int n = 0;
  TDX_CUDA_CHECK(cudaGetDeviceCount(&n));
  int prev = 0;
  cudaGetDevice(&prev);
  for (int i = 0; i < n; ++i) {
    TDX_CUDA_CHECK(cudaSetDevice(i));
    for (int j = 0; j < n; ++j) {
      if (i == j) continue;
      int can = 0;
      TDX_CUDA_CHECK(cudaDeviceCanAccessPeer(&can, i, j));
      if (!can) throw std::runtime_error("devices " + std::to_string(i) + " and " + std::to_string(j) + " have no peer access");
      cudaError_t e = cudaDeviceEnablePeerAccess(j, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) TDX_CUDA_CHECK(e);
      cudaGetLastError();
    }
  }
  cudaSetDevice(prev);
  return n;
}

}  // namespace tdx
