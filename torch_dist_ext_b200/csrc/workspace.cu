// Symmetric-workspace manager: allocates one peer-mappable buffer per rank, shares it with the
// peers, keeps the pointer table resident on the device, initialises flags and sentinels with a
// kernel, mirrors the error record into host-mapped memory and releases what it mapped.
//
// Reference counterpart: class CommWorkspace (src/ops/all_reduce_fusion.cpp:63-174) and
// enable_p2p (src/common/collectives.h:5-19). Differences by design: the table is uploaded
// once at registration (the reference rebuilds and copies it on every get_workspace call,
// :159-173); flags are zeroed and sentinels written by a device kernel at construction and by
// reset() (the reference never zeroes its barrier flags and re-fills sentinels with a blocking
// host copy whenever the dtype changes, :143-158); mappings are released in the destructor;
// sizes are 64-bit; the CUDA device is explicit instead of being equal to the rank.
//
// Two sharing tiers:
//  A  cudaMalloc + cudaIpcGetMemHandle / cudaIpcOpenMemHandle (what the reference does).
//  B  cuMemCreate with a POSIX-fd shareable handle; fds travel between processes over an abstract
//     Unix-domain socket (SCM_RIGHTS) served by a small thread of the exporting rank; every rank
//     binds its allocation to ONE multicast object created by rank 0, which gives the NVLS kernels
//     an address whose loads reduce, and whose stores replicate, inside the NVSwitch.
// Tier B falls back to tier A when any step is refused (no multicast support, no fd export).
#include <cuda.h>
#include <unistd.h>
#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include <thread>
#include "tdx/api.h"
#include "tdx/fd_channel.h"
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
  union {
    cudaIpcMemHandle_t ipc;   // tier A
    char socket_name[64];     // tier B: abstract Unix socket that serves this rank's fds
  };
  int32_t tier;               // 0 = cudaIpc, 1 = VMM allocation shared by POSIX fd
  int32_t has_multicast;      // rank 0 only: a multicast object exists and its fd is served
  uint8_t pad[kHandleBytes - 8 - 4 - 4 - 8 - 8 - 8 - 64 - 4 - 4];
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

// ---- driver entry points (resolved at run time: the library does not link libcuda) -----------
struct Driver {
  decltype(&cuMemCreate) MemCreate = nullptr;
  decltype(&cuMemRelease) MemRelease = nullptr;
  decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
  decltype(&cuMemAddressFree) MemAddressFree = nullptr;
  decltype(&cuMemMap) MemMap = nullptr;
  decltype(&cuMemUnmap) MemUnmap = nullptr;
  decltype(&cuMemSetAccess) MemSetAccess = nullptr;
  decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity = nullptr;
  decltype(&cuMemExportToShareableHandle) MemExportToShareableHandle = nullptr;
  decltype(&cuMemImportFromShareableHandle) MemImportFromShareableHandle = nullptr;
  decltype(&cuMulticastCreate) MulticastCreate = nullptr;
  decltype(&cuMulticastAddDevice) MulticastAddDevice = nullptr;
  decltype(&cuMulticastBindMem) MulticastBindMem = nullptr;
  decltype(&cuMulticastUnbind) MulticastUnbind = nullptr;
  decltype(&cuMulticastGetGranularity) MulticastGetGranularity = nullptr;
  decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
  decltype(&cuDeviceGet) DeviceGet = nullptr;
  bool ok = false;

  template <typename F>
  bool get(const char* name, F& fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return false;
    }
    fn = reinterpret_cast<F>(p);
    return true;
  }
  Driver() {
    ok = get("cuMemCreate", MemCreate) && get("cuMemRelease", MemRelease) &&
         get("cuMemAddressReserve", MemAddressReserve) && get("cuMemAddressFree", MemAddressFree) &&
         get("cuMemMap", MemMap) && get("cuMemUnmap", MemUnmap) && get("cuMemSetAccess", MemSetAccess) &&
         get("cuMemGetAllocationGranularity", MemGetAllocationGranularity) &&
         get("cuMemExportToShareableHandle", MemExportToShareableHandle) &&
         get("cuMemImportFromShareableHandle", MemImportFromShareableHandle) &&
         get("cuMulticastCreate", MulticastCreate) && get("cuMulticastAddDevice", MulticastAddDevice) &&
         get("cuMulticastBindMem", MulticastBindMem) && get("cuMulticastUnbind", MulticastUnbind) &&
         get("cuMulticastGetGranularity", MulticastGetGranularity) &&
         get("cuDeviceGetAttribute", DeviceGetAttribute) && get("cuDeviceGet", DeviceGet);
  }
};
Driver& driver() {
  static Driver d;
  return d;
}

}  // namespace

struct Workspace::Vmm {
  size_t size = 0;                 // mapped bytes (total_bytes rounded up to the granularity)
  CUmemGenericAllocationHandle mem = 0;
  int mem_fd = -1;
  CUmemGenericAllocationHandle mc = 0;
  bool mc_created = false, mc_bound = false;
  int mc_fd = -1;
  CUdeviceptr mc_va = 0;
  CUmemGenericAllocationHandle peer_mem[kMaxRanks] = {};
  CUdeviceptr peer_va[kMaxRanks] = {};
  FdServer server;                 // hands mem_fd ('m') and mc_fd ('c') to the peers
};

Workspace::Workspace(int rank, int world_size, int nblocks, uint64_t max_message_bytes,
                     uint64_t lamport_bytes, int device, int multicast)
    : rank_(rank), world_(world_size), device_(device), nblocks_(nblocks), timeout_ns_(5000000000ull) {
  if (world_size < 1 || world_size > kMaxRanks)
    throw std::invalid_argument("world_size must be between 1 and 8");
  if (rank < 0 || rank >= world_size) throw std::invalid_argument("rank out of range");
  if (device_ < 0) TDX_CUDA_CHECK(cudaGetDevice(&device_));
  DeviceGuard guard(device_);
  if (lamport_bytes == 0) lamport_bytes = 32ull << 20;
  if (multicast < 0) {
    const char* env = std::getenv("TDX_NVLS");
    multicast = (env == nullptr || (std::strcmp(env, "0") != 0 && std::strcmp(env, "off") != 0 &&
                                    std::strcmp(env, "false") != 0)) ? 1 : 0;
  }
  if (world_size == 1) multicast = 0;
  // The layout (and with it every offset the peers use) depends only on the request, never on
  // whether this rank's multicast set-up succeeds, so that all ranks agree.
  layout_ = make_layout(max_message_bytes, lamport_bytes, multicast != 0);

  if (multicast) {
    Driver& d = driver();
    int mc_ok = 0, fd_ok = 0;
    CUdevice cudev = 0;
    if (!d.ok) {
      mc_note_ = "driver entry points for virtual memory / multicast are not available";
    } else if (d.DeviceGet(&cudev, device_) != CUDA_SUCCESS ||
               d.DeviceGetAttribute(&mc_ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cudev) != CUDA_SUCCESS ||
               d.DeviceGetAttribute(&fd_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cudev) != CUDA_SUCCESS ||
               !mc_ok || !fd_ok) {
      mc_note_ = "device does not support multicast objects or POSIX-fd memory handles";
    } else {
      vmm_ = new Vmm();
      CUmemAllocationProp prop{};
      prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
      prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      prop.location.id = device_;
      prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      size_t gran = 0, mc_gran = 0;
      CUmulticastObjectProp mprop{};
      mprop.numDevices = (unsigned)world_;
      mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      mprop.size = layout_.total_bytes;
      CUresult r = d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
      if (r == CUDA_SUCCESS) r = d.MulticastGetGranularity(&mc_gran, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED);
      if (r == CUDA_SUCCESS) {
        if (mc_gran > gran) gran = mc_gran;
        vmm_->size = (layout_.total_bytes + gran - 1) / gran * gran;
        r = d.MemCreate(&vmm_->mem, vmm_->size, &prop, 0);
      }
      CUdeviceptr va = 0;
      if (r == CUDA_SUCCESS) r = d.MemAddressReserve(&va, vmm_->size, gran, 0, 0);
      if (r == CUDA_SUCCESS) r = d.MemMap(va, vmm_->size, 0, vmm_->mem, 0);
      CUmemAccessDesc acc{};
      acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      acc.location.id = device_;
      acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      if (r == CUDA_SUCCESS) r = d.MemSetAccess(va, vmm_->size, &acc, 1);
      if (r == CUDA_SUCCESS)
        r = d.MemExportToShareableHandle(&vmm_->mem_fd, vmm_->mem, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      if (r != CUDA_SUCCESS) {
        mc_note_ = "virtual-memory allocation or fd export failed (CUresult " + std::to_string((int)r) + ")";
        if (va) {
          d.MemUnmap(va, vmm_->size);
          d.MemAddressFree(va, vmm_->size);
        }
        if (vmm_->mem) d.MemRelease(vmm_->mem);
        delete vmm_;
        vmm_ = nullptr;
      } else {
        base_ = reinterpret_cast<void*>(va);
        if (rank_ == 0) {
          mprop.size = vmm_->size;
          CUresult m = d.MulticastCreate(&vmm_->mc, &mprop);
          if (m == CUDA_SUCCESS) {
            vmm_->mc_created = true;
            m = d.MemExportToShareableHandle(&vmm_->mc_fd, vmm_->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
          }
          if (m != CUDA_SUCCESS) {
            mc_note_ = "multicast object could not be created or exported (CUresult " + std::to_string((int)m) + ")";
            vmm_->mc_fd = -1;
          }
        }
        // listener that hands this rank's fds to the peers
        vmm_->server.offer('m', vmm_->mem_fd);
        vmm_->server.offer('c', vmm_->mc_fd);
        if (!vmm_->server.start(std::to_string(rank_).c_str()))
          throw std::runtime_error("could not open the Unix-domain socket that shares the workspace with the peers");
      }
    }
  }
  if (vmm_ == nullptr) TDX_CUDA_CHECK(cudaMalloc(&base_, layout_.total_bytes));
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

void Workspace::release_vmm() {
  if (vmm_ == nullptr) return;
  Driver& d = driver();
  vmm_->server.stop();
  if (vmm_->mc_va) {
    d.MemUnmap(vmm_->mc_va, vmm_->size);
    d.MemAddressFree(vmm_->mc_va, vmm_->size);
  }
  if (vmm_->mc_bound) {
    CUdevice cudev = 0;
    d.DeviceGet(&cudev, device_);
    d.MulticastUnbind(vmm_->mc, cudev, 0, vmm_->size);
  }
  if (vmm_->mc) d.MemRelease(vmm_->mc);
  for (int r = 0; r < world_; ++r) {
    if (vmm_->peer_va[r]) {
      d.MemUnmap(vmm_->peer_va[r], vmm_->size);
      d.MemAddressFree(vmm_->peer_va[r], vmm_->size);
    }
    if (vmm_->peer_mem[r]) d.MemRelease(vmm_->peer_mem[r]);
  }
  if (base_) {
    d.MemUnmap(reinterpret_cast<CUdeviceptr>(base_), vmm_->size);
    d.MemAddressFree(reinterpret_cast<CUdeviceptr>(base_), vmm_->size);
    base_ = nullptr;
  }
  if (vmm_->mem) d.MemRelease(vmm_->mem);
  if (vmm_->mem_fd >= 0) close(vmm_->mem_fd);
  if (vmm_->mc_fd >= 0) close(vmm_->mc_fd);
  delete vmm_;
  vmm_ = nullptr;
}

Workspace::~Workspace() {
  {
    std::lock_guard<std::mutex> lock(g_registry_mu);
    for (auto it = registry().begin(); it != registry().end();)
      it = (it->second == this) ? registry().erase(it) : std::next(it);
  }
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  for (int r = 0; r < world_; ++r)
    if (opened_[r] && peer_[r]) cudaIpcCloseMemHandle(peer_[r]);
  if (table_dev_) cudaFree(table_dev_);
  if (vmm_) release_vmm();
  else if (base_) cudaFree(base_);
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
  if (vmm_) {
    h.tier = 1;
    std::snprintf(h.socket_name, sizeof(h.socket_name), "%s", vmm_->server.name());
    h.has_multicast = vmm_->mc_fd >= 0 ? 1 : 0;
  } else {
    h.tier = 0;
    TDX_CUDA_CHECK(cudaIpcGetMemHandle(&h.ipc, base_));
  }
  std::memcpy(out, &h, sizeof(h));
}

void Workspace::open_handles(const std::vector<const uint8_t*>& handles) {
  if ((int)handles.size() != world_)
    throw std::invalid_argument("open_handles expects one handle per rank (" + std::to_string(world_) +
                                "), got " + std::to_string(handles.size()));
  if (registered_) throw std::runtime_error("workspace is already registered");
  DeviceGuard guard(device_);
  Driver& d = driver();
  std::vector<HandleBlob> blobs(world_);
  for (int r = 0; r < world_; ++r) {
    if (handles[r] == nullptr) throw std::invalid_argument("missing handle for rank " + std::to_string(r));
    HandleBlob& h = blobs[r];
    std::memcpy(&h, handles[r], sizeof(h));
    if (h.magic != kTableMagic) throw std::invalid_argument("handle " + std::to_string(r) + " is not a workspace handle");
    if (h.rank != r) throw std::invalid_argument("handle at position " + std::to_string(r) + " belongs to rank " + std::to_string(h.rank));
    if (h.total_bytes != layout_.total_bytes)
      throw std::invalid_argument("rank " + std::to_string(r) + " allocated a workspace of a different size "
                                  "(all ranks must pass the same sizes and the same TDX_NVLS setting)");
    if (h.tier != (vmm_ ? 1 : 0))
      throw std::invalid_argument("rank " + std::to_string(r) + " shares its workspace differently (cudaIpc versus "
                                  "file descriptor); set TDX_NVLS=0 on all ranks");
  }
  for (int r = 0; r < world_; ++r) {
    const HandleBlob& h = blobs[r];
    if (r == rank_) {
      peer_[r] = base_;
    } else if (h.pid == (int64_t)getpid() && (!vmm_ || h.device == device_)) {
      // Same process (several ranks driven by one host process): the pointer is already valid
      // here; an IPC handle cannot be opened by the process that exported it.
      if (h.device != device_) {
        int can = 0;
        TDX_CUDA_CHECK(cudaDeviceCanAccessPeer(&can, device_, h.device));
        if (!can) throw std::runtime_error("no peer access between devices " + std::to_string(device_) + " and " + std::to_string(h.device));
        cudaError_t e = cudaDeviceEnablePeerAccess(h.device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) TDX_CUDA_CHECK(e);
        cudaGetLastError();
      }
      peer_[r] = reinterpret_cast<void*>(h.local_ptr);
    } else if (vmm_) {
      const int fd = request_fd(h.socket_name, 'm');
      if (fd < 0) throw std::runtime_error("could not obtain the memory handle of rank " + std::to_string(r));
      CUresult rc = d.MemImportFromShareableHandle(&vmm_->peer_mem[r], reinterpret_cast<void*>((uintptr_t)fd),
                                                   CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      close(fd);
      CUdeviceptr va = 0;
      if (rc == CUDA_SUCCESS) rc = d.MemAddressReserve(&va, vmm_->size, 0, 0, 0);
      if (rc == CUDA_SUCCESS) rc = d.MemMap(va, vmm_->size, 0, vmm_->peer_mem[r], 0);
      CUmemAccessDesc acc{};
      acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      acc.location.id = device_;
      acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      if (rc == CUDA_SUCCESS) rc = d.MemSetAccess(va, vmm_->size, &acc, 1);
      if (rc != CUDA_SUCCESS)
        throw std::runtime_error("mapping the workspace of rank " + std::to_string(r) + " failed (CUresult " + std::to_string((int)rc) + ")");
      vmm_->peer_va[r] = va;
      peer_[r] = reinterpret_cast<void*>(va);
    } else {
      TDX_CUDA_CHECK(cudaIpcOpenMemHandle(&peer_[r], h.ipc, cudaIpcMemLazyEnablePeerAccess));
      opened_[r] = true;
    }
  }
  // multicast: import rank 0's object, join it, bind this rank's memory, map it
  void* mc_base = nullptr;
  if (vmm_ && world_ > 1) {
    if (!blobs[0].has_multicast) {
      if (mc_note_.empty()) mc_note_ = "rank 0 could not create the multicast object";
    } else {
      CUresult rc = CUDA_SUCCESS;
      if (rank_ != 0) {
        const int fd = request_fd(blobs[0].socket_name, 'c');
        if (fd < 0) rc = CUDA_ERROR_UNKNOWN;
        else {
          rc = d.MemImportFromShareableHandle(&vmm_->mc, reinterpret_cast<void*>((uintptr_t)fd),
                                              CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
          close(fd);
        }
      }
      CUdevice cudev = 0;
      if (rc == CUDA_SUCCESS) rc = d.DeviceGet(&cudev, device_);
      if (rc == CUDA_SUCCESS) rc = d.MulticastAddDevice(vmm_->mc, cudev);
      // blocks until every rank has added its device
      if (rc == CUDA_SUCCESS) rc = d.MulticastBindMem(vmm_->mc, 0, vmm_->mem, 0, vmm_->size, 0);
      if (rc == CUDA_SUCCESS) vmm_->mc_bound = true;
      CUdeviceptr va = 0;
      if (rc == CUDA_SUCCESS) rc = d.MemAddressReserve(&va, vmm_->size, 0, 0, 0);
      if (rc == CUDA_SUCCESS) rc = d.MemMap(va, vmm_->size, 0, vmm_->mc, 0);
      CUmemAccessDesc acc{};
      acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      acc.location.id = device_;
      acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      if (rc == CUDA_SUCCESS) rc = d.MemSetAccess(va, vmm_->size, &acc, 1);
      if (rc == CUDA_SUCCESS) {
        vmm_->mc_va = va;
        mc_base = reinterpret_cast<void*>(va);
      } else {
        mc_note_ = "joining the multicast object failed (CUresult " + std::to_string((int)rc) + ")";
      }
    }
  }
  table_host_ = CommTable{};
  table_host_.magic = kTableMagic;
  table_host_.rank = rank_;
  table_host_.nranks = world_;
  for (int r = 0; r < world_; ++r) table_host_.peer[r] = peer_[r];
  table_host_.mc_base = mc_base;
  table_host_.layout = layout_;
  upload_table();
  registered_ = true;
  std::lock_guard<std::mutex> lock(g_registry_mu);
  registry()[table_dev_] = this;
}

void Workspace::upload_table() {
  DeviceGuard guard(device_);
  TDX_CUDA_CHECK(cudaMemcpy(table_dev_, &table_host_, sizeof(CommTable), cudaMemcpyHostToDevice));
}

void Workspace::disable_multicast() {
  if (table_host_.mc_base == nullptr) return;
  table_host_.mc_base = nullptr;
  if (mc_note_.empty()) mc_note_ = "disabled because not every rank could join the multicast object";
  upload_table();
}

void Workspace::connect_local(const std::vector<Workspace*>& all) {
  std::vector<std::vector<uint8_t>> blobs(all.size(), std::vector<uint8_t>(kHandleBytes));
  for (size_t r = 0; r < all.size(); ++r) all[r]->export_handle(blobs[r].data());
  std::vector<const uint8_t*> ptrs;
  for (auto& b : blobs) ptrs.push_back(b.data());
  for (auto* w : all) w->open_handles(ptrs);
}

namespace {
std::atomic<int> g_waves_override{-1}, g_nvls_batch_override{-1};
}
void set_tuning(int waves, int nvls_batch) {
  g_waves_override.store(waves);
  g_nvls_batch_override.store(nvls_batch);
}

void Workspace::fill_params(ArParams* p) const {
  for (int r = 0; r < kMaxRanks; ++r) p->peer[r] = r < world_ ? peer_[r] : nullptr;
  p->mc_base = table_host_.mc_base;
  p->layout = layout_;
  p->rank = rank_;
  p->nranks = world_;
  p->timeout_ns = timeout_ns_;
  p->host_status = host_status_dev_;
  p->debug_extent = debug_extent_;
  p->trace = trace_;
  static const int waves_env = [] {
    const char* e = std::getenv("TDX_WAVES");
    return e ? std::atoi(e) : 1;
  }();
  p->waves = g_waves_override.load() >= 0 ? g_waves_override.load() : waves_env;
  static const int batch_env = [] {
    const char* e = std::getenv("TDX_NVLS_BATCH");
    return e ? std::atoi(e) : 1;
  }();
  p->nvls_batch = g_nvls_batch_override.load() >= 0 ? g_nvls_batch_override.load() : batch_env;
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

void Workspace::adopt_table_copy(const void* copy_dev) {
  std::lock_guard<std::mutex> lock(g_registry_mu);
  registry()[copy_dev] = this;
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
