// PyTorch bindings: custom class CommWorkspace and the fused-op entry points, registered in
// the `torch_dist_ext` namespace so that code written against the reference's
// torch.classes.torch_dist_ext.CommWorkspace / torch.ops.torch_dist_ext.allreduce_rms_fusion
// (src/register.cpp:4-15) keeps working. The op schema marks the tensors it writes
// (the reference's schema omits the alias annotations).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/custom_class.h>
#include <torch/library.h>
#include <torch/torch.h>
#include "tdx/api.h"
#include "tdx/bindings.h"

namespace {

using at::Tensor;

int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return tdx::kF32;
    case at::kHalf: return tdx::kF16;
    case at::kBFloat16: return tdx::kBF16;
    default: TORCH_CHECK(false, "torch_dist_ext: unsupported dtype ", t, " (float32, float16 and bfloat16 are supported)");
  }
  return -1;
}

}  // namespace

namespace tdx_torch {

CommWorkspace::CommWorkspace(int64_t rank, int64_t world_size, int64_t nblocks, int64_t size_in_bytes)
    : CommWorkspace(rank, world_size, nblocks, size_in_bytes, 0, -1, -1) {}

CommWorkspace::CommWorkspace(int64_t rank, int64_t world_size, int64_t nblocks, int64_t size_in_bytes,
                             int64_t lamport_bytes, int64_t device, int64_t multicast) {
  try {
    impl_ = std::make_unique<tdx::Workspace>((int)rank, (int)world_size, (int)nblocks, (uint64_t)size_in_bytes,
                                             (uint64_t)lamport_bytes, (int)device, (int)multicast);
  } catch (const std::exception& e) {
    TORCH_CHECK(false, "CommWorkspace: ", e.what());
  }
}

c10::intrusive_ptr<CommWorkspace> create_workspace(int64_t rank, int64_t world_size, int64_t nblocks,
                                                   int64_t size_in_bytes, int64_t lamport_bytes, int64_t device,
                                                   int64_t multicast) {
  return c10::make_intrusive<CommWorkspace>(rank, world_size, nblocks, size_in_bytes, lamport_bytes, device, multicast);
}

Tensor CommWorkspace::get_handle() {
  auto t = torch::empty({tdx::kHandleBytes}, torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCPU));
  try {
    impl_->export_handle(t.data_ptr<uint8_t>());
  } catch (const std::exception& e) {
    TORCH_CHECK(false, "CommWorkspace.get_handle: ", e.what());
  }
  return t;
}

void CommWorkspace::open_handles(std::vector<Tensor> handles) {
  std::vector<Tensor> keep;
  std::vector<const uint8_t*> ptrs;
  for (auto& h : handles) {
    TORCH_CHECK(h.device().is_cpu() && h.scalar_type() == at::kByte && h.numel() == tdx::kHandleBytes,
                "CommWorkspace.open_handles: each handle must be a CPU uint8 tensor of ", tdx::kHandleBytes, " bytes");
    keep.push_back(h.contiguous());
    ptrs.push_back(keep.back().data_ptr<uint8_t>());
  }
  try {
    impl_->open_handles(ptrs);
  } catch (const std::exception& e) {
    TORCH_CHECK(false, "CommWorkspace.open_handles: ", e.what());
  }
}

Tensor CommWorkspace::get_workspace(const Tensor& ref) {
  TORCH_CHECK(impl_->registered(), "CommWorkspace.get_workspace: call open_handles first");
  TORCH_CHECK(!ref.defined() || !ref.is_cuda() || ref.get_device() == impl_->device(),
              "CommWorkspace.get_workspace: reference tensor is on another device than the workspace");
  auto opts = torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, impl_->device());
  // The tensor views memory that the workspace owns, so it holds a reference that keeps the workspace alive.
  auto keep = c10::intrusive_ptr<CommWorkspace>::unsafe_reclaim_from_nonowning(this);
  return torch::from_blob(const_cast<tdx::CommTable*>(impl_->device_table()), {(int64_t)sizeof(tdx::CommTable)},
                          [keep](void*) mutable { keep.reset(); }, opts);
}

void CommWorkspace::adopt_table(const Tensor& copy) {
  TORCH_CHECK(copy.is_cuda() && copy.scalar_type() == at::kByte && copy.is_contiguous() &&
                  copy.numel() == (int64_t)sizeof(tdx::CommTable) && copy.get_device() == impl_->device(),
              "CommWorkspace.adopt_table: expected a device copy of the tensor returned by get_workspace");
  impl_->adopt_table_copy(copy.data_ptr());
}

void CommWorkspace::reset() { impl_->reset(); }
bool CommWorkspace::has_multicast() { return impl_->has_multicast(); }
void CommWorkspace::disable_multicast() { impl_->disable_multicast(); }
std::string CommWorkspace::multicast_note() { return impl_->multicast_note(); }
void CommWorkspace::set_timeout_ms(int64_t ms) { impl_->set_timeout_ns((uint64_t)ms * 1000000ull); }
void CommWorkspace::set_debug_extent(int64_t bytes) { impl_->set_debug_extent((uint64_t)bytes); }
int64_t CommWorkspace::errors_seen() { return impl_->errors_seen(); }
void CommWorkspace::set_trace(const c10::optional<Tensor>& buffer) {
  if (!buffer.has_value() || !buffer->defined()) {
    impl_->set_trace(nullptr);
    trace_ = Tensor();
    return;
  }
  TORCH_CHECK(buffer->is_cuda() && buffer->get_device() == impl_->device() && buffer->scalar_type() == at::kLong &&
                  buffer->is_contiguous() && buffer->numel() >= (int64_t)tdx::kMaxBarrierBlocks * tdx::kTraceSlots,
              "CommWorkspace.set_trace: need a contiguous int64 tensor of at least ", tdx::kMaxBarrierBlocks * tdx::kTraceSlots,
              " elements on the workspace's device");
  trace_ = *buffer;
  impl_->set_trace(reinterpret_cast<uint64_t*>(trace_.data_ptr<int64_t>()));
}

std::vector<int64_t> CommWorkspace::stats() {
  tdx::WorkspaceStats s = impl_->stats();
  std::vector<int64_t> v = {(int64_t)s.total_bytes, (int64_t)s.lamport_bytes, (int64_t)s.stage_bytes,
                            (int64_t)s.error_count, (int64_t)s.lamport_epoch, (int64_t)s.barrier_epoch,
                            (int64_t)s.has_multicast};
  for (int i = 0; i < 8; ++i) v.push_back(s.status[i]);
  return v;
}

void connect_local(std::vector<c10::intrusive_ptr<CommWorkspace>> all) {
  std::vector<tdx::Workspace*> ws;
  for (auto& w : all) ws.push_back(w->impl());
  try {
    tdx::Workspace::connect_local(ws);
  } catch (const std::exception& e) {
    TORCH_CHECK(false, "connect_local: ", e.what());
  }
}

// ---- fused all-reduce -------------------------------------------------------------------------

// Address under which the device sees a tensor's data. A CUDA tensor must live on `device`. With
// `allow_pinned`, a CPU tensor in page-locked memory is accepted too: the kernels then read or write it
// over PCIe themselves, which saves the staging copies of a caller whose data starts and ends on the host.
static void* device_address(const Tensor& t, int device, bool allow_pinned, const char* name) {
  if (t.is_cuda()) {
    TORCH_CHECK(t.get_device() == device, name, " is on another device than the workspace");
    return t.data_ptr();
  }
  TORCH_CHECK(allow_pinned && t.is_cpu(), name, " must be a CUDA tensor");
  cudaPointerAttributes attr{};
  const cudaError_t e = cudaPointerGetAttributes(&attr, t.data_ptr());
  if (e != cudaSuccess) (void)cudaGetLastError();
  TORCH_CHECK(e == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer != nullptr, name,
              " is a CPU tensor outside page-locked (pinned) memory: pin it or move it to the device");
  return attr.devicePointer;
}

static void fill_tensor_params(tdx::ArParams& p, const Tensor& in, const c10::optional<Tensor>& residual_in,
                               const Tensor& gamma, const c10::optional<Tensor>& residual_out,
                               const Tensor& norm_out, const c10::optional<Tensor>& scale_out, double eps,
                               int64_t out_mode, int64_t algo, bool scatter_only, int nranks, int device,
                               bool allow_pinned) {
  TORCH_CHECK(in.is_contiguous(), "allreduce_in must be contiguous");
  TORCH_CHECK(in.dim() >= 1, "allreduce_in must have at least one dimension");
  const int64_t hidden = in.size(-1);
  const int64_t tokens = hidden > 0 ? in.numel() / hidden : 0;
  TORCH_CHECK(in.numel() < (1ll << 31) * 8, "allreduce_in is too large");
  TORCH_CHECK(gamma.is_cuda() && gamma.get_device() == device && gamma.is_contiguous() && gamma.numel() == hidden &&
                  gamma.scalar_type() == in.scalar_type(),
              "rms_gamma must be a contiguous CUDA tensor of shape [hidden] and the input dtype, on the workspace's device");
  const int64_t out_rows = scatter_only ? (tokens + nranks - 1) / nranks : tokens;
  auto check_like = [&](const Tensor& t, const char* name) -> void* {
    TORCH_CHECK(t.is_contiguous() && t.scalar_type() == in.scalar_type() && t.numel() == out_rows * hidden, name,
                " must be a contiguous tensor of the input dtype with ", out_rows, " x ", hidden, " elements");
    return device_address(t, device, allow_pinned, name);
  };
  p.in = device_address(in, device, allow_pinned, "allreduce_in");
  p.residual_in = nullptr;
  if (residual_in.has_value() && residual_in->defined()) p.residual_in = check_like(*residual_in, "residual_in");
  p.residual_out = nullptr;
  if (residual_out.has_value() && residual_out->defined()) p.residual_out = check_like(*residual_out, "residual_out");
  p.gamma = gamma.data_ptr();
  if (out_mode == tdx::kOutSame) {
    p.norm_out = check_like(norm_out, "norm_out");
    p.scale_out = nullptr;
  } else {
    TORCH_CHECK(norm_out.is_contiguous() && norm_out.element_size() == 1 && norm_out.numel() == out_rows * hidden,
                "fp8 norm_out must be a contiguous 1-byte tensor with ", out_rows, " x ", hidden, " elements");
    TORCH_CHECK(scale_out.has_value() && scale_out->defined() && scale_out->is_contiguous() &&
                    scale_out->scalar_type() == at::kFloat,
                "fp8 output needs a contiguous float32 scale tensor");
    const int64_t nscale = out_mode == tdx::kOutFp8Token ? out_rows : out_rows * (hidden / 128);
    TORCH_CHECK(scale_out->numel() == nscale, "scale tensor must have ", nscale, " elements");
    p.norm_out = device_address(norm_out, device, allow_pinned, "norm_out");
    p.scale_out = static_cast<float*>(device_address(*scale_out, device, allow_pinned, "scale_out"));
  }
  p.tokens = (int32_t)tokens;
  p.hidden = (int32_t)hidden;
  p.eps = (float)eps;
  p.dtype = dtype_code(in.scalar_type());
  p.out_mode = (int32_t)out_mode;
  p.algo = (int32_t)algo;
  p.scatter_only = scatter_only ? 1 : 0;
}

static int64_t launch_fused(const Tensor& in, const c10::optional<Tensor>& residual_in, const Tensor& gamma,
                            const c10::optional<Tensor>& residual_out, const Tensor& norm_out,
                            const c10::optional<Tensor>& scale_out, double eps, const Tensor& workspace,
                            int64_t out_mode, int64_t algo, bool scatter_only, bool allow_pinned) {
  TORCH_CHECK(workspace.is_cuda(), "workspace must be the CUDA tensor returned by get_workspace");
  tdx::Workspace* ws = tdx::Workspace::from_table(workspace.data_ptr());
  TORCH_CHECK(ws != nullptr, "workspace tensor does not belong to a registered CommWorkspace");
  const c10::cuda::CUDAGuard guard(workspace.device());
  tdx::ArParams p{};
  ws->fill_params(&p);
  fill_tensor_params(p, in, residual_in, gamma, residual_out, norm_out, scale_out, eps, out_mode, algo, scatter_only,
                     p.nranks, ws->device(), allow_pinned);
  tdx::LaunchPlan used{};
  const std::string err = tdx::launch_allreduce(p, at::cuda::getCurrentCUDAStream().stream(), &used);
  TORCH_CHECK(err.empty(), "allreduce_rms_fusion: ", err);
  return used.algo;
}

int64_t allreduce_rms_fusion_ex(const Tensor& in, const c10::optional<Tensor>& residual_in, const Tensor& gamma,
                                c10::optional<Tensor> residual_out, Tensor norm_out, c10::optional<Tensor> scale_out,
                                double eps, const Tensor& workspace, int64_t out_mode, int64_t algo,
                                bool scatter_only) {
  return launch_fused(in, residual_in, gamma, residual_out, norm_out, scale_out, eps, workspace, out_mode, algo,
                      scatter_only, /*allow_pinned=*/false);
}

// Same op for callers whose data starts and ends in page-locked host memory: any of the data tensors (not
// gamma) may be a pinned CPU tensor. The reference has no counterpart; its op takes device tensors only
// (src/ops/all_reduce_fusion.cpp:14-61).
int64_t allreduce_rms_fusion_hostio(const Tensor& in, const c10::optional<Tensor>& residual_in, const Tensor& gamma,
                                    c10::optional<Tensor> residual_out, Tensor norm_out,
                                    c10::optional<Tensor> scale_out, double eps, const Tensor& workspace,
                                    int64_t out_mode, int64_t algo, bool scatter_only) {
  return launch_fused(in, residual_in, gamma, residual_out, norm_out, scale_out, eps, workspace, out_mode, algo,
                      scatter_only, /*allow_pinned=*/true);
}

void allreduce_rms_fusion(c10::SymInt rank, c10::SymInt nranks, const Tensor& allreduce_in, const Tensor& residual_in,
                          const Tensor& rms_gamma, Tensor residual_out, Tensor norm_out, double eps,
                          const Tensor& workspace) {
  tdx::Workspace* ws = tdx::Workspace::from_table(workspace.data_ptr());
  TORCH_CHECK(ws != nullptr, "workspace tensor does not belong to a registered CommWorkspace");
  TORCH_CHECK(rank.expect_int() == ws->rank() && nranks.expect_int() == ws->world_size(),
              "allreduce_rms_fusion: rank/nranks (", rank, "/", nranks, ") do not match the workspace (", ws->rank(), "/",
              ws->world_size(), ")");
  allreduce_rms_fusion_ex(allreduce_in, residual_in, rms_gamma, residual_out, norm_out, c10::nullopt, eps, workspace,
                          tdx::kOutSame, tdx::kAlgoAuto, false);
}

// All ranks as one cooperative launch on the current device (single-GPU protocol tests).
int64_t allreduce_rms_emulated(std::vector<c10::intrusive_ptr<CommWorkspace>> workspaces, std::vector<Tensor> ins,
                               std::vector<Tensor> residual_ins, const Tensor& gamma, std::vector<Tensor> residual_outs,
                               std::vector<Tensor> norm_outs, std::vector<Tensor> scale_outs, double eps,
                               int64_t out_mode, int64_t algo, bool scatter_only) {
  const int n = (int)workspaces.size();
  TORCH_CHECK(n >= 1 && n <= tdx::kMaxRanks && (int)ins.size() == n && (int)norm_outs.size() == n,
              "allreduce_rms_emulated: need one workspace, input and norm_out per rank");
  std::vector<tdx::ArParams> params(n);
  for (int r = 0; r < n; ++r) {
    tdx::Workspace* ws = workspaces[r]->impl();
    TORCH_CHECK(ws->rank() == r && ws->world_size() == n, "workspaces must be ordered by rank");
    ws->fill_params(&params[r]);
    fill_tensor_params(params[r], ins[r],
                       residual_ins.empty() ? c10::nullopt : c10::optional<Tensor>(residual_ins[r]), gamma,
                       residual_outs.empty() ? c10::nullopt : c10::optional<Tensor>(residual_outs[r]), norm_outs[r],
                       scale_outs.empty() ? c10::nullopt : c10::optional<Tensor>(scale_outs[r]), eps, out_mode, algo,
                       scatter_only, n, ws->device(), /*allow_pinned=*/true);
  }
  const c10::cuda::CUDAGuard guard(gamma.device());
  auto dev = torch::empty({(int64_t)(n * sizeof(tdx::ArParams))},
                          torch::TensorOptions().dtype(torch::kUInt8).device(gamma.device()));
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  C10_CUDA_CHECK(cudaMemcpyAsync(dev.data_ptr(), params.data(), n * sizeof(tdx::ArParams), cudaMemcpyHostToDevice, stream));
  tdx::LaunchPlan used{};
  const std::string err = tdx::launch_allreduce_emulated(
      params.data(), reinterpret_cast<const tdx::ArParams*>(dev.data_ptr()), n, stream, &used);
  TORCH_CHECK(err.empty(), "allreduce_rms_emulated: ", err);
  // the parameter copy must outlive the kernel
  C10_CUDA_CHECK(cudaStreamSynchronize(stream));
  return used.algo;
}

// Negative values leave the entry as it is.
void set_policy(int64_t nranks, int64_t oneshot_max_bytes, int64_t lamport_max_bytes, int64_t mc_oneshot, int64_t mc_twoshot,
                int64_t nvls_min_bytes) {
  TORCH_CHECK(nranks >= 1 && nranks <= tdx::kMaxRanks, "nranks out of range");
  tdx::Policy& pol = tdx::policy();
  if (oneshot_max_bytes >= 0) pol.oneshot_max_bytes[nranks] = (uint64_t)oneshot_max_bytes;
  if (lamport_max_bytes >= 0) pol.lamport_max_bytes[nranks] = (uint64_t)lamport_max_bytes;
  if (mc_oneshot >= 0) pol.mc_oneshot[nranks] = mc_oneshot != 0;
  if (mc_twoshot >= 0) pol.mc_twoshot[nranks] = mc_twoshot != 0;
  if (nvls_min_bytes >= 0) pol.nvls_min_bytes[nranks] = (uint64_t)nvls_min_bytes;
}

std::vector<int64_t> get_policy(int64_t nranks) {
  TORCH_CHECK(nranks >= 1 && nranks <= tdx::kMaxRanks, "nranks out of range");
  const tdx::Policy& pol = tdx::policy();
  return {(int64_t)pol.oneshot_max_bytes[nranks], (int64_t)pol.lamport_max_bytes[nranks], (int64_t)pol.mc_oneshot[nranks],
          (int64_t)pol.mc_twoshot[nranks], (int64_t)(pol.nvls_min_bytes[nranks] > (uint64_t)INT64_MAX ? INT64_MAX : pol.nvls_min_bytes[nranks])};
}

std::vector<int64_t> plan_allreduce(int64_t nranks, int64_t tokens, int64_t hidden, int64_t dtype, int64_t out_mode,
                                    int64_t algo, int64_t max_message_bytes, int64_t lamport_bytes) {
  // Host-only: what would be launched for this shape (no device needed except for occupancy).
  tdx::ArParams p{};
  p.nranks = (int)nranks;
  p.rank = 0;
  p.tokens = (int)tokens;
  p.hidden = (int)hidden;
  p.dtype = (int)dtype;
  p.out_mode = (int)out_mode;
  p.algo = (int)algo;
  p.layout = tdx::make_layout((uint64_t)max_message_bytes, (uint64_t)lamport_bytes);
  static char dummy[64] __attribute__((aligned(64)));
  p.in = p.gamma = dummy;
  p.norm_out = dummy;
  p.scale_out = reinterpret_cast<float*>(dummy);
  for (int r = 0; r < nranks && r < tdx::kMaxRanks; ++r) p.peer[r] = dummy;
  tdx::LaunchPlan pl{};
  const std::string err = tdx::plan_allreduce(p, 0, &pl);
  TORCH_CHECK(err.empty(), "plan_allreduce: ", err);
  return {pl.algo, pl.n_tmpl, pl.vpt, pl.threads, pl.grid};
}

}  // namespace tdx_torch

TORCH_LIBRARY(torch_dist_ext, m) {
  using tdx_torch::CommWorkspace;
  m.class_<CommWorkspace>("CommWorkspace")
      .def(torch::init<int64_t, int64_t, int64_t, int64_t>())
      .def("get_handle", &CommWorkspace::get_handle)
      .def("open_handles", &CommWorkspace::open_handles)
      .def("get_workspace", &CommWorkspace::get_workspace)
      .def("adopt_table", &CommWorkspace::adopt_table)
      .def("set_trace", &CommWorkspace::set_trace)
      .def("reset", &CommWorkspace::reset)
      .def("set_timeout_ms", &CommWorkspace::set_timeout_ms)
      .def("set_debug_extent", &CommWorkspace::set_debug_extent)
      .def("errors_seen", &CommWorkspace::errors_seen)
      .def("stats", &CommWorkspace::stats)
      .def("has_multicast", &CommWorkspace::has_multicast)
      .def("disable_multicast", &CommWorkspace::disable_multicast)
      .def("multicast_note", &CommWorkspace::multicast_note);
  m.def("create_workspace(int rank, int world_size, int nblocks, int size_in_bytes, int lamport_bytes, int device, "
        "int multicast) -> __torch__.torch.classes.torch_dist_ext.CommWorkspace", &tdx_torch::create_workspace);
  m.def("bounds_checked_build() -> bool", []() -> bool { return tdx::bounds_checked_build(); });
  m.def("set_tuning(int waves, int nvls_batch) -> ()", [](int64_t w, int64_t b) { tdx::set_tuning((int)w, (int)b); });
  m.def("tracing_build() -> bool", []() -> bool { return tdx::tracing_build(); });
  m.def("pdl_enabled() -> bool", []() -> bool { return tdx::pdl_enabled(); });
  m.def("table_nbytes() -> int", []() -> int64_t { return (int64_t)sizeof(tdx::CommTable); });
  m.def("connect_local(__torch__.torch.classes.torch_dist_ext.CommWorkspace[] workspaces) -> ()", &tdx_torch::connect_local);
  m.def(
      "allreduce_rms_fusion(SymInt rank, SymInt nranks, Tensor allreduce_in, Tensor residual_in, Tensor rms_gamma, "
      "Tensor(a!) residual_out, Tensor(b!) norm_out, float eps, Tensor workspace) -> ()");
  m.def(
      "allreduce_rms_fusion_ex(Tensor allreduce_in, Tensor? residual_in, Tensor rms_gamma, Tensor(a!)? residual_out, "
      "Tensor(b!) norm_out, Tensor(c!)? scale_out, float eps, Tensor workspace, int out_mode, int algo, "
      "bool scatter_only) -> int");
  m.def(
      "allreduce_rms_emulated(__torch__.torch.classes.torch_dist_ext.CommWorkspace[] workspaces, Tensor[] ins, "
      "Tensor[] residual_ins, Tensor rms_gamma, Tensor[] residual_outs, Tensor[] norm_outs, Tensor[] scale_outs, "
      "float eps, int out_mode, int algo, bool scatter_only) -> int",
      &tdx_torch::allreduce_rms_emulated);
  m.def(
      "allreduce_rms_fusion_hostio(Tensor allreduce_in, Tensor? residual_in, Tensor rms_gamma, Tensor(a!)? residual_out, "
      "Tensor(b!) norm_out, Tensor(c!)? scale_out, float eps, Tensor workspace, int out_mode, int algo, "
      "bool scatter_only) -> int",
      &tdx_torch::allreduce_rms_fusion_hostio);
  m.def("set_policy(int nranks, int oneshot_max_bytes, int lamport_max_bytes, int mc_oneshot=-1, int mc_twoshot=-1, int nvls_min_bytes=-1) -> ()", &tdx_torch::set_policy);
  m.def("get_policy(int nranks) -> int[]", &tdx_torch::get_policy);
  m.def(
      "plan_allreduce(int nranks, int tokens, int hidden, int dtype, int out_mode, int algo, int max_message_bytes, "
      "int lamport_bytes) -> int[]",
      &tdx_torch::plan_allreduce);
  tdx_torch::register_extra_ops(m);
}

TORCH_LIBRARY_IMPL(torch_dist_ext, CUDA, m) {
  m.impl("allreduce_rms_fusion", &tdx_torch::allreduce_rms_fusion);
  m.impl("allreduce_rms_fusion_ex", &tdx_torch::allreduce_rms_fusion_ex);
}
