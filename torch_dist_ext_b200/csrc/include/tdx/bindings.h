// Declarations shared by the PyTorch binding translation units.
#pragma once
#include <torch/custom_class.h>
#include <torch/library.h>
#include <torch/torch.h>
#include <memory>
#include "tdx/api.h"

namespace tdx_torch {

// torch.classes.torch_dist_ext.CommWorkspace — same constructor and the same three methods as
// the reference's class (src/ops/all_reduce_fusion.h:10-40), plus reset / timeout / status.
class CommWorkspace : public torch::CustomClassHolder {
 public:
  CommWorkspace(int64_t rank, int64_t world_size, int64_t nblocks, int64_t size_in_bytes);
  CommWorkspace(int64_t rank, int64_t world_size, int64_t nblocks, int64_t size_in_bytes, int64_t lamport_bytes,
                int64_t device, int64_t multicast);
  at::Tensor get_handle();
  void open_handles(std::vector<at::Tensor> handles);
  at::Tensor get_workspace(const at::Tensor& ref);
  void adopt_table(const at::Tensor& copy);
  void reset();
  bool has_multicast();
  void disable_multicast();
  std::string multicast_note();
  void set_timeout_ms(int64_t ms);
  void set_debug_extent(int64_t bytes);
  void set_trace(const c10::optional<at::Tensor>& buffer);
  int64_t errors_seen();
  std::vector<int64_t> stats();
  tdx::Workspace* impl() { return impl_.get(); }

 private:
  std::unique_ptr<tdx::Workspace> impl_;
  at::Tensor trace_;   // keeps the trace buffer alive while the kernels may write to it
};

// Registers the standalone ops, GEMMs and model kernels (defined in ops_register.cpp).
void register_extra_ops(torch::Library& m);

}  // namespace tdx_torch
