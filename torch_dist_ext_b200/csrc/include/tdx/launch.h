// Kernel launch with programmatic stream serialisation (programmatic dependent launch).
//
// Launched with the attribute below, the blocks of a kernel may be scheduled while the previous kernel
// of the stream is still running. Every kernel of this library first does the work that touches no
// memory an earlier kernel may still write or read (barrier set-up, tensor-memory allocation,
// tensor-map prefetch and, in the decode GEMMs, the first ring of WEIGHT tiles), then executes
// `griddepcontrol.wait` (the previous kernel has completed and its memory is visible) and
// `griddepcontrol.launch_dependents` (the next kernel may be scheduled), in that order: a kernel
// therefore holds its shared and tensor memory before its successor can claim any, and at most one
// successor is waiting at a time. Launch latency and prologue of a kernel so overlap the tail of its
// predecessor; kernels of other libraries before or after simply serialise as usual. TDX_PDL=0 turns
// the attribute off (the two instructions are then no-ops).
//
// The reference launches with cudaLaunchCooperativeKernel and has no launch chaining
// (src/common/all_reduce_fusion_impl.h:492-495).
#pragma once
#include <cuda_runtime.h>
#include "tdx/api.h"

namespace tdx {

// `args` as for cudaLaunchKernel: an array of pointers to the kernel's arguments.
inline cudaError_t launch_chained(const void* fn, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, void** args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelExC(&cfg, fn, args);
}

// Typed form for `kernel<<<grid, block, smem, stream>>>(args...)` call sites.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace tdx
