// Stand-in used only when the reference is built for CUDA: maps the ROCm-build guard name that
// the reference includes unconditionally onto PyTorch's CUDA guard.
#pragma once
#include <c10/cuda/CUDAGuard.h>
namespace at { namespace hip {
using OptionalHIPGuardMasqueradingAsCUDA = c10::cuda::OptionalCUDAGuard;
}}
