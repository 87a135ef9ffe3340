// Stand-in used only when the reference is built for CUDA (see HIPGuardImplMasqueradingAsCUDA.h).
#pragma once
#include <c10/cuda/CUDAStream.h>
namespace c10 { namespace hip {
inline c10::cuda::CUDAStream getCurrentHIPStreamMasqueradingAsCUDA() { return c10::cuda::getCurrentCUDAStream(); }
}}
