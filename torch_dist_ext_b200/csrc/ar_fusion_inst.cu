// Instantiates the fused all-reduce kernels for ONE element type and one launch flavour
// (real or single-GPU emulation). Compiled six times with
//   -DTDX_INST_DTYPE={0,1,2} -DTDX_INST_EMU={0,1}
// so that the instantiations build in parallel.
#include "tdx/api.h"
#include "tdx/ar_fusion_kernels.cuh"

#ifndef TDX_INST_DTYPE
#error "TDX_INST_DTYPE must be 0 (f32), 1 (f16) or 2 (bf16)"
#endif
#ifndef TDX_INST_EMU
#define TDX_INST_EMU 0
#endif

namespace tdx {
namespace {

#if TDX_INST_DTYPE == 0
using Elem = float;
#elif TDX_INST_DTYPE == 1
using Elem = __half;
#else
using Elem = __nv_bfloat16;
#endif
constexpr bool kEmu = TDX_INST_EMU != 0;

template <int kAlgo, int kN, int kVpt, int kOut>
const void* kernel_ptr() {
  if constexpr (kEmu)
    return reinterpret_cast<const void*>(&ar_fused_kernel_emu<Elem, kAlgo, kN, kVpt, kOut>);
  else
    return reinterpret_cast<const void*>(&ar_fused_kernel<Elem, kAlgo, kN, kVpt, kOut>);
}

template <int kAlgo, int kN, int kVpt>
const void* by_out(int out) {
  switch (out) {
    case kOutSame: return kernel_ptr<kAlgo, kN, kVpt, kOutSame>();
    case kOutFp8Token: return kernel_ptr<kAlgo, kN, kVpt, kOutFp8Token>();
    case kOutFp8Block128: return kernel_ptr<kAlgo, kN, kVpt, kOutFp8Block128>();
  }
  return nullptr;
}
template <int kAlgo, int kN>
const void* by_vpt(int vpt, int out) {
  switch (vpt) {
    case 1: return by_out<kAlgo, kN, 1>(out);
    case 2: return by_out<kAlgo, kN, 2>(out);
    case 4: return by_out<kAlgo, kN, 4>(out);
  }
  return nullptr;
}
template <int kAlgo>
const void* by_n(int n, int vpt, int out) {
  switch (n) {
    case 2: return by_vpt<kAlgo, 2>(vpt, out);
    case 4: return by_vpt<kAlgo, 4>(vpt, out);
    case 8: return by_vpt<kAlgo, 8>(vpt, out);
    case 0: return by_vpt<kAlgo, 0>(vpt, out);
  }
  return nullptr;
}
const void* select(const LaunchPlan& plan, int out) {
  switch (plan.algo) {
    case kAlgoLocal: return by_vpt<kAlgoLocal, 1>(plan.vpt, out);
    case kAlgoOneShotLamport: return by_n<kAlgoOneShotLamport>(plan.n_tmpl, plan.vpt, out);
    case kAlgoTwoShotLamport: return by_n<kAlgoTwoShotLamport>(plan.n_tmpl, plan.vpt, out);
    case kAlgoTwoShotBarrier: return by_n<kAlgoTwoShotBarrier>(plan.n_tmpl, plan.vpt, out);
    case kAlgoNvlsOneShot:
      if constexpr (!kEmu) return by_n<kAlgoNvlsOneShot>(plan.n_tmpl, plan.vpt, out);
      break;
    case kAlgoNvlsTwoShot:
      if constexpr (!kEmu) return by_n<kAlgoNvlsTwoShot>(plan.n_tmpl, plan.vpt, out);
      break;
    case kAlgoOneShotMc:
      if constexpr (!kEmu) return by_n<kAlgoOneShotMc>(plan.n_tmpl, plan.vpt, out);
      break;
    case kAlgoTwoShotMc:
      if constexpr (!kEmu) return by_n<kAlgoTwoShotMc>(plan.n_tmpl, plan.vpt, out);
      break;
  }
  return nullptr;
}

cudaError_t do_launch(const LaunchPlan& plan, int out, const ArParams& p, const ArParams* dev_ranks,
                      cudaStream_t stream) {
  const void* fn = select(plan, out);
  if (fn == nullptr) return cudaErrorInvalidValue;
  if constexpr (kEmu) {
    void* args[] = {const_cast<ArParams**>(&dev_ranks)};
    return cudaLaunchCooperativeKernel(fn, dim3(plan.grid, plan.emu_ranks), dim3(plan.threads), args, 0, stream);
  } else {
    // Programmatic stream serialisation: the blocks may be scheduled before the previous kernel of the stream has
    // finished; the kernel begins with griddepcontrol.wait, so nothing is read or written early.
    void* args[] = {const_cast<ArParams*>(&p)};
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(plan.grid);
    cfg.blockDim = dim3(plan.threads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelExC(&cfg, fn, args);
  }
}

int do_occupancy(const LaunchPlan& plan, int out) {
  const void* fn = select(plan, out);
  if (fn == nullptr) return 0;
  int nb = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, fn, plan.threads, 0) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return nb;
}

}  // namespace

#define TDX_CAT2(a, b) a##b
#define TDX_CAT(a, b) TDX_CAT2(a, b)
#if TDX_INST_DTYPE == 0
#define TDX_SUFFIX f32
#elif TDX_INST_DTYPE == 1
#define TDX_SUFFIX f16
#else
#define TDX_SUFFIX bf16
#endif
#if TDX_INST_EMU
#define TDX_NAME(base) TDX_CAT(TDX_CAT(base, TDX_SUFFIX), _emu)
#else
#define TDX_NAME(base) TDX_CAT(base, TDX_SUFFIX)
#endif

cudaError_t TDX_NAME(launch_ar_)(const LaunchPlan& plan, int out, const ArParams& p,
                                 const ArParams* dev_ranks, cudaStream_t stream) {
  return do_launch(plan, out, p, dev_ranks, stream);
}
int TDX_NAME(occupancy_ar_)(const LaunchPlan& plan, int out) { return do_occupancy(plan, out); }

}  // namespace tdx
