// Launch planning for the fused all-reduce kernels: validation, capacity checks, algorithm
// selection by message size, block/grid sizing from the occupancy API, and dispatch to the
// per-dtype back ends.
//
// Reference counterpart: allreduce_fusion_kernel_launcher and allreduce_rms_fusion_impl
// (src/common/all_reduce_fusion_impl.h:476-535). Unlike it, every capacity is checked before
// the launch, the launch result is returned to the caller, one-shot versus two-shot is chosen
// by bytes per rank count (a table that a measured sweep can overwrite) instead of by a fixed
// token count, any rank count from 1 to 8 is accepted, and co-residency is obtained by sizing
// the grid from the occupancy API rather than by an unchecked cooperative launch.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>
#include "tdx/api.h"

namespace tdx {

bool bounds_checked_build() {
#ifdef TDX_BOUNDS
  return true;
#else
  return false;
#endif
}

bool tracing_build() {
#ifdef TDX_TRACE
  return true;
#else
  return false;
#endif
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("TDX_PDL");
    return !(e != nullptr && (e[0] == '0' || e[0] == 'o' || e[0] == 'f'));
  }();
  return on;
}

Policy& policy() {
  static Policy pol = [] {
    Policy q{};
    for (int n = 0; n <= kMaxRanks; ++n) {
      // Egress of the one-shot push grows with (n-1) x message, so its range shrinks with n.
      // Measured on 8 x B200 at 2, 4 and 8 ranks (benchmarks/bench_fused_allreduce.py). 2 ranks: one-shot wins up to
      // 16 MiB (49 against 52 us). 4 ranks: one-shot up to 512 KiB (1 MiB: 14.2 against 13.7 us), two-shot Lamport up
      // to 16 MiB (55 against 64 us for the flag-synchronised flow; equal at 32 MiB).
      q.oneshot_max_bytes[n] = n <= 2 ? (16u << 20) : (512u << 10);
      q.lamport_max_bytes[n] = n <= 2 ? (32u << 20) : n <= 4 ? (16u << 20) : (12u << 20);
      // In-switch reduction pays off once N-1 peers' worth of traffic is saved: never at 2 ranks, and at 4 ranks the
      // flag-synchronised peer-to-peer flow measured faster at every size (186 against 219 us at 64 MiB).
      q.nvls_min_bytes[n] = n <= 4 ? ~0ull : (12ull << 20);
      // one multimem.st instead of n - 1 stores pays off from three peers on
      q.mc_oneshot[n] = n >= 4;
      q.mc_twoshot[n] = n >= 4;
    }
    q.prefer_nvls = 1;
    return q;
  }();
  return pol;
}

namespace {

size_t elem_size(int dtype) { return dtype == kF32 ? 4 : 2; }

struct DeviceInfo {
  int sms = 0;
};
const DeviceInfo& device_info(int dev) {
  static std::mutex mu;
  static std::map<int, DeviceInfo> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(dev);
  if (it != cache.end()) return it->second;
  DeviceInfo d;
  cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
  return cache.emplace(dev, d).first->second;
}

int occupancy(int dtype, bool emu, const LaunchPlan& plan, int out_mode) {
  static std::mutex mu;
  static std::map<std::tuple<int, bool, int, int, int, int, int>, int> cache;
  const auto key = std::make_tuple(dtype, emu, plan.algo, plan.n_tmpl, plan.vpt, out_mode, plan.threads);
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  int nb = 0;
  if (emu) {
    nb = dtype == kF32 ? occupancy_ar_f32_emu(plan, out_mode)
         : dtype == kF16 ? occupancy_ar_f16_emu(plan, out_mode)
                         : occupancy_ar_bf16_emu(plan, out_mode);
  } else {
    nb = dtype == kF32 ? occupancy_ar_f32(plan, out_mode)
         : dtype == kF16 ? occupancy_ar_f16(plan, out_mode)
                         : occupancy_ar_bf16(plan, out_mode);
  }
  cache[key] = nb;
  return nb;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

std::string fmt(const char* f, long long a = 0, long long b = 0, long long c = 0) {
  char buf[256];
  std::snprintf(buf, sizeof(buf), f, a, b, c);
  return buf;
}

}  // namespace

std::string plan_allreduce(const ArParams& p, int emu_ranks, LaunchPlan* plan) {
  if (p.nranks < 1 || p.nranks > kMaxRanks) return fmt("nranks must be 1..8, got %lld", p.nranks);
  if (p.rank < 0 || p.rank >= p.nranks) return fmt("rank %lld out of range for %lld ranks", p.rank, p.nranks);
  if (p.dtype != kF32 && p.dtype != kF16 && p.dtype != kBF16) return "dtype must be float32, float16 or bfloat16";
  if (p.tokens < 0 || p.hidden <= 0) return "tokens must be >= 0 and hidden > 0";
  const size_t esz = elem_size(p.dtype);
  const int vec = int(16 / esz);
  if (p.hidden % vec != 0) return fmt("hidden (%lld) must be a multiple of %lld elements (16 bytes)", p.hidden, vec);
  if (p.out_mode < kOutSame || p.out_mode > kOutFp8Block128) return "unknown output mode";
  if (p.out_mode == kOutFp8Block128 && p.hidden % 128 != 0) return fmt("1x128 block scaling needs hidden %% 128 == 0, got %lld", p.hidden);
  if (p.out_mode != kOutSame && p.scale_out == nullptr) return "fp8 output needs a scale tensor";
  if (p.in == nullptr || p.gamma == nullptr || p.norm_out == nullptr) return "null input/gamma/norm_out";
  if (!aligned16(p.in) || !aligned16(p.gamma) || !aligned16(p.residual_in) || !aligned16(p.residual_out))
    return "inputs, gamma and residual tensors must be 16-byte aligned";
  if (!(p.out_mode == kOutSame ? aligned16(p.norm_out) : (reinterpret_cast<uintptr_t>(p.norm_out) & 7u) == 0))
    return "norm_out is not sufficiently aligned";

  const int nvec = p.hidden / vec;
  LaunchPlan pl{};
  pl.emu_ranks = emu_ranks;
  // Rows up to 512 vectors: one vector per thread. Up to 1024: two per thread in 512 threads
  // (128 registers available). Up to 2048: four per thread.
  if (nvec <= 512) pl.vpt = 1;
  else if (nvec <= 1024) pl.vpt = 2;
  else if (nvec <= 2048) pl.vpt = 4;
  else return fmt("hidden %lld exceeds the supported maximum of %lld for this dtype", p.hidden, 2048LL * vec);
  pl.threads = ((nvec + pl.vpt - 1) / pl.vpt + 31) / 32 * 32;

  const uint64_t row_bytes = uint64_t(p.hidden) * esz;
  const uint64_t msg_bytes = row_bytes * uint64_t(p.tokens);
  const int n = p.nranks;
  const uint64_t groups = (uint64_t(p.tokens) + n - 1) / n;
  const uint64_t gather_bytes = uint64_t(n) * groups * row_bytes;
  const uint64_t need_oneshot = uint64_t(n) * msg_bytes;
  const uint64_t need_ts_lamport = gather_bytes + (p.scatter_only ? 0 : uint64_t(p.tokens) * (row_bytes + 16));

  int algo = p.algo;
  if (n == 1) {
    algo = kAlgoLocal;
  } else {
    for (int r = 0; r < n; ++r)
      if (p.peer[r] == nullptr) return "workspace is not registered with all peers (null peer pointer)";
    if (algo == kAlgoLocal) return "the local algorithm needs nranks == 1";
    const bool mc_ok = p.mc_base != nullptr && emu_ranks == 0;
    if (algo == kAlgoAuto) {
      const Policy& pol = policy();
      const bool nvls_ok = p.mc_base != nullptr && pol.prefer_nvls && emu_ranks == 0 &&
                           msg_bytes <= p.layout.nvls_in_bytes &&
                           uint64_t(p.tokens) * (row_bytes + 16) + 2 * p.layout.nvls_in_bytes <= p.layout.nvls_bytes;
      if (nvls_ok && msg_bytes >= pol.nvls_min_bytes[n])
        algo = kAlgoNvlsTwoShot;
      else if (!p.scatter_only && msg_bytes <= pol.oneshot_max_bytes[n] && need_oneshot <= p.layout.lamport_bytes)
        algo = (mc_ok && pol.mc_oneshot[n]) ? kAlgoOneShotMc : kAlgoOneShotLamport;
      else if (msg_bytes <= pol.lamport_max_bytes[n] && need_ts_lamport <= p.layout.lamport_bytes)
        // the multicast result hop wins at every size at 8 ranks, at fewer ranks only up to 2 MiB
        algo = (mc_ok && pol.mc_twoshot[n] && !p.scatter_only && (n >= 8 || msg_bytes <= (2u << 20))) ? kAlgoTwoShotMc
                                                                                                      : kAlgoTwoShotLamport;
      else
        algo = kAlgoTwoShotBarrier;
    }
    if ((algo == kAlgoOneShotMc || algo == kAlgoTwoShotMc) && !mc_ok)
      return "the multicast-push algorithms need a workspace with an NVSwitch multicast mapping (not available here) and real ranks";
    if (algo == kAlgoOneShotLamport || algo == kAlgoOneShotMc) {
      if (p.scatter_only) return "the one-shot algorithm cannot produce scattered output";
      if (need_oneshot > p.layout.lamport_bytes)
        return fmt("one-shot needs %lld bytes of Lamport buffer, capacity is %lld", need_oneshot, p.layout.lamport_bytes);
    } else if (algo == kAlgoTwoShotLamport || algo == kAlgoTwoShotMc) {
      if (need_ts_lamport > p.layout.lamport_bytes)
        return fmt("two-shot (Lamport) needs %lld bytes of Lamport buffer, capacity is %lld", need_ts_lamport, p.layout.lamport_bytes);
    } else if (algo == kAlgoTwoShotBarrier) {
      // gather area in the first half of the staging region, result rows + trailers in the second
      const uint64_t half = p.layout.stage_bytes / 2;
      const uint64_t need_result = p.scatter_only ? 0 : uint64_t(p.tokens) * (row_bytes + 16);
      if (gather_bytes > half || need_result > half)
        return fmt("message of %lld bytes exceeds the workspace capacity (needs %lld of %lld staging bytes)", msg_bytes,
                   2 * (gather_bytes > need_result ? gather_bytes : need_result), p.layout.stage_bytes);
    } else if (algo == kAlgoNvlsOneShot || algo == kAlgoNvlsTwoShot) {
      if (p.mc_base == nullptr || p.layout.nvls_in_bytes == 0)
        return "NVLS algorithms need a workspace with an NVSwitch multicast mapping (not available here)";
      if (emu_ranks > 0) return "NVLS algorithms cannot be emulated on one device";
      if (algo == kAlgoNvlsOneShot && p.scatter_only) return "the one-shot algorithm cannot produce scattered output";
      const uint64_t result_cap = p.layout.nvls_bytes - 2 * p.layout.nvls_in_bytes;
      if (msg_bytes > p.layout.nvls_in_bytes || uint64_t(p.tokens) * (row_bytes + 16) > result_cap)
        return fmt("message of %lld bytes exceeds the NVLS staging capacity of %lld bytes", msg_bytes, p.layout.nvls_in_bytes);
    } else {
      return fmt("unknown algorithm %lld", algo);
    }
  }
  pl.algo = algo;
  pl.n_tmpl = (n == 1) ? 1 : (n == 2 || n == 4 || n == 8) ? n : 0;

  // grid: one block per row (or row group), capped by what is co-resident
  // Work items that set the grid: rows, except on the flag-synchronised two-shot paths where block b
  // of every rank must handle the same row groups.
  const uint64_t work = (algo == kAlgoTwoShotBarrier || algo == kAlgoNvlsTwoShot) ? groups : uint64_t(p.tokens);
  int dev = 0, ndev = 0;
  int sms = 148, per_sm = 1;  // planning without a device (dry runs) assumes one block per B200 SM
  if (cudaGetDeviceCount(&ndev) == cudaSuccess && ndev > 0) {
    cudaGetDevice(&dev);
    sms = device_info(dev).sms;
    per_sm = occupancy(p.dtype, emu_ranks > 0, pl, p.out_mode);
    if (per_sm <= 0 || sms <= 0) return "kernel cannot be resident on this device (occupancy query returned 0)";
  } else {
    cudaGetLastError();
  }
  uint64_t cap = uint64_t(per_sm) * sms;
  if (emu_ranks > 0) cap /= emu_ranks;
  const bool uses_flags = algo == kAlgoTwoShotBarrier || algo == kAlgoNvlsOneShot || algo == kAlgoNvlsTwoShot;
  if (uses_flags && cap > uint64_t(kMaxBarrierBlocks)) cap = kMaxBarrierBlocks;
  if (cap == 0) return "too many emulated ranks for one cooperative launch";
  uint64_t grid = work < cap ? work : cap;
  if (grid == 0) grid = 1;
  pl.grid = int(grid);
  *plan = pl;
  return "";
}

namespace {
std::string dispatch(const LaunchPlan& pl, const ArParams& p, const ArParams* dev_ranks, cudaStream_t stream) {
  cudaError_t e;
  if (pl.emu_ranks > 0) {
    e = p.dtype == kF32 ? launch_ar_f32_emu(pl, p.out_mode, p, dev_ranks, stream)
        : p.dtype == kF16 ? launch_ar_f16_emu(pl, p.out_mode, p, dev_ranks, stream)
                          : launch_ar_bf16_emu(pl, p.out_mode, p, dev_ranks, stream);
  } else {
    e = p.dtype == kF32 ? launch_ar_f32(pl, p.out_mode, p, dev_ranks, stream)
        : p.dtype == kF16 ? launch_ar_f16(pl, p.out_mode, p, dev_ranks, stream)
                          : launch_ar_bf16(pl, p.out_mode, p, dev_ranks, stream);
  }
  if (e != cudaSuccess) return std::string("kernel launch failed: ") + cudaGetErrorString(e);
  return "";
}
}  // namespace

std::string launch_allreduce(const ArParams& p, cudaStream_t stream, LaunchPlan* used) {
  LaunchPlan pl{};
  std::string err = plan_allreduce(p, 0, &pl);
  if (!err.empty()) return err;
  if (used) *used = pl;
  if (p.tokens == 0) return "";
  return dispatch(pl, p, nullptr, stream);
}

std::string launch_allreduce_emulated(const ArParams* host_ranks, const ArParams* dev_ranks, int nranks,
                                      cudaStream_t stream, LaunchPlan* used) {
  if (nranks < 1 || nranks > kMaxRanks) return "emulated rank count must be 1..8";
  LaunchPlan pl{};
  for (int r = 0; r < nranks; ++r) {
    if (host_ranks[r].rank != r || host_ranks[r].nranks != nranks) return "emulated parameter blocks must be ordered by rank";
    LaunchPlan q{};
    std::string err = plan_allreduce(host_ranks[r], nranks, &q);
    if (!err.empty()) return err;
    if (r == 0) pl = q;
    else if (q.algo != pl.algo || q.grid != pl.grid || q.threads != pl.threads || q.vpt != pl.vpt)
      return "emulated ranks disagree on the launch plan";
  }
  if (used) *used = pl;
  if (host_ranks[0].tokens == 0) return "";
  return dispatch(pl, host_ranks[0], dev_ranks, stream);
}

}  // namespace tdx
