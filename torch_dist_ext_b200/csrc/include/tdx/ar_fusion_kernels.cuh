// Fused all-reduce + residual add + RMSNorm (+ fp8 quantisation) kernels for sm_100a.
//
// Same math as the reference's two kernels (src/common/all_reduce_fusion_impl.h:342-396
// two-shot, :417-474 one-shot Lamport, :316-340 rms_norm):
//   s            = T( sum_r float(in_r) )          fp32 accumulate in rank order, one rounding
//   residual_out = T( float(s) + float(residual_in) )
//   rstd         = rsqrtf( sum_h residual_out_h^2 / H + eps )
//   norm_out     = T( residual_out * rstd * gamma )      or its e4m3 quantisation
// but a different data flow, designed for NVSwitch (every peer one hop away at full rate):
//
//  one-shot Lamport   every rank pushes its rows into a slot of every peer's buffer and
//                     polls its own buffer; no barrier. The rank's own contribution is read
//                     from its input, never pushed to itself.
//  two-shot Lamport   rows are owned round-robin (row % N). Ranks push each row only to its
//                     owner (reduce-scatter by push, no local staging copy); the owner
//                     reduces, adds the residual, computes rstd (and the per-token fp8
//                     scale) ONCE, and pushes the finished residual row plus a 16-byte
//                     trailer {rstd, scale} to the peers, which only run the elementwise
//                     epilogue. Still no barrier: both hops are validated by sentinels.
//  two-shot barrier   the same flow through flag-synchronised staging, for messages larger
//                     than a Lamport buffer.
//  NVLS one/two-shot  the reduction is done by the switch (multimem.ld_reduce); results are
//                     replicated by multimem.st.
//
// A row is processed by one CTA; thread t holds vectors t, t+blockDim, ... (kVpt of them)
// of 16 bytes each, so hidden sizes beyond 1024 threads x 16 B are handled by kVpt > 1.
//
// kEmu: all ranks run inside ONE cooperative launch on one GPU (blockIdx.y = rank), each
// with its own parameter block and buffers. It exists so that the cross-rank protocols can
// be tested on a single GPU, where separate launches that wait on each other must never be
// used.
#pragma once
#include "tdx/comm.h"
#include "tdx/ptx.cuh"
#include "tdx/sync.cuh"
#include "tdx/vec.cuh"

namespace tdx {

constexpr float kFp8Max = 448.f;     // e4m3fn
constexpr float kAmaxFloor = 1e-10f; // keeps scales finite for all-zero rows

template <typename T, int kVpt>
struct RowView {
  static constexpr int kVec = VecTraits<T>::kVec;
  int nvec;                 // 16-byte vectors per row
  size_t row_bytes;
  __device__ __forceinline__ RowView(int hidden)
      : nvec(hidden / kVec), row_bytes((size_t)hidden * sizeof(T)) {}
  __device__ __forceinline__ int vec_index(int v) const { return threadIdx.x + v * blockDim.x; }
  __device__ __forceinline__ bool active(int v) const { return vec_index(v) < nvec; }
};

// ---- epilogue -------------------------------------------------------------------------

template <typename T, int kVpt>
__device__ __forceinline__ float row_sum_squares(const float (&x)[kVpt][VecTraits<T>::kVec]) {
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < kVpt; ++v)
#pragma unroll
    for (int i = 0; i < VecTraits<T>::kVec; ++i) ss = fmaf(x[v][i], x[v][i], ss);
  return ss;
}

// |norm| maximum of this thread's part of the row (inactive vectors hold zeros).
template <typename T, int kVpt>
__device__ __forceinline__ float thread_amax(const float (&x)[kVpt][VecTraits<T>::kVec],
                                             const uint4 (&gamma)[kVpt], float rstd) {
  float amax = 0.f;
#pragma unroll
  for (int v = 0; v < kVpt; ++v) {
    float g[VecTraits<T>::kVec];
    unpack<T>(gamma[v], g);
#pragma unroll
    for (int i = 0; i < VecTraits<T>::kVec; ++i) amax = fmaxf(amax, fabsf(x[v][i] * rstd * g[i]));
  }
  return amax;
}

template <int kVec>
__device__ __forceinline__ void store_fp8(void* dst, const float (&q)[kVec]) {
  if constexpr (kVec == 8) {
    uint2 o;
    o.x = ptx::cvt_e4m3x4(q[0], q[1], q[2], q[3]);
    o.y = ptx::cvt_e4m3x4(q[4], q[5], q[6], q[7]);
    ptx::st_stream_v2(dst, o);
  } else {
    *reinterpret_cast<uint32_t*>(dst) = ptx::cvt_e4m3x4(q[0], q[1], q[2], q[3]);
  }
}

// Writes norm_out (and block scales) for one row. `token_scale` is used by kOutFp8Token only
// and must already be the value written to scale_out for this row.
template <typename T, int kVpt, int kOut>
__device__ __forceinline__ void store_norm(const ArParams& p, const RowView<T, kVpt>& rv,
                                           int64_t out_row,
                                           const float (&x)[kVpt][VecTraits<T>::kVec],
                                           const uint4 (&gamma)[kVpt], float rstd,
                                           float token_scale) {
  constexpr int kVec = VecTraits<T>::kVec;
#pragma unroll
  for (int v = 0; v < kVpt; ++v) {
    float g[kVec], y[kVec];
    unpack<T>(gamma[v], g);
#pragma unroll
    for (int i = 0; i < kVec; ++i) y[i] = x[v][i] * rstd * g[i];
    const int64_t col = (int64_t)rv.vec_index(v) * kVec;
    if constexpr (kOut == kOutSame) {
      if (rv.active(v))
        ptx::st_stream_v4(static_cast<char*>(p.norm_out) + out_row * rv.row_bytes +
                              (size_t)rv.vec_index(v) * 16,
                          pack<T>(y));
    } else if constexpr (kOut == kOutFp8Token) {
      const float inv = 1.f / token_scale;
#pragma unroll
      for (int i = 0; i < kVec; ++i) y[i] *= inv;
      if (rv.active(v))
        store_fp8<kVec>(static_cast<char*>(p.norm_out) + out_row * p.hidden + col, y);
    } else {
      // 1x128 block scales: the 128/kVec lanes that share a block are adjacent in a warp.
      constexpr int kLanes = 128 / kVec;
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < kVec; ++i) amax = fmaxf(amax, fabsf(y[i]));
      amax = group_max<kLanes>(amax);
      const float scale = fmaxf(amax, kAmaxFloor) / kFp8Max;
      const float inv = 1.f / scale;
#pragma unroll
      for (int i = 0; i < kVec; ++i) y[i] *= inv;
      if (rv.active(v)) {
        store_fp8<kVec>(static_cast<char*>(p.norm_out) + out_row * p.hidden + col, y);
        if ((threadIdx.x & (kLanes - 1)) == 0)
          p.scale_out[out_row * (p.hidden / 128) + col / 128] = scale;
      }
    }
  }
}

// rstd, the optional per-token scale, and the norm_out store for a row held in registers.
// Every thread of the block must call it (block-wide reductions inside).
template <typename T, int kVpt, int kOut>
__device__ __forceinline__ void finish_row(const ArParams& p, const RowView<T, kVpt>& rv,
                                           int64_t out_row,
                                           const float (&x)[kVpt][VecTraits<T>::kVec],
                                           const uint4 (&gamma)[kVpt], float (*red)[32],
                                           int parity, float& rstd_out, float& scale_out_val) {
  const float ss = block_allreduce<false>(row_sum_squares<T, kVpt>(x), red[parity]);
  const float rstd = rsqrtf(ss / (float)p.hidden + p.eps);
  float token_scale = 1.f;
  if constexpr (kOut == kOutFp8Token) {
    const float amax = block_allreduce<true>(thread_amax<T, kVpt>(x, gamma, rstd), red[2 + parity]);
    token_scale = fmaxf(amax, kAmaxFloor) / kFp8Max;
    if (threadIdx.x == 0) p.scale_out[out_row] = token_scale;
  }
  store_norm<T, kVpt, kOut>(p, rv, out_row, x, gamma, rstd, token_scale);
  rstd_out = rstd;
  scale_out_val = token_scale;
}

template <typename T, int kVpt>
__device__ __forceinline__ void load_gamma(const ArParams& p, const RowView<T, kVpt>& rv,
                                           uint4 (&gamma)[kVpt]) {
#pragma unroll
  for (int v = 0; v < kVpt; ++v)
    gamma[v] = rv.active(v) ? ptx::ld_v4(static_cast<const char*>(p.gamma) + (size_t)rv.vec_index(v) * 16)
                            : make_uint4(0, 0, 0, 0);
}

// s = T(acc); x = T(s + residual). `acc` holds the fp32 sum over ranks on entry, x on exit.
template <typename T>
__device__ __forceinline__ void add_residual(float (&acc)[VecTraits<T>::kVec], const void* res_ptr) {
  constexpr int kVec = VecTraits<T>::kVec;
  round_through<T>(acc);
  if (res_ptr != nullptr) {
    float r[kVec];
    unpack<T>(ptx::ld_stream_v4(res_ptr), r);
#pragma unroll
    for (int i = 0; i < kVec; ++i) acc[i] += r[i];
    round_through<T>(acc);
  }
}

// The same with a residual vector that the caller requested earlier (before it started to wait for
// its peers, so that the DRAM latency of the residual hides behind that wait).
template <typename T>
__device__ __forceinline__ void add_residual_loaded(float (&acc)[VecTraits<T>::kVec], bool has_residual, const uint4& res) {
  constexpr int kVec = VecTraits<T>::kVec;
  round_through<T>(acc);
  if (has_residual) {
    float r[kVec];
    unpack<T>(res, r);
#pragma unroll
    for (int i = 0; i < kVec; ++i) acc[i] += r[i];
    round_through<T>(acc);
  }
}

template <typename T, int kVpt>
__device__ __forceinline__ void request_residual(const ArParams& p, const RowView<T, kVpt>& rv, int64_t res_row,
                                                 uint4 (&res)[kVpt]) {
#pragma unroll
  for (int v = 0; v < kVpt; ++v)
    res[v] = (p.residual_in != nullptr && rv.active(v))
                 ? ptx::ld_stream_v4(static_cast<const char*>(p.residual_in) + (size_t)res_row * rv.row_bytes +
                                     (size_t)rv.vec_index(v) * 16)
                 : make_uint4(0u, 0u, 0u, 0u);
}

__device__ __forceinline__ char* lamport_buf(void* base, const Layout& l, uint32_t idx) {
  return static_cast<char*>(base) + l.off_lamport + (size_t)idx * l.lamport_bytes;
}

// All blocks of this rank cooperatively re-fill the buffer that the previous Lamport call used.
__device__ __forceinline__ void clear_previous(char* buf, uint64_t dirty_bytes, int cta, int nctas) {
  const uint4 s = sentinel_vec();
  const uint64_t stride = (uint64_t)nctas * blockDim.x * 16;
  for (uint64_t off = ((uint64_t)cta * blockDim.x + threadIdx.x) * 16; off < dirty_bytes; off += stride)
    ptx::st_v4(buf + off, s);
}
__device__ __forceinline__ void clear_previous(char* buf, uint64_t dirty_bytes) {
  clear_previous(buf, dirty_bytes, blockIdx.x, gridDim.x);
}

// Poll one 16-byte vector until every 32-bit lane has been overwritten by its producer.
__device__ __forceinline__ uint4 poll_vec(const char* addr, Waiter& w, const ArParams& p,
                                          Control* ctl, uint32_t code, int peer, int phase,
                                          int row) {
  uint4 v = ptx::ld_volatile_v4(addr);
  if (all_arrived(v)) return v;
  w.begin();
  uint32_t backoff = 20;
  while (true) {
    v = ptx::ld_volatile_v4(addr);
    if (all_arrived(v)) return v;
    // back off between polls so that waiting blocks do not crowd the L2 that the producers need
    __nanosleep(backoff);
    if (backoff < 320) backoff <<= 1;
    if (!w.keep_waiting()) {
      report_error(ctl, p.host_status, code, p.rank, peer, phase, row);
      return v;
    }
  }
}

// ---- local (single rank): residual add + RMSNorm (+ quant) --------------------------------

template <typename T, int kVpt, int kOut>
__device__ __forceinline__ void local_body(const ArParams& p) {
  constexpr int kVec = VecTraits<T>::kVec;
  __shared__ float red[4][32];
  const RowView<T, kVpt> rv(p.hidden);
  uint4 gamma[kVpt];
  load_gamma<T, kVpt>(p, rv, gamma);
  int parity = 0;
  for (int row = blockIdx.x; row < p.tokens; row += gridDim.x, parity ^= 1) {
    float x[kVpt][kVec];
#pragma unroll
    for (int v = 0; v < kVpt; ++v) {
      if (rv.active(v)) {
        const size_t off = (size_t)row * rv.row_bytes + (size_t)rv.vec_index(v) * 16;
        unpack<T>(ptx::ld_stream_v4(static_cast<const char*>(p.in) + off), x[v]);
        add_residual<T>(x[v], p.residual_in ? static_cast<const char*>(p.residual_in) + off : nullptr);
        if (p.residual_out) ptx::st_stream_v4(static_cast<char*>(p.residual_out) + off, pack<T>(x[v]));
      } else {
#pragma unroll
        for (int i = 0; i < kVec; ++i) x[v][i] = 0.f;
      }
    }
    float rstd, sc;
    finish_row<T, kVpt, kOut>(p, rv, row, x, gamma, red, parity, rstd, sc);
  }
}

// ---- one-shot Lamport ------------------------------------------------------------------

// kMc: the push is one multimem.st per vector into slot `rank` of the multicast mapping; NVSwitch replicates it
// into every rank's buffer (this rank's own slot included, which nobody reads), so the sender's links carry the
// message once instead of N - 1 times and a thread issues one store instead of N - 1.
template <typename T, int kN, int kVpt, int kOut, bool kMc = false>
__device__ __forceinline__ void oneshot_lamport_body(const ArParams& p) {
  constexpr int kVec = VecTraits<T>::kVec;
  __shared__ float red[4][32];
  const int nranks = kN > 0 ? kN : p.nranks;
  const RowView<T, kVpt> rv(p.hidden);
  char* self = static_cast<char*>(p.peer[p.rank]);
  Control* ctl = reinterpret_cast<Control*>(self + p.layout.off_control);
  const uint32_t epoch = ctl->lamport_epoch;
  const uint64_t dirty_prev = ctl->lamport_dirty[(epoch + 2u) % 3u];
  const size_t msg_bytes = rv.row_bytes * p.tokens;
  const char* in = static_cast<const char*>(p.in);

  // 1. push this rank's rows into slot `rank` of every peer's current buffer. When no block has
  //    more than one row, the vectors read here stay in registers for step 3, so that the input
  //    is read once (it may live in pinned host memory, where a second read crosses PCIe again).
  const bool single_row = p.tokens <= (int)gridDim.x;
  uint4 own[kVpt];
  for (int row = blockIdx.x; row < p.tokens; row += gridDim.x) {
#pragma unroll
    for (int v = 0; v < kVpt; ++v) {
      if (!rv.active(v)) continue;
      const size_t off = (size_t)row * rv.row_bytes + (size_t)rv.vec_index(v) * 16;
      const uint4 val = scrub(ptx::ld_stream_v4(in + off));
      own[v] = val;
      const size_t dst = p.layout.off_lamport + (size_t)(epoch % 3u) * p.layout.lamport_bytes + (size_t)p.rank * msg_bytes + off;
      if constexpr (kMc) {
        ptx::multimem_st_v4(symm_mc(p, dst), val);
      } else {
#pragma unroll
        for (int r = 0; r < (kN > 0 ? kN : kMaxRanks); ++r) {
          if (r >= nranks || r == p.rank) continue;
          ptx::st_v4(symm(p, r, dst), val);
        }
      }
    }
  }
  trace_mark(p, kTracePushed);

  // 2. restore the sentinels in the buffer the previous call used
  clear_previous(lamport_buf(self, p.layout, (epoch + 2u) % 3u), dirty_prev);
  trace_mark(p, kTraceCleared);

  // 3. gather, reduce, epilogue
  uint4 gamma[kVpt];
  load_gamma<T, kVpt>(p, rv, gamma);
  Waiter w(p.timeout_ns);
  const char* mine = lamport_buf(self, p.layout, epoch % 3u);
  int parity = 0;
  for (int row = blockIdx.x; row < p.tokens; row += gridDim.x, parity ^= 1) {
    float x[kVpt][kVec];
    uint4 res[kVpt];
    request_residual<T, kVpt>(p, rv, row, res);
#pragma unroll
    for (int v = 0; v < kVpt; ++v) {
#pragma unroll
      for (int i = 0; i < kVec; ++i) x[v][i] = 0.f;
      if (!rv.active(v)) continue;
      const size_t off = (size_t)row * rv.row_bytes + (size_t)rv.vec_index(v) * 16;
      if constexpr (kN > 0) {
        uint4 vals[kN];
        // issue all polls first so that kN-1 loads are in flight together
#pragma unroll
        for (int r = 0; r < kN; ++r)
          vals[r] = (r == p.rank) ? (single_row ? own[v] : scrub(ptx::ld_v4(in + off)))
                                  : ptx::ld_volatile_v4(mine + (size_t)r * msg_bytes + off);
#pragma unroll
        for (int r = 0; r < kN; ++r)
          if (r != p.rank && !all_arrived(vals[r]))
            vals[r] = poll_vec(mine + (size_t)r * msg_bytes + off, w, p, ctl, kTimeoutLamportGather, r, 1, row);
#pragma unroll
        for (int r = 0; r < kN; ++r) {
          float f[kVec];
          unpack<T>(vals[r], f);
#pragma unroll
          for (int i = 0; i < kVec; ++i) x[v][i] += f[i];
        }
      } else {
        for (int r = 0; r < nranks; ++r) {
          const uint4 val = (r == p.rank)
                                ? (single_row ? own[v] : scrub(ptx::ld_v4(in + off)))
                                : poll_vec(mine + (size_t)r * msg_bytes + off, w, p, ctl, kTimeoutLamportGather, r, 1, row);
          float f[kVec];
          unpack<T>(val, f);
#pragma unroll
          for (int i = 0; i < kVec; ++i) x[v][i] += f[i];
        }
      }
      add_residual_loaded<T>(x[v], p.residual_in != nullptr, res[v]);
      if (p.residual_out) ptx::st_stream_v4(static_cast<char*>(p.residual_out) + off, pack<T>(x[v]));
    }
    trace_mark(p, kTraceGathered);
    float rstd, sc;
    finish_row<T, kVpt, kOut>(p, rv, row, x, gamma, red, parity, rstd, sc);
  }
  trace_mark(p, kTraceEndClk);
  trace_mark_ns(p, kTraceEndNs);
  finish_launch(ctl, true, epoch, (uint64_t)nranks * msg_bytes, 0);
}

// ---- two-shot: shared pieces ---------------------------------------------------------------
// Row `t` is owned by rank t % N and belongs to group j = t / N. Block b handles groups
// b, b + gridDim, ...  Gather area on the owner: [src rank][group][hidden]. Result area on
// every rank: [row]{hidden values, 16-byte trailer} (Lamport) or [row][hidden] followed by a
// trailer array (barrier).

struct TwoShotGeometry {
  int groups;
  size_t gather_bytes;   // size of the gather area
  size_t result_stride;  // bytes between result rows
  size_t trailer_off;    // barrier path: offset of the trailer array inside the result area
};

template <typename T, int kVpt>
__device__ __forceinline__ TwoShotGeometry twoshot_geometry(const ArParams& p, const RowView<T, kVpt>& rv,
                                                            int nranks, bool lamport) {
  TwoShotGeometry g;
  g.groups = (p.tokens + nranks - 1) / nranks;
  g.gather_bytes = (size_t)nranks * g.groups * rv.row_bytes;
  g.result_stride = lamport ? rv.row_bytes + 16 : rv.row_bytes;
  g.trailer_off = (size_t)p.tokens * rv.row_bytes;
  return g;
}

// Scatter: push every row of this block's groups to the row's owner.
template <typename T, int kN, int kVpt, bool kScrub>
__device__ __forceinline__ void twoshot_scatter(const ArParams& p, const RowView<T, kVpt>& rv,
                                                const TwoShotGeometry& g, int nranks,
                                                size_t area_off /* from peer base */) {
  const char* in = static_cast<const char*>(p.in);
  for (int j = blockIdx.x; j < g.groups; j += gridDim.x) {
#pragma unroll
    for (int r = 0; r < (kN > 0 ? kN : kMaxRanks); ++r) {
      const int row = j * nranks + r;
      if (r >= nranks || r == p.rank || row >= p.tokens) continue;
      const size_t dst_off = area_off + ((size_t)p.rank * g.groups + j) * rv.row_bytes;
#pragma unroll
      for (int v = 0; v < kVpt; ++v) {
        if (!rv.active(v)) continue;
        uint4 val = ptx::ld_stream_v4(in + (size_t)row * rv.row_bytes + (size_t)rv.vec_index(v) * 16);
        if (kScrub) val = scrub(val);
        ptx::st_v4(symm(p, r, dst_off + (size_t)rv.vec_index(v) * 16), val);
      }
    }
  }
}

// Same push, but work is split by ROW over all blocks: with sentinel-validated data any block may
// push any row (no block-to-block pairing as on the flag-barrier path), so mid-sized messages use
// tokens blocks instead of tokens / N.
template <typename T, int kVpt>
__device__ __forceinline__ void twoshot_scatter_rows(const ArParams& p, const RowView<T, kVpt>& rv,
                                                     const TwoShotGeometry& g, int nranks, size_t area_off) {
  const char* in = static_cast<const char*>(p.in);
  for (int row = blockIdx.x; row < p.tokens; row += gridDim.x) {
    const int r = row % nranks, j = row / nranks;
    if (r == p.rank) continue;
    const size_t dst_off = area_off + ((size_t)p.rank * g.groups + j) * rv.row_bytes;
#pragma unroll
    for (int v = 0; v < kVpt; ++v) {
      if (!rv.active(v)) continue;
      const uint4 val = scrub(ptx::ld_stream_v4(in + (size_t)row * rv.row_bytes + (size_t)rv.vec_index(v) * 16));
      ptx::st_v4(symm(p, r, dst_off + (size_t)rv.vec_index(v) * 16), val);
    }
  }
}

// ---- two-shot Lamport -------------------------------------------------------------------

// Owner and receive phases of the two-shot Lamport flow for the row groups cta, cta + nctas, ...
// kOwnFromBuffer: this rank's own partial row is polled from its gather slot like the peers'
// (used when the partial rows are produced by a GEMM epilogue instead of being an input tensor).
// Returns the number of bytes of the Lamport buffer that hold data after this call.
// kMc: finished rows and their trailers leave the owner as one multimem.st each, replicated by NVSwitch into every
// rank's result area (the owner's own included, which it never reads).
template <typename T, int kN, int kVpt, int kOut, bool kOwnFromBuffer, bool kMc = false>
__device__ __forceinline__ uint64_t twoshot_lamport_tail(const ArParams& p, int cta, int nctas, uint32_t epoch,
                                                         float (*red)[32]) {
  constexpr int kVec = VecTraits<T>::kVec;
  const int nranks = kN > 0 ? kN : p.nranks;
  const RowView<T, kVpt> rv(p.hidden);
  char* self = static_cast<char*>(p.peer[p.rank]);
  Control* ctl = reinterpret_cast<Control*>(self + p.layout.off_control);
  const TwoShotGeometry g = twoshot_geometry<T, kVpt>(p, rv, nranks, true);
  const size_t buf_off = p.layout.off_lamport + (size_t)(epoch % 3u) * p.layout.lamport_bytes;
  const size_t result_off = buf_off + g.gather_bytes;
  const char* in = static_cast<const char*>(p.in);
  const bool gather_back = p.scatter_only == 0;

  uint4 gamma[kVpt];
  load_gamma<T, kVpt>(p, rv, gamma);
  Waiter w(p.timeout_ns);
  int parity = 0;

  // owner phase: rows j*N + rank
  for (int j = cta; j < g.groups; j += nctas) {
    const int row = j * nranks + p.rank;
    if (row >= p.tokens) continue;
    const int64_t out_row = gather_back ? row : j;
    float x[kVpt][kVec];
    uint4 packed[kVpt];
    uint4 res[kVpt];
    request_residual<T, kVpt>(p, rv, out_row, res);
#pragma unroll
    for (int v = 0; v < kVpt; ++v) {
#pragma unroll
      for (int i = 0; i < kVec; ++i) x[v][i] = 0.f;
      packed[v] = make_uint4(0, 0, 0, 0);
      if (!rv.active(v)) continue;
      const size_t voff = (size_t)rv.vec_index(v) * 16;
      const char* slot0 = self + buf_off + (size_t)j * rv.row_bytes + voff;
      const size_t slot_stride = (size_t)g.groups * rv.row_bytes;
      if constexpr (kN > 0) {
        uint4 vals[kN];
#pragma unroll
        for (int r = 0; r < kN; ++r)
          vals[r] = (!kOwnFromBuffer && r == p.rank) ? ptx::ld_stream_v4(in + (size_t)row * rv.row_bytes + voff)
                                                     : ptx::ld_volatile_v4(slot0 + r * slot_stride);
#pragma unroll
        for (int r = 0; r < kN; ++r)
          if ((kOwnFromBuffer || r != p.rank) && !all_arrived(vals[r]))
            vals[r] = poll_vec(slot0 + r * slot_stride, w, p, ctl, kTimeoutLamportGather, r, 1, row);
#pragma unroll
        for (int r = 0; r < kN; ++r) {
          float f[kVec];
          unpack<T>(vals[r], f);
#pragma unroll
          for (int i = 0; i < kVec; ++i) x[v][i] += f[i];
        }
      } else {
        for (int r = 0; r < nranks; ++r) {
          const uint4 val = (!kOwnFromBuffer && r == p.rank)
                                ? ptx::ld_stream_v4(in + (size_t)row * rv.row_bytes + voff)
                                : poll_vec(slot0 + r * slot_stride, w, p, ctl, kTimeoutLamportGather, r, 1, row);
          float f[kVec];
          unpack<T>(val, f);
#pragma unroll
          for (int i = 0; i < kVec; ++i) x[v][i] += f[i];
        }
      }
      add_residual_loaded<T>(x[v], p.residual_in != nullptr, res[v]);
      packed[v] = scrub(pack<T>(x[v]));
      unpack<T>(packed[v], x[v]);
      if (p.residual_out)
        ptx::st_stream_v4(static_cast<char*>(p.residual_out) + (size_t)out_row * rv.row_bytes + voff, packed[v]);
      if (gather_back) {
        if constexpr (kMc) {
          ptx::multimem_st_v4(symm_mc(p, result_off + (size_t)row * g.result_stride + voff), packed[v]);
        } else {
#pragma unroll
          for (int r = 0; r < (kN > 0 ? kN : kMaxRanks); ++r) {
            if (r >= nranks || r == p.rank) continue;
            ptx::st_v4(symm(p, r, result_off + (size_t)row * g.result_stride + voff), packed[v]);
          }
        }
      }
    }
    trace_mark(p, kTraceGathered);
    float rstd, sc;
    finish_row<T, kVpt, kOut>(p, rv, out_row, x, gamma, red, parity, rstd, sc);
    parity ^= 1;
    if (gather_back) {
      const uint4 trailer = make_uint4(__float_as_uint(rstd), __float_as_uint(sc), 0u, 0u);
      if constexpr (kMc) {
        if (threadIdx.x == 0) ptx::multimem_st_v4(symm_mc(p, result_off + (size_t)row * g.result_stride + rv.row_bytes), trailer);
      } else if (threadIdx.x < nranks && (int)threadIdx.x != p.rank) {
        ptx::st_v4(symm(p, threadIdx.x, result_off + (size_t)row * g.result_stride + rv.row_bytes), trailer);
      }
    }
    trace_mark(p, kTraceOwnerDone);
  }

  // receive phase: rows owned by the peers, split by row over all blocks
  if (gather_back) {
    for (int row = cta; row < p.tokens; row += nctas) {
      const int r = row % nranks;
      if (r == p.rank) continue;
      {
        const char* src = self + result_off + (size_t)row * g.result_stride;
        const uint4 trailer = poll_vec(src + rv.row_bytes, w, p, ctl, kTimeoutLamportResult, r, 2, row);
        trace_mark(p, kTraceTrailer);
        const float rstd = __uint_as_float(trailer.x);
        const float sc = __uint_as_float(trailer.y);
        float x[kVpt][kVec];
#pragma unroll
        for (int v = 0; v < kVpt; ++v) {
#pragma unroll
          for (int i = 0; i < kVec; ++i) x[v][i] = 0.f;
          if (!rv.active(v)) continue;
          const size_t voff = (size_t)rv.vec_index(v) * 16;
          const uint4 val = poll_vec(src + voff, w, p, ctl, kTimeoutLamportResult, r, 2, row);
          unpack<T>(val, x[v]);
          if (p.residual_out)
            ptx::st_stream_v4(static_cast<char*>(p.residual_out) + (size_t)row * rv.row_bytes + voff, val);
        }
        trace_mark(p, kTraceReceived);
        if (kOut == kOutFp8Token && threadIdx.x == 0) p.scale_out[row] = sc;
        store_norm<T, kVpt, kOut>(p, rv, row, x, gamma, rstd, sc);
      }
    }
  }
  return g.gather_bytes + (gather_back ? (uint64_t)p.tokens * g.result_stride : 0);
}

template <typename T, int kN, int kVpt, int kOut, bool kMc = false>
__device__ __forceinline__ void twoshot_lamport_body(const ArParams& p) {
  __shared__ float red[4][32];
  const int nranks = kN > 0 ? kN : p.nranks;
  const RowView<T, kVpt> rv(p.hidden);
  char* self = static_cast<char*>(p.peer[p.rank]);
  Control* ctl = reinterpret_cast<Control*>(self + p.layout.off_control);
  const uint32_t epoch = ctl->lamport_epoch;
  const uint64_t dirty_prev = ctl->lamport_dirty[(epoch + 2u) % 3u];
  const TwoShotGeometry g = twoshot_geometry<T, kVpt>(p, rv, nranks, true);
  const size_t buf_off = p.layout.off_lamport + (size_t)(epoch % 3u) * p.layout.lamport_bytes;

  twoshot_scatter_rows<T, kVpt>(p, rv, g, nranks, buf_off);
  trace_mark(p, kTracePushed);
  clear_previous(lamport_buf(self, p.layout, (epoch + 2u) % 3u), dirty_prev);
  trace_mark(p, kTraceCleared);
  const uint64_t dirty = twoshot_lamport_tail<T, kN, kVpt, kOut, false, kMc>(p, blockIdx.x, gridDim.x, epoch, red);
  trace_mark(p, kTraceEndClk);
  trace_mark_ns(p, kTraceEndNs);
  finish_launch(ctl, true, epoch, dirty, 0);
}

// ---- two-shot with flag barriers (peer-to-peer staging or NVLS), pipelined in waves -------------
// Block b of every rank handles the row groups b, b + gridDim, ... . They can be processed in up to
// kMaxWaves waves (ArParams::waves, default 1) so that the three phases of different waves overlap in
// time: while one wave's finished rows are normalised locally, the next wave's partial rows already
// cross the links. Measured at 2 ranks every extra wave costs more in flag round trips (two per wave)
// than the overlap returns, so one wave is the default. Per wave w (flag values are epoch + w + 1; plane 0 = "gathered", plane 1 = "results"):
//     stage(w+1), signal(plane 0)   |  wait(plane 0, w)  reduce(w) + publish, signal(plane 1)
//                                   |  wait(plane 1, w)  epilogue(w)
// kNvls = false: stage = push my rows to their owners' gather slots; reduce reads them locally;
//                publish = peer stores into every rank's result area.
// kNvls = true : stage = copy my rows into my multicast-bound input buffer; reduce =
//                multimem.ld_reduce (the switch adds); publish = multimem.st (the switch replicates).
// The last wave's plane-1 wait also keeps a fast rank's next call from overwriting slots that a
// slow rank is still reading.
constexpr int kMaxWaves = 4;

template <typename T>
__device__ __forceinline__ uint4 mc_ld_reduce(const void* mc_addr) {
  if constexpr (sizeof(T) == 4) return ptx::multimem_ld_reduce_f32x4(mc_addr);
  else if constexpr (VecTraits<T>::kDType == kF16) return ptx::multimem_ld_reduce_f16x8(mc_addr);
  else return ptx::multimem_ld_reduce_bf16x8(mc_addr);
}

__device__ __forceinline__ size_t nvls_in_offset(const Layout& l, uint32_t bepoch) {
  return l.off_nvls + (size_t)(bepoch & 1u) * l.nvls_in_bytes;
}

template <typename T, int kN, int kVpt, int kOut, bool kNvls>
__device__ __forceinline__ void twoshot_flag_body(const ArParams& p) {
  constexpr int kVec = VecTraits<T>::kVec;
  __shared__ float red[4][32];
  const int nranks = kN > 0 ? kN : p.nranks;
  const RowView<T, kVpt> rv(p.hidden);
  char* self = static_cast<char*>(p.peer[p.rank]);
  Control* ctl = reinterpret_cast<Control*>(self + p.layout.off_control);
  const uint32_t bepoch = ctl->barrier_epoch;
  const TwoShotGeometry g = twoshot_geometry<T, kVpt>(p, rv, nranks, false);
  // staging: gather slots [src][group][hidden] (peer-to-peer) or my rows in natural order (NVLS)
  const size_t stage_off = kNvls ? nvls_in_offset(p.layout, bepoch) : p.layout.off_stage;
  // The result area sits at an offset that does not depend on the message: the epilogue reads it after the last
  // wait of the call, so a peer that runs ahead into a LARGER call must find its gather slots (pushed before any
  // wait) clear of the rows that a slower rank is still reading.
  const size_t result_off = kNvls ? p.layout.off_nvls + 2 * p.layout.nvls_in_bytes : p.layout.off_stage + p.layout.stage_bytes / 2;
  const char* in = static_cast<const char*>(p.in);
  const bool gather_back = p.scatter_only == 0;
  Waiter w(p.timeout_ns);

  // waves: the same count on every block and rank (derived from the largest per-block group count)
  const int per_block = (g.groups + gridDim.x - 1) / gridDim.x;
  const int want = p.waves < 1 ? 1 : (p.waves > kMaxWaves ? kMaxWaves : p.waves);
  const int waves = per_block < want ? (per_block > 0 ? per_block : 1) : want;
  const int wave_len = (per_block + waves - 1) / waves;

  auto stage_wave = [&](int wv) {
    for (int k = wv * wave_len; k < (wv + 1) * wave_len && k < per_block; ++k) {
      const int j = blockIdx.x + k * gridDim.x;
      if (j >= g.groups) break;
#pragma unroll
      for (int r = 0; r < (kN > 0 ? kN : kMaxRanks); ++r) {
        const int row = j * nranks + r;
        if (r >= nranks || row >= p.tokens) continue;
        if (!kNvls && r == p.rank) continue;
        const int dst_rank = kNvls ? p.rank : r;
        const size_t dst_off = kNvls ? stage_off + (size_t)row * rv.row_bytes
                                     : stage_off + ((size_t)p.rank * g.groups + j) * rv.row_bytes;
#pragma unroll
        for (int v = 0; v < kVpt; ++v) {
          if (!rv.active(v)) continue;
          const size_t voff = (size_t)rv.vec_index(v) * 16;
          ptx::st_v4(symm(p, dst_rank, dst_off + voff), ptx::ld_stream_v4(in + (size_t)row * rv.row_bytes + voff));
        }
      }
    }
  };

  uint4 gamma[kVpt];
  load_gamma<T, kVpt>(p, rv, gamma);
  int parity = 0;

  stage_wave(0);
  flag_signal(p, 0, bepoch + 1u);
  for (int wv = 0; wv < waves; ++wv) {
    if (wv + 1 < waves) {
      stage_wave(wv + 1);
      flag_signal(p, 0, bepoch + (uint32_t)wv + 2u);
    }
    flag_wait(p, ctl, 0, bepoch + (uint32_t)wv + 1u, w, 1);

    // ---- reduce + publish the rows this rank owns in this wave ----
    // NVLS: the switch-side sums of up to `batch` rows are requested before the first of them is
    // consumed. A multimem.ld_reduce takes several microseconds to come back, and one 16-byte
    // request per thread does not keep the links busy (`nvls_batch`, default 1 = one row at a time).
    constexpr int kMaxBatch = kNvls ? (kVpt == 1 ? 4 : (kVpt == 2 ? 2 : 1)) : 1;
    const int batch = !kNvls || p.nvls_batch < 1 ? 1 : (p.nvls_batch > kMaxBatch ? kMaxBatch : p.nvls_batch);
    const int k_end = min((wv + 1) * wave_len, per_block);
    for (int k0 = wv * wave_len; k0 < k_end; k0 += batch) {
      uint4 pre[kMaxBatch][kVpt];
      if constexpr (kNvls) {
#pragma unroll
        for (int b = 0; b < kMaxBatch; ++b) {
          const int j = blockIdx.x + (k0 + b) * gridDim.x;
          const int row = j * nranks + p.rank;
          if (b < batch && k0 + b < k_end && j < g.groups && row < p.tokens) {
#pragma unroll
            for (int v = 0; v < kVpt; ++v)
              if (rv.active(v))
                pre[b][v] = mc_ld_reduce<T>(static_cast<const char*>(p.mc_base) + stage_off + (size_t)row * rv.row_bytes +
                                            (size_t)rv.vec_index(v) * 16);
          }
        }
      }
#pragma unroll
      for (int b = 0; b < kMaxBatch; ++b) {
        const int k = k0 + b;
        if (b >= batch || k >= k_end) continue;
        const int j = blockIdx.x + k * gridDim.x;
        if (j >= g.groups) continue;
        const int row = j * nranks + p.rank;
        if (row >= p.tokens) continue;
        const int64_t out_row = gather_back ? row : j;
        float x[kVpt][kVec];
#pragma unroll
        for (int v = 0; v < kVpt; ++v) {
#pragma unroll
          for (int i = 0; i < kVec; ++i) x[v][i] = 0.f;
          if (!rv.active(v)) continue;
          const size_t voff = (size_t)rv.vec_index(v) * 16;
          if constexpr (kNvls) {
            unpack<T>(pre[b][v], x[v]);
          } else {
            const char* slot0 = self + stage_off + (size_t)j * rv.row_bytes + voff;
            const size_t slot_stride = (size_t)g.groups * rv.row_bytes;
#pragma unroll
            for (int r = 0; r < (kN > 0 ? kN : kMaxRanks); ++r) {
              if (r >= nranks) continue;
              const uint4 val = (r == p.rank) ? ptx::ld_stream_v4(in + (size_t)row * rv.row_bytes + voff)
                                              : ptx::ld_volatile_v4(slot0 + r * slot_stride);
              float f[kVec];
              unpack<T>(val, f);
#pragma unroll
              for (int i = 0; i < kVec; ++i) x[v][i] += f[i];
            }
          }
          add_residual<T>(x[v], p.residual_in ? static_cast<const char*>(p.residual_in) +
                                                    (size_t)out_row * rv.row_bytes + voff
                                              : nullptr);
          const uint4 packed = pack<T>(x[v]);
          if (p.residual_out)
            ptx::st_stream_v4(static_cast<char*>(p.residual_out) + (size_t)out_row * rv.row_bytes + voff, packed);
          if (gather_back) {
            if constexpr (kNvls) {
              // one store, replicated by the switch into every rank's result area
              ptx::multimem_st_v4(static_cast<char*>(p.mc_base) + result_off + (size_t)row * rv.row_bytes + voff, packed);
            } else {
#pragma unroll
              for (int r = 0; r < (kN > 0 ? kN : kMaxRanks); ++r) {
                if (r >= nranks || r == p.rank) continue;
                ptx::st_v4(symm(p, r, result_off + (size_t)row * rv.row_bytes + voff), packed);
              }
            }
          }
        }
        float rstd, sc;
        finish_row<T, kVpt, kOut>(p, rv, out_row, x, gamma, red, parity, rstd, sc);
        parity ^= 1;
        if (gather_back) {
          const uint4 trailer = make_uint4(__float_as_uint(rstd), __float_as_uint(sc), 0u, 0u);
          if constexpr (kNvls) {
            if (threadIdx.x == 0)
              ptx::multimem_st_v4(static_cast<char*>(p.mc_base) + result_off + g.trailer_off + (size_t)row * 16, trailer);
          } else if (threadIdx.x < nranks && (int)threadIdx.x != p.rank) {
            ptx::st_v4(symm(p, threadIdx.x, result_off + g.trailer_off + (size_t)row * 16), trailer);
          }
        }
      }
    }
    flag_signal(p, 1, bepoch + (uint32_t)wv + 1u);
    flag_wait(p, ctl, 1, bepoch + (uint32_t)wv + 1u, w, 2);

    // ---- epilogue of the rows the peers own in this wave ----
    if (gather_back) {
      for (int k = wv * wave_len; k < (wv + 1) * wave_len && k < per_block; ++k) {
        const int j = blockIdx.x + k * gridDim.x;
        if (j >= g.groups) break;
        for (int r = 0; r < nranks; ++r) {
          const int row = j * nranks + r;
          if (r == p.rank || row >= p.tokens) continue;
          const char* src = self + result_off + (size_t)row * rv.row_bytes;
          const uint4 trailer = ptx::ld_volatile_v4(self + result_off + g.trailer_off + (size_t)row * 16);
          const float rstd = __uint_as_float(trailer.x);
          const float sc = __uint_as_float(trailer.y);
          float x[kVpt][kVec];
#pragma unroll
          for (int v = 0; v < kVpt; ++v) {
#pragma unroll
            for (int i = 0; i < kVec; ++i) x[v][i] = 0.f;
            if (!rv.active(v)) continue;
            const size_t voff = (size_t)rv.vec_index(v) * 16;
            const uint4 val = ptx::ld_volatile_v4(src + voff);
            unpack<T>(val, x[v]);
            if (p.residual_out)
              ptx::st_stream_v4(static_cast<char*>(p.residual_out) + (size_t)row * rv.row_bytes + voff, val);
          }
          if (kOut == kOutFp8Token && threadIdx.x == 0) p.scale_out[row] = sc;
          store_norm<T, kVpt, kOut>(p, rv, row, x, gamma, rstd, sc);
        }
      }
    }
  }
  // every plane was used with values up to epoch + waves (other kernels use up to epoch + 2 on plane 0)
  finish_launch(ctl, false, 0, 0, waves > 2 ? waves : 2);
}

template <typename T, int kN, int kVpt, int kOut>
__device__ __forceinline__ void twoshot_barrier_body(const ArParams& p) {
  twoshot_flag_body<T, kN, kVpt, kOut, false>(p);
}

// ---- NVLS (NVSwitch multicast) ---------------------------------------------------------------
// Every rank's symmetric allocation is bound to one multicast object; `mc_base` addresses all
// copies at once. multimem.ld_reduce returns the sum over ranks computed inside the switch
// (fp32 accumulation for 16-bit types, one rounding to T; the order of the additions is the
// switch's). The input is first copied into the NVLS staging buffer selected by the parity of the
// barrier epoch, so that a rank that runs ahead never overwrites data a peer is still reducing.

template <typename T, int kVpt>
__device__ __forceinline__ void nvls_copy_in_row(const ArParams& p, const RowView<T, kVpt>& rv, char* dst_base, int row) {
  const char* in = static_cast<const char*>(p.in);
#pragma unroll
  for (int v = 0; v < kVpt; ++v) {
    if (!rv.active(v)) continue;
    const size_t off = (size_t)row * rv.row_bytes + (size_t)rv.vec_index(v) * 16;
    ptx::st_v4(dst_base + off, ptx::ld_stream_v4(in + off));
  }
}

template <typename T, int kN, int kVpt, int kOut>
__device__ __forceinline__ void nvls_oneshot_body(const ArParams& p) {
  constexpr int kVec = VecTraits<T>::kVec;
  __shared__ float red[4][32];
  const RowView<T, kVpt> rv(p.hidden);
  char* self = static_cast<char*>(p.peer[p.rank]);
  Control* ctl = reinterpret_cast<Control*>(self + p.layout.off_control);
  const uint32_t bepoch = ctl->barrier_epoch;
  const size_t in_off = nvls_in_offset(p.layout, bepoch);
  Waiter w(p.timeout_ns);

  for (int row = blockIdx.x; row < p.tokens; row += gridDim.x) nvls_copy_in_row<T, kVpt>(p, rv, self + in_off, row);
  flag_barrier(p, ctl, bepoch + 1u, w, 1);

  uint4 gamma[kVpt];
  load_gamma<T, kVpt>(p, rv, gamma);
  const char* mc_in = static_cast<const char*>(p.mc_base) + in_off;
  int parity = 0;
  for (int row = blockIdx.x; row < p.tokens; row += gridDim.x, parity ^= 1) {
    float x[kVpt][kVec];
#pragma unroll
    for (int v = 0; v < kVpt; ++v) {
#pragma unroll
      for (int i = 0; i < kVec; ++i) x[v][i] = 0.f;
      if (!rv.active(v)) continue;
      const size_t off = (size_t)row * rv.row_bytes + (size_t)rv.vec_index(v) * 16;
      unpack<T>(mc_ld_reduce<T>(mc_in + off), x[v]);
      add_residual<T>(x[v], p.residual_in ? static_cast<const char*>(p.residual_in) + off : nullptr);
      if (p.residual_out) ptx::st_stream_v4(static_cast<char*>(p.residual_out) + off, pack<T>(x[v]));
    }
    float rstd, sc;
    finish_row<T, kVpt, kOut>(p, rv, row, x, gamma, red, parity, rstd, sc);
  }
  finish_launch(ctl, false, 0, 0, 1);
}

template <typename T, int kN, int kVpt, int kOut>
__device__ __forceinline__ void nvls_twoshot_body(const ArParams& p) {
  twoshot_flag_body<T, kN, kVpt, kOut, true>(p);
}

// ---- kernel wrappers ---------------------------------------------------------------------

template <typename T, int kAlgo, int kN, int kVpt, int kOut>
__device__ __forceinline__ void ar_dispatch_body(const ArParams& p) {
  if constexpr (kAlgo == kAlgoLocal) local_body<T, kVpt, kOut>(p);
  else if constexpr (kAlgo == kAlgoOneShotLamport) oneshot_lamport_body<T, kN, kVpt, kOut>(p);
  else if constexpr (kAlgo == kAlgoTwoShotLamport) twoshot_lamport_body<T, kN, kVpt, kOut>(p);
  else if constexpr (kAlgo == kAlgoTwoShotBarrier) twoshot_barrier_body<T, kN, kVpt, kOut>(p);
  else if constexpr (kAlgo == kAlgoNvlsOneShot) nvls_oneshot_body<T, kN, kVpt, kOut>(p);
  else if constexpr (kAlgo == kAlgoNvlsTwoShot) nvls_twoshot_body<T, kN, kVpt, kOut>(p);
  else if constexpr (kAlgo == kAlgoOneShotMc) oneshot_lamport_body<T, kN, kVpt, kOut, true>(p);
  else if constexpr (kAlgo == kAlgoTwoShotMc) twoshot_lamport_body<T, kN, kVpt, kOut, true>(p);
}

// kVpt == 1 kernels may run with up to 1024 threads (64 registers); wider rows use at most
// 512 threads with 2 or 4 vectors each and may use up to 128 registers.
template <int kVpt>
constexpr int kMaxThreadsFor = (kVpt == 1) ? 1024 : 512;

template <typename T, int kAlgo, int kN, int kVpt, int kOut>
__global__ void __launch_bounds__(kMaxThreadsFor<kVpt>, 1) ar_fused_kernel(const __grid_constant__ ArParams p) {
  // Launched with programmatic stream serialisation (ar_fusion_inst.cu), the blocks of this kernel are scheduled
  // while the previous kernel of the stream still runs, and wait here until it has completed and its memory
  // is visible; the next kernel may then be scheduled in the same way. A plain launch passes straight through.
  ptx::pdl_wait();
  ptx::pdl_launch_dependents();
  trace_mark_ns(p, kTraceStartNs);
  trace_mark(p, kTraceStartClk);
  ar_dispatch_body<T, kAlgo, kN, kVpt, kOut>(p);
}

// All ranks in one cooperative launch on one GPU; blockIdx.y selects the rank.
template <typename T, int kAlgo, int kN, int kVpt, int kOut>
__global__ void __launch_bounds__(kMaxThreadsFor<kVpt>, 1) ar_fused_kernel_emu(const ArParams* __restrict__ ranks) {
  ar_dispatch_body<T, kAlgo, kN, kVpt, kOut>(ranks[blockIdx.y]);
}

}  // namespace tdx
