// Causal self-attention for the prompt phase on the tensor cores (tcgen05 / TMEM), head dimension 128,
// bf16, grouped-query heads. One CTA owns 128 consecutive query positions of one query head and walks
// the key/value positions 0 .. (its last query) in chunks of 128:
//
//   S[q 128, keys 128] = Q[q, d] * K[keys, d]^T        both operands K-major, as TMA delivers them
//   O[q 128, d 128]   += P[q, keys] * V[keys, d]        P written by the softmax warps (K-major over keys),
//                                                       V read MN-major (d contiguous) straight from its TMA tile
//
// Eight softmax warps: two threads per query row, one per 64-key half of a chunk (so that every warp
// scheduler has two of them to alternate between); the two halves exchange their partial row maxima
// through shared memory once per chunk. A thread fetches its 64 scores of a chunk with ONE tcgen05.ld
// (one TMEM round trip per chunk) and gives the score buffer back at once; S is double-buffered, so the
// scores of chunk c+1 are computed while chunk c is in the softmax. O stays in tensor memory and is
// accumulated there by the P*V products of all chunks. A row's running maximum is only raised - and its part of O rescaled in
// tensor memory - when the new maximum exceeds it by more than 2^8 (a warp-uniform decision); until
// then the probabilities are taken against the older maximum, which changes neither O / l nor the
// accuracy of bf16 probabilities below 256. A ninth warp issues the TMA copies (separate rings for
// K, 2 stages, freed as soon as the scores are computed, and V, 3 stages, freed after P*V) and all MMAs.
//
// Every wait is bounded; a wait that runs out records a status word and raises the CTA's abort flag,
// and all threads still reach the common exit. Not part of the reference (it has no attention).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cfloat>
#include <mutex>
#include <set>
#include <string>
#include "tdx/comm.h"
#include "tdx/launch.h"
#include "tdx/ops.h"
#include "tdx/ptx.cuh"
#include "tdx/tc.cuh"
#include "tdx/tma_host.h"

namespace tdx {
namespace {

constexpr int kD = 128;
constexpr int kRows = 128;                        // query rows per CTA = key positions per chunk
constexpr int kStagesK = 2;
constexpr int kStagesV = 3;
constexpr int kSoftmaxThreads = 256;          // two warp groups: 64 key positions of every chunk each
constexpr int kHalfKeys = 64;
constexpr int kThreads = kSoftmaxThreads + 32;
constexpr int kMmaWarp = kSoftmaxThreads / 32;
constexpr int kHalfBytes = kRows * 128;           // one 64-column half of a 128-row tile
constexpr int kTileBytes = 2 * kHalfBytes;        // Q, P, one K chunk or one V chunk
constexpr int kNumBarriers = 2 * kStagesK + 2 * kStagesV + 4 + 3;   // k/v full+free, s full+free [2], q_full, p_full, o_full
constexpr int kBarrierBytes = 256;                // the mbarriers, the TMEM address and the abort flag
static_assert(kNumBarriers * 8 + 8 <= kBarrierBytes, "barrier area too small");
constexpr int kSmem = (kStagesK + kStagesV + 2) * kTileBytes + kBarrierBytes + 2 * 2 * kRows * (int)sizeof(float);
static_assert(kSmem <= 227 * 1024, "shared memory of one CTA");
constexpr uint32_t kTmemCols = 512;               // S buffers at columns 0 and 128, O at 256
constexpr uint32_t kColO = 256;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr float kRescaleThreshold = 8.f;          // log2 units

struct PrefillArgs {
  __nv_bfloat16* out;          // [S, Hq, D] contiguous
  int S, Hq, Hkv;
  float scale_log2;            // softmax scale * log2(e)
  uint32_t idesc_s, idesc_pv;
  uint32_t* status;
};

__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const PrefillArgs a) {
  // The tiles need 1024-byte alignment (128-byte swizzle) and fill the shared memory of the SM to within a
  // kilobyte, so there is no room for alignment slack: the dynamic region is declared aligned, and a kernel
  // that finds it otherwise reports that instead of running.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if ((tc::smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0 && a.status) atomicExch(a.status, (uint32_t)kTimeoutGemmPipeline);
    return;
  }
  uint8_t* k_ring = smem_raw;
  uint8_t* v_ring = k_ring + kStagesK * kTileBytes;
  uint8_t* q_tile = v_ring + kStagesV * kTileBytes;
  uint8_t* p_tile = q_tile + kTileBytes;
  uint64_t* k_full = reinterpret_cast<uint64_t*>(p_tile + kTileBytes);
  uint64_t* k_free = k_full + kStagesK;
  uint64_t* v_full = k_free + kStagesK;
  uint64_t* v_free = v_full + kStagesV;
  uint64_t* s_full = v_free + kStagesV;     // [2]
  uint64_t* s_free = s_full + 2;            // [2]
  uint64_t* q_full = s_free + 2;
  uint64_t* p_full = q_full + 1;
  uint64_t* o_full = p_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  // partial row maxima (and, at the end, sums) of the two warp groups: [chunk parity][warp group][row]
  float (*xmax)[2][kRows] = reinterpret_cast<float (*)[2][kRows]>(p_tile + kTileBytes + kBarrierBytes);

  // the blocks with the most key chunks start first
  const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int h = blockIdx.y;
  const int hkv = h / (a.Hq / a.Hkv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int q0 = qb * kRows;
  const int nchunks = qb + 1;               // key positions 0 .. q0 + 127 (causal)

  if (tid == 0) {
    for (int s = 0; s < kStagesK; ++s) {
      tc::mbar_init(&k_full[s], 1);
      tc::mbar_init(&k_free[s], 1);
    }
    for (int s = 0; s < kStagesV; ++s) {
      tc::mbar_init(&v_full[s], 1);
      tc::mbar_init(&v_free[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&s_full[i], 1);
      tc::mbar_init(&s_free[i], kSoftmaxThreads);
    }
    tc::mbar_init(q_full, 1);
    tc::mbar_init(p_full, kSoftmaxThreads);
    tc::mbar_init(o_full, 1);
    *abort_flag = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_desc(&map_q);
    tc::tma_prefetch_desc(&map_k);
    tc::tma_prefetch_desc(&map_v);
  }
  if (warp == kMmaWarp) {
    tc::tmem_alloc(tmem_slot, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::fence_before_thread_sync();
  __syncthreads();
  tc::fence_after_thread_sync();
  const uint32_t tmem_base = *tmem_slot;
  ptx::pdl_wait();                // q, k and v come from earlier kernels of the stream
  ptx::pdl_launch_dependents();

  auto fail = [&]() {
    *abort_flag = 1;
    if (a.status) atomicExch(a.status, (uint32_t)kTimeoutGemmPipeline);
  };

  if (warp == kMmaWarp) {
    if (lane == 0) {
      // ---- copies and MMAs ----
      auto load_k = [&](int c) {
        uint8_t* base = k_ring + (c % kStagesK) * kTileBytes;
        tc::mbar_arrive_expect_tx(&k_full[c % kStagesK], kTileBytes);
        tc::tma_load_3d(base, &map_k, &k_full[c % kStagesK], 0, hkv, c * kRows);
        tc::tma_load_3d(base + kHalfBytes, &map_k, &k_full[c % kStagesK], 64, hkv, c * kRows);
      };
      auto load_v = [&](int c) {
        uint8_t* base = v_ring + (c % kStagesV) * kTileBytes;
        tc::mbar_arrive_expect_tx(&v_full[c % kStagesV], kTileBytes);
        tc::tma_load_3d(base, &map_v, &v_full[c % kStagesV], 0, hkv, c * kRows);
        tc::tma_load_3d(base + kHalfBytes, &map_v, &v_full[c % kStagesV], 64, hkv, c * kRows);
      };
      auto issue_scores = [&](int c) {   // S[buf c & 1] = Q * K chunk^T; the K stage is free once these complete
        const uint32_t kbase = tc::smem_u32(k_ring + (c % kStagesK) * kTileBytes);
        const uint32_t qbase = tc::smem_u32(q_tile);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            tc::umma<false>(tmem_base + (uint32_t)(c & 1) * kRows, tc::make_smem_desc_sw128(qbase + kb * kHalfBytes) + (uint64_t)(ks * 2),
                            tc::make_smem_desc_sw128(kbase + kb * kHalfBytes) + (uint64_t)(ks * 2), a.idesc_s, (kb | ks) ? 1u : 0u);
        tc::umma_commit(&s_full[c & 1]);
        tc::umma_commit(&k_free[c % kStagesK]);
      };
      auto issue_pv = [&](int c) {       // O (+)= P * V chunk, 16 key positions per instruction
        const uint32_t vbase = tc::smem_u32(v_ring + (c % kStagesV) * kTileBytes);
        const uint32_t pbase = tc::smem_u32(p_tile);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          tc::umma<false>(tmem_base + kColO, tc::make_smem_desc_sw128(pbase + (j >> 2) * kHalfBytes) + (uint64_t)((j & 3) * 2),
                          tc::make_smem_desc_mn_sw128(vbase + j * 2048, kHalfBytes), a.idesc_pv, (c | j) ? 1u : 0u);
        tc::umma_commit(o_full);
        tc::umma_commit(&v_free[c % kStagesV]);
      };
      tc::mbar_arrive_expect_tx(q_full, kTileBytes);
      tc::tma_load_3d(q_tile, &map_q, q_full, 0, h, q0);
      tc::tma_load_3d(q_tile + kHalfBytes, &map_q, q_full, 64, h, q0);
      for (int c = 0; c < nchunks && c < kStagesK; ++c) load_k(c);
      for (int c = 0; c < nchunks && c < kStagesV; ++c) load_v(c);
      bool ok = tc::mbar_wait(q_full, 0, kWaitLimit, abort_flag) && tc::mbar_wait(&k_full[0], 0, kWaitLimit, abort_flag);
      if (ok) {
        tc::fence_after_thread_sync();
        issue_scores(0);
      }
      for (int i = 0; i < nchunks && ok; ++i) {
        if (i + 1 < nchunks) {
          // scores of the next chunk: its K tile has landed and the softmax has taken chunk i - 1 out of the buffer
          const int n = i + 1;
          ok = tc::mbar_wait(&k_full[n % kStagesK], (n / kStagesK) & 1, kWaitLimit, abort_flag) &&
               (n < 2 || tc::mbar_wait(&s_free[n & 1], ((n >> 1) - 1) & 1, kWaitLimit, abort_flag));
          if (!ok) break;
          tc::fence_after_thread_sync();
          issue_scores(n);
        }
        if (i + kStagesK < nchunks) {
          // K stage of chunk i is free once its scores are complete (long before P*V of the chunk)
          ok = tc::mbar_wait(&k_free[i % kStagesK], (i / kStagesK) & 1, kWaitLimit, abort_flag);
          if (!ok) break;
          load_k(i + kStagesK);
        }
        if (i >= 1 && i - 1 + kStagesV < nchunks) {
          // V stage of chunk i - 1 is free once its P*V product is complete
          ok = tc::mbar_wait(&v_free[(i - 1) % kStagesV], ((i - 1) / kStagesV) & 1, kWaitLimit, abort_flag);
          if (!ok) break;
          load_v(i - 1 + kStagesV);
        }
        ok = tc::mbar_wait(p_full, i & 1, kWaitLimit, abort_flag) &&
             tc::mbar_wait(&v_full[i % kStagesV], (i / kStagesV) & 1, kWaitLimit, abort_flag);
        if (!ok) break;
        tc::fence_after_thread_sync();
        issue_pv(i);
      }
      if (!ok) fail();
    }
  } else {
    // ---- softmax warps: two threads per query row, one per 64-key half of a chunk ----
    // Thread (wg, t): row q0 + t, keys [64 wg, 64 wg + 64) of every chunk and columns [64 wg, 64 wg + 64) of O.
    // Both warp groups reach all 128 TMEM lanes (a warp addresses the lane quarter warp % 4). The two threads
    // of a row exchange their partial row maxima through shared memory once per chunk (one named barrier among
    // the 256 softmax threads; the exchange buffer alternates with the chunk parity, so no second barrier is
    // needed) and therefore take identical decisions on the running maximum. A thread whose wait ran out keeps
    // walking the loop (its waits return at once because the abort flag is up) so that every thread executes
    // the same number of barriers.
    const int wg = warp >> 2;
    const int t = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const int q_pos = q0 + t;
    float m_run = -FLT_MAX, l_part = 0.f;
    bool ok = true;
    for (int i = 0; i < nchunks; ++i) {
      const int buf = i & 1;
      if (!tc::mbar_wait(&s_full[buf], (i >> 1) & 1, kWaitLimit, abort_flag) && ok) {
        ok = false;
        fail();
      }
      tc::fence_after_thread_sync();
      uint32_t sv[kHalfKeys];
      tc::tmem_ld_x64(lane_addr + (uint32_t)buf * kRows + (uint32_t)wg * kHalfKeys, sv);
      tc::fence_before_thread_sync();
      tc::mbar_arrive(&s_free[buf]);            // the scores are in registers: the buffer can take chunk i + 2
      const int key0 = i * kRows + wg * kHalfKeys;
      const bool diagonal = i == nchunks - 1;   // only the last chunk crosses the causal boundary
      // scores in units of log2 (multiplied by scale * log2 e), masked on the diagonal chunk; partial row maximum
      float cmax = -FLT_MAX;
#pragma unroll
      for (int j = 0; j < kHalfKeys; ++j) {
        float x = __uint_as_float(sv[j]) * a.scale_log2;
        if (diagonal && key0 + j > q_pos) x = -FLT_MAX;
        sv[j] = __float_as_uint(x);
        cmax = fmaxf(cmax, x);
      }
      xmax[buf][wg][t] = cmax;
      tc::named_barrier_sync(1, kSoftmaxThreads);
      cmax = fmaxf(cmax, xmax[buf][wg ^ 1][t]);
      if (i == 0) {
        m_run = cmax;                           // the diagonal element is always live, so this is finite
      } else {
        // P*V of the previous chunk is complete: the P tile may be overwritten and O is stable
        if (!tc::mbar_wait(o_full, (i - 1) & 1, kWaitLimit, abort_flag) && ok) {
          ok = false;
          fail();
        }
        tc::fence_after_thread_sync();
        const bool grow = cmax - m_run > kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          const float f = grow ? exp2f(m_run - cmax) : 1.f;
          if (grow) {
            m_run = cmax;
            l_part *= f;
          }
#pragma unroll 1
          for (int c = 0; c < kHalfKeys; c += 32) {
            uint32_t ov[32];
            tc::tmem_ld_x32(lane_addr + kColO + wg * kHalfKeys + c, ov);
#pragma unroll
            for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * f);
            tc::tmem_st_x32(lane_addr + kColO + wg * kHalfKeys + c, ov);
          }
        }
      }
      // probabilities against m_run, partial row sum, this thread's half of the P row (bf16, K-major over the key
      // positions, 128-byte swizzle: key block wg of the tile)
      float psum = 0.f;
      uint8_t* row = p_tile + wg * kHalfBytes + t * 128;
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float p0 = exp2f(__uint_as_float(sv[cc * 8 + 2 * j]) - m_run);
          const float p1 = exp2f(__uint_as_float(sv[cc * 8 + 2 * j + 1]) - m_run);
          psum += p0 + p1;
          __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
          w[j] = *reinterpret_cast<uint32_t*>(&hh);
        }
        *reinterpret_cast<uint4*>(row + ((cc ^ (t & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      l_part += psum;
      tc::fence_proxy_async();          // P was written by threads and is read by the tensor core
      tc::fence_before_thread_sync();   // orders the rescaled O (tcgen05.st) before the MMA that the arrival releases
      tc::mbar_arrive(p_full);
    }
    if (!tc::mbar_wait(o_full, (nchunks - 1) & 1, kWaitLimit, abort_flag) && ok) {
      ok = false;
      fail();
    }
    tc::fence_after_thread_sync();
    // row sum = the two halves' partial sums (same running maximum in both threads of a row)
    xmax[0][wg][t] = l_part;
    tc::named_barrier_sync(1, kSoftmaxThreads);
    const float l_run = l_part + xmax[0][wg ^ 1][t];
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    uint4* dst = reinterpret_cast<uint4*>(a.out + ((int64_t)q_pos * a.Hq + h) * kD + wg * kHalfKeys);
#pragma unroll 1
    for (int c = 0; c < kHalfKeys; c += 32) {
      uint32_t ov[32];
      tc::tmem_ld_x32(lane_addr + kColO + wg * kHalfKeys + c, ov);   // every lane of the warp takes part, rows beyond S included
      if (ok && q_pos < a.S) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(ov[g * 8 + 2 * j]) * inv, __uint_as_float(ov[g * 8 + 2 * j + 1]) * inv);
            w[j] = *reinterpret_cast<uint32_t*>(&hh);
          }
          dst[c / 8 + g] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
    tc::fence_before_thread_sync();
  }

  tc::fence_before_thread_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);   // copies already issued land before shared memory goes away
  }
  if (warp == kMmaWarp) {
    tc::fence_after_thread_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

std::string attention_prefill_tc(const void* q, const void* k, const void* v, void* out, int S, int Hq, int Hkv, int D,
                                 int64_t q_stride_s, int64_t k_stride_s, int64_t v_stride_s, float scale, cudaStream_t stream,
                                 uint32_t* status) {
  if (D != kD) return "prefill attention supports head dimension 128";
  if (Hkv <= 0 || Hq % Hkv) return "query heads must be a multiple of KV heads";
  if (S <= 0) return "";
  PrefillArgs a{};
  a.out = static_cast<__nv_bfloat16*>(out);
  a.S = S; a.Hq = Hq; a.Hkv = Hkv;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.idesc_s = tc::make_idesc(kRows, kRows, 1, 1);                  // both operands K-major bf16
  a.idesc_pv = tc::make_idesc(kRows, kD, 1, 1) | tc::kIdescBMnMajor;       // B (the V chunk) is read MN-major
  a.status = status;
  CUtensorMap mq, mk, mv;
  std::string err = tma::head_rows_3d(&mq, q, S, Hq, q_stride_s, kRows, "q");
  if (!err.empty()) return err;
  err = tma::head_rows_3d(&mk, k, S, Hkv, k_stride_s, kRows, "k");
  if (!err.empty()) return err;
  err = tma::head_rows_3d(&mv, v, S, Hkv, v_stride_s, kRows, "v");
  if (!err.empty()) return err;
  auto kern = attn_prefill_tc_kernel;
  const std::string smem_err = reserve_dynamic_smem(kern, kSmem);
  if (!smem_err.empty()) return smem_err;
  const dim3 grid((S + kRows - 1) / kRows, Hq, 1);
  const cudaError_t e = launch_chained(kern, grid, dim3(kThreads), kSmem, stream, mq, mk, mv, a);
  return e == cudaSuccess ? "" : cudaGetErrorString(e);
}

}  // namespace tdx
