// Causal self-attention for the prompt phase on the tensor cores (tcgen05 / TMEM), head dimension 128,
// bf16, grouped-query heads. One CTA owns 128 consecutive query positions of one query head and walks
// the key/value positions 0 .. (its last query) in chunks of 64:
//
//   S[q 128, keys 64] = Q[q, d] * K[keys, d]^T         both operands K-major, as TMA delivers them
//   O[q 128, d 128]  += P[q, keys] * V[keys, d]         P written by the softmax warps (K-major over keys),
//                                                       V read MN-major (d contiguous) straight from its TMA tile
//
// Two softmax warpgroups of four warps, one query row per thread in each: group g takes the chunks
// c = g, g + 2, ... - score buffer g, probability tile g and its OWN output accumulator O_g in tensor
// memory, with its own running maximum and sum - so two chunks are in the softmax at any time and every
// scheduler has two warps to choose from (one warp per scheduler issued an instruction in one cycle out of
// five: the softmax is a latency chain, not a throughput limit). At the end both groups combine
// O = (O_0 2^(m_0 - m) + O_1 2^(m_1 - m)) / (l_0 2^(m_0 - m) + l_1 2^(m_1 - m)), each writing one half of
// the head dimension. A thread fetches its 64 scores of a chunk with ONE tcgen05.ld and gives the score
// buffer back at once. A group has TWO probability tiles (chunk c uses tile c % 4), so before it writes
// the probabilities of a chunk it waits for the P*V product of its chunk before last, which has long
// completed - never for the product of its previous chunk, whose issue and completion would otherwise sit
// in the group's cycle (measured: half of it). A row's running maximum is only raised - and its row of O_g
// rescaled in tensor memory - when the new maximum exceeds it by more than 2^8 (a warp-uniform
// decision); until then the probabilities are taken against the older maximum, which changes neither
// O / l nor the accuracy of bf16 probabilities below 256 (that rescale does wait for the group's latest
// product). Five more warps hold one single-thread role
// each: the TMA copies (four-stage rings for K, freed as soon as the scores are computed, and for V, freed
// after P*V), the score MMAs of the even and of the odd chunks, and the P*V MMAs into O_0 and into O_1.
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
constexpr int kRows = 128;                        // query rows per CTA
constexpr int kKeys = 64;                         // key positions per chunk
constexpr int kStagesK = 4;
constexpr int kStagesV = 4;
constexpr int kSoftmaxThreads = 128;              // per warpgroup; two groups
constexpr int kLoadWarp = 2 * kSoftmaxThreads / 32;   // also owns the tensor-memory allocation
constexpr int kScoreWarp = kLoadWarp + 1;              // and kScoreWarp + 1: one issuer per score buffer
constexpr int kPvWarp = kLoadWarp + 3;                 // and kPvWarp + 1: one issuer per accumulator
constexpr int kThreads = 2 * kSoftmaxThreads + 5 * 32;
constexpr int kPTiles = 4;                             // probability tiles: chunk c uses tile c % 4, so a group has two
constexpr int kQHalfBytes = kRows * 128;          // 64 head-dimension columns of the 128 query rows
constexpr int kQBytes = 2 * kQHalfBytes;
constexpr int kKVHalfBytes = kKeys * 128;         // 64 head-dimension columns of the 64 positions of a chunk
constexpr int kKVBytes = 2 * kKVHalfBytes;        // one K chunk or one V chunk
constexpr int kPBytes = kRows * kKeys * 2;        // probabilities of a chunk: one 64-key K block of 128 rows
constexpr int kNumBarriers = 2 * kStagesK + 2 * kStagesV + 4 + 2 + 2 * kPTiles;   // k/v full+free, s full+free [2], q_full, o_final, p_full [4], pv_done [4]
constexpr int kBarrierBytes = 256;                // the mbarriers, the TMEM address and the abort flag
static_assert(kNumBarriers * 8 + 8 <= kBarrierBytes, "barrier area too small");
constexpr int kSmem = kQBytes + kPTiles * kPBytes + (kStagesK + kStagesV) * kKVBytes + kBarrierBytes;
static_assert(kSmem <= 227 * 1024, "shared memory of one CTA");
constexpr uint32_t kTmemCols = 512;               // S buffers at columns 0 and 64, O_0 at 128, O_1 at 256
constexpr uint32_t kColO = 128;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr float kRescaleThreshold = 8.f;          // log2 units

// Timing probe (the tracing flavour of the library, -DTDX_TRACE): the block with the most chunks of head 0 stamps
// clock64 at fixed points of every chunk, per role: role 0 = the issuers (slots 0-2 by the score issuer of the chunk:
// loop top, waits passed, MMAs and commits issued; slots 3-4 by its P*V issuer: waits passed, issued), roles 1 and 2 =
// thread 0 of the softmax groups (scores ready, loaded, maximum done, tile free, probabilities stored, arrived).
// attention_prefill_probe() copies the stamps out; benchmarks/trace_prefill_attention.py prints them.
#if defined(TDX_TRACE) && !defined(TDX_ATTN_PROBE)
#define TDX_ATTN_PROBE 1
#endif
#ifdef TDX_ATTN_PROBE
__device__ unsigned long long g_attn_probe[3 * 64 * 8];
#define TDX_PROBE(role, chunk, slot)                                                        \
  do {                                                                                      \
    if (probe_on && (chunk) < 64) g_attn_probe[((role) * 64 + (chunk)) * 8 + (slot)] = clock64(); \
  } while (0)
#else
#define TDX_PROBE(role, chunk, slot) \
  do {                               \
  } while (0)
#endif

struct PrefillArgs {
  __nv_bfloat16* out;          // [S, Hq, D] contiguous
  int S, Hq, Hkv;
  float scale_log2;            // softmax scale * log2(e)
  uint32_t idesc_s, idesc_pv;
  uint32_t* status;
};

// exp2 of a non-positive (or slightly positive) argument, flushing what underflows to zero
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const PrefillArgs a) {
  // The tiles need 1024-byte alignment (128-byte swizzle): the dynamic region is declared aligned, and a kernel
  // that finds it otherwise reports that instead of running.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if ((tc::smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0 && a.status) atomicExch(a.status, (uint32_t)kTimeoutGemmPipeline);
    return;
  }
  uint8_t* q_tile = smem_raw;
  uint8_t* p_tile = q_tile + kQBytes;
  uint8_t* k_ring = p_tile + kPTiles * kPBytes;
  uint8_t* v_ring = k_ring + kStagesK * kKVBytes;
  uint64_t* k_full = reinterpret_cast<uint64_t*>(v_ring + kStagesV * kKVBytes);
  uint64_t* k_free = k_full + kStagesK;
  uint64_t* v_full = k_free + kStagesK;
  uint64_t* v_free = v_full + kStagesV;
  uint64_t* s_full = v_free + kStagesV;     // [2]
  uint64_t* s_free = s_full + 2;            // [2]
  uint64_t* q_full = s_free + 2;
  uint64_t* p_full = q_full + 1;            // [4]: probabilities of chunk c are in tile c & 3
  uint64_t* pv_done = p_full + kPTiles;     // [4]: the P*V product that read tile c & 3 has completed
  uint64_t* o_final = pv_done + kPTiles;    // every product has completed (one arrival per P*V issuer)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_final + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  // The blocks with the most key chunks start first, for all heads (blockIdx.x runs fastest): the short blocks of
  // the causal triangle fill the tail of the grid. Neighbouring blocks are the query heads of one KV head and
  // read the same K / V tiles out of L2.
  const int qb = (int)gridDim.y - 1 - (int)blockIdx.y;
  const int h = blockIdx.x;
  const int hkv = h / (a.Hq / a.Hkv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int q0 = qb * kRows;
  const int nchunks = (q0 + kRows) / kKeys;  // key positions 0 .. q0 + 127 (causal)
#ifdef TDX_ATTN_PROBE
  const bool probe_on = blockIdx.x == 0 && blockIdx.y == 0 && ((tid & (kSoftmaxThreads - 1)) == 0 || (warp >= kLoadWarp && lane == 0));
#endif

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
    for (int i = 0; i < kPTiles; ++i) {
      tc::mbar_init(&p_full[i], kSoftmaxThreads);
      tc::mbar_init(&pv_done[i], 1);
    }
    tc::mbar_init(o_final, 2);
    *abort_flag = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_desc(&map_q);
    tc::tma_prefetch_desc(&map_k);
    tc::tma_prefetch_desc(&map_v);
  }
  if (warp == kLoadWarp) {
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

  // Three single-thread roles in three warps, each with its own chain of waits, so that none of them queues behind
  // the others' (one thread doing all three spent about 2300 cycles per chunk issuing copies, MMAs and commits one
  // after the other, twice what a softmax group needs for the chunk):
  //   loader        TMA copies of Q, K and V; refills a K stage when its scores are complete, a V stage after P*V
  //   score issuers S_(c & 1) = Q K_c^T as soon as K_c has landed and the group has taken chunk c - 2 out of the buffer
//                 (two of them: one for the even chunks, one for the odd ones)
  //   P*V issuers   O_(c & 1) += P_c V_c as soon as the group has written P_c and V_c has landed (one per accumulator)
  // MMAs of the two issuers touch different tensor-memory columns and different tiles; what orders them against the
  // softmax groups are the barriers below, and each issuer's commits cover its own MMAs.
  if (warp == kLoadWarp) {
    if (lane == 0) {
      auto load_k = [&](int c) {
        uint8_t* base = k_ring + (c % kStagesK) * kKVBytes;
        tc::mbar_arrive_expect_tx(&k_full[c % kStagesK], kKVBytes);
        tc::tma_load_3d(base, &map_k, &k_full[c % kStagesK], 0, hkv, c * kKeys);
        tc::tma_load_3d(base + kKVHalfBytes, &map_k, &k_full[c % kStagesK], 64, hkv, c * kKeys);
      };
      auto load_v = [&](int c) {
        uint8_t* base = v_ring + (c % kStagesV) * kKVBytes;
        tc::mbar_arrive_expect_tx(&v_full[c % kStagesV], kKVBytes);
        tc::tma_load_3d(base, &map_v, &v_full[c % kStagesV], 0, hkv, c * kKeys);
        tc::tma_load_3d(base + kKVHalfBytes, &map_v, &v_full[c % kStagesV], 64, hkv, c * kKeys);
      };
      tc::mbar_arrive_expect_tx(q_full, kQBytes);
      tc::tma_load_3d(q_tile, &map_q, q_full, 0, h, q0);
      tc::tma_load_3d(q_tile + kQHalfBytes, &map_q, q_full, 64, h, q0);
      for (int c = 0; c < nchunks && c < kStagesK; ++c) load_k(c);
      for (int c = 0; c < nchunks && c < kStagesV; ++c) load_v(c);
      bool ok = true;
      // The P*V products trail the score MMAs by about two chunks, so the V stages come free two chunks after the
      // K stages: the K refill of chunk j shares an iteration with the V refill of chunk j - 2, and neither wait
      // holds the other's copies back.
      for (int j = 0; j < nchunks + 2 && ok; ++j) {
        if (j + kStagesK < nchunks) {
          // K stage of chunk j is free once its scores are complete (long before P*V of the chunk)
          ok = tc::mbar_wait(&k_free[j % kStagesK], (j / kStagesK) & 1, kWaitLimit, abort_flag);
          if (!ok) break;
          load_k(j + kStagesK);
        }
        const int i = j - 2;
        if (i >= 0 && i + kStagesV < nchunks) {
          // V stage of chunk i is free once its P*V product is complete
          ok = tc::mbar_wait(&v_free[i % kStagesV], (i / kStagesV) & 1, kWaitLimit, abort_flag);
          if (!ok) break;
          load_v(i + kStagesV);
        }
      }
      if (!ok) fail();
    }
  } else if (warp == kScoreWarp || warp == kScoreWarp + 1) {
    if (lane == 0) {
      // issuing the eight MMAs and two commits of a chunk takes one thread longer than a softmax group needs for
      // the chunk, so the even and the odd chunks have an issuer each
      const uint32_t qbase = tc::smem_u32(q_tile);
      bool ok = tc::mbar_wait(q_full, 0, kWaitLimit, abort_flag);
      for (int c = warp - kScoreWarp; c < nchunks && ok; c += 2) {
        TDX_PROBE(0, c, 0);
        ok = tc::mbar_wait(&k_full[c % kStagesK], (c / kStagesK) & 1, kWaitLimit, abort_flag) &&
             (c < 2 || tc::mbar_wait(&s_free[c & 1], ((c >> 1) - 1) & 1, kWaitLimit, abort_flag));
        if (!ok) break;
        TDX_PROBE(0, c, 1);
        tc::fence_after_thread_sync();
        const uint32_t kbase = tc::smem_u32(k_ring + (c % kStagesK) * kKVBytes);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)     // the two 64-column halves of the head dimension
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)   // 16 columns per instruction, stepped inside the swizzle span
            tc::umma<false>(tmem_base + (uint32_t)(c & 1) * kKeys, tc::make_smem_desc_sw128(qbase + kb * kQHalfBytes) + (uint64_t)(ks * 2),
                            tc::make_smem_desc_sw128(kbase + kb * kKVHalfBytes) + (uint64_t)(ks * 2), a.idesc_s, (kb | ks) ? 1u : 0u);
        tc::umma_commit(&s_full[c & 1]);
        tc::umma_commit(&k_free[c % kStagesK]);    // the K stage is free once these complete
        TDX_PROBE(0, c, 2);
      }
      if (!ok) fail();
    }
  } else if (warp == kPvWarp || warp == kPvWarp + 1) {
    if (lane == 0) {
      bool ok = true;
      for (int c = warp - kPvWarp; c < nchunks && ok; c += 2) {
        ok = tc::mbar_wait(&p_full[c & 3], (c >> 2) & 1, kWaitLimit, abort_flag) &&
             tc::mbar_wait(&v_full[c % kStagesV], (c / kStagesV) & 1, kWaitLimit, abort_flag);
        if (!ok) break;
        TDX_PROBE(0, c, 3);
        tc::fence_after_thread_sync();
        const uint32_t vbase = tc::smem_u32(v_ring + (c % kStagesV) * kKVBytes);
        const uint32_t pbase = tc::smem_u32(p_tile + (c & 3) * kPBytes);
#pragma unroll
        for (int j = 0; j < kKeys / 16; ++j)   // 16 key positions per instruction
          tc::umma<false>(tmem_base + kColO + (uint32_t)(c & 1) * kD, tc::make_smem_desc_sw128(pbase) + (uint64_t)(j * 2),
                          tc::make_smem_desc_mn_sw128(vbase + j * 2048, kKVHalfBytes), a.idesc_pv, (c >= 2 || j > 0) ? 1u : 0u);
        tc::umma_commit(&pv_done[c & 3]);
        tc::umma_commit(&v_free[c % kStagesV]);
        if (c + 2 >= nchunks) tc::umma_commit(o_final);      // this issuer's last chunk
        TDX_PROBE(0, c, 4);
      }
      if (!ok) fail();
    }
  } else {
    // ---- softmax warps: group g = warp / 4 takes the chunks g, g + 2, ...; its thread t owns query row q0 + t ----
    // A thread whose wait ran out keeps walking the loop (its waits return at once because the abort flag is up),
    // so that the warp-wide tensor-memory instructions and the named barrier below are always executed by all.
    const int g = warp >> 2;
    const int t = tid & (kSoftmaxThreads - 1);
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t o_addr = lane_addr + kColO + (uint32_t)g * kD;
    const int q_pos = q0 + t;
    float m_run = -1e30f, l_run = 0.f;
    bool ok = true;
    // The exponentials of a chunk keep the special-function unit busy for 512 cycles per warp; two groups that run
    // them at the same time (they fall into step by themselves) both take twice as long, while the rest of a
    // group's cycle - waiting for scores, loading them, the row maximum - needs no exponentials. So the groups take
    // turns: a group enters its exponential phase through named barrier 2 + g, which the other group completes when
    // it leaves its own. Group 1 hands group 0 the first turn; both run the same number of chunks.
    if (g == 1) tc::named_barrier_arrive(2, 2 * kSoftmaxThreads);
    for (int i = g; i < nchunks; i += 2) {
      if (!tc::mbar_wait(&s_full[g], (i >> 1) & 1, kWaitLimit, abort_flag) && ok) {
        ok = false;
        fail();
      }
      TDX_PROBE(1 + g, i, 0);
      tc::fence_after_thread_sync();
      uint32_t sv[kKeys];
      tc::tmem_ld_x64(lane_addr + (uint32_t)g * kKeys, sv);
      TDX_PROBE(1 + g, i, 1);
      tc::fence_before_thread_sync();
      tc::mbar_arrive(&s_free[g]);              // the scores are in registers: the buffer can take chunk i + 2
      const int key0 = i * kKeys;
      const bool diagonal = key0 + kKeys - 1 > q0;   // the last two chunks cross the causal boundary of some row
      // row maximum of the raw scores, masked where the key lies after the query; the softmax scale (times log2 e)
      // is positive, so it commutes with the maximum and is folded into the exponent's multiply-add below
      if (diagonal) {
#pragma unroll
        for (int j = 0; j < kKeys; ++j)
          if (key0 + j > q_pos) sv[j] = __float_as_uint(-FLT_MAX);
      }
      float cm[4] = {-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX};   // four chains instead of one of 64 dependent maxima
#pragma unroll
      for (int j = 0; j < kKeys; j += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) cm[u] = fmaxf(cm[u], __uint_as_float(sv[j + u]));
      }
      // in units of log2 from here on; a chunk that the mask removes entirely for this row (the group of the odd
      // chunks, first rows of the prompt) must not become the reference: keep the maximum above -1e30
      const float cmax = fmaxf(fmaxf(fmaxf(cm[0], cm[1]), fmaxf(cm[2], cm[3])) * a.scale_log2, -1e30f);
      TDX_PROBE(1 + g, i, 2);
      if (i < 2) {
        m_run = cmax;
      } else {
        const bool grow = cmax - m_run > kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          // O_g may only be touched when the group's latest product, the one of chunk i - 2, has completed
          if (!tc::mbar_wait(&pv_done[(i - 2) & 3], ((i - 2) >> 2) & 1, kWaitLimit, abort_flag) && ok) {
            ok = false;
            fail();
          }
          tc::fence_after_thread_sync();
          const float f = grow ? ex2(m_run - cmax) : 1.f;
          if (grow) {
            m_run = cmax;
            l_run *= f;
          }
#pragma unroll 1
          for (int c = 0; c < kD; c += 32) {
            uint32_t ov[32];
            tc::tmem_ld_x32(o_addr + c, ov);
#pragma unroll
            for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * f);
            tc::tmem_st_x32(o_addr + c, ov);
          }
        }
      }
      TDX_PROBE(1 + g, i, 3);
      // the probability tile of this chunk was last read by the P*V product of chunk i - 4: the group never waits
      // for the product of its previous chunk, which is still being issued while these probabilities are computed
      if (i >= 4 && !tc::mbar_wait(&pv_done[i & 3], ((i >> 2) - 1) & 1, kWaitLimit, abort_flag) && ok) {
        ok = false;
        fail();
      }
      tc::named_barrier_sync(2 + g, 2 * kSoftmaxThreads);      // this group's turn at the exponentials
      // probabilities against m_run, row sum, this row of the P tile (bf16, K-major over the 64 key positions,
      // 128-byte swizzle). A masked score is -FLT_MAX and comes out as zero.
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
      uint8_t* row = p_tile + (i & 3) * kPBytes + t * 128;
      const float neg_m = -m_run;
#pragma unroll
      for (int cc = 0; cc < kKeys / 8; ++cc) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float p0 = ex2(fmaf(__uint_as_float(sv[cc * 8 + 2 * j]), a.scale_log2, neg_m));
          const float p1 = ex2(fmaf(__uint_as_float(sv[cc * 8 + 2 * j + 1]), a.scale_log2, neg_m));
          ps[j] += p0 + p1;
          __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
          w[j] = *reinterpret_cast<uint32_t*>(&hh);
        }
        *reinterpret_cast<uint4*>(row + ((cc ^ (t & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      l_run += (ps[0] + ps[1]) + (ps[2] + ps[3]);
      if (g == 0 || i + 2 < nchunks) tc::named_barrier_arrive(2 + (g ^ 1), 2 * kSoftmaxThreads);   // the other group's turn
      TDX_PROBE(1 + g, i, 4);
      tc::fence_proxy_async();          // P was written by threads and is read by the tensor core
      tc::fence_before_thread_sync();   // orders the rescaled O (tcgen05.st) before the MMA that the arrival releases
      tc::mbar_arrive(&p_full[i & 3]);
      TDX_PROBE(1 + g, i, 5);
    }
    // every product has completed: both accumulators are final and the probability tiles are free
    if (!tc::mbar_wait(o_final, 0, kWaitLimit, abort_flag) && ok) {
      ok = false;
      fail();
    }
    tc::fence_after_thread_sync();
    // the two groups tell each other maximum and sum of their rows (through the first probability tile)
    float2* ml = reinterpret_cast<float2*>(p_tile);
    ml[g * kSoftmaxThreads + t] = make_float2(m_run, l_run);
    tc::named_barrier_sync(1, 2 * kSoftmaxThreads);
    const float2 other = ml[(g ^ 1) * kSoftmaxThreads + t];
    const float m = fmaxf(m_run, other.x);
    const float w_own = ex2(m_run - m), w_other = ex2(other.x - m);
    const float l = l_run * w_own + other.y * w_other;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const float w0 = (g == 0 ? w_own : w_other) * inv, w1 = (g == 0 ? w_other : w_own) * inv;
    // group g writes the head-dimension columns 64 g .. 64 g + 63 of its rows
    uint4* dst = reinterpret_cast<uint4*>(a.out + ((int64_t)q_pos * a.Hq + h) * kD + g * 64);
#pragma unroll 1
    for (int c = 0; c < 64; c += 32) {
      uint32_t o0[32], o1[32];
      tc::tmem_ld_x32(lane_addr + kColO + (uint32_t)(g * 64 + c), o0);        // every lane of the warp takes part,
      tc::tmem_ld_x32(lane_addr + kColO + kD + (uint32_t)(g * 64 + c), o1);   // rows beyond S included
      if (ok && q_pos < a.S) {
#pragma unroll
        for (int gg = 0; gg < 4; ++gg) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int e = gg * 8 + 2 * j;
            __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(o0[e]) * w0 + __uint_as_float(o1[e]) * w1,
                                                      __uint_as_float(o0[e + 1]) * w0 + __uint_as_float(o1[e + 1]) * w1);
            w[j] = *reinterpret_cast<uint32_t*>(&hh);
          }
          dst[c / 8 + gg] = make_uint4(w[0], w[1], w[2], w[3]);
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
  if (warp == kLoadWarp) {
    tc::fence_after_thread_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

std::string attention_prefill_probe(unsigned long long* dst, size_t count) {
#ifdef TDX_ATTN_PROBE
  if (count != 3 * 64 * 8) return "the probe holds 3 x 64 x 8 stamps";
  const cudaError_t e = cudaMemcpyFromSymbol(dst, g_attn_probe, count * sizeof(unsigned long long));
  return e == cudaSuccess ? "" : cudaGetErrorString(e);
#else
  (void)dst;
  (void)count;
  return "the clock stamps exist in the tracing flavour of the library only (TDX_TRACE=1)";
#endif
}

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
  a.idesc_s = tc::make_idesc(kRows, kKeys, 1, 1);                  // both operands K-major bf16
  a.idesc_pv = tc::make_idesc(kRows, kD, 1, 1) | tc::kIdescBMnMajor;       // B (the V chunk) is read MN-major
  a.status = status;
  CUtensorMap mq, mk, mv;
  std::string err = tma::head_rows_3d(&mq, q, S, Hq, q_stride_s, kRows, "q");
  if (!err.empty()) return err;
  err = tma::head_rows_3d(&mk, k, S, Hkv, k_stride_s, kKeys, "k");
  if (!err.empty()) return err;
  err = tma::head_rows_3d(&mv, v, S, Hkv, v_stride_s, kKeys, "v");
  if (!err.empty()) return err;
  auto kern = attn_prefill_tc_kernel;
  const std::string smem_err = reserve_dynamic_smem(kern, kSmem);
  if (!smem_err.empty()) return smem_err;
  const dim3 grid(Hq, (S + kRows - 1) / kRows, 1);
  const cudaError_t e = launch_chained(kern, grid, dim3(kThreads), kSmem, stream, mq, mk, mv, a);
  return e == cudaSuccess ? "" : cudaGetErrorString(e);
}

}  // namespace tdx
