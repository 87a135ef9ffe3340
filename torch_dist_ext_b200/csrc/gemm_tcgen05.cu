// tcgen05 / TMEM GEMM for sm_100a:  D[x, y] = sum_k X[x, k] * Y[y, k]   (both operands K-major).
//
// One CTA computes a 128 x kBN tile of D. Warp 0 streams operand tiles with TMA into a ring of
// 128-byte-swizzled shared-memory stages; warp 1 owns the tensor memory and issues tcgen05.mma
// (one elected thread) into an fp32 accumulator in TMEM; warps 2-5 read the accumulator back with
// tcgen05.ld and write the output. "X" and "Y" are roles, not matrices: a linear layer
// out[M, N] = a[M, K] * w[N, K]^T runs either as (X = a, Y = w) for large M, or as (X = w, Y = a)
// for decode-sized M, so that the weights fill the 128-row dimension of the instruction and the
// few tokens sit on the narrow N side; the output strides (sx, sy) place D either way round.
// K can be split over gridDim.z; partial tiles are then reduced in an fp32 workspace with
// red.global.add and finished by whichever CTA arrives last at the tile. That finalizer can do more than
// store: with the weights on the 128-row side it holds 128 output features of up to kBN tokens, enough to
// rotate a head of a fused qkv projection and append it to the KV cache (rotate-half pairs element i with
// i + 64), or to form silu(gate) * up when the tile was loaded as 64 gate rows and the 64 up rows of the
// same features. Either saves a kernel of the decode layer's latency chain.
//
// fp8 (e4m3) operands use kind::f8f6f4. With block scales (1x128 on one operand, 128x128 on the
// other, fp32) each 128-wide K block is multiplied into its own TMEM buffer and promoted by the
// epilogue warps: acc += partial * x_scale * y_scale, with two TMEM buffers so that the next
// block's MMAs overlap the promotion.
//
// Every mbarrier wait is bounded; a wait that runs out records a status word, raises the CTA's
// abort flag, lets copies in flight land, frees the tensor memory and returns.
//
// The reference (xytpai/torch_dist_ext) has no GEMM; this kernel exists for the tensor-parallel
// decoder layers around its fused all-reduce.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdlib>
#include <mutex>
#include "tdx/comm.h"
#include "tdx/gemm.h"
#include "tdx/gemm_core.cuh"
#include "tdx/launch.h"
#include "tdx/ptx.cuh"
#include "tdx/tc.cuh"
#include "tdx/tma_host.h"

namespace tdx {
namespace {

using gemm_core::store_chunk;

using gemm_core::kBM;
using gemm_core::kSwizzleBytes;
using gemm_core::kWaitLimit;
using gemm_core::SmemLayout;
constexpr int kThreads = 192;

struct GemmArgs {
  int x_rows, y_rows;
  int kblocks;             // K / (128 / elem_size)
  int kblocks_per_split;
  void* out;
  int64_t sx, sy;          // D[x, y] -> out[x * sx + y * sy]
  int out_dtype;           // kF32 / kF16 / kBF16
  uint32_t idesc;
  float* ws;               // split-K: fp32 tiles [tile][column][128 rows], zero on entry and on exit
  int ws_ld;
  uint32_t* counters;      // split-K: one per output tile, zero on entry and on exit
  uint32_t* status;        // device word: non-zero after a wait ran out
  // block scales (scaled kernels only); *_per_row: one scale per row and K block, else per 128 rows
  const float* x_scale;
  const float* y_scale;
  int x_scale_per_row, y_scale_per_row;
  int scale_kb;            // K blocks per scale row (= total K / 128)
  int x_static;            // X is never written by a kernel (weights): its first tiles may be requested before the
                           // previous kernel of the stream has finished
  PairEpilogue epi;        // what the split-K finalizer does with rows r and r + 64 of a tile (kEpiNone: plain store)
};

// ---- pair epilogues ---------------------------------------------------------------------------------------
// The finalizer of a tile whose rows r and r + 64 belong together. The 128 epilogue threads split the work as 64 row
// pairs x 2 column halves; a thread walks its half in steps of kPairW columns. Everything a step needs is requested
// before anything is used - the two sums per column from the split-K scratch, the angles of the columns' positions -
// and the positions themselves are fetched one step ahead (those of the first step before the CTA even knows whether
// it is the finalizer), so that a step costs one round trip to L2, not three dependent ones.
template <int kBN>
struct PairShape {
  static constexpr int kHalf = kBN / 2;                  // columns per thread
  static constexpr int kW = kHalf < 16 ? kHalf : 16;     // columns per step
  static constexpr int kSteps = kHalf / kW;
};

template <int kW>
__device__ __forceinline__ void pair_positions(const GemmArgs& a, int y0, int (&pos)[kW]) {
#pragma unroll
  for (int j = 0; j < kW; ++j) pos[j] = y0 + j < a.y_rows ? (int)__ldg(a.epi.positions + y0 + j) : 0;
}

// `tile_ws`: this tile's fp32 sums, [column][128 rows]; `pos`: positions of the first step's columns (rope only).
template <int kBN>
__device__ __forceinline__ void pair_finalize(const GemmArgs& a, int tile_x, float* tile_ws, int r, int half, int y_base,
                                              int (&pos)[PairShape<kBN>::kW]) {
  using S = PairShape<kBN>;
  constexpr int kW = S::kW;
  const PairEpilogue& e = a.epi;
  const bool rope = e.kind == kEpiRopeKv;
  // rope: tile_x is the head (queries, then keys, then values)
  const bool is_q = tile_x < e.q_heads;
  const bool is_v = tile_x >= e.q_heads + e.kv_heads;
  const bool rotate = rope && !is_v;
  __nv_bfloat16* cache = (!rope || is_q) ? nullptr : static_cast<__nv_bfloat16*>(is_v ? e.v_cache : e.k_cache);
  const int kv_head = tile_x - e.q_heads - (is_v ? e.kv_heads : 0);
  const int64_t x_lo = rope ? (int64_t)tile_x * kBM + r : (int64_t)tile_x * 64 + r;
  float* src = tile_ws + r;
#pragma unroll 1
  for (int s = 0; s < S::kSteps; ++s) {
    const int c = half * S::kHalf + s * kW;
    float lo[kW], hi[kW], cs[kW], sn[kW];
    int cur[kW];
#pragma unroll
    for (int j = 0; j < kW; ++j) {
      lo[j] = __ldcg(src + (size_t)(c + j) * kBM);
      hi[j] = __ldcg(src + (size_t)(c + j) * kBM + 64);
      cur[j] = pos[j];
    }
    if (rotate) {
#pragma unroll
      for (int j = 0; j < kW; ++j) {
        const int p = cur[j] < 0 ? 0 : (cur[j] >= e.max_pos ? e.max_pos - 1 : cur[j]);
        cs[j] = __ldg(e.cos_sin + (int64_t)p * 128 + r);
        sn[j] = __ldg(e.cos_sin + (int64_t)p * 128 + 64 + r);
      }
    }
    if (rope && s + 1 < S::kSteps) pair_positions<kW>(a, y_base + c + kW, pos);
#pragma unroll
    for (int j = 0; j < kW; ++j) {
      __stcg(src + (size_t)(c + j) * kBM, 0.f);
      __stcg(src + (size_t)(c + j) * kBM + 64, 0.f);
    }
#pragma unroll
    for (int j = 0; j < kW; ++j) {
      const int y = y_base + c + j;
      if (y >= a.y_rows) continue;
      if (!rope) {   // silu(gate) * up
        gemm_core::store_out(a, x_lo * a.sx + (int64_t)y * a.sy, lo[j] / (1.f + __expf(-lo[j])) * hi[j]);
        continue;
      }
      float o_lo = lo[j], o_hi = hi[j];
      if (rotate) {
        o_lo = lo[j] * cs[j] - hi[j] * sn[j];
        o_hi = hi[j] * cs[j] + lo[j] * sn[j];
      }
      gemm_core::store_out(a, x_lo * a.sx + (int64_t)y * a.sy, o_lo);
      gemm_core::store_out(a, (x_lo + 64) * a.sx + (int64_t)y * a.sy, o_hi);
      if (cache != nullptr && cur[j] >= 0 && cur[j] < e.cache_seq) {
        __nv_bfloat16* dst = cache + (int64_t)y * e.cache_batch_stride + (int64_t)cur[j] * e.cache_pos_stride + kv_head * 128 + r;
        dst[0] = __float2bfloat16(o_lo);
        dst[64] = __float2bfloat16(o_hi);
      }
    }
  }
}

template <int kBN, int kStages, bool kFp8, bool kScaled>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y, const GemmArgs a) {
  using L = SmemLayout<kBN, kStages>;
  constexpr int kElemsPerBlock = kFp8 ? 128 : 64;   // K elements per 128-byte block
  constexpr uint32_t kTmemCols = kScaled ? (2 * kBN < 32 ? 32 : 2 * kBN) : (kBN < 32 ? 32 : kBN);
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "TMEM columns must be a power of two");

  extern __shared__ uint8_t smem_raw[];
  gemm_core::Pipeline<kBN, kStages> pipe;
  pipe.init(smem_raw, kTmemCols, &map_x, &map_y);
  uint64_t* acc_full = pipe.acc_full;
  uint64_t* acc_empty = pipe.acc_empty;
  volatile uint32_t* abort_flag = pipe.abort_flag;
  uint32_t* last_flag = pipe.scratch;
  const uint32_t tmem_base = pipe.tmem_base;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_x = blockIdx.x, tile_y = blockIdx.y;
  const int kb0 = blockIdx.z * a.kblocks_per_split;
  const int kb1 = min(a.kblocks, kb0 + a.kblocks_per_split);
  const int nkb = kb1 - kb0;

  if (warp == 0) {
    if (lane == 0) {
      // With static X (decode orientation: the weights) the first ring of X tiles is requested before the wait for
      // the previous kernel of the stream; everything else is read and written after it.
      if (!a.x_static) ptx::pdl_wait();
      // silu(gate) * up: 64 gate rows and the 64 up rows of the same features make one 128-row tile
      const bool halves = a.epi.kind == kEpiSiluMul;
      pipe.template produce<kElemsPerBlock>(&map_x, &map_y, halves ? tile_x * 64 : tile_x * kBM, tile_y * kBN, kb0, nkb, a.status, [] {
        ptx::pdl_wait();
        return true;
      }, halves ? a.epi.ffn + tile_x * 64 : -1);
      ptx::pdl_launch_dependents();
    }
  } else if (warp == 1) {
    if (lane == 0) pipe.template issue<kFp8, kScaled>(nkb, a.idesc, a.status);
  } else {
    ptx::pdl_wait();   // scales, split-K scratch and the output belong to the stream's order
    // ---- epilogue (warps 2..5): TMEM lane quarter = warp % 4 -----------------------------------------
    const int q = warp & 3;
    const int x = tile_x * kBM + q * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const int y_base = tile_y * kBN;
    bool ok = true;
    float acc[kScaled ? kBN : 1];
    if constexpr (kScaled) {
#pragma unroll
      for (int i = 0; i < kBN; ++i) acc[i] = 0.f;
      // Scales of a K block: one per thread for its X row, and the kBN (<= 64) column scales held two per lane
      // and handed round with shuffles. Those of block i + 1 are requested before the wait for block i's partial
      // product, so their latency hides behind the MMAs instead of sitting in front of every multiply-add.
      static_assert(kBN <= 64, "the promoting epilogue keeps the column scales of a K block in two registers per lane");
      const float* xs_ptr = a.x_scale + (size_t)(a.x_scale_per_row ? min(x, a.x_rows - 1) : (x < a.x_rows ? x / 128 : 0)) * a.scale_kb;
      const int y_lo = min(y_base + lane, a.y_rows - 1), y_hi = min(y_base + 32 + lane, a.y_rows - 1);
      const float* ys_lo_ptr = a.y_scale + (size_t)(a.y_scale_per_row ? y_lo : y_lo / 128) * a.scale_kb;
      const float* ys_hi_ptr = a.y_scale + (size_t)(a.y_scale_per_row ? y_hi : y_hi / 128) * a.scale_kb;
      float xs_next = nkb > 0 ? xs_ptr[kb0] : 0.f;
      float lo_next = nkb > 0 ? ys_lo_ptr[kb0] : 0.f;
      float hi_next = (nkb > 0 && kBN > 32) ? ys_hi_ptr[kb0] : 0.f;
      for (int i = 0; i < nkb && ok; ++i) {
        const int buf = i & 1;
        const float xs = xs_next, ys_lo = lo_next, ys_hi = hi_next;
        if (i + 1 < nkb) {
          xs_next = xs_ptr[kb0 + i + 1];
          lo_next = ys_lo_ptr[kb0 + i + 1];
          if (kBN > 32) hi_next = ys_hi_ptr[kb0 + i + 1];
        }
        // (the shuffles below are warp-wide: the warp gives up as a whole)
        ok = __all_sync(0xffffffffu, tc::mbar_wait(&acc_full[buf], (i >> 1) & 1, kWaitLimit, abort_flag));
        if (!ok) break;
        tc::fence_after_thread_sync();
        gemm_core::promote_block<kBN>(lane_addr + buf * kBN, xs, ys_lo, ys_hi, acc);
        tc::fence_before_thread_sync();
        tc::mbar_arrive(&acc_empty[buf]);
      }
    } else {
      ok = nkb <= 0 || tc::mbar_wait(&acc_full[0], 0, kWaitLimit, abort_flag);
      tc::fence_after_thread_sync();
    }
    if (!ok) {
      *abort_flag = 1;
      if (a.status) atomicExch(a.status, kTimeoutGemmPipeline);
    }
    const bool split = gridDim.z > 1;
    if (ok && nkb > 0) {
#pragma unroll
      for (int c = 0; c < kBN; c += 16) {
        float v[16];
        if constexpr (kScaled) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = acc[c + j];
        } else {
          tc::tmem_ld_16(lane_addr + c, v);
        }
        if (!split) {
          store_chunk(a, x, y_base + c, v);
        } else {
          // scratch tile is column-major ([column][128 rows]): the lanes of a warp add to 32
          // consecutive floats, one 128-byte line per instruction
          float* dst = a.ws + (size_t)(tile_y * gridDim.x + tile_x) * (kBM * kBN) + (size_t)c * kBM + q * 32 + lane;
#pragma unroll
          for (int j = 0; j < 16; ++j) atomicAdd(dst + j * kBM, v[j]);
        }
      }
    }
    int pair_pos[PairShape<kBN>::kW] = {};
    if (split && a.epi.kind == kEpiRopeKv) pair_positions<PairShape<kBN>::kW>(a, y_base + (q >> 1) * PairShape<kBN>::kHalf, pair_pos);
    if (split) {
      // the CTA that arrives last at this tile turns the fp32 sums into the output and re-zeroes them
      __threadfence();
      tc::named_barrier_sync(1, 128);
      if (threadIdx.x == 64) {
        const uint32_t prev = atomicAdd(&a.counters[tile_y * gridDim.x + tile_x], 1u);
        *last_flag = (prev == gridDim.z - 1) ? 1u : 0u;
      }
      tc::named_barrier_sync(1, 128);
      if (*last_flag) {
        __threadfence();
        float* src = a.ws + (size_t)(tile_y * gridDim.x + tile_x) * (kBM * kBN) + q * 32 + lane;
        if (a.epi.kind == kEpiNone) {
#pragma unroll
          for (int c = 0; c < kBN; c += 16) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              v[j] = __ldcg(src + (size_t)(c + j) * kBM);
              __stcg(src + (size_t)(c + j) * kBM, 0.f);
            }
            store_chunk(a, x, y_base + c, v);
          }
        } else {
          pair_finalize<kBN>(a, tile_x, a.ws + (size_t)(tile_y * gridDim.x + tile_x) * (kBM * kBN), (q & 1) * 32 + lane, q >> 1,
                             y_base, pair_pos);
        }
        if (threadIdx.x == 64) a.counters[tile_y * gridDim.x + tile_x] = 0;
      }
    }
  }

  pipe.finish(kTmemCols);
}

// ---- host side -------------------------------------------------------------------------------------

template <int kBN, int kStages, bool kFp8, bool kScaled>
std::string launch(const CUtensorMap& mx, const CUtensorMap& my, const GemmArgs& a, dim3 grid, cudaStream_t stream) {
  using L = SmemLayout<kBN, kStages>;
  auto kern = gemm_tn_kernel<kBN, kStages, kFp8, kScaled>;
  const std::string err = reserve_dynamic_smem(kern, L::kTotal);
  if (!err.empty()) return err;
  const cudaError_t e = launch_chained(kern, grid, dim3(kThreads), L::kTotal, stream, mx, my, a);
  return e == cudaSuccess ? "" : std::string("GEMM launch failed: ") + cudaGetErrorString(e);
}

// TDX_GEMM_CTAS_PER_SM=2 halves the operand ring of the tiles up to 128 columns so that two CTAs share an SM:
// a weight-streaming grid of up to 296 tiles is then resident at once and its CTAs finish together,
// instead of a full wave followed by a partly filled one. Default 1 (the measured configuration).
bool two_ctas_per_sm() {
  static const bool on = [] {
    const char* e = std::getenv("TDX_GEMM_CTAS_PER_SM");
    return e != nullptr && std::atoi(e) == 2;
  }();
  return on;
}

template <bool kFp8, bool kScaled>
std::string launch_bn(int bn, const CUtensorMap& mx, const CUtensorMap& my, const GemmArgs& a, dim3 grid, cudaStream_t s) {
  if (two_ctas_per_sm()) {
    switch (bn) {
      case 16: return launch<16, 5, kFp8, kScaled>(mx, my, a, grid, s);
      case 32: return launch<32, 4, kFp8, kScaled>(mx, my, a, grid, s);
      case 64: return launch<64, 4, kFp8, kScaled>(mx, my, a, grid, s);
      case 128:   // 3 x 32 KB per CTA: the epilogue of one CTA overlaps the main loop of the other
        if constexpr (!kScaled) return launch<128, 3, kFp8, kScaled>(mx, my, a, grid, s);
        break;
    }
  }
  switch (bn) {
    case 16: return launch<16, 10, kFp8, kScaled>(mx, my, a, grid, s);
    case 32: return launch<32, 8, kFp8, kScaled>(mx, my, a, grid, s);
    case 64: return launch<64, 8, kFp8, kScaled>(mx, my, a, grid, s);
    case 128:
      if constexpr (!kScaled) return launch<128, 6, kFp8, kScaled>(mx, my, a, grid, s);
      break;
    case 256:
      if constexpr (!kScaled) return launch<256, 4, kFp8, kScaled>(mx, my, a, grid, s);
      break;
  }
  return "unsupported tile width";
}

}  // namespace

int gemm_pick_block_n(int y_rows, bool scaled) {
  const int cap = scaled ? 64 : 256;   // the promoting epilogue keeps one fp32 accumulator per column in registers
  for (int bn : {16, 32, 64, 128, 256})
    if (bn <= cap && y_rows <= bn) return bn;
  return cap;
}

std::string gemm_tn(const GemmProblem& g, cudaStream_t stream) {
  const bool fp8 = g.elem_size == 1;
  const bool scaled = g.x_scale != nullptr || g.y_scale != nullptr;
  if (scaled && !(fp8 && g.x_scale && g.y_scale)) return "block scales need fp8 operands and scales for both of them";
  const int epb = kSwizzleBytes / g.elem_size;
  if (g.k <= 0 || g.k % epb) return "K must be a positive multiple of " + std::to_string(epb);
  if (g.x_rows <= 0 || g.y_rows <= 0) return "";
  const int bn = g.block_n > 0 ? g.block_n : gemm_pick_block_n(g.y_rows, scaled);
  GemmArgs a{};
  a.x_rows = g.x_rows;
  a.y_rows = g.y_rows;
  a.kblocks = g.k / epb;
  int splits = g.splits < 1 ? 1 : g.splits;
  const int epi = g.epi.kind;
  if (epi != kEpiNone) {
    // the pair epilogues live in the split-K finalizer
    if (a.kblocks < 2) return "a pair epilogue needs K of at least two 128-byte blocks";
    if (splits < 2) splits = 2;
    if (epi == kEpiRopeKv) {
      if (g.epi.q_heads < 0 || g.epi.kv_heads < 1 || g.x_rows != (g.epi.q_heads + 2 * g.epi.kv_heads) * kBM)
        return "rope epilogue: X must hold (q_heads + 2 kv_heads) heads of 128 rows";
      if (!g.epi.positions || !g.epi.cos_sin || !g.epi.k_cache || !g.epi.v_cache || g.epi.max_pos < 1 || g.epi.cache_seq < 1)
        return "rope epilogue: positions, angle table and caches are required";
    } else if (epi == kEpiSiluMul) {
      if (scaled) return "silu epilogue: block-scaled operands are not supported";
      if (g.epi.ffn < 64 || g.epi.ffn % 64 || g.x_rows != 2 * g.epi.ffn) return "silu epilogue: X must be [2 ffn, k] with ffn a multiple of 64";
    } else {
      return "unknown pair epilogue";
    }
  }
  if (splits > a.kblocks) splits = a.kblocks;
  a.kblocks_per_split = (a.kblocks + splits - 1) / splits;
  splits = (a.kblocks + a.kblocks_per_split - 1) / a.kblocks_per_split;
  a.out = g.out;
  a.sx = g.sx;
  a.sy = g.sy;
  a.out_dtype = g.out_dtype;
  a.idesc = fp8 ? tc::make_idesc(kBM, bn, 0, 0) : tc::make_idesc(kBM, bn, g.elem_kind == kBF16 ? 1 : 0, g.elem_kind == kBF16 ? 1 : 0);
  a.status = g.status;
  const dim3 grid(epi == kEpiSiluMul ? g.epi.ffn / 64 : (g.x_rows + kBM - 1) / kBM, (g.y_rows + bn - 1) / bn, splits);
  if (epi != kEpiNone && splits < 2) return "a pair epilogue needs at least two K splits";
  a.epi = g.epi;
  if (splits > 1) {
    if (!g.ws || !g.counters) return "split-K needs a workspace";
    a.ws_ld = grid.y * bn;
    if ((size_t)grid.x * grid.y * kBM * bn * sizeof(float) > g.ws_bytes || (size_t)grid.x * grid.y > g.counter_count)
      return "split-K workspace is too small for this problem";
    a.ws = g.ws;
    a.counters = g.counters;
  }
  a.x_scale = g.x_scale;
  a.y_scale = g.y_scale;
  a.x_scale_per_row = g.x_scale_per_row;
  a.y_scale_per_row = g.y_scale_per_row;
  a.scale_kb = a.kblocks;
  a.x_static = g.x_static;
  CUtensorMap mx, my;
  // silu epilogue: the X tile arrives as two boxes of 64 rows (gate rows, then the up rows of the same features)
  std::string err = tma::kmajor_2d(&mx, g.x, g.x_rows, g.k, g.ldx, g.elem_size, g.elem_kind, epi == kEpiSiluMul ? 64 : kBM);
  if (!err.empty()) return err;
  err = tma::kmajor_2d(&my, g.y, g.y_rows, g.k, g.ldy, g.elem_size, g.elem_kind, bn);
  if (!err.empty()) return err;
  if (fp8) return scaled ? launch_bn<true, true>(bn, mx, my, a, grid, stream) : launch_bn<true, false>(bn, mx, my, a, grid, stream);
  return launch_bn<false, false>(bn, mx, my, a, grid, stream);
}

}  // namespace tdx
