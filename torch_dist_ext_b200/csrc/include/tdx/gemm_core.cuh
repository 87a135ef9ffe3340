// Building blocks shared by the tcgen05 GEMM kernels: tile constants, the shared-memory ring,
// barrier set-up with TMEM allocation, the TMA producer loop and the MMA issue loop. A kernel
// composes them with its own epilogue (plain store, split-K reduction, block-scale promotion, or
// a push of the tile into a peer GPU's memory).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "tdx/comm.h"
#include "tdx/tc.cuh"

namespace tdx {
namespace gemm_core {

constexpr int kBM = 128;            // tile rows (tcgen05.mma M)
constexpr int kSwizzleBytes = 128;  // one K block = 128 bytes per row (64 bf16 / 128 fp8)
constexpr uint32_t kWaitLimit = 1u << 22;

// ---- output of a tile -----------------------------------------------------------------------------------
// `Args` describes the destination: out, sx, sy (D[x, y] -> out[x * sx + y * sy]), out_dtype (kF32 / kF16 /
// kBF16), x_rows, y_rows.
template <typename Args>
__device__ __forceinline__ void store_out(const Args& a, int64_t idx, float v) {
  if (a.out_dtype == kBF16) static_cast<__nv_bfloat16*>(a.out)[idx] = __float2bfloat16(v);
  else if (a.out_dtype == kF16) static_cast<__half*>(a.out)[idx] = __float2half(v);
  else static_cast<float*>(a.out)[idx] = v;
}

// Writes 16 consecutive y columns of row x (values already final): two 16-byte stores when the 16 columns are
// contiguous 16-bit values at an aligned address, else element by element with bounds checks.
template <typename Args>
__device__ __forceinline__ void store_chunk(const Args& a, int x, int y0, const float (&v)[16]) {
  if (x >= a.x_rows) return;
  if (a.sy == 1 && a.out_dtype != kF32 && y0 + 16 <= a.y_rows && ((a.sx * 2) % 16 == 0) && (y0 % 8 == 0) &&
      (reinterpret_cast<uintptr_t>(a.out) % 16 == 0)) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (a.out_dtype == kBF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(a.out) + ((int64_t)x * a.sx + y0) * 2);
    dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
    dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (y0 + i < a.y_rows) store_out(a, (int64_t)x * a.sx + (int64_t)(y0 + i) * a.sy, v[i]);
  }
}

// Block-scale promotion of one K block: acc[j] += partial[j] * xs * ys[j] for the kBN (<= 64) columns of this
// thread's row. The partial products are fetched from tensor memory with ONE load (one round trip per K block);
// the column scales sit two per lane (`ys_lo`: columns 0-31, `ys_hi`: 32-63) and are handed round by shuffles.
// Warp-wide: every lane of the warp calls it.
template <int kBN>
__device__ __forceinline__ void promote_block(uint32_t taddr, float xs, float ys_lo, float ys_hi, float (&acc)[kBN]) {
  static_assert(kBN == 16 || kBN == 32 || kBN == 64, "promotion handles 16, 32 or 64 columns");
  uint32_t v[kBN];
  if constexpr (kBN == 64) {
    tc::tmem_ld_x64(taddr, v);
  } else if constexpr (kBN == 32) {
    tc::tmem_ld_x32(taddr, v);
  } else {
    float f[16];
    tc::tmem_ld_16(taddr, f);
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(f[j]);
  }
#pragma unroll
  for (int j = 0; j < kBN; ++j) {
    const float ys = __shfl_sync(0xffffffffu, j < 32 ? ys_lo : ys_hi, j & 31);
    acc[j] = fmaf(__uint_as_float(v[j]), xs * ys, acc[j]);
  }
}

template <int kBN, int kStages>
struct SmemLayout {
  static constexpr int kXBytes = kBM * kSwizzleBytes;
  static constexpr int kYBytes = kBN * kSwizzleBytes;
  static constexpr int kStageBytes = kXBytes + kYBytes;
  static constexpr int kBarrierOffset = kStages * kStageBytes;
  static constexpr int kPipelineBytes = kBarrierOffset + 1024;      // ring + barriers/scratch
  static constexpr int kTotal = kPipelineBytes + 1024;              // + alignment slack
};

template <int kBN, int kStages>
struct Pipeline {
  uint8_t* smem;            // 1024-byte aligned ring
  uint64_t* full;
  uint64_t* empty;
  uint64_t* acc_full;       // [2]
  uint64_t* acc_empty;      // [2]
  uint32_t* tmem_slot;
  volatile uint32_t* abort_flag;
  uint32_t* scratch;        // a few words for the kernel's own use
  uint32_t tmem_base;

  // Called by every thread of the CTA. Warp 1 allocates `tmem_cols` TMEM columns.
  __device__ __forceinline__ void init(uint8_t* smem_raw, uint32_t tmem_cols, const CUtensorMap* mx, const CUtensorMap* my) {
    using L = SmemLayout<kBN, kStages>;
    smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    full = reinterpret_cast<uint64_t*>(smem + L::kBarrierOffset);
    empty = full + kStages;
    acc_full = empty + kStages;
    acc_empty = acc_full + 2;
    tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    abort_flag = tmem_slot + 1;
    scratch = tmem_slot + 2;
    if (threadIdx.x == 0) {
      for (int s = 0; s < kStages; ++s) {
        tc::mbar_init(&full[s], 1);
        tc::mbar_init(&empty[s], 1);
      }
      for (int i = 0; i < 2; ++i) {
        tc::mbar_init(&acc_full[i], 1);
        tc::mbar_init(&acc_empty[i], 128);
      }
      *abort_flag = 0;
      tc::fence_barrier_init();
      tc::tma_prefetch_desc(mx);
      tc::tma_prefetch_desc(my);
    }
    if ((threadIdx.x >> 5) == 1) {
      tc::tmem_alloc(tmem_slot, tmem_cols);
      tc::tmem_relinquish();
    }
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    tmem_base = *tmem_slot;
  }

  __device__ __forceinline__ void fail(uint32_t* status) {
    *abort_flag = 1;
    if (status) atomicExch(status, (uint32_t)kTimeoutGemmPipeline);
  }

  // One thread. Streams `nkb` K blocks starting at block `kb0`. `gate_y` is called once, before the
  // first Y (narrow-side) tile is requested; X tiles of the first ring pass are requested before it,
  // so that a wait inside the gate overlaps the fetch of the wide operand.
  // `x_row1 >= 0`: the X tile is two runs of 64 rows, starting at x_row0 and x_row1, fetched by two copies through a
  // tensor map whose box is 64 rows (the second run lands 8 KB into the stage, where a 128-row box would have put
  // its rows 64-127: the swizzle pattern repeats every 1 KB, so the MMA sees one 128-row tile).
  template <int kElemsPerBlock, typename Gate>
  __device__ __forceinline__ void produce(const CUtensorMap* mx, const CUtensorMap* my, int x_row0, int y_row0, int kb0,
                                          int nkb, uint32_t* status, Gate gate_y, int x_row1 = -1) {
    produce_pick<kElemsPerBlock>(mx, x_row0, y_row0, kb0, nkb, status, gate_y, [my] { return my; }, x_row1);
  }

  // The same with the Y tensor map chosen only after the gate has passed (`*parity` odd: my1, else my0), for a Y
  // operand whose buffer is selected by state that may be read only behind the gate.
  template <int kElemsPerBlock, typename Gate>
  __device__ __forceinline__ void produce_late_y(const CUtensorMap* mx, const CUtensorMap* my0, const CUtensorMap* my1,
                                                 const uint32_t* parity, int x_row0, int y_row0, int kb0, int nkb,
                                                 uint32_t* status, Gate gate_y) {
    produce_pick<kElemsPerBlock>(mx, x_row0, y_row0, kb0, nkb, status, gate_y, [=] { return (*parity & 1u) ? my1 : my0; });
  }

  template <int kElemsPerBlock, typename Gate, typename PickY>
  __device__ __forceinline__ void produce_pick(const CUtensorMap* mx, int x_row0, int y_row0, int kb0, int nkb,
                                               uint32_t* status, Gate gate_y, PickY pick_y, int x_row1 = -1) {
    using L = SmemLayout<kBN, kStages>;
    const int first = nkb < kStages ? nkb : kStages;
    for (int i = 0; i < first; ++i) {
      tc::mbar_arrive_expect_tx(&full[i], L::kStageBytes);
      tc::tma_load_2d(smem + i * L::kStageBytes, mx, &full[i], (kb0 + i) * kElemsPerBlock, x_row0);
      if (x_row1 >= 0) tc::tma_load_2d(smem + i * L::kStageBytes + L::kXBytes / 2, mx, &full[i], (kb0 + i) * kElemsPerBlock, x_row1);
    }
    if (!gate_y()) {
      fail(status);
      return;
    }
    const CUtensorMap* my = pick_y();
    for (int i = 0; i < first; ++i)
      tc::tma_load_2d(smem + i * L::kStageBytes + L::kXBytes, my, &full[i], (kb0 + i) * kElemsPerBlock, y_row0);
    for (int i = first; i < nkb; ++i) {
      const int s = i % kStages;
      if (!tc::mbar_wait(&empty[s], ((i / kStages) - 1) & 1, kWaitLimit, abort_flag)) {
        fail(status);
        return;
      }
      uint8_t* sx = smem + s * L::kStageBytes;
      tc::mbar_arrive_expect_tx(&full[s], L::kStageBytes);
      tc::tma_load_2d(sx, mx, &full[s], (kb0 + i) * kElemsPerBlock, x_row0);
      if (x_row1 >= 0) tc::tma_load_2d(sx + L::kXBytes / 2, mx, &full[s], (kb0 + i) * kElemsPerBlock, x_row1);
      tc::tma_load_2d(sx + L::kXBytes, my, &full[s], (kb0 + i) * kElemsPerBlock, y_row0);
    }
  }

  // One thread. kScaled: every K block goes to its own TMEM buffer (two, alternating) and is handed to
  // the epilogue through acc_full/acc_empty; else all blocks accumulate into one buffer.
  template <bool kFp8, bool kScaled>
  __device__ __forceinline__ void issue(int nkb, uint32_t idesc, uint32_t* status) {
    using L = SmemLayout<kBN, kStages>;
    for (int i = 0; i < nkb; ++i) {
      const int s = i % kStages;
      if (!tc::mbar_wait(&full[s], (i / kStages) & 1, kWaitLimit, abort_flag)) {
        fail(status);
        return;
      }
      uint32_t acc_col = 0;
      if constexpr (kScaled) {
        const int buf = i & 1;
        if (i >= 2 && !tc::mbar_wait(&acc_empty[buf], ((i >> 1) - 1) & 1, kWaitLimit, abort_flag)) {
          fail(status);
          return;
        }
        acc_col = buf * kBN;
      }
      tc::fence_after_thread_sync();
      const uint32_t xa = tc::smem_u32(smem + s * L::kStageBytes);
      const uint64_t dx = tc::make_smem_desc_sw128(xa);
      const uint64_t dy = tc::make_smem_desc_sw128(xa + L::kXBytes);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        // one instruction covers 32 bytes of K; step the start address inside the swizzle span
        const uint32_t accumulate = kScaled ? (k > 0) : (i > 0 || k > 0);
        tc::umma<kFp8>(tmem_base + acc_col, dx + (uint64_t)(k * 2), dy + (uint64_t)(k * 2), idesc, accumulate);
      }
      tc::umma_commit(&empty[s]);  // stage reusable once these MMAs have read it
      if constexpr (kScaled) tc::umma_commit(&acc_full[i & 1]);
    }
    if constexpr (!kScaled) tc::umma_commit(&acc_full[0]);
  }

  // Called by every thread at the end of the kernel.
  __device__ __forceinline__ void finish(uint32_t tmem_cols) {
    tc::fence_before_thread_sync();
    __syncthreads();
    if (*abort_flag) {
      // let TMA copies that were already issued land before the CTA's shared memory goes away
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    if ((threadIdx.x >> 5) == 1) {
      tc::fence_after_thread_sync();
      tc::tmem_dealloc(tmem_base, tmem_cols);
    }
  }
};

}  // namespace gemm_core
}  // namespace tdx
