// Registration of the standalone ops (normalisation, quantisation, RoPE, activation), the
// tcgen05 GEMMs, the fused GEMM+collective ops and the decode-attention kernel.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "tdx/bindings.h"
#include "tdx/gemm.h"
#include "tdx/ops.h"

namespace tdx_torch {

using at::Tensor;

static int dtype_code(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return tdx::kF32;
    case at::kHalf: return tdx::kF16;
    case at::kBFloat16: return tdx::kBF16;
    default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
  }
  return -1;
}

static cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// residual add + RMSNorm (+ fp8 quant) without communication: the single-rank form of the fused op.
int64_t fused_add_rmsnorm(const Tensor& x, const c10::optional<Tensor>& residual_in, const Tensor& gamma,
                          c10::optional<Tensor> residual_out, Tensor norm_out, c10::optional<Tensor> scale_out,
                          double eps, int64_t out_mode) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "x must be a contiguous CUDA tensor");
  const c10::cuda::CUDAGuard guard(x.device());
  tdx::ArParams p{};
  p.rank = 0;
  p.nranks = 1;
  p.hidden = (int32_t)x.size(-1);
  p.tokens = (int32_t)(x.numel() / std::max<int64_t>(1, x.size(-1)));
  p.in = x.data_ptr();
  p.residual_in = residual_in.has_value() && residual_in->defined() ? residual_in->data_ptr() : nullptr;
  p.residual_out = residual_out.has_value() && residual_out->defined() ? residual_out->data_ptr() : nullptr;
  p.gamma = gamma.data_ptr();
  p.norm_out = norm_out.data_ptr();
  p.scale_out = scale_out.has_value() && scale_out->defined() ? scale_out->data_ptr<float>() : nullptr;
  p.eps = (float)eps;
  p.dtype = dtype_code(x);
  p.out_mode = (int32_t)out_mode;
  p.algo = tdx::kAlgoLocal;
  TORCH_CHECK(gamma.numel() == p.hidden && gamma.scalar_type() == x.scalar_type(), "gamma must be [hidden] in x's dtype");
  TORCH_CHECK(norm_out.numel() == x.numel(), "norm_out has the wrong size");
  tdx::LaunchPlan used{};
  const std::string err = tdx::launch_allreduce(p, cur_stream(), &used);
  TORCH_CHECK(err.empty(), "fused_add_rmsnorm: ", err);
  return used.grid;
}

void quant_fp8(const Tensor& x, Tensor q, Tensor scales, bool block128) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && q.is_contiguous() && scales.is_contiguous(), "contiguous CUDA tensors expected");
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t cols = x.size(-1), rows = x.numel() / std::max<int64_t>(1, cols);
  TORCH_CHECK(q.numel() == x.numel() && q.element_size() == 1, "q must be a 1-byte tensor of x's shape");
  TORCH_CHECK(scales.scalar_type() == at::kFloat && scales.numel() == (block128 ? rows * (cols / 128) : rows), "scales has the wrong size");
  const std::string err = tdx::quant_fp8(x.data_ptr(), q.data_ptr(), scales.data_ptr<float>(), (int)rows, (int)cols,
                                         dtype_code(x), block128, cur_stream());
  TORCH_CHECK(err.empty(), "quant_fp8: ", err);
}

void silu_mul(const Tensor& gate_up, Tensor out, c10::optional<Tensor> scales) {
  TORCH_CHECK(gate_up.is_cuda() && gate_up.is_contiguous() && out.is_contiguous(), "contiguous CUDA tensors expected");
  const c10::cuda::CUDAGuard guard(gate_up.device());
  const int64_t inter = gate_up.size(-1) / 2, rows = gate_up.numel() / std::max<int64_t>(1, gate_up.size(-1));
  const bool quant = scales.has_value() && scales->defined();
  TORCH_CHECK(out.numel() == rows * inter, "out must be [rows, inter]");
  if (quant) {
    TORCH_CHECK(out.element_size() == 1 && scales->scalar_type() == at::kFloat && scales->numel() == rows * (inter / 128),
                "fp8 output needs [rows, inter/128] fp32 scales");
  } else {
    TORCH_CHECK(out.scalar_type() == gate_up.scalar_type(), "out must have the input dtype");
  }
  const std::string err = tdx::silu_mul(gate_up.data_ptr(), out.data_ptr(), quant ? scales->data_ptr<float>() : nullptr,
                                        (int)rows, (int)inter, dtype_code(gate_up), quant, cur_stream());
  TORCH_CHECK(err.empty(), "silu_mul: ", err);
}

Tensor attention_prefill_probe() {
  Tensor out = at::zeros({3, 64, 8}, at::TensorOptions().dtype(at::kLong));
  const std::string err = tdx::attention_prefill_probe(reinterpret_cast<unsigned long long*>(out.data_ptr<int64_t>()), 3 * 64 * 8);
  TORCH_CHECK(err.empty(), "attention_prefill_probe: ", err);
  return out;
}

void argmax_pack(const Tensor& logits, int64_t index_base, int64_t rank, int64_t nranks, Tensor pack) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.scalar_type() == at::kFloat && logits.stride(1) == 1,
              "logits must be a CUDA fp32 [tokens, vocab] tensor with unit stride along the vocabulary");
  TORCH_CHECK(pack.is_cuda() && pack.device() == logits.device() && pack.scalar_type() == at::kFloat && pack.is_contiguous() &&
              pack.numel() == logits.size(0) * 4 * nranks, "pack must be a contiguous fp32 [tokens, 4 * nranks] tensor");
  const c10::cuda::CUDAGuard guard(logits.device());
  const std::string err = tdx::argmax_pack(logits.data_ptr<float>(), logits.stride(0), (int)logits.size(0), (int)logits.size(1),
                                           (int)index_base, (int)rank, (int)nranks, pack.data_ptr<float>(), cur_stream());
  TORCH_CHECK(err.empty(), "argmax_pack: ", err);
}

void select_token(const Tensor& gathered, int64_t nranks, Tensor out) {
  TORCH_CHECK(gathered.is_cuda() && gathered.scalar_type() == at::kFloat && gathered.is_contiguous() && gathered.dim() == 2 &&
              gathered.size(1) == 4 * nranks, "candidates must be a contiguous fp32 [tokens, 4 * nranks] tensor");
  TORCH_CHECK(out.is_cuda() && out.device() == gathered.device() && out.scalar_type() == at::kLong && out.is_contiguous() &&
              out.numel() == gathered.size(0), "out must be a contiguous int64 [tokens] tensor");
  const c10::cuda::CUDAGuard guard(gathered.device());
  const std::string err = tdx::select_token(gathered.data_ptr<float>(), (int)gathered.size(0), (int)nranks,
                                            out.data_ptr<int64_t>(), cur_stream());
  TORCH_CHECK(err.empty(), "select_token: ", err);
}

void rope_impl(Tensor q, Tensor k, const Tensor& positions, const Tensor& cos_sin_cache, const c10::optional<Tensor>& v,
               c10::optional<Tensor> k_cache, c10::optional<Tensor> v_cache);

void rope_(Tensor q, Tensor k, const Tensor& positions, const Tensor& cos_sin_cache) {
  rope_impl(q, k, positions, cos_sin_cache, c10::nullopt, c10::nullopt, c10::nullopt);
}

// rope on q and k, and append of the rotated k row and the v row to the decode KV cache, in one kernel
void rope_append_kv_(Tensor q, Tensor k, const Tensor& v, const Tensor& positions, const Tensor& cos_sin_cache, Tensor k_cache,
                     Tensor v_cache) {
  rope_impl(q, k, positions, cos_sin_cache, v, k_cache, v_cache);
}

void rope_impl(Tensor q, Tensor k, const Tensor& positions, const Tensor& cos_sin_cache, const c10::optional<Tensor>& v,
               c10::optional<Tensor> k_cache, c10::optional<Tensor> v_cache) {
  TORCH_CHECK(q.is_cuda() && k.is_cuda() && q.dim() == 3 && k.dim() == 3, "q and k must be [tokens, heads, dim] CUDA tensors");
  TORCH_CHECK(q.stride(2) == 1 && k.stride(2) == 1 && q.stride(1) == q.size(2) && k.stride(1) == k.size(2), "heads must be densely packed");
  TORCH_CHECK(positions.scalar_type() == at::kLong && positions.is_cuda() && positions.numel() == q.size(0), "positions must be int64 [tokens]");
  TORCH_CHECK(cos_sin_cache.scalar_type() == at::kFloat && cos_sin_cache.is_contiguous() && cos_sin_cache.size(-1) == q.size(2), "cos_sin_cache must be fp32 [max_pos, dim]");
  TORCH_CHECK(q.scalar_type() == k.scalar_type() && q.size(2) == k.size(2) && q.size(0) == k.size(0), "q and k must agree in dtype, tokens and dim");
  const int64_t esz = q.element_size();
  TORCH_CHECK((q.stride(0) * esz) % 16 == 0 && (k.stride(0) * esz) % 16 == 0 && (uintptr_t)q.data_ptr() % 16 == 0 && (uintptr_t)k.data_ptr() % 16 == 0,
              "q and k rows must be 16-byte aligned");
  const c10::cuda::CUDAGuard guard(q.device());
  const void* vp = nullptr;
  void *kc = nullptr, *vc = nullptr;
  int64_t vs = 0, cb = 0, cs = 0;
  if (k_cache.has_value() && k_cache->defined()) {
    TORCH_CHECK(v.has_value() && v_cache.has_value(), "rope_append_kv_: v and both caches are needed");
    TORCH_CHECK(k_cache->dim() == 4 && k_cache->sizes() == v_cache->sizes() && k_cache->strides() == v_cache->strides() &&
                    k_cache->size(2) == k.size(1) && k_cache->size(3) == k.size(2) && k_cache->size(0) >= q.size(0) &&
                    k_cache->stride(3) == 1 && k_cache->stride(2) == k.size(2) && k_cache->scalar_type() == k.scalar_type(),
                "rope_append_kv_: caches must be [B >= tokens, S, k_heads, dim] with dense heads, in k's dtype");
    TORCH_CHECK(v->dim() == 3 && v->sizes() == k.sizes() && v->stride(2) == 1 && v->stride(1) == v->size(2) &&
                    (v->stride(0) * esz) % 16 == 0 && (uintptr_t)v->data_ptr() % 16 == 0, "rope_append_kv_: v must look like k");
    TORCH_CHECK((k_cache->stride(1) * esz) % 16 == 0 && (k_cache->stride(0) * esz) % 16 == 0, "rope_append_kv_: cache rows must be 16-byte aligned");
    vp = v->data_ptr(); vs = v->stride(0);
    kc = k_cache->data_ptr(); vc = v_cache->data_ptr();
    cb = k_cache->stride(0); cs = k_cache->stride(1);
  }
  const std::string err = tdx::rope_inplace(q.data_ptr(), k.data_ptr(), positions.data_ptr<int64_t>(), cos_sin_cache.data_ptr<float>(),
                                            (int)q.size(0), (int)q.size(1), (int)k.size(1), (int)q.size(2), q.stride(0),
                                            k.stride(0), dtype_code(q), cur_stream(), vp, vs, kc, vc, cb, cs);
  TORCH_CHECK(err.empty(), "rope: ", err);
}

// D[x, y] = sum_k X[x, k] * Y[y, k] written to out.flatten()[x * sx + y * sy] (tcgen05 GEMM).
// `out_x_rows`: how many x rows the output holds when that is not X's row count (the silu epilogue halves it).
static tdx::GemmProblem gemm_problem(const Tensor& x, const Tensor& y, Tensor& out, int64_t sx, int64_t sy,
                                     const c10::optional<Tensor>& status, int64_t out_x_rows = -1) {
  TORCH_CHECK(x.is_cuda() && y.is_cuda() && out.is_cuda() && x.dim() == 2 && y.dim() == 2, "gemm_tn: 2-D CUDA operands expected");
  TORCH_CHECK(x.stride(1) == 1 && y.stride(1) == 1, "gemm_tn: operands must be K-major (unit stride along K)");
  TORCH_CHECK(x.size(1) == y.size(1) && x.scalar_type() == y.scalar_type(), "gemm_tn: operands disagree in K or dtype");
  tdx::GemmProblem g{};
  g.x = x.data_ptr();
  g.y = y.data_ptr();
  g.x_rows = (int)x.size(0);
  g.y_rows = (int)y.size(0);
  g.k = (int)x.size(1);
  g.ldx = x.stride(0);
  g.ldy = y.stride(0);
  g.elem_size = (int)x.element_size();
  TORCH_CHECK(g.elem_size == 1 || x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf,
              "gemm_tn: operands must be bfloat16, float16 or float8_e4m3fn");
  g.elem_kind = x.scalar_type() == at::kHalf ? tdx::kF16 : tdx::kBF16;
  g.out = out.data_ptr();
  g.sx = sx;
  g.sy = sy;
  g.out_dtype = dtype_code(out);
  const int64_t max_idx = ((out_x_rows >= 0 ? out_x_rows : g.x_rows) - 1) * sx + (g.y_rows - 1) * sy;
  TORCH_CHECK(g.x_rows == 0 || g.y_rows == 0 || (max_idx < out.numel() && sx >= 1 && sy >= 1), "gemm_tn: output strides exceed the output tensor");
  if (status.has_value() && status->defined()) g.status = reinterpret_cast<uint32_t*>(status->data_ptr<int>());
  return g;
}

void gemm_tn(const Tensor& x, const Tensor& y, Tensor out, int64_t sx, int64_t sy, int64_t block_n, int64_t splits,
             const c10::optional<Tensor>& ws, const c10::optional<Tensor>& counters, const c10::optional<Tensor>& status,
             const c10::optional<Tensor>& x_scale, const c10::optional<Tensor>& y_scale, bool x_scale_per_row,
             bool y_scale_per_row, bool x_static) {
  tdx::GemmProblem g = gemm_problem(x, y, out, sx, sy, status);
  g.x_static = x_static;
  const c10::cuda::CUDAGuard guard(x.device());
  g.block_n = (int)block_n;
  g.splits = (int)splits;
  if (ws.has_value() && ws->defined()) {
    TORCH_CHECK(ws->scalar_type() == at::kFloat && counters.has_value() && counters->scalar_type() == at::kInt, "gemm_tn: workspace dtypes");
    g.ws = ws->data_ptr<float>();
    g.ws_bytes = (size_t)ws->numel() * 4;
    g.counters = reinterpret_cast<uint32_t*>(counters->data_ptr<int>());
    g.counter_count = (size_t)counters->numel();
  }
  if (x_scale.has_value() && x_scale->defined()) {
    TORCH_CHECK(y_scale.has_value() && y_scale->defined(), "gemm_tn: both operands need scales");
    TORCH_CHECK(x_scale->scalar_type() == at::kFloat && y_scale->scalar_type() == at::kFloat && x_scale->is_contiguous() && y_scale->is_contiguous(), "gemm_tn: scales must be contiguous float32");
    const int64_t kb = g.k / 128;
    TORCH_CHECK(x_scale->numel() == (x_scale_per_row ? g.x_rows : (g.x_rows + 127) / 128) * kb, "gemm_tn: x_scale has the wrong size");
    TORCH_CHECK(y_scale->numel() == (y_scale_per_row ? g.y_rows : (g.y_rows + 127) / 128) * kb, "gemm_tn: y_scale has the wrong size");
    g.x_scale = x_scale->data_ptr<float>();
    g.y_scale = y_scale->data_ptr<float>();
    g.x_scale_per_row = x_scale_per_row;
    g.y_scale_per_row = y_scale_per_row;
  }
  const std::string err = tdx::gemm_tn(g, cur_stream());
  TORCH_CHECK(err.empty(), "gemm_tn: ", err);
}

static void gemm_scratch(tdx::GemmProblem& g, const Tensor& ws, const Tensor& counters, const char* who) {
  TORCH_CHECK(ws.is_cuda() && counters.is_cuda() && ws.scalar_type() == at::kFloat && counters.scalar_type() == at::kInt, who,
              ": the split-K scratch must be float32 / int32 CUDA tensors");
  g.ws = ws.data_ptr<float>();
  g.ws_bytes = (size_t)ws.numel() * 4;
  g.counters = reinterpret_cast<uint32_t*>(counters.data_ptr<int>());
  g.counter_count = (size_t)counters.numel();
}

// Fused qkv projection of a decode step whose split-K finalizer rotates the query and key heads and appends keys and
// values to the caches: out[t, :] = rope(a[t] @ w^T), k_cache[t, positions[t]] / v_cache[t, positions[t]] = the new rows.
// w [(q_heads + 2 kv_heads) * 128, K] (bf16 / fp16, or e4m3 with 128 x 128 scales and 1 x 128 scales on a).
void gemm_tn_rope_kv(const Tensor& w, const Tensor& a, Tensor out, int64_t block_n, int64_t splits, const Tensor& ws,
                     const Tensor& counters, const c10::optional<Tensor>& status, const c10::optional<Tensor>& w_scale,
                     const c10::optional<Tensor>& a_scale, const Tensor& positions, const Tensor& cos_sin, Tensor k_cache,
                     Tensor v_cache, int64_t q_heads, int64_t kv_heads) {
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.stride(1) == 1 && out.size(0) == a.size(0) && out.size(1) == w.size(0),
              "gemm_tn_rope_kv: out must be [tokens, (q_heads + 2 kv_heads) * 128] with unit stride along the features");
  tdx::GemmProblem g = gemm_problem(w, a, out, 1, out.stride(0), status);
  const c10::cuda::CUDAGuard guard(w.device());
  g.x_static = 1;
  g.block_n = (int)block_n;
  g.splits = (int)splits;
  gemm_scratch(g, ws, counters, "gemm_tn_rope_kv");
  if (w_scale.has_value() && w_scale->defined()) {
    TORCH_CHECK(a_scale.has_value() && a_scale->defined(), "gemm_tn_rope_kv: both operands need scales");
    TORCH_CHECK(w_scale->scalar_type() == at::kFloat && a_scale->scalar_type() == at::kFloat && w_scale->is_contiguous() && a_scale->is_contiguous(),
                "gemm_tn_rope_kv: scales must be contiguous float32");
    const int64_t kb = g.k / 128;
    TORCH_CHECK(w_scale->numel() == (g.x_rows + 127) / 128 * kb && a_scale->numel() == (int64_t)g.y_rows * kb, "gemm_tn_rope_kv: scales have the wrong size");
    g.x_scale = w_scale->data_ptr<float>();
    g.y_scale = a_scale->data_ptr<float>();
    g.x_scale_per_row = 0;
    g.y_scale_per_row = 1;
  }
  TORCH_CHECK(positions.is_cuda() && positions.scalar_type() == at::kLong && positions.is_contiguous() && positions.numel() >= a.size(0),
              "gemm_tn_rope_kv: positions must be a contiguous int64 CUDA tensor with one entry per token");
  TORCH_CHECK(cos_sin.is_cuda() && cos_sin.scalar_type() == at::kFloat && cos_sin.is_contiguous() && cos_sin.dim() == 2 && cos_sin.size(1) == 128,
              "gemm_tn_rope_kv: the angle table must be contiguous float32 [max_pos, 128]");
  for (const Tensor* c : {&k_cache, &v_cache})
    TORCH_CHECK(c->is_cuda() && c->scalar_type() == at::kBFloat16 && c->dim() == 4 && c->size(0) >= a.size(0) && c->size(2) == kv_heads &&
                    c->size(3) == 128 && c->stride(3) == 1 && c->stride(2) == 128,
                "gemm_tn_rope_kv: caches must be bfloat16 [batch >= tokens, seq, kv_heads, 128] with contiguous heads");
  TORCH_CHECK(k_cache.sizes() == v_cache.sizes() && k_cache.strides() == v_cache.strides(), "gemm_tn_rope_kv: the caches must agree in shape");
  for (const Tensor* t : std::initializer_list<const Tensor*>{&a, &out, &ws, &counters, &positions, &cos_sin, &k_cache, &v_cache})
    TORCH_CHECK(t->device() == w.device(), "gemm_tn_rope_kv: every tensor must live on the weights' device");
  g.epi.kind = tdx::kEpiRopeKv;
  g.epi.q_heads = (int)q_heads;
  g.epi.kv_heads = (int)kv_heads;
  g.epi.positions = positions.data_ptr<int64_t>();
  g.epi.cos_sin = cos_sin.data_ptr<float>();
  g.epi.max_pos = (int)cos_sin.size(0);
  g.epi.cache_seq = (int)k_cache.size(1);
  g.epi.k_cache = k_cache.data_ptr();
  g.epi.v_cache = v_cache.data_ptr();
  g.epi.cache_batch_stride = k_cache.stride(0);
  g.epi.cache_pos_stride = k_cache.stride(1);
  const std::string err = tdx::gemm_tn(g, cur_stream());
  TORCH_CHECK(err.empty(), "gemm_tn_rope_kv: ", err);
}

// Gate/up projection of a decode step whose split-K finalizer applies the activation:
// out[t, f] = silu(a[t] . w[f]) * (a[t] . w[ffn + f]) for w [2 ffn, K] (bf16 / fp16).
void gemm_tn_silu_mul(const Tensor& w, const Tensor& a, Tensor out, int64_t block_n, int64_t splits, const Tensor& ws,
                      const Tensor& counters, const c10::optional<Tensor>& status) {
  TORCH_CHECK(w.dim() == 2 && w.size(0) % 2 == 0, "gemm_tn_silu_mul: w must be [2 ffn, K]");
  const int64_t ffn = w.size(0) / 2;
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.stride(1) == 1 && out.size(0) == a.size(0) && out.size(1) == ffn,
              "gemm_tn_silu_mul: out must be [tokens, ffn] with unit stride along the features");
  tdx::GemmProblem g = gemm_problem(w, a, out, 1, out.stride(0), status, ffn);
  const c10::cuda::CUDAGuard guard(w.device());
  g.x_static = 1;
  g.block_n = (int)block_n;
  g.splits = (int)splits;
  gemm_scratch(g, ws, counters, "gemm_tn_silu_mul");
  for (const Tensor* t : std::initializer_list<const Tensor*>{&a, &out, &ws, &counters})
    TORCH_CHECK(t->device() == w.device(), "gemm_tn_silu_mul: every tensor must live on the weights' device");
  g.epi.kind = tdx::kEpiSiluMul;
  g.epi.ffn = (int)ffn;
  const std::string err = tdx::gemm_tn(g, cur_stream());
  TORCH_CHECK(err.empty(), "gemm_tn_silu_mul: ", err);
}

// The same product on 256 x 256 tiles computed by CTA pairs (tcgen05.mma.cta_group::2).
void gemm_tn_pair(const Tensor& x, const Tensor& y, Tensor out, int64_t sx, int64_t sy, const c10::optional<Tensor>& status,
                  const c10::optional<Tensor>& ws, const c10::optional<Tensor>& counters) {
  tdx::GemmProblem g = gemm_problem(x, y, out, sx, sy, status);
  if (ws.has_value() && ws->defined() && counters.has_value() && counters->defined()) {
    TORCH_CHECK(ws->scalar_type() == at::kFloat && counters->scalar_type() == at::kInt && ws->is_cuda() && counters->is_cuda(),
                "gemm_tn_pair: scratch must be float32 / int32 CUDA tensors");
    g.ws = ws->data_ptr<float>();
    g.ws_bytes = (size_t)ws->numel() * 4;
    g.counters = reinterpret_cast<uint32_t*>(counters->data_ptr<int>());
    g.counter_count = (size_t)counters->numel();
  }
  const c10::cuda::CUDAGuard guard(x.device());
  const std::string err = tdx::gemm_tn_pair(g, cur_stream());
  TORCH_CHECK(err.empty(), "gemm_tn_pair: ", err);
}

// The same product by a persistent grid with the accumulator double-buffered in tensor memory.
void gemm_tn_persistent(const Tensor& x, const Tensor& y, Tensor out, int64_t sx, int64_t sy, const c10::optional<Tensor>& status) {
  tdx::GemmProblem g = gemm_problem(x, y, out, sx, sy, status);
  const c10::cuda::CUDAGuard guard(x.device());
  const std::string err = tdx::gemm_tn_persistent(g, cur_stream());
  TORCH_CHECK(err.empty(), "gemm_tn_persistent: ", err);
}

static void attention_decode_impl(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& seq_lens, Tensor& out,
                                  Tensor& partial, int64_t nsplit, double scale, const c10::optional<Tensor>& status,
                                  bool tensor_cores) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 3 && k_cache.dim() == 4 && v_cache.dim() == 4, "attention_decode: q [B, Hq, D], caches [B, S, Hkv, D]");
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k_cache.scalar_type() == at::kBFloat16 && v_cache.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16, "attention_decode: bfloat16 tensors");
  TORCH_CHECK(q.stride(2) == 1 && q.stride(1) == q.size(2) && out.is_contiguous(), "attention_decode: q heads densely packed, out contiguous");
  TORCH_CHECK(k_cache.stride(3) == 1 && k_cache.stride(2) == k_cache.size(3) && k_cache.strides() == v_cache.strides() && k_cache.sizes() == v_cache.sizes(), "attention_decode: cache layout [B, S, Hkv, D] with dense heads");
  TORCH_CHECK(seq_lens.scalar_type() == at::kInt && seq_lens.is_cuda() && seq_lens.numel() == q.size(0), "attention_decode: seq_lens int32 [B]");
  TORCH_CHECK(partial.scalar_type() == at::kFloat && partial.is_contiguous(), "attention_decode: partial must be contiguous fp32");
  TORCH_CHECK(q.size(2) == 128 && k_cache.size(3) == 128, "attention_decode: head dimension must be 128");
  TORCH_CHECK(out.numel() == q.size(0) * q.size(1) * q.size(2), "attention_decode: out must hold [B, Hq, D] elements");
  TORCH_CHECK(k_cache.size(0) == q.size(0), "attention_decode: q and the caches disagree on the batch size");
  for (const Tensor* t : {&k_cache, &v_cache, &seq_lens, (const Tensor*)&out, (const Tensor*)&partial})
    TORCH_CHECK(t->is_cuda() && t->device() == q.device(), "attention_decode: every tensor must live on q's device");
  if (status.has_value() && status->defined())
    TORCH_CHECK(status->is_cuda() && status->device() == q.device() && status->scalar_type() == at::kInt, "attention_decode: status must be an int32 tensor on q's device");
  const c10::cuda::CUDAGuard guard(q.device());
  const auto fn = tensor_cores ? &tdx::attention_decode_tc : &tdx::attention_decode;
  const std::string err = fn(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), seq_lens.data_ptr<int>(),
                                                partial.data_ptr<float>(), (size_t)partial.numel(), out.data_ptr(), (int)q.size(0),
                                                (int)q.size(1), (int)k_cache.size(2), (int)q.size(2), (int)k_cache.size(1),
                                                q.stride(0), k_cache.stride(0), k_cache.stride(1), (int)nsplit, (float)scale, cur_stream(),
                                                status.has_value() && status->defined() ? reinterpret_cast<uint32_t*>(status->data_ptr<int>()) : nullptr);
  TORCH_CHECK(err.empty(), "attention_decode: ", err);
}

void attention_decode(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& seq_lens, Tensor out,
                      Tensor partial, int64_t nsplit, double scale, const c10::optional<Tensor>& status) {
  attention_decode_impl(q, k_cache, v_cache, seq_lens, out, partial, nsplit, scale, status, false);
}

// Both products of a chunk on the tensor cores (tcgen05).
void attention_decode_tc(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& seq_lens, Tensor out,
                         Tensor partial, int64_t nsplit, double scale, const c10::optional<Tensor>& status) {
  attention_decode_impl(q, k_cache, v_cache, seq_lens, out, partial, nsplit, scale, status, true);
}

// Causal attention over one prompt, both products on the tensor cores (tcgen05).
void attention_prefill_tc(const Tensor& q, const Tensor& k, const Tensor& v, Tensor out, double scale,
                          const c10::optional<Tensor>& status) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "attention_prefill_tc: q [S, Hq, D], k / v [S, Hkv, D]");
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16 &&
                  out.scalar_type() == at::kBFloat16, "attention_prefill_tc: bfloat16 tensors");
  auto dense_heads = [](const Tensor& t) { return t.stride(2) == 1 && t.stride(1) == t.size(2); };
  TORCH_CHECK(dense_heads(q) && dense_heads(k) && dense_heads(v) && out.is_contiguous(),
              "attention_prefill_tc: heads densely packed inside a row, out contiguous");
  TORCH_CHECK(k.size(0) == q.size(0) && v.sizes() == k.sizes() && out.numel() == q.size(0) * q.size(1) * q.size(2),
              "attention_prefill_tc: shapes disagree");
  const c10::cuda::CUDAGuard guard(q.device());
  const std::string err = tdx::attention_prefill_tc(
      q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), (int)q.size(0), (int)q.size(1), (int)k.size(1), (int)q.size(2),
      q.stride(0), k.stride(0), v.stride(0), (float)scale, cur_stream(),
      status.has_value() && status->defined() ? reinterpret_cast<uint32_t*>(status->data_ptr<int>()) : nullptr);
  TORCH_CHECK(err.empty(), "attention_prefill_tc: ", err);
}

static tdx::Workspace* workspace_of(const Tensor& table) {
  TORCH_CHECK(table.is_cuda(), "workspace must be the CUDA tensor returned by get_workspace");
  tdx::Workspace* ws = tdx::Workspace::from_table(table.data_ptr());
  TORCH_CHECK(ws != nullptr, "workspace tensor does not belong to a registered CommWorkspace");
  return ws;
}

// Row-parallel linear + all-reduce (or reduce-scatter) + residual + RMSNorm in one kernel.
void gemm_ar_rmsnorm(const Tensor& a, const Tensor& w, const c10::optional<Tensor>& residual_in, const Tensor& gamma,
                     c10::optional<Tensor> residual_out, Tensor norm_out, c10::optional<Tensor> scale_out, double eps,
                     const Tensor& workspace, int64_t out_mode, bool scatter_only, const c10::optional<Tensor>& status,
                     int64_t splits, const c10::optional<Tensor>& splitk_ws, const c10::optional<Tensor>& splitk_counters,
                     const c10::optional<Tensor>& a_scale, const c10::optional<Tensor>& w_scale, bool one_hop) {
  tdx::Workspace* ws = workspace_of(workspace);
  TORCH_CHECK(a.is_cuda() && w.is_cuda() && a.dim() == 2 && w.dim() == 2 && a.size(1) == w.size(1), "gemm_ar_rmsnorm: a [tokens, k], w [hidden, k]");
  const bool fp8 = a.scalar_type() == at::kFloat8_e4m3fn;
  TORCH_CHECK((fp8 || a.scalar_type() == at::kBFloat16) && w.scalar_type() == a.scalar_type() && gamma.scalar_type() == at::kBFloat16,
              "gemm_ar_rmsnorm: bfloat16 operands, or float8_e4m3fn operands with block scales; bfloat16 gamma");
  TORCH_CHECK(a.stride(1) == 1 && w.stride(1) == 1 && gamma.is_contiguous() && norm_out.is_contiguous(), "gemm_ar_rmsnorm: K-major operands, contiguous outputs");
  const c10::cuda::CUDAGuard guard(a.device());
  tdx::FusedGemmProblem g{};
  ws->fill_params(&g.ar);
  const int64_t tokens = a.size(0), hidden = w.size(0);
  const int64_t rows = scatter_only ? (tokens + g.ar.nranks - 1) / g.ar.nranks : tokens;
  g.ar.tokens = (int)tokens;
  g.ar.hidden = (int)hidden;
  g.ar.in = nullptr;
  auto opt_ptr = [&](const c10::optional<Tensor>& t, const char* name) -> void* {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->is_contiguous() && t->numel() == rows * hidden && t->scalar_type() == at::kBFloat16, name, " must be contiguous bf16 [", rows, ", ", hidden, "]");
    return t->data_ptr();
  };
  g.elem_size = fp8 ? 1 : 2;
  if (fp8) {
    const int64_t kb = a.size(1) / 128;
    TORCH_CHECK(a.size(1) % 128 == 0 && a_scale.has_value() && w_scale.has_value() && a_scale->defined() && w_scale->defined(),
                "gemm_ar_rmsnorm: e4m3 operands need K % 128 == 0 and both scale tensors");
    TORCH_CHECK(a_scale->is_cuda() && w_scale->is_cuda() && a_scale->scalar_type() == at::kFloat && w_scale->scalar_type() == at::kFloat &&
                    a_scale->is_contiguous() && w_scale->is_contiguous() && a_scale->numel() == tokens * kb &&
                    w_scale->numel() == ((hidden + 127) / 128) * kb,
                "gemm_ar_rmsnorm: scales must be contiguous float32 [tokens, K/128] and [hidden/128, K/128]");
    g.a_scale = a_scale->data_ptr<float>();
    g.w_scale = w_scale->data_ptr<float>();
  }
  g.ar.residual_in = opt_ptr(residual_in, "residual_in");
  g.ar.residual_out = opt_ptr(residual_out, "residual_out");
  g.ar.gamma = gamma.data_ptr();
  g.one_hop = one_hop;
  TORCH_CHECK(gamma.numel() == hidden && norm_out.numel() == rows * hidden, "gemm_ar_rmsnorm: gamma / norm_out sizes");
  g.ar.norm_out = norm_out.data_ptr();
  g.ar.scale_out = nullptr;
  if (out_mode != tdx::kOutSame) {
    TORCH_CHECK(scale_out.has_value() && scale_out->scalar_type() == at::kFloat && scale_out->numel() == rows * (hidden / 128) && norm_out.element_size() == 1,
                "gemm_ar_rmsnorm: fp8 output needs 1-byte norm_out and [rows, hidden/128] fp32 scales");
    g.ar.scale_out = scale_out->data_ptr<float>();
  } else {
    TORCH_CHECK(norm_out.scalar_type() == at::kBFloat16, "gemm_ar_rmsnorm: norm_out must be bf16");
  }
  g.ar.eps = (float)eps;
  g.ar.dtype = tdx::kBF16;
  g.ar.out_mode = (int)out_mode;
  g.ar.scatter_only = scatter_only ? 1 : 0;
  g.a = a.data_ptr();
  g.w = w.data_ptr();
  g.k = (int)a.size(1);
  g.lda = a.stride(0);
  g.ldw = w.stride(0);
  g.status = status.has_value() && status->defined() ? reinterpret_cast<uint32_t*>(status->data_ptr<int>()) : nullptr;
  g.splits = (int)splits;
  if (splitk_ws.has_value() && splitk_ws->defined() && splitk_counters.has_value() && splitk_counters->defined()) {
    TORCH_CHECK(splitk_ws->scalar_type() == at::kFloat && splitk_counters->scalar_type() == at::kInt, "gemm_ar_rmsnorm: split-K scratch dtypes");
    g.ws = splitk_ws->data_ptr<float>();
    g.ws_bytes = (size_t)splitk_ws->numel() * 4;
    g.counters = reinterpret_cast<uint32_t*>(splitk_counters->data_ptr<int>());
    g.counter_count = (size_t)splitk_counters->numel();
  }
  const std::string err = tdx::gemm_ar_rmsnorm(g, cur_stream());
  TORCH_CHECK(err.empty(), "gemm_ar_rmsnorm: ", err);
}

// All-gather of the sequence-parallel activation shards fused with a column-parallel linear.
void ag_gemm(const Tensor& x_shard, const Tensor& w, Tensor out, int64_t tokens, const Tensor& workspace,
             const c10::optional<Tensor>& status) {
  tdx::Workspace* ws = workspace_of(workspace);
  TORCH_CHECK(x_shard.is_cuda() && x_shard.is_contiguous() && w.is_cuda() && w.stride(1) == 1 && out.is_contiguous(), "ag_gemm: contiguous CUDA tensors");
  TORCH_CHECK(x_shard.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16, "ag_gemm: bfloat16 tensors");
  const c10::cuda::CUDAGuard guard(x_shard.device());
  tdx::AgGemmProblem g{};
  g.rank = ws->rank();
  g.nranks = ws->world_size();
  for (int r = 0; r < g.nranks; ++r) g.peer[r] = ws->peer_base(r);
  g.layout = ws->layout();
  g.tokens = (int)tokens;
  g.k = (int)w.size(1);
  const int64_t my_rows = (tokens - g.rank + g.nranks - 1) / g.nranks;
  TORCH_CHECK(x_shard.dim() == 2 && x_shard.size(1) == g.k && x_shard.size(0) >= my_rows, "ag_gemm: x_shard must hold this rank's rows [", my_rows, ", ", g.k, "]");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == tokens && out.size(1) == w.size(0), "ag_gemm: out must be [tokens, weight rows]");
  g.x_shard = x_shard.data_ptr();
  g.w = w.data_ptr();
  g.ldw = w.stride(0);
  g.out_rows = (int)w.size(0);
  g.out = out.data_ptr();
  g.ldo = out.stride(0);
  g.status = status.has_value() && status->defined() ? reinterpret_cast<uint32_t*>(status->data_ptr<int>()) : nullptr;
  g.timeout_ns = ws->timeout_ns();
  g.host_status = ws->host_status_device_ptr();
  const std::string err = tdx::ag_gemm(g, cur_stream());
  TORCH_CHECK(err.empty(), "ag_gemm: ", err);
}

void register_extra_ops(torch::Library& m) {
  m.def("gemm_ar_rmsnorm(Tensor a, Tensor w, Tensor? residual_in, Tensor gamma, Tensor(a!)? residual_out, Tensor(b!) norm_out, "
        "Tensor(c!)? scale_out, float eps, Tensor workspace, int out_mode, bool scatter_only, Tensor(d!)? status, "
        "int splits, Tensor(e!)? splitk_ws, Tensor(f!)? splitk_counters, Tensor? a_scale=None, Tensor? w_scale=None, "
        "bool one_hop=False) -> ()",
        &gemm_ar_rmsnorm);
  m.def("attention_decode(Tensor q, Tensor k_cache, Tensor v_cache, Tensor seq_lens, Tensor(a!) out, Tensor(b!) partial, "
        "int nsplit, float scale, Tensor(c!)? status) -> ()", &attention_decode);
  m.def("attention_decode_tc(Tensor q, Tensor k_cache, Tensor v_cache, Tensor seq_lens, Tensor(a!) out, Tensor(b!) partial, "
        "int nsplit, float scale, Tensor(c!)? status) -> ()", &attention_decode_tc);
  m.def("attention_prefill_tc(Tensor q, Tensor k, Tensor v, Tensor(a!) out, float scale, Tensor(b!)? status) -> ()",
        &attention_prefill_tc);
  m.def("ag_gemm(Tensor x_shard, Tensor w, Tensor(a!) out, int tokens, Tensor workspace, Tensor(b!)? status) -> ()", &ag_gemm);
  m.def("gemm_tn(Tensor x, Tensor y, Tensor(a!) out, int sx, int sy, int block_n, int splits, Tensor(b!)? ws, "
        "Tensor(c!)? counters, Tensor(d!)? status, Tensor? x_scale, Tensor? y_scale, bool x_scale_per_row, "
        "bool y_scale_per_row, bool x_static=False) -> ()", &gemm_tn);
  m.def("gemm_tn_rope_kv(Tensor w, Tensor a, Tensor(a!) out, int block_n, int splits, Tensor(b!) ws, Tensor(c!) counters, "
        "Tensor(d!)? status, Tensor? w_scale, Tensor? a_scale, Tensor positions, Tensor cos_sin, Tensor(e!) k_cache, "
        "Tensor(f!) v_cache, int q_heads, int kv_heads) -> ()", &gemm_tn_rope_kv);
  m.def("gemm_tn_silu_mul(Tensor w, Tensor a, Tensor(a!) out, int block_n, int splits, Tensor(b!) ws, Tensor(c!) counters, "
        "Tensor(d!)? status) -> ()", &gemm_tn_silu_mul);
  m.def("gemm_tn_pair(Tensor x, Tensor y, Tensor(a!) out, int sx, int sy, Tensor(b!)? status, Tensor(c!)? ws=None, "
        "Tensor(d!)? counters=None) -> ()", &gemm_tn_pair);
  m.def("gemm_tn_persistent(Tensor x, Tensor y, Tensor(a!) out, int sx, int sy, Tensor(b!)? status) -> ()", &gemm_tn_persistent);
  m.def("fused_add_rmsnorm(Tensor x, Tensor? residual_in, Tensor gamma, Tensor(a!)? residual_out, Tensor(b!) norm_out, "
        "Tensor(c!)? scale_out, float eps, int out_mode) -> int", &fused_add_rmsnorm);
  m.def("quant_fp8(Tensor x, Tensor(a!) q, Tensor(b!) scales, bool block128) -> ()", &quant_fp8);
  m.def("silu_mul(Tensor gate_up, Tensor(a!) out, Tensor(b!)? scales) -> ()", &silu_mul);
  m.def("attention_prefill_probe() -> Tensor", &attention_prefill_probe);
  m.def("argmax_pack(Tensor logits, int index_base, int rank, int nranks, Tensor(a!) pack) -> ()", &argmax_pack);
  m.def("select_token(Tensor gathered, int nranks, Tensor(a!) out) -> ()", &select_token);
  m.def("rope_(Tensor(a!) q, Tensor(b!) k, Tensor positions, Tensor cos_sin_cache) -> ()", &rope_);
  m.def("rope_append_kv_(Tensor(a!) q, Tensor(b!) k, Tensor v, Tensor positions, Tensor cos_sin_cache, Tensor(c!) k_cache, "
        "Tensor(d!) v_cache) -> ()", &rope_append_kv_);
}

}  // namespace tdx_torch
