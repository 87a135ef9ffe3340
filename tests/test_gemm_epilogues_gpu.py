"""Decode GEMMs whose split-K finalizer does the next kernel's work: rotary embedding + KV append inside the qkv
projection, silu(gate) * up inside the gate/up projection. Each against a plain PyTorch fp32 statement of the same op."""
import pytest
import torch

from torch_dist_ext_b200.ops import gemm, quant, rope

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def tol(ref: torch.Tensor) -> float:
    return float(ref.abs().max()) * 2.0 ** -6 + 1e-3


def rope_kv_reference(qkv, positions, cos_sin, q_heads, kv_heads):
    t = qkv.shape[0]
    q = qkv[:, : q_heads * 128].view(t, q_heads, 128)
    k = qkv[:, q_heads * 128: (q_heads + kv_heads) * 128].view(t, kv_heads, 128)
    v = qkv[:, (q_heads + kv_heads) * 128:].view(t, kv_heads, 128)
    half = 64
    cs = cos_sin[positions].float()
    cos, sin = cs[:, None, :half], cs[:, None, half:]

    def rot(x):
        a, b = x[..., :half], x[..., half:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)

    return rot(q), rot(k), v


@pytest.mark.parametrize("tokens,hidden,q_heads,kv_heads", [(1, 512, 4, 1), (16, 4096, 4, 1), (50, 1024, 2, 2), (128, 512, 8, 8)])
def test_qkv_projection_rotates_and_appends(tokens, hidden, q_heads, kv_heads):
    g = torch.Generator(device=DEV).manual_seed(tokens)
    seq, batch = 96, tokens + 3
    a = torch.randn(tokens, hidden, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn((q_heads + 2 * kv_heads) * 128, hidden, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    positions = torch.randint(0, seq, (tokens,), device=DEV, generator=g)
    cos_sin = rope.build_cos_sin_cache(seq, 128, 5e5, DEV)
    k_cache = torch.zeros(batch, seq, kv_heads, 128, dtype=torch.bfloat16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    out = gemm.linear_rope_kv(a, w, positions, cos_sin, k_cache, v_cache, q_heads, kv_heads)
    ref = a.float() @ w.float().t()
    q, k, v = rope_kv_reference(ref, positions, cos_sin, q_heads, kv_heads)
    want = torch.cat([q.reshape(tokens, -1), k.reshape(tokens, -1), v.reshape(tokens, -1)], dim=1)
    assert (out.float() - want).abs().max() <= tol(want)
    rows = torch.arange(tokens, device=DEV)
    assert (k_cache[rows, positions].float() - k).abs().max() <= tol(k)
    assert (v_cache[rows, positions].float() - v).abs().max() <= tol(v)
    # nothing but the appended rows was written
    k_cache[rows, positions] = 0
    v_cache[rows, positions] = 0
    assert not k_cache.any() and not v_cache.any()
    # the split-K scratch is zero again: a plain product right after comes out right
    plain = gemm.linear(a, w)
    assert (plain.float() - ref).abs().max() <= tol(ref)
    assert gemm.pipeline_status(DEV) == 0


@pytest.mark.parametrize("tokens", [1, 16, 64])
def test_block_scaled_qkv_projection_rotates_and_appends(tokens):
    g = torch.Generator(device=DEV).manual_seed(100 + tokens)
    hidden, q_heads, kv_heads, seq = 1024, 3, 1, 40
    a = torch.randn(tokens, hidden, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn((q_heads + 2 * kv_heads) * 128, hidden, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    w_q, w_s = gemm.quantize_weight_block128(w)
    a_q, a_s = quant.quant_fp8(a, block_scaled=True)
    positions = torch.randint(0, seq, (tokens,), device=DEV, generator=g)
    cos_sin = rope.build_cos_sin_cache(seq, 128, 5e5, DEV)
    k_cache = torch.zeros(tokens, seq, kv_heads, 128, dtype=torch.bfloat16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    out = gemm.linear_rope_kv(a_q, w_q, positions, cos_sin, k_cache, v_cache, q_heads, kv_heads, a_scale=a_s, w_scale=w_s)
    # the oracle multiplies the dequantised operands: what is tested is the epilogue, not the quantisation
    a_d = (a_q.float().view(tokens, hidden // 128, 128) * a_s.view(tokens, hidden // 128, 1)).view(tokens, hidden)
    n = w_q.shape[0]
    w_d = (w_q.float().view(n // 128, 128, hidden // 128, 128) * w_s.view(n // 128, 1, hidden // 128, 1)).view(n, hidden)
    q, k, v = rope_kv_reference(a_d @ w_d.t(), positions, cos_sin, q_heads, kv_heads)
    want = torch.cat([q.reshape(tokens, -1), k.reshape(tokens, -1), v.reshape(tokens, -1)], dim=1)
    assert (out.float() - want).abs().max() <= tol(want)
    rows = torch.arange(tokens, device=DEV)
    assert (k_cache[rows, positions].float() - k).abs().max() <= tol(k)
    assert (v_cache[rows, positions].float() - v).abs().max() <= tol(v)
    assert gemm.pipeline_status(DEV) == 0


@pytest.mark.parametrize("tokens,hidden,ffn", [(1, 512, 64), (16, 4096, 1792), (37, 1024, 320), (128, 512, 1024)])
def test_gate_up_projection_applies_the_activation(tokens, hidden, ffn):
    g = torch.Generator(device=DEV).manual_seed(7 * tokens)
    a = torch.randn(tokens, hidden, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * ffn, hidden, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    out = gemm.linear_silu_mul(a, w)
    gu = a.float() @ w.float().t()
    want = torch.nn.functional.silu(gu[:, :ffn]) * gu[:, ffn:]
    assert out.shape == (tokens, ffn)
    assert (out.float() - want).abs().max() <= tol(want)
    plain = gemm.linear(a, w)
    assert (plain.float() - gu).abs().max() <= tol(gu)
    assert gemm.pipeline_status(DEV) == 0


def test_fused_epilogues_refuse_what_they_cannot_take():
    a = torch.randn(300, 512, device=DEV).to(torch.bfloat16)                       # prompt-sized: the tokens fill the 128-row side
    w = torch.randn(2 * 64, 512, device=DEV).to(torch.bfloat16)
    assert not gemm.fused_epilogue_fits(300, 512)
    with pytest.raises(AssertionError):
        gemm.linear_silu_mul(a, w)
    assert not gemm.fused_epilogue_fits(16, 64)                                     # one K block: nothing to split
