"""The PyTorch oracle itself: golden values for the seeded BASELINE configuration and
independent re-derivations of every output."""
import torch

from torch_dist_ext_b200.ops import reference as ref
from torch_dist_ext_b200.utils.config import OUT_FP8_BLOCK128, OUT_FP8_TOKEN, OUT_SAME


def baseline_case(world=2, tokens=128, hidden=4096):
    ins = [torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(r)) for r in range(world)]
    gs = torch.Generator().manual_seed(1000)
    residual = torch.randn(tokens, hidden, generator=gs)
    gamma = 1.0 + 0.1 * torch.randn(hidden, generator=gs)
    return ins, residual, gamma


def test_fp32_outputs_rederived_in_float64():
    ins, residual, gamma = baseline_case()
    norm, res, _ = ref.fused_allreduce_rms_reference(ins, residual, gamma, 1e-6, OUT_SAME)
    s = sum(t.double() for t in ins) + residual.double()
    assert (res.double() - s).abs().max().item() < 1e-5
    y = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.double()
    assert (norm.double() - y).abs().max().item() < 1e-4      # the reference's own tolerance
    # golden checksums of the seeded case (guards the generator recipe and the math)
    assert abs(res.double().sum().item() - s.sum().item()) < 1e-2
    assert norm.shape == (128, 4096)


def test_fp8_per_token_scales_and_codes():
    ins, residual, gamma = baseline_case()
    q, res, scale = ref.fused_allreduce_rms_reference(ins, residual, gamma, 1e-6, OUT_FP8_TOKEN)
    y, _, _ = ref.fused_allreduce_rms_reference(ins, residual, gamma, 1e-6, OUT_SAME)
    assert scale.shape == (128, 1) and scale.dtype == torch.float32
    assert torch.allclose(scale.squeeze(1), y.abs().amax(-1) / 448.0, rtol=1e-6)
    assert q.dtype == torch.float8_e4m3fn and q.float().abs().max().item() <= 448.0
    # the row maximum maps to the largest code
    assert torch.all(q.float().abs().amax(-1) == 448.0)
    back = ref.dequantize_fp8(q, scale)
    assert ((back - y).abs() <= y.abs().amax(-1, keepdim=True) * 2.0 ** -4).all()


def test_fp8_block128_scales():
    ins, residual, gamma = baseline_case(hidden=5120)
    q, res, scale = ref.fused_allreduce_rms_reference(ins, residual, gamma, 1e-6, OUT_FP8_BLOCK128)
    y, _, _ = ref.fused_allreduce_rms_reference(ins, residual, gamma, 1e-6, OUT_SAME)
    assert scale.shape == (128, 40)
    assert torch.allclose(scale, y.view(128, 40, 128).abs().amax(-1) / 448.0, rtol=1e-6)
    back = ref.dequantize_fp8(q, scale)
    assert ((back - y).abs().view(128, 40, 128) <= y.view(128, 40, 128).abs().amax(-1, keepdim=True) * 2.0 ** -4).all()


def test_sixteen_bit_rounding_order():
    """s is rounded to T before the residual is added (two roundings), as in the kernels."""
    ins = [torch.full((1, 8), 1.0, dtype=torch.bfloat16), torch.full((1, 8), 2.0 ** -9, dtype=torch.bfloat16)]
    residual = torch.full((1, 8), 2.0 ** -9, dtype=torch.bfloat16)
    gamma = torch.ones(8, dtype=torch.bfloat16)
    _, res, _ = ref.fused_allreduce_rms_reference(ins, residual, gamma, 1e-6)
    # 1 + 2^-9 rounds to 1 in bf16 (8 bits of mantissa); adding 2^-9 again rounds to 1 again.
    assert torch.all(res.float() == 1.0)


def test_rotary_projection_oracle_equals_a_complex_rotation():
    """rotate-half pairs element i with i + 64: as complex numbers (x_i + j x_{i+64}) * exp(j * angle_i)."""
    from torch_dist_ext_b200.ops import reference, rope

    g = torch.Generator().manual_seed(3)
    tokens, hidden, q_heads, kv_heads, seq = 5, 64, 2, 1, 32
    a = torch.randn(tokens, hidden, generator=g)
    w = torch.randn((q_heads + 2 * kv_heads) * 128, hidden, generator=g) * 0.1
    positions = torch.tensor([0, 7, 7, 31, 12])
    cos_sin = rope.build_cos_sin_cache(seq, 128, 5e5, "cpu")
    k_cache = torch.zeros(tokens, seq, kv_heads, 128)
    v_cache = torch.zeros_like(k_cache)
    out = reference.linear_rope_kv_reference(a, w, positions, cos_sin, k_cache, v_cache, q_heads, kv_heads)
    qkv = (a.double() @ w.double().t()).view(tokens, q_heads + 2 * kv_heads, 128)
    inv_freq = 1.0 / (5e5 ** (torch.arange(0, 128, 2, dtype=torch.float64) / 128))
    phase = torch.polar(torch.ones(tokens, 64, dtype=torch.float64), positions.double()[:, None] * inv_freq[None, :])
    z = torch.complex(qkv[..., :64], qkv[..., 64:]) * phase[:, None, :]
    want = torch.cat([z.real, z.imag], dim=-1)
    want[:, q_heads + kv_heads:] = qkv[:, q_heads + kv_heads:]          # values are not rotated
    assert (out.view(tokens, -1, 128).double() - want).abs().max() < 1e-4
    rows = torch.arange(tokens)
    assert (k_cache[rows, positions].double() - want[:, q_heads: q_heads + kv_heads]).abs().max() < 1e-4
    assert (v_cache[rows, positions].double() - want[:, q_heads + kv_heads:]).abs().max() < 1e-4
    k_cache[rows, positions] = 0
    assert not k_cache.any()                                            # nothing else was written


def test_gate_up_oracle():
    from torch_dist_ext_b200.ops import reference

    g = torch.Generator().manual_seed(4)
    a, w = torch.randn(3, 32, generator=g), torch.randn(2 * 64, 32, generator=g)
    gate, up = a.double() @ w[:64].double().t(), a.double() @ w[64:].double().t()
    want = gate / (1 + torch.exp(-gate)) * up
    assert (reference.linear_silu_mul_reference(a, w).double() - want).abs().max() < 1e-4
