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
