"""Standalone hot ops against plain PyTorch fp32 statements of the same math."""
import pytest
import torch

import torch_dist_ext_b200  # noqa: F401  (loads the library)
from torch_dist_ext_b200.ops import activation, norm, quant, rope
from torch_dist_ext_b200.ops import reference as ref
from torch_dist_ext_b200.utils.config import OUT_FP8_BLOCK128, OUT_FP8_TOKEN

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,cols", [(1, 4096), (33, 5120), (257, 7168), (16, 128)])
def test_rmsnorm(dtype, rows, cols):
    x = torch.randn(rows, cols, device="cuda").to(dtype)
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).to(dtype)
    y = norm.rmsnorm(x, w, 1e-6)
    xf = x.float()
    e = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float())
    tol = {torch.float32: 2e-5, torch.float16: 4e-3, torch.bfloat16: 3.2e-2}[dtype]
    assert (y.float() - e).abs().max().item() <= tol * max(1.0, e.abs().max().item())


@pytest.mark.parametrize("block", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_quant_fp8(dtype, block):
    x = (torch.randn(131, 7168, device="cuda") * 3).to(dtype)
    q, s = quant.quant_fp8(x, block_scaled=block)
    e_q, e_s = ref.quantize_fp8(x.float(), OUT_FP8_BLOCK128 if block else OUT_FP8_TOKEN)
    assert torch.allclose(s, e_s, rtol=1e-6)
    # codes equal up to one step where the product x * (1/scale) lands on a rounding boundary
    got, want = q.float(), e_q.float()
    assert bool(((got - want).abs() <= torch.maximum(got.abs(), want.abs()) * 0.125 + 2.0 ** -9).all())
    assert (q.view(torch.uint8) != e_q.view(torch.uint8)).float().mean().item() < 0.02
    back = ref.dequantize_fp8(q, s)
    assert (back - x.float()).abs().max().item() <= x.float().abs().max().item() * 2.0 ** -4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_silu_mul(dtype):
    gu = torch.randn(67, 2 * 14336 // 8, device="cuda").to(dtype)
    out, _ = activation.silu_mul(gu)
    inter = gu.shape[-1] // 2
    e = torch.nn.functional.silu(gu[:, :inter].float()) * gu[:, inter:].float()
    assert (out.float() - e).abs().max().item() <= 2e-2 * max(1.0, e.abs().max().item())
    q, s = activation.silu_mul(gu, quant_block128=True)
    back = ref.dequantize_fp8(q, s)
    assert (back - e).abs().max().item() <= e.abs().max().item() * 2.0 ** -3


def test_rope_matches_rotate_half():
    tokens, hq, hk, dim = 19, 32, 8, 128
    cache = rope.build_cos_sin_cache(4096, dim, theta=5e5)
    pos = torch.randint(0, 4096, (tokens,), device="cuda")
    qkv = torch.randn(tokens, (hq + 2 * hk) * dim, device="cuda", dtype=torch.bfloat16)
    q = qkv[:, : hq * dim].view(tokens, hq, dim)
    k = qkv[:, hq * dim: (hq + hk) * dim].view(tokens, hk, dim)
    e_q, e_k = rope.rope_reference(q, pos, cache), rope.rope_reference(k, pos, cache)
    rope.rope_(q, k, pos, cache)   # strided views into the fused qkv buffer, rotated in place
    assert (q.float() - e_q.float()).abs().max().item() <= 3.2e-2
    assert (k.float() - e_k.float()).abs().max().item() <= 3.2e-2


def test_rope_append_kv_writes_the_cache_rows():
    tokens, hq, hk, dim, smax = 5, 8, 2, 128, 40
    cache = rope.build_cos_sin_cache(smax, dim)
    pos = torch.tensor([3, 0, 39, 17, 8], device="cuda")
    qkv = torch.randn(tokens, (hq + 2 * hk) * dim, device="cuda", dtype=torch.bfloat16)
    q = qkv[:, : hq * dim].view(tokens, hq, dim)
    k = qkv[:, hq * dim: (hq + hk) * dim].view(tokens, hk, dim)
    v = qkv[:, (hq + hk) * dim:].view(tokens, hk, dim)
    e_k = rope.rope_reference(k, pos, cache)
    e_q = rope.rope_reference(q, pos, cache)
    kc = torch.zeros(8, smax, hk, dim, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    rope.rope_append_kv_(q, k, v, pos, cache, kc, vc)
    idx = torch.arange(tokens, device="cuda")
    assert (q.float() - e_q.float()).abs().max().item() <= 3.2e-2
    assert torch.equal(kc[idx, pos], k) and (k.float() - e_k.float()).abs().max().item() <= 3.2e-2
    assert torch.equal(vc[idx, pos], v)
    assert kc.abs().sum().item() == kc[idx, pos].abs().sum().item()      # nothing else was touched
