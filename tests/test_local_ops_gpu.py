"""Single-rank (world_size == 1) path: residual add + RMSNorm (+ fp8 quant) without communication,
through the public API."""
import pytest
import torch

import torch_dist_ext_b200 as tdx
from helpers import TOL
from torch_dist_ext_b200.utils.config import OUT_FP8_BLOCK128, OUT_FP8_TOKEN, OUT_SAME

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def env():
    tdx.setup_env(0, 1, max_size_in_bytes=8 << 20)
    yield
    tdx.teardown_env()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tokens,hidden", [(1, 4096), (129, 1024), (300, 8192), (7, 508 * 2), (64, 16384)])
def test_public_api_world1(dtype, tokens, hidden):
    if dtype == torch.float32 and hidden > 8192:
        pytest.skip("fp32 rows are limited to 8192 columns")
    g = torch.Generator().manual_seed(tokens)
    x = torch.randn(tokens, hidden, generator=g).to(dtype).cuda()
    r = torch.randn(tokens, hidden, generator=g).to(dtype).cuda()
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype).cuda()
    ws = tdx.get_workspace(x)
    norm, res = tdx.allreduce_rms(0, 1, x, r, w, 1e-6, ws)
    e_norm, e_res, _ = tdx.reference.fused_allreduce_rms_reference([x], r, w, 1e-6)
    assert torch.equal(res, e_res)
    assert (norm.float() - e_norm.float()).abs().max().item() <= TOL[dtype] * max(1.0, e_norm.float().abs().max().item())
    tdx.check_status()


@pytest.mark.parametrize("block", [False, True])
def test_fp8_world1(block):
    x = torch.randn(77, 7168, device="cuda", dtype=torch.bfloat16)
    r = torch.randn_like(x)
    w = torch.ones(7168, device="cuda", dtype=torch.bfloat16)
    q, scales, res = tdx.allreduce_rms_fp8(x, r, w, 1e-6, block_scaled=block)
    mode = OUT_FP8_BLOCK128 if block else OUT_FP8_TOKEN
    e_q, e_res, e_s = tdx.reference.fused_allreduce_rms_reference([x], r, w, 1e-6, mode)
    assert torch.equal(res, e_res)
    assert torch.allclose(scales, e_s, rtol=1e-5)
    y = tdx.reference.dequantize_fp8(q, scales)
    e_y, _, _ = tdx.reference.fused_allreduce_rms_reference([x], r, w, 1e-6, OUT_SAME)
    # e4m3 keeps 3 mantissa bits: relative error <= 2^-4 of the block/token maximum
    assert (y - e_y.float()).abs().max().item() <= e_y.float().abs().max().item() * 2.0 ** -4


def test_float64_inputs_give_the_fp32_result_as_doubles():
    """The reference's dispatch covers double but its arithmetic stays in fp32; so does this path."""
    x = torch.randn(9, 1024, device="cuda", dtype=torch.float64)
    r = torch.randn_like(x)
    w = 1 + 0.1 * torch.randn(1024, device="cuda", dtype=torch.float64)
    norm, res = tdx.allreduce_rms(0, 1, x, r, w, 1e-6, tdx.get_workspace(x))
    assert norm.dtype == torch.float64 and res.dtype == torch.float64
    n32, r32 = tdx.allreduce_rms(0, 1, x.float(), r.float(), w.float(), 1e-6, tdx.get_workspace(x))
    assert torch.equal(norm, n32.double()) and torch.equal(res, r32.double())
    want = (x + r)
    want = want * torch.rsqrt(want.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    assert (norm - want).abs().max().item() <= 1e-4
