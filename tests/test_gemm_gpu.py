"""tcgen05 GEMM against torch.matmul in fp32 on the same (rounded) inputs."""
import pytest
import torch

from torch_dist_ext_b200.ops import gemm, quant
from torch_dist_ext_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def check(out, a, w, rtol):
    want = a.float() @ w.float().t()
    err = (out.float() - want).abs().max().item()
    assert err <= rtol * want.abs().max().item() + 1e-3, f"max err {err} vs scale {want.abs().max().item()}"


@pytest.mark.parametrize("m,n,k", [(1, 768, 4096), (16, 4096, 512), (64, 3584, 4096), (7, 256, 128), (128, 1024, 1792)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_decode_shapes_swapped(m, n, k, dtype):
    a = torch.randn(m, k, device="cuda").to(dtype)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(dtype)
    out = gemm.linear(a, w)
    assert out.shape == (m, n) and out.dtype == dtype
    check(out, a, w, 8e-3)
    assert gemm.pipeline_status() == 0


@pytest.mark.parametrize("m,n,k", [(256, 512, 1024), (2048, 1280, 4096), (300, 200, 192), (129, 4096, 512)])
def test_prefill_shapes_normal(m, n, k):
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    out = gemm.linear(a, w)
    check(out, a, w, 8e-3)
    assert gemm.pipeline_status() == 0


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
@pytest.mark.parametrize("swap", [True, False])
def test_split_k_and_orientation_agree(splits, swap):
    a = torch.randn(48, 2048, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(640, 2048, device="cuda") * 0.05).to(torch.bfloat16)
    out = gemm.linear(a, w, swap=swap, splits=splits)
    check(out, a, w, 8e-3)
    # the workspace must be left zeroed: a second call gives the same result
    out2 = gemm.linear(a, w, swap=swap, splits=splits)
    # (fp32 atomics add in varying order: the two results may differ by a bf16 rounding step)
    assert (out.float() - out2.float()).abs().max().item() <= 8e-3 * out.float().abs().max().item()


def test_fp32_output_and_strided_operands():
    big = torch.randn(32, 3 * 1024, device="cuda", dtype=torch.bfloat16)
    a = big[:, 1024:2048]            # row pitch 3072, K-major view
    w = (torch.randn(512, 1024, device="cuda") * 0.05).to(torch.bfloat16)
    out = gemm.linear(a, w, out_dtype=torch.float32)
    assert out.dtype == torch.float32
    check(out, a, w, 2e-3)


def test_fp8_plain():
    a = torch.randn(32, 1024, device="cuda").to(torch.float8_e4m3fn)
    w = (torch.randn(768, 1024, device="cuda")).to(torch.float8_e4m3fn)
    out = gemm.linear(a, w)
    check(out, a, w, 8e-3)


@pytest.mark.parametrize("m,n,k", [(1, 1280, 8192), (64, 1024, 1024), (33, 7168, 3584), (200, 512, 2048)])
def test_fp8_block_scaled(m, n, k):
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    a_q, a_s = quant.quant_fp8(a, block_scaled=True)
    w_q, w_s = gemm.quantize_weight_block128(w)
    out = gemm.linear_fp8_blockscaled(a_q, a_s, w_q, w_s)
    a_d = ref.dequantize_fp8(a_q, a_s)
    w_d = (w_q.float().view(n // 128, 128, k // 128, 128) * w_s.view(n // 128, 1, k // 128, 1)).view(n, k)
    want = a_d @ w_d.t()
    err = (out.float() - want).abs().max().item()
    assert err <= 1e-2 * want.abs().max().item() + 1e-3, err
    # and the quantised product stays close to the bf16 one
    full = a.float() @ w.float().t()
    assert (out.float() - full).abs().max().item() <= 0.08 * full.abs().max().item()
    assert gemm.pipeline_status() == 0
