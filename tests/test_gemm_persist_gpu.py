"""The persistent tcgen05 GEMM (one CTA per SM walks the tiles, double-buffered accumulator) against
fp32 PyTorch math and against the one-tile-per-CTA kernel.

The kernel is the library's default for prefill-sized problems (``TDX_GEMM_PERSIST=0`` turns it off).
Shapes cover fewer tiles than SMs, several tiles per CTA (accumulator buffers reused), ragged M and N,
one K block, and K loops longer than the operand ring."""
import pytest
import torch

from torch_dist_ext_b200.ops import gemm

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (256, 512, 1024), (300, 520, 512), (2048, 4096, 256), (4096, 28672, 128),
                                   (1024, 256, 8192)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_persistent_gemm_matches_fp32(m, n, k, dtype):
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = (torch.randn(m, k, device="cuda", generator=g) * 0.5).to(dtype)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.5).to(dtype)
    out = gemm.linear(a, w, persistent=True)
    torch.cuda.synchronize()
    assert gemm.pipeline_status() == 0
    base = gemm.linear(a, w, persistent=False, splits=1)
    # same products accumulated in fp32 in the same K order: at most a last-bit difference of the output type
    assert torch.allclose(out.float(), base.float(), rtol=1e-2, atol=1e-2)
    if m * n * k <= 1 << 32:
        ref = a.float() @ w.float().t()
        assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2
