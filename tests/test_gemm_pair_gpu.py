"""The two-CTA (tcgen05.mma.cta_group::2) GEMM against fp32 PyTorch math.

The kernel is selected with ``linear(..., cta_pair=True)`` or ``TDX_GEMM_PAIR=1``. Shapes cover full tiles, ragged M and N, a single K block and a K loop longer
than the operand ring; every wait in the kernel is bounded, and the device status word is checked."""
import pytest
import torch

from torch_dist_ext_b200.ops import gemm

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (256, 256, 1024), (512, 768, 4096), (300, 520, 512), (1024, 256, 8192)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_pair_gemm_matches_fp32(m, n, k, dtype):
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = (torch.randn(m, k, device="cuda", generator=g) * 0.5).to(dtype)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.5).to(dtype)
    out = gemm.linear(a, w, cta_pair=True)
    torch.cuda.synchronize()
    assert gemm.pipeline_status() == 0
    ref = a.float() @ w.float().t()
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-2, err
    # the one-CTA kernel computes the same sums in the same order per K block: results agree closely
    base = gemm.linear(a, w, cta_pair=False)
    assert (out.float() - base.float()).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2


def test_pair_gemm_fp8_unscaled():
    g = torch.Generator(device="cuda").manual_seed(7)
    a = torch.randn(256, 512, device="cuda", generator=g).to(torch.float8_e4m3fn)
    w = torch.randn(512, 512, device="cuda", generator=g).to(torch.float8_e4m3fn)
    out = gemm.linear(a, w, cta_pair=True)
    torch.cuda.synchronize()
    assert gemm.pipeline_status() == 0
    ref = a.float() @ w.float().t()
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("m,n,k", [(2304, 2560, 512), (2304, 2560, 2048), (2100, 2500, 4096), (2048, 3584, 8192),
                                   (2048, 4096, 14336)])
def test_partly_filled_last_round_is_split_along_k(m, n, k):
    """More tiles than CTA pairs with a remainder: where K is long enough to pay for it the tail tiles are cut along
    K, every piece stores its partial tile in a scratch slice and the last arriver adds them up. The scratch may hold
    anything beforehand (NaN here); two calls in a row: the second finds the counters as the first left them."""
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = (torch.randn(m, k, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    ref = a.float() @ w.float().t()
    gemm._pair_scratch(a.device).fill_(float("nan"))
    outs = []
    for _ in range(2):
        out = gemm.linear(a, w, cta_pair=True)
        torch.cuda.synchronize()
        assert gemm.pipeline_status() == 0
        err = (out.float() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item() + 1e-2, err
        outs.append(out)
    assert torch.equal(outs[0], outs[1]), "the sum must not depend on which piece arrives last"
    ws, counters, _ = gemm._workspace(a.device)
    assert int(counters.abs().sum()) == 0 and float(ws.abs().max()) == 0.0
