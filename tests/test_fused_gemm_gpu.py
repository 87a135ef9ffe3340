"""GEMM fused with its collective, single rank (world_size 1): the kernels run their full flow -
tcgen05 GEMM, tile push into the Lamport gather slots, reduce + residual + RMSNorm tail, and the
all-gather staging with its arrival flag - with this rank as its own only peer."""
import pytest
import torch

import torch_dist_ext_b200 as tdx
from torch_dist_ext_b200.ops import fused_gemm, gemm
from torch_dist_ext_b200.ops import reference as ref
from torch_dist_ext_b200.utils.config import OUT_FP8_BLOCK128, OUT_SAME

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def env():
    tdx.setup_env(0, 1, max_size_in_bytes=16 << 20)
    yield
    tdx.teardown_env()


def tol(expected):
    """Two bf16 roundings (the GEMM output, then the sum with the residual) at the magnitude of the largest value."""
    return 0.03 + 2.0 ** -7 * expected.float().abs().max().item()


def oracle(a, w, residual, gamma, eps, out_mode=OUT_SAME):
    y = (a.float() @ w.float().t()).to(torch.bfloat16)       # each rank's GEMM output is rounded to bf16
    return ref.residual_rmsnorm_reference(y.float(), residual, gamma, eps, out_mode)


@pytest.mark.parametrize("one_hop", [None, True, False])
@pytest.mark.parametrize("tokens,hidden,k", [(1, 4096, 512), (16, 4096, 1792), (64, 8192, 1024), (33, 1024, 256), (100, 2048, 128)])
def test_gemm_allreduce_rms_world1(tokens, hidden, k, one_hop):
    """Both tails of the fused kernel: one hop (tiles pushed to every rank, each rank reduces all rows) and two hops
    (reduce-scatter to the owners, gather back); None lets the op choose by message size."""
    a = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(hidden, k, device="cuda") * 0.05).to(torch.bfloat16)
    r = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    g = (1 + 0.1 * torch.randn(hidden, device="cuda")).to(torch.bfloat16)
    for _ in range(3):   # repeated calls walk through the three Lamport buffers
        norm, res, _ = fused_gemm.gemm_allreduce_rms(a, w, r, g, 1e-6, one_hop=one_hop)
    e_norm, e_res, _ = oracle(a, w, r, g, 1e-6)
    assert (res.float() - e_res.float()).abs().max().item() <= tol(e_res)
    assert (norm.float() - e_norm.float()).abs().max().item() <= tol(e_norm)
    tdx.check_status()
    assert gemm.pipeline_status() == 0


def test_gemm_allreduce_rms_fp8_output_world1():
    tokens, hidden, k = 16, 4096, 512
    a = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(hidden, k, device="cuda") * 0.05).to(torch.bfloat16)
    r = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    g = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
    q, res, scales = fused_gemm.gemm_allreduce_rms(a, w, r, g, 1e-6, out_mode=OUT_FP8_BLOCK128)
    e_norm, _, _ = oracle(a, w, r, g, 1e-6)
    back = ref.dequantize_fp8(q, scales)
    assert (back - e_norm.float()).abs().max().item() <= e_norm.float().abs().max().item() * 2.0 ** -3


@pytest.mark.parametrize("tokens,hidden,k", [(1, 4096, 512), (16, 8192, 1024), (64, 8192, 3584), (33, 1024, 256)])
@pytest.mark.parametrize("out_mode", [OUT_SAME, OUT_FP8_BLOCK128])
def test_gemm_allreduce_rms_block_scaled_fp8_operands_world1(tokens, hidden, k, out_mode):
    """e4m3 activations (1x128 scales) times e4m3 weights (128x128 scales) inside the fused kernel, against the
    dequantised operands multiplied in fp32."""
    from torch_dist_ext_b200.ops import quant

    a = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(hidden, k, device="cuda") * 0.05).to(torch.bfloat16)
    r = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    g = (1 + 0.1 * torch.randn(hidden, device="cuda")).to(torch.bfloat16)
    aq, ascale = quant.quant_fp8(a, block_scaled=True)
    wq, wscale = gemm.quantize_weight_block128(w)
    for hop in (True, False, None):
        norm, res, scales = fused_gemm.gemm_allreduce_rms(aq, wq, r, g, 1e-6, out_mode=out_mode, a_scale=ascale, w_scale=wscale,
                                                          one_hop=hop)
    a_deq = (aq.float().view(tokens, k // 128, 128) * ascale.view(tokens, k // 128, 1)).view(tokens, k)
    w_deq = (wq.float().view(hidden // 128, 128, k // 128, 128) * wscale.view(hidden // 128, 1, k // 128, 1)).view(hidden, k)
    y = (a_deq @ w_deq.t()).to(torch.bfloat16)
    e_norm, e_res, _ = ref.residual_rmsnorm_reference(y.float(), r, g, 1e-6, OUT_SAME)
    assert (res.float() - e_res.float()).abs().max().item() <= tol(e_res)
    if out_mode == OUT_SAME:
        assert (norm.float() - e_norm.float()).abs().max().item() <= tol(e_norm)
    else:
        back = ref.dequantize_fp8(norm, scales)
        assert (back - e_norm.float()).abs().max().item() <= e_norm.float().abs().max().item() * 2.0 ** -3
    # the unfused route (block-scaled GEMM, then the all-reduce op) agrees
    u_norm, u_res, _ = fused_gemm.gemm_allreduce_rms(aq, wq, r, g, 1e-6, out_mode=OUT_SAME, a_scale=ascale, w_scale=wscale,
                                                     force_unfused=True)
    assert (res.float() - u_res.float()).abs().max().item() <= 0.07
    tdx.check_status()
    assert gemm.pipeline_status() == 0


@pytest.mark.parametrize("tokens,n_out,k", [(1, 768, 4096), (16, 3584, 4096), (64, 1280, 8192), (40, 256, 128)])
def test_allgather_gemm_world1(tokens, n_out, k):
    x = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(n_out, k, device="cuda") * 0.05).to(torch.bfloat16)
    for _ in range(3):   # both staging buffers and the epoch flags
        out = fused_gemm.allgather_gemm(x, w, tokens)
    want = x.float() @ w.float().t()
    assert (out.float() - want).abs().max().item() <= 8e-3 * want.abs().max().item() + 1e-3
    tdx.check_status()
    assert gemm.pipeline_status() == 0


def _standalone_allreduce_calls():
    from torch_dist_ext_b200.parallel import comm
    return sum(comm.get_comm().algo_counts.values())


@pytest.mark.parametrize("tokens,hidden,k", [(2048, 4096, 512), (4096, 1024, 256), (1000, 4096, 1792), (300, 8192, 1024),
                                             (2049, 2048, 64)])
@pytest.mark.parametrize("out_mode", [OUT_SAME, OUT_FP8_BLOCK128])
def test_prompt_sized_token_counts_stay_fused(tokens, hidden, k, out_mode):
    """More tiles than SMs: the persistent kernel walks them and still ends in the reduce / normalise tail; no
    standalone all-reduce launch is involved."""
    a = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(hidden, k, device="cuda") * 0.05).to(torch.bfloat16)
    r = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    g = (1 + 0.1 * torch.randn(hidden, device="cuda")).to(torch.bfloat16)
    before = _standalone_allreduce_calls()
    for _ in range(3):   # repeated calls walk through the three Lamport buffers
        norm, res, scales = fused_gemm.gemm_allreduce_rms(a, w, r, g, 1e-6, out_mode=out_mode)
    assert _standalone_allreduce_calls() == before, "the call fell back to GEMM + all-reduce"
    e_norm, e_res, _ = oracle(a, w, r, g, 1e-6)
    assert (res.float() - e_res.float()).abs().max().item() <= tol(e_res)
    if out_mode == OUT_SAME:
        assert (norm.float() - e_norm.float()).abs().max().item() <= tol(e_norm)
    else:
        back = ref.dequantize_fp8(norm, scales)
        assert (back - e_norm.float()).abs().max().item() <= e_norm.float().abs().max().item() * 2.0 ** -3
    tdx.check_status()
    assert gemm.pipeline_status() == 0
    # a decode-sized call afterwards finds the communication state intact
    n2, r2, _ = fused_gemm.gemm_allreduce_rms(a[:16], w, r[:16], g, 1e-6)
    assert (r2.float() - e_res[:16].float()).abs().max().item() <= tol(e_res)


def test_messages_beyond_the_lamport_buffers_take_the_unfused_route():
    tokens, hidden, k = 8192, 4096, 64                                    # 64 MiB of partial sums
    a = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(hidden, k, device="cuda") * 0.05).to(torch.bfloat16)
    g = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
    before = _standalone_allreduce_calls()
    norm, res, _ = fused_gemm.gemm_allreduce_rms(a, w, None, g, 1e-6)
    assert _standalone_allreduce_calls() == before + 1
    e_norm, e_res, _ = oracle(a, w, None, g, 1e-6)
    assert (norm.float() - e_norm.float()).abs().max().item() <= tol(e_norm)
