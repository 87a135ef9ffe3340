"""Multi-rank protocols of the fused all-reduce kernels, emulated on ONE GPU.

All ranks run inside a single cooperative launch (blockIdx.y = rank), each with its own
workspace, so the Lamport and flag-barrier protocols, the phase logic across repeated calls and
every epilogue are exercised without a second GPU. Shapes follow the reference's C++ harness
(test/unit_test.cpp:322-323: ragged token counts, hidden sizes that leave partial warps) and its
Python test (test/test_all_reduce_fusion.py:70-87: tokens 128/129, three dtypes), with real
assertions: the residual stream must match the oracle exactly, the normalised output within
dtype tolerance, and all ranks must agree bitwise.
"""
import pytest
import torch

import torch_dist_ext_b200 as tdx
from helpers import check_against_oracle, make_inputs, run_emulated
from torch_dist_ext_b200.utils.config import ALGO_CODES, OUT_FP8_BLOCK128, OUT_FP8_TOKEN, OUT_SAME

pytestmark = pytest.mark.gpu
EPS = 1e-6
ALGOS = ["oneshot", "twoshot", "twoshot_barrier"]


@pytest.fixture(scope="module")
def workspaces():
    cache = {}

    def get(n):
        if n not in cache:
            cache[n] = tdx.local_workspaces(n, size_in_bytes=8 << 20, timeout_ms=2000)
        return cache[n]

    yield get
    torch.cuda.synchronize()
    cache.clear()


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_matches_oracle(workspaces, nranks, dtype, algo):
    ws = workspaces(nranks)
    for tokens, hidden in [(3, 1024), (127, 512), (130, 1024), (17, 4096)]:
        ins, residual, gamma = make_inputs(nranks, tokens, hidden, dtype, "cuda", seed=tokens + hidden)
        used, norm, res, scales = run_emulated(ws, ins, residual, gamma, EPS, OUT_SAME, algo)
        assert used == ALGO_CODES[algo]
        check_against_oracle(ins, residual, gamma, EPS, OUT_SAME, norm, res, scales)
    assert all(w.errors_seen() == 0 for w in ws)


@pytest.mark.parametrize("algo", ALGOS)
def test_reference_harness_shapes_fp32(workspaces, algo):
    """tokens x hidden grid of the reference's unit test, fp32, uniform [0, 0.5) inputs."""
    ws = workspaces(4)
    for tokens in (513, 127, 778, 3):
        for hidden in (1024, 508, 124):
            g = torch.Generator().manual_seed(tokens * 7 + hidden)
            ins = [(torch.rand(tokens, hidden, generator=g) * 0.5).cuda() for _ in range(4)]
            residual = (torch.rand(tokens, hidden, generator=g) * 0.5).cuda()
            gamma = (torch.rand(hidden, generator=g) * 0.5).cuda()
            _, norm, res, scales = run_emulated(ws, ins, residual, gamma, EPS, OUT_SAME, algo)
            check_against_oracle(ins, residual, gamma, EPS, OUT_SAME, norm, res, scales)
            # the reference's own criterion: absolute error <= 1e-4
            exp, _, _ = tdx.reference.fused_allreduce_rms_reference(ins, residual, gamma, EPS)
            assert (norm[0] - exp).abs().max().item() <= 1e-4


@pytest.mark.parametrize("nranks", [3, 5, 7])
def test_odd_rank_counts(workspaces, nranks):
    ws = workspaces(nranks)
    for algo in ALGOS:
        ins, residual, gamma = make_inputs(nranks, 37, 768, torch.bfloat16, "cuda", seed=nranks)
        _, norm, res, scales = run_emulated(ws, ins, residual, gamma, EPS, OUT_SAME, algo)
        check_against_oracle(ins, residual, gamma, EPS, OUT_SAME, norm, res, scales)


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("out_mode", [OUT_FP8_TOKEN, OUT_FP8_BLOCK128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fp8_epilogues(workspaces, dtype, out_mode, algo):
    ws = workspaces(8)
    for tokens, hidden in [(5, 5120), (64, 7168), (33, 1024)]:
        if dtype == torch.float32 and hidden > 4096 * 2:
            continue
        ins, residual, gamma = make_inputs(8, tokens, hidden, dtype, "cuda", seed=hidden)
        _, norm, res, scales = run_emulated(ws, ins, residual, gamma, EPS, out_mode, algo)
        check_against_oracle(ins, residual, gamma, EPS, out_mode, norm, res, scales)


@pytest.mark.parametrize("algo", ["twoshot", "twoshot_barrier"])
@pytest.mark.parametrize("out_mode", [OUT_SAME, OUT_FP8_TOKEN])
def test_reduce_scatter_variant(workspaces, algo, out_mode):
    ws = workspaces(4)
    for tokens in (64, 61, 2):
        ins, residual, gamma = make_inputs(4, tokens, 2048, torch.bfloat16, "cuda", seed=tokens)
        _, norm, res, scales = run_emulated(ws, ins, residual, gamma, EPS, out_mode, algo, scatter_only=True)
        exp_norm, exp_res, exp_scale = tdx.reference.fused_allreduce_rms_reference(ins, residual, gamma, EPS, out_mode)
        for r in range(4):
            k = exp_res[r::4].shape[0]
            if k == 0:      # fewer tokens than ranks: this rank owns no row
                continue
            assert torch.equal(res[r][:k].float(), exp_res[r::4].float())
            if out_mode == OUT_SAME:
                assert (norm[r][:k].float() - exp_norm[r::4].float()).abs().max().item() <= 3.2e-2 * 4
            else:
                assert torch.allclose(scales[r][:k], exp_scale[r::4], rtol=1e-5)


def test_repeated_calls_mixed_sizes_and_dtypes(workspaces):
    """Phase logic: triple buffering, dirty-extent clearing and barrier epochs across calls whose
    size, dtype, algorithm and grid all change (the reference only gets this from its shape sweep)."""
    ws = workspaces(4)
    seq = [
        ("oneshot", 8, 1024, torch.float32), ("oneshot", 120, 1024, torch.bfloat16),
        ("twoshot", 300, 512, torch.float16), ("oneshot", 1, 4096, torch.bfloat16),
        ("twoshot_barrier", 700, 256, torch.float32), ("twoshot", 5, 8192, torch.bfloat16),
        ("oneshot", 64, 2048, torch.float32), ("twoshot_barrier", 9, 1024, torch.bfloat16),
        ("oneshot", 64, 2048, torch.float32), ("oneshot", 2, 128, torch.float16),
        ("twoshot", 1000, 128, torch.float32), ("oneshot", 3, 128, torch.float32),
    ]
    for i, (algo, tokens, hidden, dtype) in enumerate(seq * 2):
        ins, residual, gamma = make_inputs(4, tokens, hidden, dtype, "cuda", seed=i)
        _, norm, res, scales = run_emulated(ws, ins, residual, gamma, EPS, OUT_SAME, algo)
        check_against_oracle(ins, residual, gamma, EPS, OUT_SAME, norm, res, scales)
    s = ws[0].stats()
    assert s[3] == 0  # error_count


def test_negative_zero_payload(workspaces):
    """Inputs full of -0.0 / +0.0 pairs equal the sentinel bit pattern and must still arrive."""
    ws = workspaces(2)
    for dtype in (torch.float32, torch.bfloat16):
        ins = [torch.zeros(16, 1024, dtype=dtype, device="cuda") for _ in range(2)]
        ins[0][:, ::2] = -0.0
        ins[1][:, 1::2] = -0.0
        residual = torch.ones(16, 1024, dtype=dtype, device="cuda")
        gamma = torch.ones(1024, dtype=dtype, device="cuda")
        for algo in ("oneshot", "twoshot"):
            _, norm, res, _ = run_emulated(ws, ins, residual, gamma, EPS, OUT_SAME, algo)
            assert torch.equal(res[0], residual) and torch.equal(res[1], residual)
    assert all(w.errors_seen() == 0 for w in ws)


def test_auto_policy_picks_by_bytes(workspaces):
    ws = workspaces(8)
    ins, residual, gamma = make_inputs(8, 4, 1024, torch.bfloat16, "cuda")
    used, *_ = run_emulated(ws, ins, residual, gamma, EPS, OUT_SAME, "auto")
    assert used == ALGO_CODES["oneshot"]
    ins, residual, gamma = make_inputs(8, 512, 1024, torch.bfloat16, "cuda")
    used, norm, res, scales = run_emulated(ws, ins, residual, gamma, EPS, OUT_SAME, "auto")
    assert used == ALGO_CODES["twoshot"]
    check_against_oracle(ins, residual, gamma, EPS, OUT_SAME, norm, res, scales)


def test_capacity_and_shape_errors(workspaces):
    ws = workspaces(2)
    ins, residual, gamma = make_inputs(2, 4, 1024, torch.float32, "cuda")
    with pytest.raises(RuntimeError, match="multiple of"):
        bad = [t[:, :1022].contiguous() for t in ins]
        run_emulated(ws, bad, residual[:, :1022].contiguous(), gamma[:1022].contiguous(), EPS, OUT_SAME, "oneshot")
    big = [torch.zeros(4096, 8192, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    with pytest.raises(RuntimeError, match="capacity"):
        run_emulated(ws, big, big[0], torch.ones(8192, dtype=torch.bfloat16, device="cuda"), EPS, OUT_SAME, "oneshot")
