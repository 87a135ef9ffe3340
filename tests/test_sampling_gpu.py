"""Greedy sampling kernels against torch.argmax: one rank through the public op, and several ranks' candidate rows
summed on one GPU the way the fused all-reduce sums them across GPUs."""
import pytest
import torch

import torch_dist_ext_b200 as tdx
from torch_dist_ext_b200 import _lib
from torch_dist_ext_b200.ops import sampling

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def env():
    tdx.setup_env(0, 1, max_size_in_bytes=8 << 20)
    yield
    tdx.teardown_env()


@pytest.mark.parametrize("tokens,vocab", [(1, 128256), (64, 16032), (7, 33), (300, 1000)])
def test_single_rank_matches_argmax(tokens, vocab):
    g = torch.Generator().manual_seed(vocab)
    logits = torch.randn(tokens, vocab, generator=g).cuda()
    got = sampling.greedy_sample_sharded(logits, 0, 1, 0)
    assert got.dtype == torch.int64 and torch.equal(got.cpu(), logits.cpu().argmax(dim=-1))


@pytest.mark.parametrize("first,last", [(1000, 3000), (1001, 3000), (1002, 2999), (0, 20481)])
def test_rows_of_a_wider_matrix_and_an_index_base(first, last):
    """Row stride 32768, unit column stride; rows that start off a 16-byte boundary take the element-wise loads."""
    g = torch.Generator().manual_seed(3)
    wide = torch.randn(16, 32768, generator=g).cuda()
    view = wide[:, first:last]
    got = sampling.greedy_sample_sharded(view, 0, 1, 50000)
    assert torch.equal(got.cpu(), view.cpu().argmax(dim=-1) + 50000)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_candidates_of_several_ranks_summed(world):
    shard, tokens = 2004, 65
    g = torch.Generator().manual_seed(world)
    full = torch.randn(tokens, world * shard, generator=g)
    full[3, 11] = full[3, world * shard - 1] = 8.0              # equal logits on the first and the last rank
    full[4, :] = -1.0                                           # a constant row: index 0
    full[6, shard + 5] = float("nan")                           # a NaN never wins
    want = torch.where(full.isnan(), torch.full_like(full, -float("inf")), full).argmax(dim=-1)
    want[3], want[4] = 11, 0
    ops = _lib.ops()
    total = torch.zeros(tokens, 4 * world, device="cuda")
    for r in range(world):
        pack = torch.full((tokens, 4 * world), 123.0, device="cuda")     # stale contents must be overwritten
        ops.argmax_pack(full[:, r * shard:(r + 1) * shard].contiguous().cuda(), r * shard, r, world, pack)
        own = pack.view(tokens, world, 4)
        others = torch.ones(world, dtype=torch.bool)
        others[r] = False
        assert bool((own[:, others] == 0).all()) and bool((own[:, r, 2:] == 0).all())
        total += pack
    out = torch.empty(tokens, dtype=torch.int64, device="cuda")
    ops.select_token(total, world, out)
    assert torch.equal(out.cpu(), want)


def test_index_range_is_checked():
    logits = torch.zeros(2, 64, device="cuda")
    pack = torch.empty(2, 4, device="cuda")
    with pytest.raises(RuntimeError, match="2\\^24"):
        _lib.ops().argmax_pack(logits, 1 << 24, 0, 1, pack)
