"""Bounded device-side waits: a rank whose peer never launches must return with an error
record instead of hanging, and the workspace must be usable again after reset().

The failure is made on the host (the peer's kernel is simply never launched; nothing ever
writes the flag or the Lamport slot). No GPU fault, trap or endless loop is involved: the
waiting kernel gives up after its time budget and exits normally.
"""
import pytest
import torch

import torch_dist_ext_b200 as tdx
from helpers import check_against_oracle, make_inputs, run_emulated
from torch_dist_ext_b200.utils.config import ALGO_CODES, OUT_SAME

pytestmark = pytest.mark.gpu


# two-shot: the blocks that own a row wait for the peer's partial sums (1), the others for the rows that the peer owns
# (2); both budgets run out together and the first report wins
@pytest.mark.parametrize("algo,codes", [("oneshot", (1,)), ("twoshot", (1, 2)), ("twoshot_barrier", (3,))])
def test_missing_peer_times_out_and_reports(algo, codes):
    ws = tdx.local_workspaces(2, size_in_bytes=4 << 20, timeout_ms=200)
    ins, residual, gamma = make_inputs(2, 8, 1024, torch.bfloat16, "cuda")
    table0 = ws[0].get_workspace(ins[0])
    norm = torch.empty_like(ins[0])
    res = torch.empty_like(ins[0])
    # rank 0 launches alone; rank 1 never does
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    torch.ops.torch_dist_ext.allreduce_rms_fusion_ex(ins[0], residual, gamma, res, norm, None, 1e-6, table0,
                                                     OUT_SAME, ALGO_CODES[algo], False)
    end.record()
    torch.cuda.synchronize()  # returns: the kernel exits by itself
    assert 150 <= start.elapsed_time(end) <= 3000
    code = ws[0].errors_seen()
    assert code in codes
    st = ws[0].stats()
    assert st[3] >= 1           # error_count
    assert st[7] == code        # status[0] = code
    assert st[8] == 0           # status[1] = reporting rank
    assert st[9] == 1           # status[2] = the peer that never arrived
    # recover: both ranks idle -> reset both -> the emulated pair works again
    for w in ws:
        w.reset()
    assert ws[0].errors_seen() == 0
    _, norm2, res2, scales = run_emulated(ws, ins, residual, gamma, 1e-6, OUT_SAME, algo)
    check_against_oracle(ins, residual, gamma, 1e-6, OUT_SAME, norm2, res2, scales)
