"""Child process of test_checked_build_gpu.py: runs with TDX_BOUNDS=1, i.e. on the range-checking
flavour of the library (a process can load only one flavour, hence the child)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch_dist_ext_b200 as tdx  # noqa: E402
from helpers import check_against_oracle, make_inputs, run_emulated  # noqa: E402
from torch_dist_ext_b200.utils.config import ALGO_CODES, OUT_FP8_TOKEN, OUT_SAME  # noqa: E402

EPS = 1e-6
BOUNDS_VIOLATION = 7


def main():
    assert torch.ops.torch_dist_ext.bounds_checked_build(), "TDX_BOUNDS=1 must load the checked flavour"
    # 1. correct offsets: every protocol runs clean under the checks and still matches the oracle
    for nranks in (2, 4, 8):
        ws = tdx.local_workspaces(nranks, size_in_bytes=8 << 20, timeout_ms=2000)
        for algo in ("oneshot", "twoshot", "twoshot_barrier"):
            for tokens, hidden, mode in [(3, 1024, OUT_SAME), (130, 1024, OUT_SAME), (17, 4096, OUT_FP8_TOKEN)]:
                ins, residual, gamma = make_inputs(nranks, tokens, hidden, torch.bfloat16, "cuda", seed=tokens)
                _, norm, res, scales = run_emulated(ws, ins, residual, gamma, EPS, mode, algo)
                check_against_oracle(ins, residual, gamma, EPS, mode, norm, res, scales)
        assert all(w.errors_seen() == 0 for w in ws), f"{nranks} ranks: a correct run tripped a bounds check"
        del ws
    # 2. an extent that ends before the Lamport buffers: rank 0's pushes leave it, are recorded and go to
    #    the scratch slots instead of the peer; the peer (never launched) gets nothing, so rank 0's own wait
    #    runs out afterwards - the FIRST record is the violation
    ws = tdx.local_workspaces(2, size_in_bytes=4 << 20, timeout_ms=200)
    ins, residual, gamma = make_inputs(2, 8, 1024, torch.bfloat16, "cuda")
    ws[0].set_debug_extent(64 << 10)
    norm, res = torch.empty_like(ins[0]), torch.empty_like(ins[0])
    torch.ops.torch_dist_ext.allreduce_rms_fusion_ex(ins[0], residual, gamma, res, norm, None, EPS,
                                                     ws[0].get_workspace(ins[0]), OUT_SAME, ALGO_CODES["oneshot"], False)
    torch.cuda.synchronize()
    assert ws[0].errors_seen() == BOUNDS_VIOLATION, ws[0].errors_seen()
    st = ws[0].stats()
    assert st[7] == BOUNDS_VIOLATION and st[8] == 0 and st[9] == 1, list(st[7:13])
    # 3. recovery: real extent again, reset, and the pair works
    ws[0].set_debug_extent(0)
    for w in ws:
        w.reset()
    _, norm2, res2, scales = run_emulated(ws, ins, residual, gamma, EPS, OUT_SAME, "oneshot")
    check_against_oracle(ins, residual, gamma, EPS, OUT_SAME, norm2, res2, scales)
    assert all(w.errors_seen() == 0 for w in ws)
    torch.cuda.synchronize()
    print("checked build ok")


if __name__ == "__main__":
    main()
