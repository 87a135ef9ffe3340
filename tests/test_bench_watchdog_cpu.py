"""The reference arm of bench.py turns a hang of the reference (its device-side waits have no limit) into its
``unavailable`` line: a watchdog thread that sees no progress ends the process with exit code 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys, time
sys.path.insert(0, {root!r})
import bench
bench._watchdog = bench._ReferenceWatchdog(limit_s=0.6)
bench._progress("setup_env")
{body}
print("finished", flush=True)
"""


def run_child(body: str, rank: str):
    env = dict(os.environ, RANK=rank)
    return subprocess.run([sys.executable, "-c", CHILD.format(root=ROOT, body=body)], capture_output=True, text=True, timeout=120,
                          env=env)


def test_a_stuck_arm_prints_unavailable_and_exits_zero():
    r = run_child("time.sleep(30)", "0")
    assert r.returncode == 0
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1 and "finished" not in r.stdout
    msg = json.loads(lines[0])
    assert msg["impl"] == "reference" and "setup_env" in msg["unavailable"]


def test_other_ranks_leave_silently():
    r = run_child("time.sleep(30)", "1")
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_progress_keeps_the_arm_alive():
    r = run_child("for _ in range(8):\n    time.sleep(0.3)\n    bench._progress('step')", "0")
    assert r.returncode == 0 and "finished" in r.stdout and "unavailable" not in r.stdout


def test_the_arm_declines_by_default_after_the_recorded_hang(monkeypatch):
    """One run of the arm at 2 ranks never returned: by default the arm says so instead of launching that code again."""
    import argparse

    sys.path.insert(0, ROOT)
    import bench
    from benchmarks import common

    monkeypatch.delenv("TDX_BENCH_REFERENCE_RUN", raising=False)
    for world in (2, 4, 8):
        monkeypatch.setattr(common, "init_dist", lambda gpus, w=world: (0, w, 0))
        args = argparse.Namespace(gpus=world, steps=5, warmup=3, impl="reference", tokens=128, hidden=4096, no_extras=True,
                                  no_pinned_io=True)
        msg = bench.run(args)
        assert msg["impl"] == "reference" and "hung" in msg["unavailable"] and "TDX_BENCH_REFERENCE_RUN" in msg["unavailable"]
    monkeypatch.setattr(common, "init_dist", lambda gpus: (0, 1, 0))
    args.gpus = 1
    assert "2, 4 or 8 ranks" in bench.run(args)["unavailable"]
