"""API surface, launch planning and configuration - everything that needs no GPU."""
import json

import pytest
import torch

import torch_dist_ext_b200 as tdx
from torch_dist_ext_b200.ops import reference as ref
from torch_dist_ext_b200.utils.config import ALGO_CODES, OUT_FP8_BLOCK128, OUT_SAME, Config

MB = 1 << 20


def plan(n, tokens, hidden, dtype=2, out=0, algo=0, cap=128 * MB, lam=32 * MB):
    return list(torch.ops.torch_dist_ext.plan_allreduce(n, tokens, hidden, dtype, out, algo, cap, lam))


def test_reference_api_names_exist():
    for name in ("setup_env", "get_workspace", "allreduce_rms", "CommProcess", "CommWorkspace",
                 "allreduce_rms_fusion_impl"):
        assert hasattr(tdx, name), name
    assert torch.ops.torch_dist_ext.allreduce_rms is not None
    assert torch.ops.torch_dist_ext.get_workspace is not None


def test_algorithm_selection_by_bytes_not_tokens():
    # 128 tokens x 8192 bf16 = 2 MiB at 8 ranks: the reference would push 8 x 2 MiB one-shot
    assert plan(8, 128, 8192)[0] == ALGO_CODES["twoshot"]
    assert plan(8, 8, 4096)[0] == ALGO_CODES["oneshot"]
    assert plan(8, 32, 8192)[0] == ALGO_CODES["oneshot"]       # 512 KiB: measured crossover at 8 ranks
    assert plan(2, 128, 4096)[0] == ALGO_CODES["oneshot"]
    assert plan(8, 8192, 8192)[0] == ALGO_CODES["twoshot_barrier"]      # 128 MiB
    assert plan(1, 77, 4096)[0] == ALGO_CODES["local"]
    assert plan(3, 64, 1024)[1] == 0 and plan(4, 64, 1024)[1] == 4        # generic vs specialised rank count


def test_block_shapes_cover_wide_rows():
    # hidden 8192 bf16: 1024 vectors -> 512 threads x 2; hidden 16384 -> 512 x 4
    assert plan(8, 16, 8192)[2:4] == [2, 512]
    assert plan(8, 16, 16384)[2:4] == [4, 512]
    assert plan(8, 16, 4096)[2:4] == [1, 512]
    assert plan(4, 16, 124, dtype=0)[2:4] == [1, 32]


def test_set_policy_moves_the_crossover():
    old = list(torch.ops.torch_dist_ext.get_policy(8))
    try:
        torch.ops.torch_dist_ext.set_policy(8, 4 * MB, 16 * MB)
        assert plan(8, 128, 8192)[0] == ALGO_CODES["oneshot"]
    finally:
        torch.ops.torch_dist_ext.set_policy(8, *old)
    assert plan(8, 128, 8192)[0] == ALGO_CODES["twoshot"]


@pytest.mark.parametrize("args,msg", [
    (dict(n=9, tokens=1, hidden=1024), "nranks"),
    (dict(n=2, tokens=1, hidden=1022, dtype=0), "multiple of"),
    (dict(n=2, tokens=1, hidden=1000, out=OUT_FP8_BLOCK128), "128"),
    (dict(n=2, tokens=4, hidden=65536), "exceeds"),
    (dict(n=8, tokens=8192, hidden=8192, algo=ALGO_CODES["oneshot"]), "capacity"),
    (dict(n=8, tokens=65536, hidden=8192, cap=64 * MB), "capacity"),
])
def test_invalid_requests_are_rejected_before_launch(args, msg):
    with pytest.raises(RuntimeError, match=msg):
        plan(**args)


def test_fake_impls_trace_without_a_device():
    from torch._subclasses.fake_tensor import FakeTensorMode

    tdx.setup_env(0, 1)
    with FakeTensorMode():
        x = torch.empty(4, 64)
        r = torch.empty(4, 64)
        g = torch.empty(64)
        ws = tdx.get_workspace(x)
        assert ws.dtype == torch.uint8
        norm, res = tdx.allreduce_rms(0, 1, x, r, g, 1e-6, ws)
        assert norm.shape == x.shape and res.shape == r.shape


def test_cpu_world1_op_equals_oracle():
    tdx.setup_env(0, 1)
    g = torch.Generator().manual_seed(0)
    x, r = torch.randn(8, 256, generator=g), torch.randn(8, 256, generator=g)
    w = 1 + 0.1 * torch.randn(256, generator=g)
    norm, res = tdx.allreduce_rms(0, 1, x, r, w, 1e-6, tdx.get_workspace(x))
    e_norm, e_res, _ = ref.fused_allreduce_rms_reference([x], r, w, 1e-6)
    assert torch.equal(norm, e_norm) and torch.equal(res, e_res)
    with pytest.raises(ValueError):
        tdx.allreduce_rms(1, 2, x, r, w, 1e-6, tdx.get_workspace(x))


def test_config_env_and_policy_file(tmp_path, monkeypatch):
    p = tmp_path / "policy.json"
    p.write_text(json.dumps({"8": {"oneshot_max_bytes": 123, "lamport_max_bytes": 456},
                             "4": {"oneshot_max_bytes": 1, "lamport_max_bytes": 2, "mc_oneshot": 1, "mc_twoshot": 0,
                                   "nvls_min_bytes": 789}}))
    monkeypatch.setenv("TDX_ALGO", "twoshot")
    monkeypatch.setenv("TDX_TIMEOUT_MS", "250")
    monkeypatch.setenv("TDX_NVLS", "0")
    monkeypatch.setenv("TDX_POLICY_JSON", str(p))
    c = Config.from_env()
    assert c.algo_code == ALGO_CODES["twoshot"] and c.timeout_ms == 250 and not c.nvls
    assert c.policy[8] == (123, 456, -1, -1, -1)      # -1: keep the built-in value
    assert c.policy[4] == (1, 2, 1, 0, 789)
    monkeypatch.setenv("TDX_ALGO", "bogus")
    with pytest.raises(ValueError):
        Config.from_env()


def test_pinned_entry_point_fails_cleanly_without_a_device():
    x, g = torch.randn(4, 64), torch.ones(64)
    o1, o2 = torch.empty_like(x), torch.empty_like(x)
    with pytest.raises(RuntimeError, match="workspace must be the CUDA tensor"):
        torch.ops.torch_dist_ext.allreduce_rms_fusion_hostio(x, x, g, o1, o2, None, 1e-6,
                                                             torch.zeros(tdx.parallel.comm.table_nbytes(), dtype=torch.uint8),
                                                             OUT_SAME, 0, False)
    if torch.cuda.is_available():
        return
    tdx.setup_env(0, 1)
    with pytest.raises(RuntimeError, match="needs the CUDA workspace"):
        tdx.allreduce_rms_pinned(x, x, g, 1e-6, out=(o1, o2))


def test_nvtx_ranges_follow_the_flag():
    from torch_dist_ext_b200.utils import tracing

    calls = []
    tracing.set_backend(lambda name: calls.append(("push", name)), lambda: calls.append(("pop",)))
    tdx.setup_env(0, 1)
    x, g = torch.randn(4, 64), torch.ones(64)
    try:
        tracing.enable(False)
        tdx.fused_allreduce_rms(x, x, g, 1e-6)
        assert calls == []
        tracing.enable(True)
        tdx.fused_allreduce_rms(x, x, g, 1e-6)
        with tracing.nvtx_range("outer"):
            pass
        assert calls == [("push", "tdx.fused_allreduce_rms"), ("pop",), ("push", "outer"), ("pop",)]
    finally:
        tracing.enable(False)
        tracing.set_backend(None, None)


def test_clock_sampler_parses_the_query_output(tmp_path, monkeypatch):
    import importlib.util
    import os
    import stat
    import time

    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/sh\necho '1342, 1965, 987.12, Not Active, Not Active, Not Active, Active'\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    spec = importlib.util.spec_from_file_location(
        "_timing_under_test", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                           "torch_dist_ext_b200", "utils", "timing.py"))
    timing = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(timing)
    with timing.ClockSampler(0, period_s=0.01) as s:
        time.sleep(0.3)
    out = s.summary()
    assert out["sm_mhz"] == 1342.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"] and out["samples"] >= 1


def test_drop_in_module_keeps_the_reference_globals():
    import torch_dist_ext as ref_name

    ref_name.setup_env(0, 1)
    assert type(ref_name.comm).__name__ == "CommProcess" and ref_name.world_size_ == 1
    assert ref_name.allreduce_rms is tdx.allreduce_rms


def test_cmake_project_lists_every_native_source():
    """The ninja build globs the sources, the CMake project names them: a new file must be added there too, or the
    CMake-built library fails to load with an undefined symbol."""
    import pathlib

    root = pathlib.Path(__file__).resolve().parent.parent
    cmake = (root / "CMakeLists.txt").read_text()
    csrc = root / "torch_dist_ext_b200" / "csrc"
    missing = [p.name for p in sorted(csrc.glob("*.cu")) + sorted(csrc.glob("*.cpp")) if f"/{p.name}" not in cmake]
    assert not missing, missing
