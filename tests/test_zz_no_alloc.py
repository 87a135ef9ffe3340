"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some callers may not allocate device memory: a CUDA-graph capture region of an engine that forbids it,
a serving loop whose pool is owned by someone else, a plug-in that only receives input and output
pointers. For them the library carries its split-KV scratch as a fixed device array. This test calls
`tdx_attention_decode_noalloc` with ctypes (no torch op in between), twice in a row with different
shapes - the second call finds the first call's leftovers in the shared array - and compares each
result with the regular entry point, which uses a caller-provided scratch buffer. It also checks that
an oversized request is refused with a message instead of being launched.

Collected last on purpose (file name), so a run that stops at the first failure has already run
everything else; it also passes alone in a fresh process.
"""
import ctypes
import math

import pytest
import torch

import torch_dist_ext_b200 as tdx  # noqa: F401  (loads the library)
from torch_dist_ext_b200 import _lib
from torch_dist_ext_b200.ops import attention

pytestmark = pytest.mark.gpu


def _entry():
    lib = ctypes.CDLL(str(_lib.lib_path()))
    fn = lib.tdx_attention_decode_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 4 + [ctypes.c_int64] * 3 + [ctypes.c_int, ctypes.c_float,
                                                                                      ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    return fn


def _call(fn, q, k, v, lens, nsplit):
    out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    err = ctypes.create_string_buffer(256)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), lens.data_ptr(), out.data_ptr(), q.shape[0], q.shape[1], k.shape[2],
            k.shape[1], q.stride(0), k.stride(0), k.stride(1), nsplit, 1.0 / math.sqrt(q.shape[2]),
            torch.cuda.current_stream().cuda_stream, err, 256)
    return rc, out, err.value.decode()


def test_matches_regular_entry_point_on_two_calls_in_a_row():
    fn = _entry()
    torch.manual_seed(0)
    for b, hq, hkv, smax, nsplit in [(16, 4, 1, 1024, 6), (3, 32, 8, 777, 2)]:
        q = torch.randn(b, hq, 128, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(b, smax, hkv, 128, device="cuda", dtype=torch.bfloat16)
        v = torch.randn_like(k)
        lens = torch.randint(1, smax + 1, (b,), device="cuda", dtype=torch.int32)
        lens[0] = smax
        rc, got, msg = _call(fn, q, k, v, lens, nsplit)
        assert rc == 0, msg
        want = attention.decode_attention(q, k, v, lens, smax, nsplit=nsplit)
        torch.cuda.synchronize()
        assert (got.float() - want.float()).abs().max().item() <= 2e-2
        ref = attention.decode_attention_reference(q, k, v, lens)
        assert (got.float() - ref.float()).abs().max().item() <= 2e-2


def test_more_sequence_head_pairs_than_arrival_counters_leaves_the_counters_intact():
    """More (sequence, KV head) pairs than the 4096 arrival counters: the splits are merged by the separate
    combine kernel and the partial rows still start behind the counters, so the small call that follows
    (which merges inside the kernel and relies on zeroed counters) is correct too."""
    fn = _entry()
    torch.manual_seed(1)
    for b, hq, hkv, smax, nsplit in [(4100, 1, 1, 256, 2), (3, 8, 2, 512, 4)]:
        q = torch.randn(b, hq, 128, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(b, smax, hkv, 128, device="cuda", dtype=torch.bfloat16)
        v = torch.randn_like(k)
        lens = torch.randint(1, smax + 1, (b,), device="cuda", dtype=torch.int32)
        rc, got, msg = _call(fn, q, k, v, lens, nsplit)
        assert rc == 0, msg
        want = attention.decode_attention(q, k, v, lens, smax, nsplit=nsplit)
        torch.cuda.synchronize()
        assert (got.float() - want.float()).abs().max().item() <= 2e-2
        if b <= 16:
            ref = attention.decode_attention_reference(q, k, v, lens)
            assert (got.float() - ref.float()).abs().max().item() <= 2e-2


def test_oversized_request_is_refused_with_a_message():
    fn = _entry()
    q = torch.zeros(64, 32, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.zeros(64, 128, 8, 128, device="cuda", dtype=torch.bfloat16)
    lens = torch.ones(64, device="cuda", dtype=torch.int32)
    rc, _, msg = _call(fn, q, k, k, lens, 16)        # 64 * 32 * 16 = 32768 rows > 16384
    assert rc != 0 and "exceeds" in msg
