"""Split-KV decode attention against an fp32 softmax(QK^T)V written in PyTorch."""
import pytest
import torch

from torch_dist_ext_b200.ops import attention

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("b,hq,hkv,smax", [(1, 4, 1, 2048), (16, 4, 1, 2048), (64, 8, 1, 300), (3, 32, 8, 777), (2, 8, 8, 129)])
def test_decode_attention(b, hq, hkv, smax):
    q = torch.randn(b, hq, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(b, smax, hkv, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(b, smax, hkv, 128, device="cuda", dtype=torch.bfloat16)
    lens = torch.randint(1, smax + 1, (b,), device="cuda", dtype=torch.int32)
    lens[0] = smax
    want = attention.decode_attention_reference(q, k, v, lens)
    for nsplit in (None, 1, 5):
        got = attention.decode_attention(q, k, v, lens, smax, nsplit=nsplit)
        assert (got.float() - want.float()).abs().max().item() <= 2e-2, nsplit


def test_strided_q_view_from_fused_qkv():
    b, hq, hkv = 4, 4, 1
    qkv = torch.randn(b, (hq + 2 * hkv) * 128, device="cuda", dtype=torch.bfloat16)
    q = qkv[:, : hq * 128].view(b, hq, 128)
    k = torch.randn(b, 512, hkv, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    lens = torch.full((b,), 512, device="cuda", dtype=torch.int32)
    got = attention.decode_attention(q, k, v, lens, 512)
    want = attention.decode_attention_reference(q, k, v, lens)
    assert (got.float() - want.float()).abs().max().item() <= 2e-2


def test_more_head_pairs_than_arrival_counters_then_a_small_call():
    """batch * kv_heads beyond the 4096 arrival counters of the cached scratch buffer: the splits are merged by the
    separate kernel and the counters stay zero, so the in-kernel merge of the next small call still fires."""
    b, h, smax = 256, 32, 128
    q = torch.randn(b, h, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(b, smax, h, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    lens = torch.randint(1, smax + 1, (b,), device="cuda", dtype=torch.int32)
    one = attention.decode_attention(q, k, v, lens, smax, nsplit=1)
    two = attention.decode_attention(q, k, v, lens, smax, nsplit=2)
    assert (one.float() - two.float()).abs().max().item() <= 2e-2
    want = attention.decode_attention_reference(q[:4], k[:4], v[:4], lens[:4])
    assert (two[:4].float() - want.float()).abs().max().item() <= 2e-2
    q2, k2, v2 = q[:3, :8].contiguous(), k[:3, :, :2].contiguous(), v[:3, :, :2].contiguous()
    got = attention.decode_attention(q2, k2, v2, lens[:3], smax, nsplit=4)
    want = attention.decode_attention_reference(q2, k2, v2, lens[:3])
    assert (got.float() - want.float()).abs().max().item() <= 2e-2
