"""Tensor-core (tcgen05) decode attention against an fp32 softmax(QK^T)V written in PyTorch.

These kernels are the library's defaults for decode and prompt attention. The probabilities are rounded to bf16 before the second product, hence the slightly wider
tolerance than for the SIMT kernel, which is also used as a cross-check."""
import pytest
import torch

from torch_dist_ext_b200.ops import attention, gemm

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("b,hq,hkv,smax", [(1, 4, 1, 128), (1, 4, 1, 2048), (16, 4, 1, 2048), (64, 8, 1, 300), (3, 32, 8, 777),
                                           (2, 8, 8, 129), (2, 2, 1, 500), (2, 8, 1, 640)])
def test_decode_attention_tc(b, hq, hkv, smax):
    g = torch.Generator(device="cuda").manual_seed(b * 1000 + smax)
    q = torch.randn(b, hq, 128, device="cuda", dtype=torch.bfloat16, generator=g)
    k = torch.randn(b, smax, hkv, 128, device="cuda", dtype=torch.bfloat16, generator=g)
    v = torch.randn(b, smax, hkv, 128, device="cuda", dtype=torch.bfloat16, generator=g)
    lens = torch.randint(1, smax + 1, (b,), device="cuda", dtype=torch.int32, generator=g)
    lens[0] = smax
    want = attention.decode_attention_reference(q, k, v, lens)
    for nsplit in (None, 1, 3):
        got = attention.decode_attention(q, k, v, lens, smax, nsplit=nsplit, tensor_cores=True)
        torch.cuda.synchronize()
        assert gemm.pipeline_status() == 0
        assert (got.float() - want.float()).abs().max().item() <= 3e-2, nsplit
        simt = attention.decode_attention(q, k, v, lens, smax, nsplit=nsplit, tensor_cores=False)
        assert (got.float() - simt.float()).abs().max().item() <= 3e-2, nsplit


def test_prefill_attention_tc_rescales_and_masked_groups():
    """Scores with a large spread make a row's running maximum jump by more than the lazy threshold between chunks
    (the accumulators are rescaled in tensor memory); prompts shorter than 64 tokens leave the softmax group of the
    odd chunks with nothing but masked scores."""
    g = torch.Generator(device="cuda").manual_seed(7)
    for s, hq, hkv, gain in [(1024, 4, 1, 8.0), (640, 2, 2, 16.0), (40, 4, 1, 1.0), (64, 2, 1, 4.0), (100, 2, 1, 1.0)]:
        qkv = torch.randn(s, (hq + 2 * hkv) * 128, device="cuda", dtype=torch.bfloat16, generator=g)
        qkv[:, : hq * 128] *= gain
        # keys that grow along the sequence: later chunks keep raising the row maxima
        ramp = torch.linspace(0.2, 1.5, s, device="cuda").view(s, 1).to(torch.bfloat16)
        qkv[:, hq * 128: (hq + hkv) * 128] *= ramp
        q = qkv[:, : hq * 128].view(s, hq, 128)
        k = qkv[:, hq * 128: (hq + hkv) * 128].view(s, hkv, 128)
        v = qkv[:, (hq + hkv) * 128:].view(s, hkv, 128)
        got = attention.prefill_attention(q, k, v)
        torch.cuda.synchronize()
        assert gemm.pipeline_status() == 0
        want = attention.prefill_attention_reference(q, k, v)
        assert bool(torch.isfinite(got.float()).all())
        assert (got.float() - want.float()).abs().max().item() <= 4e-2, (s, hq, hkv, gain)


@pytest.mark.parametrize("s,hq,hkv", [(128, 1, 1), (256, 4, 1), (300, 4, 2), (1000, 8, 8), (2048, 4, 1)])
def test_prefill_attention_tc(s, hq, hkv):
    g = torch.Generator(device="cuda").manual_seed(s + hq)
    # q, k, v as views of one fused projection, the way the model produces them
    qkv = torch.randn(s, (hq + 2 * hkv) * 128, device="cuda", dtype=torch.bfloat16, generator=g)
    q = qkv[:, : hq * 128].view(s, hq, 128)
    k = qkv[:, hq * 128: (hq + hkv) * 128].view(s, hkv, 128)
    v = qkv[:, (hq + hkv) * 128:].view(s, hkv, 128)
    got = attention.prefill_attention(q, k, v)
    torch.cuda.synchronize()
    assert gemm.pipeline_status() == 0
    want = attention.prefill_attention_reference(q, k, v)
    assert (got.float() - want.float()).abs().max().item() <= 3e-2
