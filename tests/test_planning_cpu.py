"""Host-side launch planning of the GEMM and of decode attention (pure Python, no GPU)."""
import pytest

from torch_dist_ext_b200.ops import attention, gemm

SMS = 148


@pytest.mark.parametrize("m", [1, 16, 64, 128])
@pytest.mark.parametrize("n,k", [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (768, 4096), (512, 1792)])
def test_decode_shapes_run_swapped_and_fill_the_sms(m, n, k):
    swap, bn, splits = gemm.plan(m, n, k)
    assert swap, "up to 128 tokens the weights take the 128-row side of the tile"
    assert bn in (16, 32, 64, 128) and bn >= min(m, 128)
    tiles = -(-n // 128) * -(-m // bn)
    kblocks = k // 64
    assert 1 <= splits <= max(1, kblocks // 2)
    if tiles >= SMS:
        assert splits == 1
    else:
        assert tiles * splits <= SMS            # one wave
        assert splits == max(1, min(kblocks // 2, SMS // tiles))


@pytest.mark.parametrize("m,n,k", [(2048, 28672, 4096), (8192, 4096, 14336), (256, 256, 64), (300, 520, 512)])
def test_prefill_shapes_run_unswapped_with_wide_tiles(m, n, k):
    swap, bn, splits = gemm.plan(m, n, k)
    assert not swap and bn in (128, 256)
    if (m // 128) * (n // 256) >= SMS:
        assert bn == 256 and splits == 1


def test_block_scaled_plan_keeps_the_epilogue_in_registers():
    for m in (1, 16, 64, 2048):
        swap, bn, splits = gemm.plan(m, 28672, 8192, elem_size=1, scaled=True)
        assert swap and bn <= 64, "the promoting epilogue holds one fp32 accumulator per column"
        assert splits >= 1


@pytest.mark.parametrize("batch,kv_heads,max_len", [(1, 8, 2048), (16, 8, 2048), (64, 8, 2048), (64, 1, 2048), (1, 1, 64),
                                                     (256, 8, 4096), (3, 2, 100000)])
def test_attention_splits_fit_one_wave_and_keep_128_positions(batch, kv_heads, max_len):
    s = attention.pick_splits(batch, kv_heads, max_len)
    assert s >= 1
    assert s <= max(1, -(-max_len // 128))                       # at least 128 positions per split
    assert s == 1 or batch * kv_heads * s <= 2 * SMS             # two CTAs per SM, one wave
    t = attention.pick_splits(batch, kv_heads, max_len, ctas_per_sm=1)
    assert 1 <= t <= max(1, -(-max_len // 128))
    assert t == 1 or batch * kv_heads * t <= SMS                 # the tensor-core kernel holds one CTA per SM


def test_tensor_core_attention_splits_follow_the_measured_costs():
    pick = lambda b, h, n: attention.pick_splits(b, h, n, ctas_per_sm=1)
    assert pick(1, 1, 2048) == 8                                 # 16 chunks: 8 x 2, not 16 x 1 (merge grows with the splits)
    assert pick(16, 1, 2048) == 4                                # not 9: 9 splits leave 2 chunks to most CTAs, like 8
    assert pick(64, 1, 2048) == 1                                # a third of the SMs already busy: the merge costs more
    assert pick(16, 8, 2048) == 1
    assert pick(1, 1, 128) == 1
    assert pick(3, 2, 100000) > 8                                # long contexts still spread over the SMs


def test_fused_decode_epilogues_need_the_weights_on_the_wide_side_and_a_split():
    assert gemm.fused_epilogue_fits(1, 4096) and gemm.fused_epilogue_fits(128, 4096)
    assert not gemm.fused_epilogue_fits(129, 4096)                 # the tokens take the 128-row side
    assert gemm.fused_epilogue_fits(2048, 8192, 1, scaled=True)    # block-scaled operands always run weights-wide
    assert not gemm.fused_epilogue_fits(16, 64)                    # one 128-byte K block: no split, no finalizer
    assert gemm.fused_epilogue_fits(16, 128) and not gemm.fused_epilogue_fits(16, 128, 1, scaled=True)


@pytest.mark.parametrize("bn", [16, 32, 64, 128, 256])
def test_pair_finalizer_threads_cover_every_row_pair_and_column_once(bn):
    """The finalizer's work split (gemm_tcgen05.cu: PairShape, pair_finalize): epilogue warp w has TMEM quarter
    q = w % 4; row pair r = (q % 2) * 32 + lane, column half = q // 2, walked in steps of min(16, bn / 2) columns."""
    half_cols = bn // 2
    width = min(16, half_cols)
    steps = half_cols // width
    seen = {}
    for warp in range(2, 6):
        q = warp % 4
        for lane in range(32):
            r, half = (q % 2) * 32 + lane, q // 2
            for s in range(steps):
                for j in range(width):
                    c = half * half_cols + s * width + j
                    for row in (r, r + 64):
                        assert (row, c) not in seen
                        seen[(row, c)] = (warp, lane)
    assert len(seen) == 128 * bn
