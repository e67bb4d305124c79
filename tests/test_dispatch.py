"""The decisions the kernels' dispatch takes from sizes alone (how a context is cut into ranges, which tile
shape a prompt portion's products get, whether they are cut along K), for a stated number of SMs: no GPU and
no library needed, so a change to a cost model shows here first.  The GPU tests measure nothing either; they
check the same rules on the device's own SM count and that every choice gives the right numbers."""

import pytest


@pytest.fixture(params=[148, 132, 80])
def ops_with_sms(request, monkeypatch):
    import sllm_b200.ops as ops
    cached = [getattr(ops, n) for n in dir(ops) if hasattr(getattr(ops, n), "cache_clear")]
    for f in cached:
        f.cache_clear()
    monkeypatch.setattr(ops, "num_sms", lambda: request.param)
    yield ops, request.param
    for f in cached:                   # nothing decided for this SM count outlives the test
        f.cache_clear()


def test_the_cut_of_a_context_fills_whole_waves(ops_with_sms):
    ops, sms = ops_with_sms
    slots = 2 * sms
    for requests in (1, 2, 3, 8, 12, 16, 20, 33, 48, 64, 100, 128):
        for nkv in (1, 2, 4, 8):
            for ctx in (1, 127, 128, 255, 256, 1000, 4096, 5000, 17000, 32768):
                s = ops.choose_splits(requests, nkv, ctx, 2)
                assert 1 <= s <= max(1, min(ops.MAX_SPLITS, ctx // ops.SPLIT_MIN_KEYS)), (requests, nkv, ctx, s)
                tiles = -(-(-(-ctx // s)) // 64)
                assert -(-ctx // (tiles * 64)) == s, (requests, nkv, ctx, s)          # no range without keys
                ctas = requests * nkv * s
                if s > 1 and ctas > slots:                                            # a second wave only if well filled
                    assert ctas / (-(-ctas // slots) * slots) > 0.6, (requests, nkv, ctx, s)
                # the mma.sync form's merge walks the ranges one by one: its cap holds
                assert ops.choose_splits(requests, nkv, ctx, 2, ops.MMA_MAX_SPLITS) <= ops.MMA_MAX_SPLITS
    if sms == 148:
        assert ops.choose_splits(8, 4, 4096, 2) in (8, 9)          # 256 or 288 CTAs for 296 places
        assert ops.choose_splits(16, 4, 4096, 2) == 4              # five ranges would be 320 CTAs: two waves
        assert ops.choose_splits(64, 4, 4096, 2) == 1
        assert ops.choose_splits(1, 4, 32768, 2) == 74             # 296 CTAs of seven key tiles
        assert ops.choose_splits(1, 4, 1024, 2) == 8               # ranges of two key tiles, not fewer


def test_tile_shapes_of_a_prompt_portions_products(ops_with_sms):
    ops, sms = ops_with_sms
    pairs = sms // 2
    for M in (129, 256, 512, 1024, 2048, 4096, 8192):
        for N in (896, 1536, 2048, 3584, 4608, 5120, 8192, 18944, 37888):
            form = ops.pair_wide_cols(M, N)
            assert form in (False, True, 448, 384, 320)
            mt = -(-M // 256)
            if form is True:
                assert ops.pair_tiles_wide(M, N)
            if form not in (False, True):       # no more waves than the 512-wide tiles would take
                assert -(-(mt * -(-N // form)) // pairs) <= -(-(mt * -(-N // 512)) // pairs)
            if form is not False:               # wide tiles only where a pair has few tiles anyway
                assert -(-(mt * -(-N // 256)) // pairs) < 4
            if ops.pair_tiles_slim(M, N):
                assert 2 * mt * -(-N // 256) <= pairs
    if sms == 148:
        assert ops.pair_wide_cols(2048, 3584) == 448 and ops.pair_wide_cols(2048, 4608) is True
        assert ops.pair_wide_cols(1024, 5120) == 320 and ops.pair_wide_cols(4096, 1536) == 384
        assert ops.pair_wide_cols(2048, 18944) is False and ops.pair_wide_cols(2048, 5120) is False
        assert ops.pair_tiles_slim(512, 4608) and not ops.pair_tiles_slim(2048, 3584)


def test_slices_of_k_for_results_of_few_tiles(ops_with_sms):
    ops, sms = ops_with_sms
    for M in (129, 197, 256, 512, 768, 1024, 2048, 4096):
        for N, K in ((3584, 3584), (3584, 18944), (4608, 3584), (5120, 5120), (5120, 27648), (896, 4864), (8, 520)):
            s = ops.pair_splits(M, N, K)
            assert 1 <= s <= ops.PAIR_SPLIT_MAX
            if s > 1:                           # a slice keeps at least PAIR_SPLIT_MIN_BLOCKS k blocks
                assert -(-K // 64) // s >= ops.PAIR_SPLIT_MIN_BLOCKS
    if sms == 148:
        assert ops.pair_splits(197, 3584, 18944) > 1 and ops.pair_splits(512, 3584, 18944) > 1
        assert ops.pair_splits(2048, 3584, 18944) == 1 and ops.pair_splits(2048, 37888, 3584) == 1
