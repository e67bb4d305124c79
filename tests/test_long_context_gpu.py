"""The attention kernels at the context lengths the engine is benchmarked and profiled at (8k to 32k
tokens), where the tests at other sizes do not reach: the decode forms with their context cut 32 ways,
block tables of more than 2,048 pages (which the decode kernels no longer keep in shared memory), and
the tcgen05 prefill form on a portion of 512 tokens at the end of 32k with its context cut into many
ranges.  Each against the float32 statement, and with one far key made to stand out."""

import pytest
import torch

from tests import torch_ops as ref
from tests.conftest import cuda_or_skip
from tests.test_kernels_gpu import _paged_case, _starts

pytestmark = pytest.mark.gpu


def _ops():
    cuda_or_skip()
    import sllm_b200.ops as ops
    return ops


def _decode_forms(ops, hd, ps):
    forms = [("mma", lambda *a: ops.attention_mma(*a[:7], True, a[7], *a[8:]))]
    if ops.tma_attention_supports(hd, ps):
        forms.append(("tma", lambda *a: ops.attention_tma_decode(*a)))
    return forms


@pytest.mark.parametrize("ctx,ps", [(8192, 16), (32768, 16), (32768, 64), (17000, 8)])
@pytest.mark.parametrize("nq,nkv,hd", [(4, 2, 128), (6, 1, 64)])
def test_decode_forms_at_long_contexts(ctx, ps, nq, nkv, hd):
    """Single decoded tokens over 8k to 32k keys: a few numbers of splits and the one the engine picks (above 32 at 32k), requests of
    other lengths in the same batch, and (pages of 8 at 17,000 tokens: 2,125 pages) a block table longer than
    the 2,048 entries the kernels cache."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(31)
    lens = [ctx, ctx - 37, 300, 1]
    q_lens = [1] * len(lens)
    q, kc, vc, bt, pos, seq = _paged_case(g, lens, q_lens, nq, nkv, hd, ps, torch.bfloat16, consecutive="runs")
    assert ctx != 17000 or bt.shape[1] > 2048
    q_start, ctx_len = _starts(q_lens, lens)
    scale = hd ** -0.5
    want = ref.attention_simt(q.float(), kc.float(), vc.float(), bt, pos, seq, nq, nkv, hd, scale, None)
    small, large = ops.attention_tiles(q_lens, nq // nkv, "cuda")
    assert large is None
    picked = ops.choose_splits(1, 1, ctx)                      # what the engine picks for one request at this length
    assert 24 <= picked <= ops.MAX_SPLITS and (ctx < 32768 or picked > 32)
    for name, form in _decode_forms(ops, hd, ps):
        for splits in sorted({1, 7, picked, 32}):
            out = torch.full_like(q, float("nan"))
            form(q, kc, vc, bt, q_start, ctx_len, small, splits, nq, nkv, hd, scale, None, out)
            ops.check_tcgen05_status()
            assert not out.isnan().any(), f"{name}, {splits} splits: a row was not written"
            torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2, msg=lambda m: f"{name}, {splits} splits: {m}")


@pytest.mark.parametrize("ctx,ps", [(32768, 16), (17000, 8)])
def test_decode_forms_find_a_far_key_at_long_contexts(ctx, ps):
    """One key among 32k stands out: at the very start, at split and page edges, in the last page."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(32)
    nq, nkv, hd = 4, 2, 128
    per_split = -(-ctx // 32)
    for far in (0, ps - 1, ps, per_split - 1, per_split, 16383, 16384, ctx - ps - 1, ctx - 1):
        q, kc, vc, bt, pos, seq = _paged_case(g, [ctx], [1], nq, nkv, hd, ps, torch.bfloat16)
        q_start, ctx_len = _starts([1], [ctx])
        page, off = int(bt[0, far // ps]), far % ps
        direction = torch.randn(hd, device="cuda", generator=g)
        direction /= direction.norm()
        kc[page, :, off, :] = (direction * 16).bfloat16()
        q[0] = (direction * 16).repeat(nq).bfloat16()
        want = vc[page, :, off, :].float().repeat_interleave(nq // nkv, dim=0)
        small, _ = ops.attention_tiles([1], nq // nkv, "cuda")
        for name, form in _decode_forms(ops, hd, ps):
            for splits in (1, 32):
                out = torch.full_like(q, float("nan"))
                form(q, kc, vc, bt, q_start, ctx_len, small, splits, nq, nkv, hd, 1.0, None, out)
                ops.check_tcgen05_status()
                torch.testing.assert_close(out.float().reshape(nq, hd), want, rtol=2e-2, atol=2e-2,
                                           msg=lambda m: f"{name}, {splits} splits, key {far}: {m}")


@pytest.mark.parametrize("nq,nkv,hd,ps", [(4, 2, 128, 16), (6, 1, 64, 32)])
def test_prefill_form_on_a_portion_at_32k(nq, nkv, hd, ps):
    """A portion of 512 tokens whose context ends at 32,768, beside a short request: the context split the
    engine would choose (many ranges), the most ranges the kernel takes, and none; against the float32
    statement and with a far key that every query must find."""
    ops = _ops()
    if not ops.tc_attention_supports(hd, ps):
        pytest.skip("not taken by the tcgen05 form")
    g = torch.Generator(device="cuda").manual_seed(33)
    ctx, portion = 32768, 512
    lens, q_lens = [ctx, 200], [portion, 200]
    q, kc, vc, bt, pos, seq = _paged_case(g, lens, q_lens, nq, nkv, hd, ps, torch.bfloat16, consecutive="runs")
    q_start, ctx_len = _starts(q_lens, lens)
    scale = hd ** -0.5
    want = ref.attention_simt(q.float(), kc.float(), vc.float(), bt, pos, seq, nq, nkv, hd, scale, None)
    _, large = ops.attention_tiles(q_lens, nq // nkv, "cuda", lens, 128)
    chosen = ops.choose_tc_splits(large[2], nkv, ctx)
    assert chosen[0] > 2 and chosen[0] * chosen[1] * 64 >= ctx
    for splits in (chosen, (32, 16), (1, 0)):
        out = torch.full_like(q, float("nan"))
        ops.attention_tc(q, kc, vc, bt, q_start, ctx_len, large, nq, nkv, hd, scale, out, splits=splits)
        ops.check_tcgen05_status()
        assert not out.isnan().any(), f"splits {splits}: a row was not written"
        torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2, msg=lambda m: f"splits {splits}: {m}")
    # a far key: all 512 queries of the long request return its value
    for far in (0, 1023, 1024, 20000, ctx - portion - 1):
        k2, q2 = kc.clone(), q.clone()
        page, off = int(bt[0, far // ps]), far % ps
        direction = torch.randn(hd, device="cuda", generator=g)
        direction /= direction.norm()
        k2[page, :, off, :] = (direction * 18).bfloat16()
        q2[:portion] = (direction * 18).repeat(nq).bfloat16()
        out = torch.full_like(q, float("nan"))
        ops.attention_tc(q2, k2, vc, bt, q_start, ctx_len, large, nq, nkv, hd, 1.0, out, splits=chosen)
        ops.check_tcgen05_status()
        value = vc[page, :, off, :].float().repeat_interleave(nq // nkv, dim=0)
        torch.testing.assert_close(out.float()[:portion].reshape(portion, nq, hd), value.expand(portion, nq, hd),
                                   rtol=2e-2, atol=2e-2, msg=lambda m: f"far key {far}: {m}")


def test_the_cut_of_the_context_fills_whole_waves():
    """The number of ranges the decode form cuts a context into: no range without keys, at least `ops.SPLIT_MIN_KEYS` keys a
    range, at most `ops.MAX_SPLITS` ranges, and never a few CTAs more than the GPU holds at once (16 requests of 4 KV heads
    at 4,096 keys were cut five ways, 320 CTAs for 296 places, and ran two waves: 47 us against 31 cut four ways)."""
    ops = _ops()
    slots = 2 * ops.num_sms()
    for requests in (1, 2, 3, 8, 12, 16, 20, 33, 48, 64, 100, 128):
        for nkv in (1, 4, 8):
            for ctx in (1, 255, 256, 1000, 4096, 5000, 17000, 32768):
                s = ops.choose_splits(requests, nkv, ctx, 2)
                assert 1 <= s <= max(1, min(ops.MAX_SPLITS, ctx // ops.SPLIT_MIN_KEYS))
                tiles = -(-(-(-ctx // s)) // 64)
                assert -(-ctx // (tiles * 64)) == s, (requests, nkv, ctx, s)
                ctas = requests * nkv * s
                if s > 1 and ctas > slots:        # more than a wave only when the waves are well filled
                    assert ctas / (-(-ctas // slots) * slots) > 0.6, (requests, nkv, ctx, s)
    assert 16 * 4 * ops.choose_splits(16, 4, 4096, 2) <= slots


@pytest.mark.parametrize("nq,nkv,hd", [(4, 2, 128), (6, 1, 64)])
def test_the_decode_forms_merge_leaves_other_kernels_rows_alone(nq, nkv, hd):
    """A step with a prompt portion beside decoding requests: the decode form runs on the decoding requests' tiles
    only, with the context cut into ranges, and its merge kernel writes the decoded tokens' rows and not one value of
    the portion's."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(33)
    lens = [3000, 40, 1500]                       # the second request brings a portion of 40 tokens (rows 1..40)
    q_lens = [1, 40, 1]
    q, kc, vc, bt, pos, seq = _paged_case(g, lens, q_lens, nq, nkv, hd, 16, torch.bfloat16, consecutive="runs")
    q_start, ctx_len = _starts(q_lens, lens)
    want = ref.attention_simt(q.float(), kc.float(), vc.float(), bt, pos, seq, nq, nkv, hd, hd ** -0.5, None)
    small, large = ops.attention_tiles(q_lens, nq // nkv, "cuda", lens, 128)
    assert small[2] == 2 and large is not None
    for name, form in _decode_forms(ops, hd, 16):
        for splits in (1, 5):
            out = torch.full_like(q, 77.0)
            form(q, kc, vc, bt, q_start, ctx_len, small, splits, nq, nkv, hd, hd ** -0.5, None, out)
            ops.check_tcgen05_status()
            assert bool((out[1:41] == 77.0).all()), f"{name}, {splits} ranges: the portion's rows were written"
            torch.testing.assert_close(out[[0, 41]].float(), want[[0, 41]], rtol=2e-2, atol=2e-2,
                                       msg=lambda m: f"{name}, {splits} ranges: {m}")
