"""Each kernel alone against its plain PyTorch float32 statement (tests/torch_ops.py),
at sizes other than the engine's: widths and vocabularies that are no power of two,
head sizes in steps of 16, odd head counts and groups."""

import numpy as np
import pytest
import torch

from tests import torch_ops as ref
from tests.conftest import cuda_or_skip

pytestmark = pytest.mark.gpu


def _ops():
    cuda_or_skip()
    import sllm_b200.ops as ops
    return ops


def _close(got, want, dtype, scale=1.0):
    tol = 2e-5 if dtype == torch.float32 else 1.6e-2
    torch.testing.assert_close(got.float(), want.float(), rtol=tol, atol=tol * scale)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,H,T", [(300, 72, 19), (1000, 1000, 3)])
def test_embed_gather(dtype, V, H, T):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(0)
    table = torch.randn(V, H, device="cuda", generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), device="cuda", generator=g, dtype=torch.int32)
    assert torch.equal(ops.embed_gather(table, ids), ref.embed_gather(table, ids))


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("delta_kind", ["none", "f32", "bf16", "parts"])
@pytest.mark.parametrize("rows,H,eps", [(5, 72, 1e-6), (33, 3584, 1e-5), (2, 1000, 1e-6), (130, 1000, 1e-6),
                                        (200, 3584, 1e-5), (70, 16400, 1e-6)])
def test_add_rmsnorm(out_dtype, delta_kind, rows, H, eps):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(1)
    res = torch.randn(rows, H, device="cuda", generator=g) * 3
    w = 1 + 0.1 * torch.randn(H, device="cuda", generator=g)
    delta = None
    if delta_kind == "f32":
        delta = torch.randn(rows, H, device="cuda", generator=g)
    elif delta_kind == "bf16":
        delta = torch.randn(rows, H, device="cuda", generator=g).bfloat16()
    elif delta_kind == "parts":
        delta = torch.randn(3, rows, H, device="cuda", generator=g)
    r1, r2 = res.clone(), res.clone()
    got = ops.add_rmsnorm(r1, delta, w, eps, out_dtype)
    want = ref.add_rmsnorm(r2, delta, w, eps, out_dtype)
    torch.testing.assert_close(r1, r2, rtol=1e-6, atol=1e-6)
    _close(got, want, out_dtype, scale=4.0)


@pytest.mark.parametrize("M,N,K", [(1, 300, 72), (37, 130, 1000), (64, 64, 16), (130, 257, 333), (3, 1000, 18)])
@pytest.mark.parametrize("bias", [False, True])
def test_gemm_f32(M, N, K, bias):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g) / K ** 0.5
    b = torch.randn(N, device="cuda", generator=g) if bias else None
    got = ops.linear(x, w, b, torch.float32)
    want = (x.double() @ w.double().t() + (b.double() if bias else 0)).float()
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)


def test_gemm_f32_rows_do_not_depend_on_the_batch():
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(150, 333, device="cuda", generator=g)
    w = torch.randn(200, 333, device="cuda", generator=g)
    full = ops.linear(x, w, None, torch.float32)
    for lo, hi in ((0, 1), (7, 9), (64, 150), (149, 150)):
        assert torch.equal(ops.linear(x[lo:hi].contiguous(), w, None, torch.float32), full[lo:hi])


@pytest.mark.parametrize("M,N,K", [(1, 300, 72), (8, 1000, 336), (77, 130, 1000), (300, 512, 256)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_linear_bf16(M, N, K, out_dtype):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, device="cuda", generator=g)
    got = ops.linear(x, w, b, out_dtype)
    want = x.float() @ w.float().t() + b
    _close(got, want, out_dtype if out_dtype == torch.bfloat16 else torch.float32, scale=4.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,I,blk", [(5, 40, 8), (3, 37, 37), (17, 1000, 8)])
def test_silu_mul(dtype, T, I, blk):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(5)
    gu = (torch.randn(T, 2 * I, device="cuda", generator=g) * 2).to(dtype)
    _close(ops.silu_mul(gu, blk, dtype), ref.silu_mul(gu, blk, dtype), dtype, scale=4.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,rot,ps", [(4, 2, 16, 16, 16), (3, 1, 32, 32, 8), (6, 3, 48, 24, 4), (7, 7, 80, 80, 32)])
def test_rope_kv_write(dtype, nq, nkv, hd, rot, ps):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(6)
    T, pages, max_pos = 21, 9, 200
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, device="cuda", generator=g)
    bias = torch.randn((nq + 2 * nkv) * hd, device="cuda", generator=g)
    pos = torch.randint(0, max_pos, (T,), device="cuda", generator=g, dtype=torch.int32)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * (1e4 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot))[None]
    table = torch.stack([ang.cos(), ang.sin()], 1).float().cuda()
    slots = torch.randperm(pages * ps, device="cuda", generator=g)[:T].int()
    kc = [torch.zeros(pages, nkv, ps, hd, device="cuda", dtype=dtype) for _ in range(2)]
    vc = [torch.zeros(pages, nkv, ps, hd, device="cuda", dtype=dtype) for _ in range(2)]
    got = ops.rope_kv_write(qkv, bias, pos, table, rot, nq, nkv, hd, slots, kc[0], vc[0], dtype)
    want = ref.rope_kv_write(qkv, bias, pos, table, rot, nq, nkv, hd, slots, kc[1], vc[1], dtype)
    _close(got, want, dtype, scale=4.0)
    _close(kc[0], kc[1], dtype, scale=4.0)
    _close(vc[0], vc[1], dtype, scale=4.0)
    # no bias, no cache write (a run that borrows another run's cache), no rotation
    k2, v2 = torch.zeros_like(kc[0]), torch.zeros_like(vc[0])
    got = ops.rope_kv_write(qkv, None, pos, None, 0, nq, nkv, hd, None, k2, v2, dtype)
    _close(got, qkv[:, :nq * hd].to(dtype), dtype, scale=4.0)
    assert not k2.any() and not v2.any()


@pytest.mark.parametrize("in_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [21, 150])
@pytest.mark.parametrize("nq,nkv,hd,rot,ps", [(4, 2, 16, 16, 16), (3, 1, 32, 32, 8), (5, 1, 64, 32, 4), (7, 7, 80, 80, 32),
                                             (6, 2, 128, 128, 16)])
def test_rope_kv_write_wide_form(in_dtype, T, nq, nkv, hd, rot, ps):
    """A bfloat16 cache, one part, rotary_dim a multiple of 16: the 16-byte form of the kernel, few and many tokens."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(16)
    pages, max_pos = -(-T // ps) + 3, 300
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, device="cuda", generator=g).to(in_dtype)
    bias = torch.randn((nq + 2 * nkv) * hd, device="cuda", generator=g)
    pos = torch.randint(0, max_pos, (T,), device="cuda", generator=g, dtype=torch.int32)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * (1e4 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot))[None]
    table = torch.stack([ang.cos(), ang.sin()], 1).float().cuda()
    slots = torch.randperm(pages * ps, device="cuda", generator=g)[:T].int()
    dtype = torch.bfloat16
    for b in (bias, None):
        kc = [torch.zeros(pages, nkv, ps, hd, device="cuda", dtype=dtype) for _ in range(2)]
        vc = [torch.zeros(pages, nkv, ps, hd, device="cuda", dtype=dtype) for _ in range(2)]
        got = ops.rope_kv_write(qkv, b, pos, table, rot, nq, nkv, hd, slots, kc[0], vc[0], dtype)
        want = ref.rope_kv_write(qkv, b, pos, table, rot, nq, nkv, hd, slots, kc[1], vc[1], dtype)
        _close(got, want, dtype, scale=4.0)
        _close(kc[0], kc[1], dtype, scale=4.0)
        _close(vc[0], vc[1], dtype, scale=4.0)
    k2, v2 = torch.zeros_like(kc[0]), torch.zeros_like(vc[0])
    got = ops.rope_kv_write(qkv, None, pos, None, 0, nq, nkv, hd, None, k2, v2, dtype)
    assert torch.equal(got, qkv[:, :nq * hd].bfloat16())
    assert not k2.any() and not v2.any()


@pytest.mark.parametrize("M", [1, 5, 8, 9, 13, 16, 17, 32])
@pytest.mark.parametrize("nq,nkv,hd,K,ps", [(28, 4, 128, 3584, 16), (14, 2, 64, 896, 64), (4, 2, 16, 64, 16), (3, 1, 32, 96, 8),
                                            (6, 3, 48, 160, 16), (2, 2, 256, 128, 32)])
def test_linear_rope_kv_write(M, nq, nkv, hd, K, ps):
    """The fused q|k|v product whose epilogue adds the bias, rotates query and key heads and writes the
    new keys and values into their pages, against the product followed by the rotary kernel's statement:
    every head kind, head sizes from 16 to 256, rows that have no slot (padding), no bias, no rotation,
    a borrowed cache (nothing written)."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(31)
    N, pages, max_pos = (nq + 2 * nkv) * hd, 7, 300
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    bias = torch.randn(N, device="cuda", generator=g)
    pos = torch.randint(0, max_pos, (M,), device="cuda", generator=g, dtype=torch.int32)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * (1e4 ** (-torch.arange(0, hd, 2, dtype=torch.float64) / hd))[None]
    table = torch.stack([ang.cos(), ang.sin()], 1).float().cuda()
    slots = torch.randperm(pages * ps, device="cuda", generator=g)[:M].int()
    # (the dispatch sends 17..32 tokens here only for matrices with rows enough for one and a half CTAs an SM)
    assert ops.qkv_rope_supports(x, w, table, hd, nq, nkv, hd, torch.zeros(1, nkv, ps, hd, device="cuda", dtype=torch.bfloat16)) \
        == (M <= 16 or 2 * -(-N // 16) >= 3 * ops.num_sms())
    dtype = torch.bfloat16
    for b, tab, rot in ((bias, table, hd), (None, table, hd), (bias, None, 0)):
        kc = [torch.zeros(pages, nkv, ps, hd, device="cuda", dtype=dtype) for _ in range(2)]
        vc = [torch.zeros(pages, nkv, ps, hd, device="cuda", dtype=dtype) for _ in range(2)]
        sl = slots.clone()
        if M > 1:
            sl[M - 1] = -1                                      # a padding row: its queries are computed, nothing is written
        got = ops.linear_rope_kv_write(x, w, b, pos, tab, rot, nq, nkv, hd, sl, kc[0], vc[0])
        qkv = x.float() @ w.float().t()
        keep = sl >= 0
        want = ref.rope_kv_write(qkv[keep], b, pos[keep], tab, rot, nq, nkv, hd, sl[keep], kc[1], vc[1], dtype)
        _close(got[keep], want, dtype, scale=4.0)
        _close(kc[0], kc[1], dtype, scale=4.0)
        _close(vc[0], vc[1], dtype, scale=4.0)
        if M > 1:
            last = ref.rope_kv_write(qkv[M - 1:], b, pos[M - 1:], tab, rot, nq, nkv, hd, None, kc[1], vc[1], dtype)
            _close(got[M - 1:], last, dtype, scale=4.0)
    k2, v2 = torch.zeros_like(kc[0]), torch.zeros_like(vc[0])
    got = ops.linear_rope_kv_write(x, w, bias, pos, table, hd, nq, nkv, hd, None, k2, v2)
    _close(got, ref.rope_kv_write(x.float() @ w.float().t(), bias, pos, table, hd, nq, nkv, hd, None, k2, v2, dtype), dtype, scale=4.0)
    assert not k2.any() and not v2.any()
    # what it does not take: a rotation of part of the head, many tokens
    assert not ops.qkv_rope_supports(x, w, table[:, :, :hd // 4].contiguous(), hd // 2, nq, nkv, hd, k2)
    assert not ops.qkv_rope_supports(torch.zeros(40, K, device="cuda", dtype=dtype), w, table, hd, nq, nkv, hd, k2)


def _paged_case(g, lens, q_lens, nq, nkv, hd, ps, dtype, spare_pages=3, consecutive=False):
    """Random cache content for requests of `lens` tokens whose last `q_lens` are queries; their pages
    scattered over the pool, or (`consecutive`) each request's pages with consecutive ids."""
    S = len(lens)
    n_pages = sum(-(-n // ps) for n in lens) + spare_pages
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(9)).tolist()
    if consecutive == "runs":
        # runs of six consecutive ids, the runs in scrambled order: some key tiles lie inside a run
        # (one box), some straddle two (a box a page)
        ids = list(range(n_pages))
        blocks = [ids[i:i + 6] for i in range(0, n_pages, 6)]
        order = torch.randperm(len(blocks), generator=torch.Generator().manual_seed(10)).tolist()
        perm = [x for b in order for x in blocks[b]][::-1]
    elif consecutive:
        perm = list(range(n_pages - 1, -1, -1))           # popped from the end: 0, 1, 2, ...
    kc = torch.randn(n_pages, nkv, ps, hd, device="cuda", generator=g).to(dtype)
    vc = torch.randn(n_pages, nkv, ps, hd, device="cuda", generator=g).to(dtype)
    max_pages = max(-(-n // ps) for n in lens)
    bt = torch.full((S, max_pages), -1, dtype=torch.int32)
    for s, n in enumerate(lens):
        for i in range(-(-n // ps)):
            bt[s, i] = perm.pop()
    positions, seq = [], []
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        positions += list(range(n - ql, n))
        seq += [s] * ql
    T = len(positions)
    q = torch.randn(T, nq * hd, device="cuda", generator=g).to(dtype)
    return q, kc, vc, bt.cuda(), torch.tensor(positions, dtype=torch.int32).cuda(), torch.tensor(seq, dtype=torch.int32).cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,ps,window", [(4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 2, 48, 4, 10),
                                                 (5, 5, 80, 16, None), (14, 2, 64, 16, None), (8, 1, 128, 32, 33),
                                                 (2, 1, 256, 16, None)])
def test_attention_simt(dtype, nq, nkv, hd, ps, window):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(7)
    lens, q_lens = [70, 1, 33, 129], [5, 1, 33, 2]
    q, kc, vc, bt, pos, seq = _paged_case(g, lens, q_lens, nq, nkv, hd, ps, dtype)
    scale = hd ** -0.5
    got = ops.attention_simt(q, kc, vc, bt, pos, seq, nq, nkv, hd, scale, window)
    want = ref.attention_simt(q.float(), kc.float(), vc.float(), bt, pos, seq, nq, nkv, hd, scale, window)
    _close(got, want, dtype, scale=2.0)


def test_attention_finds_a_far_key():
    """One key far back among hundreds, made to stand out by scaling it and the query:
    the output must be that key's value row.  Random weights alone would hide a kernel
    that drops or misplaces a single far page."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(8)
    nq, nkv, hd, ps = 4, 2, 32, 16
    for dtype in (torch.float32, torch.bfloat16):
        for far in (0, 15, 16, 17, 255, 256, 300, 511):
            q, kc, vc, bt, pos, seq = _paged_case(g, [512], [1], nq, nkv, hd, ps, dtype)
            page, off = int(bt[0, far // ps]), far % ps
            direction = torch.randn(hd, device="cuda", generator=g)
            direction /= direction.norm()
            kc[page, :, off, :] = (direction * 12).to(dtype)
            q[0] = (direction * 12).repeat(nq).to(dtype)
            got = ops.attention_simt(q, kc, vc, bt, pos, seq, nq, nkv, hd, 1.0, None).float().reshape(nq, hd)
            want = vc[page, :, off, :].float().repeat_interleave(nq // nkv, dim=0)
            torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2)


def test_attention_window_edge():
    """A standing-out key exactly at the window's edge is seen, one step beyond it is not."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(9)
    nq, nkv, hd, ps, window = 2, 1, 16, 8, 24
    q, kc, vc, bt, pos, seq = _paged_case(g, [100], [1], nq, nkv, hd, ps, torch.float32)
    direction = torch.ones(hd, device="cuda") / hd ** 0.5
    q[0] = (direction * 10).repeat(nq)
    for key, seen in ((99 - window + 1, True), (99 - window, False)):
        k2 = kc.clone()
        page, off = int(bt[0, key // ps]), key % ps
        k2[page, :, off, :] = direction * 10
        got = ops.attention_simt(q, k2, vc, bt, pos, seq, nq, nkv, hd, 1.0, window).reshape(nq, hd)
        is_value = torch.allclose(got[0], vc[page, 0, off], rtol=1e-2, atol=1e-2)
        assert is_value == seen


@pytest.mark.parametrize("R,V", [(1, 256), (5, 1000), (3, 152064)])
def test_sample_rows(R, V):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(10)
    logits = torch.randn(R, V, device="cuda", generator=g) * 3
    logits[0, 7] = logits[0, 3] = logits[0].max() + 1          # a tie: the first maximum wins
    assert ops.sample_rows(logits).tolist() == [3] + logits[1:].argmax(-1).tolist()
    temps = torch.tensor([0.8, 0.0, 1.3, 0.5, 2.0][:R], device="cuda")
    for trial in range(4):
        u = torch.rand(R, device="cuda", generator=g, dtype=torch.float64)
        got = ops.sample_rows(logits, temps, u).tolist()
        want = ref.sample_rows(logits, temps, u).tolist()
        assert got == want
    # the ends of the unit interval
    lo = ops.sample_rows(logits, temps, torch.zeros(R, device="cuda", dtype=torch.float64)).tolist()
    hi = ops.sample_rows(logits, temps, torch.ones(R, device="cuda", dtype=torch.float64)).tolist()
    for r in range(R):
        if float(temps[r]) > 0:
            assert lo[r] == 0 and hi[r] >= V - 2


@pytest.mark.parametrize("V", [97, 1000, 50257, 152064])
def test_sample_rows_top_k_and_top_p(V):
    """The kept set against the float64 sampler, over many uniforms: a token outside the set is
    never returned and the kept ones come at the uniforms the plain sampler gives them."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(V)
    cases = [(0.7, 5, -1.0), (1.0, 0, 0.8), (1.3, 40, 0.5), (0.9, 1, -1.0), (0.5, 0, 0.0), (1.0, 3, 1.0),
             (2.0, V, 0.95), (1.0, V + 5, -1.0), (0.0, 4, 0.3), (1.1, 1000, 0.999), (0.9, 200, 0.7), (1.2, 256, -1.0)]
    R = len(cases)
    logits = torch.randn(R, V, device="cuda", generator=g) * 2.5
    logits[1, V // 2] = logits[1].max() + 3                   # one token holds most of the mass
    temps = torch.tensor([c[0] for c in cases], device="cuda")
    top_k = torch.tensor([c[1] for c in cases], device="cuda", dtype=torch.int32)
    top_p = torch.tensor([c[2] for c in cases], device="cuda")
    for trial in range(6):
        u = torch.rand(R, device="cuda", generator=g, dtype=torch.float64)
        if trial == 4:
            u.fill_(1e-300)                                   # (at exactly 0 the plain sampler names token 0, kept or not)
        if trial == 5:
            u.fill_(1.0 - 1e-12)
        got = ops.sample_rows(logits, temps, u, top_k, top_p).tolist()
        want = ref.sample_rows(logits, temps, u, top_k, top_p).tolist()
        assert got == want, (trial, got, want)
    # only one of the two filters given
    u = torch.rand(R, device="cuda", generator=g, dtype=torch.float64)
    assert ops.sample_rows(logits, temps, u, top_k, None).tolist() == ref.sample_rows(logits, temps, u, top_k, None).tolist()
    assert ops.sample_rows(logits, temps, u, None, top_p).tolist() == ref.sample_rows(logits, temps, u, None, top_p).tolist()
    with pytest.raises(ops.KernelError):
        ops.sample_rows(logits, None, None, top_k, None)


def test_sample_rows_filters_with_ties():
    """Equal logits at the cut: top-k keeps exactly k tokens and top-p exactly as many of the
    ties as reach its mass, the first ones by index; every kept token can be drawn, no other."""
    ops = _ops()
    V = 300
    logits = torch.full((3, V), -4.0, device="cuda")
    tied = [250, 11, 40, 199, 120, 77]                        # six tokens share the top value
    logits[:, tied] = 2.0
    logits[:, 5] = 3.0                                        # and one lies above them
    temps = torch.ones(3, device="cuda")
    top_k = torch.tensor([4, 0, 5], device="cuda", dtype=torch.int32)     # 5 and three of the ties; -; 5 and four ties
    p5, p_tie = np.exp(3.0), np.exp(2.0)
    tot = p5 + 6 * p_tie + (V - 7) * np.exp(-4.0)
    # row 1: top-p reaches its mass inside the ties: after the top token and two of them
    tp1 = (p5 + 1.5 * p_tie) / tot
    # row 2: top-k keeps 5 (the top token and four ties); top-p of that set ends after three ties
    tp2 = (p5 + 2.5 * p_tie) / (p5 + 4 * p_tie)
    top_p = torch.tensor([-1.0, tp1, tp2], device="cuda", dtype=torch.float32)
    want = [sorted([5] + sorted(tied)[:3]), sorted([5] + sorted(tied)[:2]), sorted([5] + sorted(tied)[:3])]
    seen = [set(), set(), set()]
    for i in range(400):
        u = torch.full((3,), (i + 0.5) / 400, device="cuda", dtype=torch.float64)
        for r, t in enumerate(ops.sample_rows(logits, temps, u, top_k, top_p).tolist()):
            seen[r].add(t)
    assert [sorted(s) for s in seen] == want


def test_sample_rows_small_top_k_when_one_thread_holds_the_largest():
    """The one-pass form for a small top_k keeps four candidates a thread; a row whose largest logits
    all fall to one thread (indices 1024 apart) must come out the same, through the general form."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(77)
    V, R = 20000, 4
    logits = torch.randn(R, V, device="cuda", generator=g)
    for r in range(R):
        logits[r, 7 + 1024 * torch.arange(8 + r, device="cuda")] = 6.0 + torch.rand(8 + r, device="cuda", generator=g)
    temps = torch.tensor([1.0, 0.7, 1.5, 1.0], device="cuda")
    top_k = torch.tensor([6, 8, 5, 10], device="cuda", dtype=torch.int32)       # 5: four candidates are not enough either
    top_p = torch.tensor([-1.0, 0.9, -1.0, 0.6], device="cuda")
    for trial in range(8):
        u = torch.rand(R, device="cuda", generator=g, dtype=torch.float64)
        got = ops.sample_rows(logits, temps, u, top_k, top_p).tolist()
        want = ref.sample_rows(logits, temps, u, top_k, top_p).tolist()
        assert got == want, (trial, got, want)
        assert all((t - 7) % 1024 == 0 for t in got)


def test_seen_table_marks_and_penalises():
    """The table of seen ids on the device: a step's tokens are recorded under their requests' slots
    (ids and slots out of range ignored), and the penalty changes exactly the seen ids of the rows
    that have one."""
    from types import SimpleNamespace
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(5)
    V, slots = 1000, 5
    seen = torch.zeros(slots, V, dtype=torch.uint8, device="cuda")
    seen[3, 17] = 1                                            # what an earlier step left
    i32 = dict(device="cuda", dtype=torch.int32)
    step = SimpleNamespace(num_tokens=7, token_ids=torch.tensor([5, 999, 5, 17, 1000, 2, 8], **i32),
                           seq_of_token=torch.tensor([0, 0, 0, 1, 1, 2, 3], **i32),
                           state_slots=torch.tensor([3, 0, 4, 7], **i32),          # the last slot lies outside the table
                           logit_rows=torch.tensor([2, 4, 5], **i32))
    want_seen = seen.clone()
    ref.mark_seen(want_seen, step)
    ops.mark_seen(seen, step)
    assert torch.equal(seen, want_seen)
    assert seen[3].nonzero().flatten().tolist() == [5, 17, 999] and seen[0].nonzero().flatten().tolist() == [17]
    assert seen[4].nonzero().flatten().tolist() == [2] and int(seen.sum()) == 5
    logits = torch.randn(3, V, device="cuda", generator=g) * 3
    pen = torch.tensor([1.3, 1.0, 0.5], device="cuda")
    want = ref.penalty_from_seen_(logits.clone(), seen, step, pen)
    got = ops.penalty_from_seen_(logits.clone(), seen, step, pen)
    torch.testing.assert_close(got, want, rtol=1e-6, atol=0)
    assert torch.equal(got[1], logits[1])                      # penalty 1: untouched
    assert (got[0] != logits[0]).nonzero().flatten().tolist() == [5, 17, 999]
    assert (got[2] != logits[2]).nonzero().flatten().tolist() == [2]


def test_repetition_penalty_in_place():
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(4)
    R, V = 4, 1000
    logits = torch.randn(R, V, device="cuda", generator=g) * 3
    rows = torch.tensor([0, 0, 0, 2, 2, 3, 3], device="cuda", dtype=torch.int32)
    ids = torch.tensor([5, 999, 17, 0, 5, 1000, -1], device="cuda", dtype=torch.int32)      # the last two lie outside
    pen = torch.tensor([1.5, 1.5, 1.5, 0.7, 0.7, 2.0, 2.0], device="cuda")
    want = ref.repetition_penalty_(logits.clone(), rows, ids, pen)
    got = ops.repetition_penalty_(logits.clone(), rows, ids, pen)
    torch.testing.assert_close(got, want, rtol=1e-6, atol=0)
    assert torch.equal(got[1], logits[1]) and torch.equal(got[3], logits[3])
    assert not torch.equal(got[0], logits[0])


def test_gather_rows():
    ops = _ops()
    x = torch.randn(40, 1000, device="cuda")
    rows = torch.tensor([39, 0, 7, 7], dtype=torch.int32, device="cuda")
    assert torch.equal(ops.gather_rows(x, rows), x[rows.long()])
    assert torch.equal(ops.gather_rows(x.bfloat16(), rows), x.bfloat16()[rows.long()])


def test_kernels_refuse_what_they_cannot_do():
    ops = _ops()
    from sllm_b200.ops import KernelError
    with pytest.raises(KernelError, match="CUDA"):
        ops.embed_gather(torch.zeros(4, 4), torch.zeros(2, dtype=torch.int32))
    x = torch.zeros(4, 8, device="cuda")
    with pytest.raises(KernelError):
        ops.linear(x, torch.zeros(4, 9, device="cuda"), None, torch.float32)
    q = torch.zeros(1, 2 * 272, device="cuda")
    kc = torch.zeros(2, 1, 16, 272, device="cuda")
    with pytest.raises(KernelError, match="head_dim"):
        ops.attention_simt(q, kc, kc, torch.zeros(1, 1, dtype=torch.int32, device="cuda"),
                           torch.zeros(1, dtype=torch.int32, device="cuda"),
                           torch.zeros(1, dtype=torch.int32, device="cuda"), 2, 1, 272, 1.0, None)


def _starts(q_lens, lens):
    qs = [0]
    for n in q_lens:
        qs.append(qs[-1] + n)
    return (torch.tensor(qs, dtype=torch.int32).cuda(), torch.tensor(lens, dtype=torch.int32).cuda())


@pytest.mark.parametrize("nq,nkv,hd,ps,window", [(4, 2, 16, 16, None), (3, 1, 32, 8, None), (14, 2, 64, 16, None),
                                                 (28, 4, 128, 16, None), (8, 1, 128, 32, 40), (6, 3, 64, 4, 9),
                                                 (40, 2, 32, 16, None)])
@pytest.mark.parametrize("case", ["prefill", "decode", "decode_split", "mixed"])
def test_attention_mma(nq, nkv, hd, ps, window, case):
    """The tensor-core kernel in both forms against the float32 statement: portions that
    start in mid-context, single tokens, split contexts, and both in one batch."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(11)
    lens, q_lens = {"prefill": ([70, 33, 200], [70, 5, 131]), "decode": ([300, 1, 17, 64], [1, 1, 1, 1]),
                    "decode_split": ([1500, 700, 3], [1, 1, 1]), "mixed": ([90, 400, 2, 65], [37, 1, 2, 1])}[case]
    q, kc, vc, bt, pos, seq = _paged_case(g, lens, q_lens, nq, nkv, hd, ps, torch.bfloat16)
    q_start, ctx_len = _starts(q_lens, lens)
    scale = hd ** -0.5
    want = ref.attention_simt(q.float(), kc.float(), vc.float(), bt, pos, seq, nq, nkv, hd, scale, window)
    G = nq // nkv
    small, large = ops.attention_tiles(q_lens, G, "cuda")
    out = torch.full_like(q, float("nan"))
    if small:
        splits = {"decode_split": 5, "decode": 2}.get(case, 1) if not large else 1
        ops.attention_mma(q, kc, vc, bt, q_start, ctx_len, small, True, splits, nq, nkv, hd, scale, window, out)
    if large:
        ops.attention_mma(q, kc, vc, bt, q_start, ctx_len, large, False, 1, nq, nkv, hd, scale, window, out)
    assert not out.isnan().any(), "a row was not written"
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nq,nkv,hd,ps", [(28, 4, 128, 16), (14, 2, 64, 16), (8, 8, 128, 8), (6, 1, 64, 32), (4, 2, 128, 64)])
@pytest.mark.parametrize("case", ["prefill", "long", "mixed", "peaked"])
@pytest.mark.parametrize("row_tiles", [1, 2])
@pytest.mark.parametrize("consecutive", [False, True, "runs"])
def test_attention_tc(nq, nkv, hd, ps, case, row_tiles, consecutive):
    """The tcgen05 prefill form against the float32 statement: portions that start in mid-context, rows
    of several requests, many key tiles, and scores so peaked that the running maximum jumps from tile
    to tile (the output in tensor memory is rescaled)."""
    ops = _ops()
    if not ops.tc_attention_supports(hd, ps):
        pytest.skip("not taken by the tcgen05 form")
    g = torch.Generator(device="cuda").manual_seed(21)
    lens, q_lens = {"prefill": ([70, 33, 200], [70, 5, 131]), "long": ([1000, 2100], [1000, 300]),
                    "mixed": ([90, 400, 2, 65, 129], [37, 1, 2, 1, 128]), "peaked": ([700], [650])}[case]
    q, kc, vc, bt, pos, seq = _paged_case(g, lens, q_lens, nq, nkv, hd, ps, torch.bfloat16, consecutive=consecutive)
    q_start, ctx_len = _starts(q_lens, lens)
    scale = 1.0 if case == "peaked" else hd ** -0.5
    want = ref.attention_simt(q.float(), kc.float(), vc.float(), bt, pos, seq, nq, nkv, hd, scale, None)
    G = nq // nkv
    small, large = ops.attention_tiles(q_lens, G, "cuda", lens, 128 * row_tiles)
    out = torch.full_like(q, float("nan"))
    if small:
        ops.attention_mma(q, kc, vc, bt, q_start, ctx_len, small, True, 1, nq, nkv, hd, scale, None, out)
    assert large
    ops.attention_tc(q, kc, vc, bt, q_start, ctx_len, large, nq, nkv, hd, scale, out, row_tiles=row_tiles)
    ops.check_tcgen05_status()
    assert not out.isnan().any(), "a row was not written"
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nq,nkv,hd,ps", [(28, 4, 128, 16), (6, 1, 64, 32), (4, 2, 128, 64)])
@pytest.mark.parametrize("case", ["long", "mixed", "peaked", "far"])
@pytest.mark.parametrize("splits", [(2, 20), (3, 11), (5, 7), (9, 4), (40, 1)])
def test_attention_tc_context_split(nq, nkv, hd, ps, case, splits):
    """The prefill form with its context cut into ranges that run as CTAs of their own and are merged:
    ranges that hold no key of a row tile (a portion's early rows), ranges of one key tile, rows of
    decoded tokens that another kernel wrote and the merge must leave alone, and a key that stands
    out in one range."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(23)
    lens, q_lens = {"long": ([1000, 2100], [1000, 300]), "mixed": ([90, 400, 2, 65, 2200], [37, 1, 2, 1, 128]),
                    "peaked": ([2300], [650]), "far": ([2500], [200])}[case]
    if splits[0] * splits[1] * 64 < max(lens):
        splits = (-(-max(lens) // (64 * splits[1])), splits[1])         # the ranges must cover the longest context
    q, kc, vc, bt, pos, seq = _paged_case(g, lens, q_lens, nq, nkv, hd, ps, torch.bfloat16, consecutive="runs")
    q_start, ctx_len = _starts(q_lens, lens)
    scale = 1.0 if case == "peaked" else hd ** -0.5
    if case == "far":
        far = 777                                                       # one key of the second range or so wins every row
        direction = torch.randn(hd, device="cuda", generator=g)
        direction /= direction.norm()
        kc[int(bt[0, far // ps]), :, far % ps, :] = (direction * 16).bfloat16()
        q[:] = (direction * 16).repeat(nq).bfloat16()
        scale = 1.0
    want = ref.attention_simt(q.float(), kc.float(), vc.float(), bt, pos, seq, nq, nkv, hd, scale, None)
    small, large = ops.attention_tiles(q_lens, nq // nkv, "cuda", lens, 128)
    out = torch.full_like(q, float("nan"))
    if small:
        ops.attention_mma(q, kc, vc, bt, q_start, ctx_len, small, True, 1, nq, nkv, hd, scale, None, out)
    before = out.clone()
    ops.attention_tc(q, kc, vc, bt, q_start, ctx_len, large, nq, nkv, hd, scale, out, splits=splits)
    ops.check_tcgen05_status()
    assert not out.isnan().any(), "a row was not written"
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)
    kept = ~before.isnan().any(dim=1)
    assert torch.equal(out[kept], before[kept]), "the merge touched rows of another kernel"
    if case == "far":
        torch.testing.assert_close(out.float().reshape(-1, nq, hd)[0], vc[int(bt[0, far // ps]), :, far % ps, :].float()
                                   .repeat_interleave(nq // nkv, dim=0), rtol=2e-2, atol=2e-2)


def test_choose_tc_splits_covers_the_context():
    ops = _ops()
    for tiles, nkv, ctx in ((112, 4, 2048), (28, 4, 32768), (7, 4, 32768), (1, 1, 100), (3, 2, 5000), (28, 4, 1025)):
        n, per = ops.choose_tc_splits(tiles, nkv, ctx)
        assert n >= 1 and n * per * 64 >= ctx and (n - 1) * per * 64 < ctx
        assert n == 1 or per >= 16
    assert ops.choose_tc_splits(112, 4, 2048)[0] == 1 and ops.choose_tc_splits(28, 4, 32768)[0] == 2


def test_a_wait_that_nothing_ends_gives_up_and_says_so():
    """The bounded wait of the TMA-fed kernels: a barrier nothing arrives at, a limit of 3 ms; the kernel
    returns with its status word set, in about that time, and the device goes on working."""
    ops = _ops()
    status, waited = ops.wait_probe(3_000_000)
    assert status == 99
    assert 3_000_000 <= waited < 50_000_000
    x = torch.arange(1000, device="cuda", dtype=torch.float32)
    assert float(x.sum()) == 499500.0
    with pytest.raises(ops.KernelError):
        ops.wait_probe(10 ** 9)             # longer than the probe allows: refused on the host


def test_attention_tc_far_key_and_page_edges():
    """One key stands out for every query, at page and tile edges of a long prompt."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(22)
    nq, nkv, hd, ps = 8, 2, 128, 16
    n = 1100
    for far in (0, 15, 16, 63, 64, 65, 127, 128, 1023, 1024):
        q, kc, vc, bt, pos, seq = _paged_case(g, [n], [n], nq, nkv, hd, ps, torch.bfloat16)
        q_start, ctx_len = _starts([n], [n])
        page, off = int(bt[0, far // ps]), far % ps
        direction = torch.randn(hd, device="cuda", generator=g)
        direction /= direction.norm()
        kc[page, :, off, :] = (direction * 16).bfloat16()
        q[:] = (direction * 16).repeat(nq).bfloat16()
        row_tiles = 1 + (far % 2)
        _, large = ops.attention_tiles([n], nq // nkv, "cuda", [n], 128 * row_tiles)
        got = ops.attention_tc(q, kc, vc, bt, q_start, ctx_len, large, nq, nkv, hd, 1.0, row_tiles=row_tiles)
        ops.check_tcgen05_status()
        # queries at or after the far key return its value; the ones before it cannot see it
        want = vc[page, :, off, :].float().repeat_interleave(nq // nkv, dim=0)
        torch.testing.assert_close(got.float().reshape(n, nq, hd)[far:], want.expand(n - far, nq, hd), rtol=2e-2, atol=2e-2)
        if far > 0:
            full = ref.attention_simt(q.float(), kc.float(), vc.float(), bt, pos, seq, nq, nkv, hd, 1.0, None)
            torch.testing.assert_close(got.float()[:far], full[:far], rtol=2e-2, atol=2e-2)


def test_attention_mma_far_key_and_page_edges():
    """A standing-out key at page and tile edges of a long context, in the split form."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(12)
    nq, nkv, hd, ps = 8, 2, 64, 16
    for far in (0, 15, 16, 63, 64, 65, 1023, 1024, 2047):
        q, kc, vc, bt, pos, seq = _paged_case(g, [2048], [1], nq, nkv, hd, ps, torch.bfloat16)
        q_start, ctx_len = _starts([1], [2048])
        page, off = int(bt[0, far // ps]), far % ps
        direction = torch.randn(hd, device="cuda", generator=g)
        direction /= direction.norm()
        kc[page, :, off, :] = (direction * 14).bfloat16()
        q[0] = (direction * 14).repeat(nq).bfloat16()
        small, _ = ops.attention_tiles([1], nq // nkv, "cuda")
        for splits in (1, 4):
            got = ops.attention_mma(q, kc, vc, bt, q_start, ctx_len, small, True, splits, nq, nkv, hd, 1.0, None)
            want = vc[page, :, off, :].float().repeat_interleave(nq // nkv, dim=0)
            torch.testing.assert_close(got.float().reshape(nq, hd), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("N,K", [(144, 128), (1000, 384), (4608, 3584), (264, 1152)])
def test_linear_stream(M, N, K):
    """The weight-streaming kernel against the float32 statement: every token count up to
    64, widths that are no multiple of the tile, direct and k-split results, both dtypes."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(13)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, device="cuda", generator=g)
    want = x.float() @ w.float().t() + b
    assert ops.stream_supports(min(M, ops.STREAM_MAX_ROWS), N, K)
    got = ops.linear_stream(x, w, b, torch.float32)
    torch.testing.assert_close(got, want, rtol=2e-3, atol=2e-3)
    got = ops.linear_stream(x, w, b, torch.bfloat16)
    torch.testing.assert_close(got.float(), want, rtol=1.6e-2, atol=1.6e-2)
    for splits in (2, 3, 16):
        parts = ops.linear_stream(x, w, b, torch.float32, splits=splits)
        if K // 128 == 1:
            assert parts.dim() == 2
        else:
            assert parts.dim() == 3 and parts.shape[0] <= splits
            parts = parts.sum(0)
        torch.testing.assert_close(parts, want, rtol=2e-3, atol=2e-3)
    # through ops.linear: the same kernel, splits chosen by the width
    got = ops.linear(x, w, b, torch.float32, True)
    torch.testing.assert_close(got.sum(0) if got.dim() == 3 else got, want, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("M", [1, 8, 19, 64])
@pytest.mark.parametrize("I,K", [(72, 128), (4864, 896), (1000, 256)])
def test_linear_stream_silu(M, I, K):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(14)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    wg = (torch.randn(I, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    wu = (torch.randn(I, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    gu = torch.stack([wg.reshape(I // 8, 8, K), wu.reshape(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()
    gate, up = x.float() @ wg.float().t(), x.float() @ wu.float().t()
    want = gate * torch.sigmoid(gate) * up
    got = ops.linear_silu_mul(x, gu, 8, torch.bfloat16)
    torch.testing.assert_close(got.float(), want, rtol=1.6e-2, atol=1.6e-2)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (200, 300, 72), (2048, 512, 3584), (77, 1000, 336),
                                   (513, 264, 128)])
def test_gemm_tcgen05(M, N, K):
    """The tcgen05 product against the float32 statement: whole tiles, ragged M and N, a k tail."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(15)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, device="cuda", generator=g)
    want = x.float() @ w.float().t() + b
    got = ops.gemm_tcgen05(x, w, b, torch.float32)
    ops.check_tcgen05_status()
    torch.testing.assert_close(got, want, rtol=2e-3, atol=2e-3)
    got = ops.gemm_tcgen05(x, w, b, torch.bfloat16)
    ops.check_tcgen05_status()
    torch.testing.assert_close(got.float(), want, rtol=1.6e-2, atol=1.6e-2)


@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (300, 200, 136), (1024, 4864, 896)])
def test_gemm_tcgen05_silu(M, I, K):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(16)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    wg = (torch.randn(I, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    wu = (torch.randn(I, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    gu = torch.stack([wg.reshape(I // 8, 8, K), wu.reshape(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()
    gate, up = x.float() @ wg.float().t(), x.float() @ wu.float().t()
    want = gate * torch.sigmoid(gate) * up
    got = ops.gemm_tcgen05(x, gu, None, torch.bfloat16, silu=True)
    ops.check_tcgen05_status()
    torch.testing.assert_close(got.float(), want, rtol=1.6e-2, atol=1.6e-2)


@pytest.mark.parametrize("wide", [False, True, 448, 384, 320])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (256, 512, 64), (129, 304, 72), (300, 300, 72), (333, 1000, 136), (512, 1040, 520),
                                   (1000, 3008, 264), (2048, 4608, 3584), (600, 3584, 18944)])
def test_gemm_pair(M, N, K, wide):
    """The product by pairs of CTAs (tcgen05.mma with cta_group::2), on tiles of 256 x 256 and of 256 x 512, all
    three epilogues, and on tiles of 256 x 448, 384 and 320 (the second product of a k step narrower than the
    first) with the float32 result: one tile with one k block, several tiles a pair, edges in M and N (rows and
    columns of a tile that lie outside the result; results whose rows are no whole 16-byte pieces leave lane by
    lane instead of through TMA stores), a long reduction."""
    ops = _ops()
    assert ops.pair_supports(M, N, K)
    g = torch.Generator(device="cuda").manual_seed(51)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, device="cuda", generator=g)
    want = x.float() @ w.float().t()
    torch.testing.assert_close(ops.gemm_pair(x, w, b, torch.float32, wide=wide), want + b, rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(ops.gemm_pair(x, w, None, torch.float32, wide=wide), want, rtol=2e-3, atol=2e-3)
    if wide not in (False, True):
        with pytest.raises(ops.KernelError, match="only with a float32 result or a residual"):
            ops.gemm_pair(x, w, b, torch.bfloat16, wide=wide)
    else:
        torch.testing.assert_close(ops.gemm_pair(x, w, b, torch.bfloat16, wide=wide).float(), want + b, rtol=1.6e-2, atol=1.6e-2)
    if N % 16 == 0 and wide in (False, True):
        gu = want.reshape(M, N // 16, 2, 8)
        act = (torch.nn.functional.silu(gu[:, :, 0]) * gu[:, :, 1]).reshape(M, N // 2)
        torch.testing.assert_close(ops.gemm_pair(x, w, None, torch.bfloat16, silu=True, wide=wide).float(), act, rtol=2e-2, atol=2e-2)
    ops.check_tcgen05_status()
    # the same bits from both tile shapes and from the one-CTA form: every element sums its k in one order
    assert torch.equal(ops.gemm_pair(x, w, b, torch.float32, wide=wide), ops.gemm_tcgen05(x, w, b, torch.float32))


@pytest.mark.parametrize("wide", [False, True, 448, 384, 320])
@pytest.mark.parametrize("M,H,K", [(256, 256, 64), (300, 3584, 520), (2048, 3584, 3584), (333, 1000, 136), (129, 904, 72)])
def test_gemm_pair_owes_and_pays_an_rmsnorm(M, H, K, wide):
    """A prompt portion's products take the RMSNorm between them apart as the decode step's do: the product that
    completes the residual stream adds into it in place and writes bfloat16(stream * gain) with sums of squares per
    row and block of 128 columns; the products that follow (plain, and gate|up with SiLU*mul) multiply their rows by
    the reciprocal root mean square (y = x * rsqrt(mean(x^2) + eps) * gain, ref/standard.py:25-31)."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(61)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(H, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(H, device="cuda", generator=g)
    gain = 1 + 0.3 * torch.randn(H, device="cuda", generator=g)
    eps = 1e-5
    res = 3 * torch.randn(M, H, device="cuda", generator=g)
    stream = res + x.float() @ w.float().t() + b
    # the residual update alone
    alone = res.clone()
    assert ops.gemm_pair(x, w, b, torch.float32, wide=wide, residual=alone) is None
    torch.testing.assert_close(alone, stream, rtol=2e-3, atol=2e-3)
    # with the next norm's input
    xg, scale = ops.gemm_pair(x, w, b, torch.float32, wide=wide, residual=res, next_gain=gain)
    scale.eps = eps
    ops.check_tcgen05_status()
    assert torch.equal(res, alone)
    torch.testing.assert_close(xg.float(), (res * gain).bfloat16().float(), rtol=1e-2, atol=1e-2)
    if wide in (False, True):
        assert scale.parts == -(-H // 128)
    else:       # four blocks a tile (128, 128 and twice the rest of the half); of the last tile those that start inside H
        starts = [t * wide + o for t in range(-(-H // wide)) for o in (0, 128, wide // 2, wide // 2 + 128)]
        assert scale.parts == sum(1 for n in starts if n < H)
    assert scale.width == H
    torch.testing.assert_close(scale.ssq[:, :scale.parts].sum(1), (res ** 2).sum(1), rtol=1e-4, atol=1e-4)
    normed = res * torch.rsqrt((res ** 2).mean(1, keepdim=True) + eps) * gain
    for wide2 in (False, True):
        N2 = 528
        w2 = (torch.randn(N2, H, device="cuda", generator=g) / H ** 0.5).bfloat16()
        b2 = torch.randn(N2, device="cuda", generator=g)
        want = normed @ w2.float().t() + b2
        torch.testing.assert_close(ops.gemm_pair(xg, w2, b2, torch.float32, wide=wide2, scale=scale), want, rtol=2e-2, atol=2e-2)
        gu = (want - b2).reshape(M, N2 // 16, 2, 8)
        act = (torch.nn.functional.silu(gu[:, :, 0]) * gu[:, :, 1]).reshape(M, N2 // 2)
        torch.testing.assert_close(ops.gemm_pair(xg, w2, None, torch.bfloat16, silu=True, wide=wide2, scale=scale).float(), act,
                                   rtol=2e-2, atol=2e-2)
    ops.check_tcgen05_status()


def test_the_width_of_the_wide_tiles_goes_by_waves():
    """`ops.pair_wide_cols`: 512-wide tiles where they fill the pairs of SMs, narrower ones where those leave fewer
    pairs idle, 256-wide ones where a pair walks many tiles; the default of `gemm_pair` follows it."""
    ops = _ops()
    pairs = ops.num_sms() // 2
    for M in (256, 512, 1024, 2048, 4096, 8192):
        for N in (896, 1536, 2048, 3584, 4608, 5120, 8192, 18944):
            form = ops.pair_wide_cols(M, N)
            assert form in (False, True, 448, 384, 320)
            if form not in (False, True):     # fewer waves than the 512-wide tiles need, or the same with less width
                mt = -(-M // 256)
                assert -(-(mt * -(-N // form)) // pairs) <= -(-(mt * -(-N // 512)) // pairs)
    if pairs == 74:
        assert ops.pair_wide_cols(2048, 3584) == 448 and ops.pair_wide_cols(2048, 4608) is True
        assert ops.pair_wide_cols(2048, 18944) is False and ops.pair_wide_cols(1024, 5120) == 320
    g = torch.Generator(device="cuda").manual_seed(71)
    M, N, K = 1024, 5120, 200
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    assert torch.equal(ops.gemm_pair(x, w, None, torch.float32), ops.gemm_pair(x, w, None, torch.float32, wide=False))
    ops.check_tcgen05_status()


@pytest.mark.parametrize("M,N,K", [(130, 264, 1160), (200, 3584, 3584), (512, 1000, 18944), (700, 520, 1024), (257, 8, 520)])
def test_gemm_pair_in_slices_of_k(M, N, K):
    """The CTA-pair product cut along K: a stack of float32 partial sums whose sum is the product (bias once), every
    number of slices up to what K gives, ragged edges, both tile widths; and through the dispatch, which cuts where
    the result has few tiles."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(23)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, device="cuda", generator=g)
    want = x.float() @ w.float().t() + b
    for splits in (2, 3, 5, 8, 1000):
        for wide in (False, "slim"):
            parts = ops.gemm_pair(x, w, b, torch.float32, splits=splits, wide=wide)
            assert parts.dim() == 3 and 2 <= parts.shape[0] <= min(splits, -(-K // 64)), parts.shape
            torch.testing.assert_close(parts.sum(0), want, rtol=2e-3, atol=2e-3, msg=lambda m: f"{splits} slices, {wide}: {m}")
            torch.testing.assert_close(parts[1:].sum(0) + parts[0], want, rtol=2e-3, atol=2e-3)
    ops.check_tcgen05_status()
    with pytest.raises(ops.KernelError):
        ops.gemm_pair(x, w, b, torch.bfloat16, splits=2)
    stack = ops.linear(x, w, b, torch.float32, allow_partials=True)
    assert (stack.dim() == 3) == (ops.pair_splits(M, N, K) > 1)
    torch.testing.assert_close(stack.sum(0) if stack.dim() == 3 else stack, want, rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(ops.linear(x, w, b, torch.float32), want, rtol=2e-3, atol=2e-3)
    ops.check_tcgen05_status()


@pytest.mark.parametrize("M", [1, 9, 17, 24, 32, 33, 64, 65, 100, 128])
@pytest.mark.parametrize("N,K", [(128, 64), (136, 72), (1000, 264), (4608, 3584), (3584, 18944), (9480, 3584), (75784, 512)])
def test_linear_tc(M, N, K):
    """The tcgen05 streaming product against the float32 statement: one and several slices of K (their
    sum is the product, bias once), ragged rows, a k tail, both accumulator widths, and a row's result
    does not depend on the other rows of the batch.  Few tokens too: the dispatch sends large matrices
    to it from 17 tokens on and very wide ones (an output head) from 9."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(18)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, device="cuda", generator=g)
    want = x.float() @ w.float().t() + b
    assert ops.linear_tc_supports(M, N, K) == (M >= ops._tc_from_rows(N, K))
    assert ops._tc_from_rows(N, K) == (9 if N > 70000 else 17 if N * K >= 1 << 25 else 33)
    whole = ops.linear_tc(x, w, b, torch.float32)
    torch.testing.assert_close(whole, want, rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(ops.linear_tc(x, w, None, torch.bfloat16).float(), want - b, rtol=1.6e-2, atol=1.6e-2)
    for splits in (2, 5, 1000):
        parts = ops.linear_tc(x, w, b, torch.float32, splits=splits)
        if K > 64:
            assert parts.dim() == 3 and 2 <= parts.shape[0] <= min(splits, -(-K // 64))
            parts = parts.sum(0)
        torch.testing.assert_close(parts, want, rtol=2e-3, atol=2e-3)
    ops.check_tcgen05_status()
    fewer = ops.linear_tc(x[M // 2:].contiguous(), w, b, torch.float32)
    assert torch.equal(fewer[-1], whole[-1])
    # and through the dispatch, as the engine calls it
    torch.testing.assert_close(ops.linear(x, w, b, torch.float32), want, rtol=2e-3, atol=2e-3)
    stack = ops.linear(x, w, b, torch.float32, allow_partials=True)
    if ops.linear_tc_supports(M, N, K):
        assert (stack.dim() == 3) == (K >= ops.LINEAR_TC_SPLIT_MIN_K and M <= ops.LINEAR_TC_SPLIT_MAX_ROWS)
    torch.testing.assert_close(stack.sum(0) if stack.dim() == 3 else stack, want, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("M,I,K", [(40, 128, 64), (64, 200, 136), (128, 4864, 896), (96, 18944, 3584), (17, 18944, 3584),
                                   (24, 4744, 3584), (1, 128, 64), (48, 18944, 3584)])
def test_linear_tc_silu(M, I, K):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(19)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    wg = (torch.randn(I, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    wu = (torch.randn(I, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    gu = torch.stack([wg.reshape(I // 8, 8, K), wu.reshape(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()
    gate, up = x.float() @ wg.float().t(), x.float() @ wu.float().t()
    want = gate * torch.sigmoid(gate) * up
    got = ops.linear_tc(x, gu, None, torch.bfloat16, silu=True)
    ops.check_tcgen05_status()
    torch.testing.assert_close(got.float(), want, rtol=1.6e-2, atol=1.6e-2)
    torch.testing.assert_close(ops.linear_silu_mul(x, gu, 8, torch.bfloat16).float(), want, rtol=1.6e-2, atol=1.6e-2)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 25, 32])
@pytest.mark.parametrize("N,K", [(16, 32), (100, 96), (3584, 3584), (4608, 3584), (200, 18944), (1000, 320)])
def test_linear_ws(M, N, K):
    """The warp-split streaming kernel: stores in both dtypes, and the fused residual add."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(17)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, device="cuda", generator=g)
    want = x.float() @ w.float().t() + b
    # what the dispatch sends here: 17..32 tokens only a short reduction into rows enough for one and a half CTAs an SM
    picked = M <= 16 or (K <= ops.WS_ROWS32_MAX_K and N * K <= ops.WS_ROWS32_MAX_ELEMENTS and 2 * -(-N // 16) >= 3 * ops.num_sms())
    assert ops.ws_supports(M, N, K) == picked
    torch.testing.assert_close(ops.linear_ws(x, w, b, torch.float32), want, rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(ops.linear_ws(x, w, None, torch.bfloat16).float(), want - b, rtol=1.6e-2, atol=1.6e-2)
    res = torch.randn(M, N, device="cuda", generator=g)
    expect = res + want
    assert ops.can_accumulate(x, w) == picked
    ops.linear_ws(x, w, b, torch.float32, residual=res)
    torch.testing.assert_close(res, expect, rtol=2e-3, atol=2e-3)
    # the sum does not depend on the other tokens of the batch
    if M > 1:
        one = ops.linear_ws(x[M - 1:].contiguous(), w, b, torch.float32)
        assert torch.equal(one[0], ops.linear_ws(x, w, b, torch.float32)[M - 1])


@pytest.mark.parametrize("M", [1, 3, 8, 11, 16, 21, 32])
@pytest.mark.parametrize("H,K", [(3584, 3584), (3584, 18944), (896, 4864), (1000, 320), (96, 64), (5120, 13824), (8192, 512), (2048, 2048)])
def test_an_rmsnorm_owed_by_one_product_and_paid_by_the_next(M, H, K):
    """The product that completes the residual stream also writes the next RMSNorm's input as
    bfloat16(stream * gain) with partial sums of squares, and the products that consume it (plain, the
    fused q|k|v with its rotary epilogue, gate|up with SiLU*mul) scale their rows by the reciprocal root
    mean square: the same numbers as the norm kernel followed by the plain products, to bfloat16 rounding
    (y = x * rsqrt(mean(x^2) + eps) * gain, ref/standard.py:25-31)."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(41)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(H, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(H, device="cuda", generator=g)
    gain = 1 + 0.3 * torch.randn(H, device="cuda", generator=g)
    eps = 1e-5
    res = 3 * torch.randn(M, H, device="cuda", generator=g)
    stream = res + x.float() @ w.float().t() + b
    assert ops.can_accumulate_norm(x[:8].contiguous(), w)

    def produce(into):
        if M <= 16:
            return ops.linear_accumulate_norm(x, w, b, into, gain, eps)      # as the engine calls it
        # 17..32 tokens: the dispatch has no use for the warp-split kernel with a norm here (the matrices it sends
        # there at so many tokens have more CTAs than the four-tile table holds); the kernel is called directly
        xg_, scale_ = ops.linear_ws(x, w, b, torch.float32, residual=into, next_gain=gain)
        scale_.eps = eps
        return xg_, scale_
    if M > 16 and (H % 32 != 0 or K % 32 != 0 or int(ops.lib().sllm_linear_ws_parts(H, K)) > ops.MAX_SCALE_PARTS_ROWS32):
        return
    xg, scale = produce(res)
    torch.testing.assert_close(res, stream, rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(xg.float(), (res * gain).bfloat16().float(), rtol=1e-2, atol=1e-2)
    assert scale.parts <= ops.MAX_SCALE_PARTS and scale.width == H and scale.eps == eps
    torch.testing.assert_close(scale.ssq[:, :scale.parts].sum(1), (res ** 2).sum(1), rtol=1e-4, atol=1e-4)
    normed = res * torch.rsqrt((res ** 2).mean(1, keepdim=True) + eps) * gain          # what the norm kernel returns
    # a plain product of the normed activations
    N2 = 272
    w2 = (torch.randn(N2, H, device="cuda", generator=g) / H ** 0.5).bfloat16()
    b2 = torch.randn(N2, device="cuda", generator=g)
    want = normed @ w2.float().t() + b2
    if H % 32 == 0:
        got = ops.linear_ws(xg, w2, b2, torch.float32, scale=scale)
        torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2)
        res2 = torch.randn(M, N2, device="cuda", generator=g)
        expect = res2 + want
        ops.linear_ws(xg, w2, b2, torch.float32, residual=res2, scale=scale)
        torch.testing.assert_close(res2, expect, rtol=2e-2, atol=2e-2)
    # gate|up with SiLU*mul
    inter = 264
    wgu = (torch.randn(2 * inter, H, device="cuda", generator=g) / H ** 0.5).bfloat16()
    if ops.silu_scaled_supports(xg, wgu, 8, torch.bfloat16):
        got = ops.linear_silu_mul(xg, wgu, 8, torch.bfloat16, scale=scale).float()
        gu = (normed @ wgu.float().t()).reshape(M, inter // 8, 2, 8)
        want = (torch.nn.functional.silu(gu[:, :, 0]) * gu[:, :, 1]).reshape(M, inter)
        torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2)
    else:
        assert H % 128 != 0
    # the fused q|k|v product with bias, rotation and the cache write
    nq, nkv, hd, ps, pages, max_pos = 3, 1, 32, 8, 9, 100
    wq = (torch.randn((nq + 2 * nkv) * hd, H, device="cuda", generator=g) / H ** 0.5).bfloat16()
    bq = torch.randn((nq + 2 * nkv) * hd, device="cuda", generator=g)
    pos = torch.randint(0, max_pos, (M,), device="cuda", generator=g, dtype=torch.int32)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * (1e4 ** (-torch.arange(0, hd, 2, dtype=torch.float64) / hd))[None]
    table = torch.stack([ang.cos(), ang.sin()], 1).float().cuda()
    slots = torch.randperm(pages * ps, device="cuda", generator=g)[:M].int()
    kc = [torch.zeros(pages, nkv, ps, hd, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    vc = [torch.zeros(pages, nkv, ps, hd, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    if H % 32 == 0:
        got = ops.linear_rope_kv_write(xg, wq, bq, pos, table, hd, nq, nkv, hd, slots, kc[0], vc[0], scale=scale)
        want = ref.rope_kv_write(normed @ wq.float().t(), bq, pos, table, hd, nq, nkv, hd, slots, kc[1], vc[1], torch.bfloat16)
        _close(got, want, torch.bfloat16, scale=4.0)
        _close(kc[0], kc[1], torch.bfloat16, scale=4.0)
        _close(vc[0], vc[1], torch.bfloat16, scale=4.0)
    # the partial sums are written per CTA and added in a fixed order: the same call gives the same bits
    again = stream - (x.float() @ w.float().t() + b)
    first = again.clone()
    xg_a, scale_a = produce(first)
    xg_b, scale_b = produce(again)
    assert torch.equal(xg_a, xg_b) and torch.equal(scale_a.ssq[:, :scale_a.parts], scale_b.ssq[:, :scale_b.parts])


@pytest.mark.parametrize("nq,nkv,hd,ps,window", [(28, 4, 128, 16, None), (14, 2, 64, 16, None), (8, 1, 128, 32, 40),
                                                 (6, 3, 64, 8, 9), (16, 2, 128, 64, None), (7, 7, 64, 16, None)])
@pytest.mark.parametrize("case", ["decode", "decode_split", "short"])
@pytest.mark.parametrize("consecutive", [False, True, "runs"])
def test_attention_tma_decode(nq, nkv, hd, ps, window, case, consecutive):
    """The TMA-fed decode form against the float32 statement: contexts that end inside a page and
    inside a tile, requests shorter than a tile (slots without a page), split contexts, a window;
    pages scattered (a box a page) and with consecutive ids (a box a tile)."""
    ops = _ops()
    assert ops.tma_attention_supports(hd, ps)
    g = torch.Generator(device="cuda").manual_seed(18)
    lens = {"decode": [300, 1, 17, 64, 65], "decode_split": [1500, 700, 3, 129], "short": [5, 2, 1, 33]}[case]
    q_lens = [1] * len(lens)
    if case == "short" and nq // nkv <= 8:
        q_lens[0] = 2                                   # two tokens of one request still fit a 16-row tile
    q, kc, vc, bt, pos, seq = _paged_case(g, lens, q_lens, nq, nkv, hd, ps, torch.bfloat16, consecutive=consecutive)
    # poison what lies outside the requests' pages: a kernel that read it would show NaN
    q_start, ctx_len = _starts(q_lens, lens)
    scale = hd ** -0.5
    want = ref.attention_simt(q.float(), kc.float(), vc.float(), bt, pos, seq, nq, nkv, hd, scale, window)
    small, large = ops.attention_tiles(q_lens, nq // nkv, "cuda")
    assert large is None
    for splits in ((1, 2) if case != "decode_split" else (1, 5, 9)):
        out = torch.full_like(q, float("nan"))
        ops.attention_tma_decode(q, kc, vc, bt, q_start, ctx_len, small, splits, nq, nkv, hd, scale, window, out)
        ops.check_tcgen05_status()
        assert not out.isnan().any(), "a row was not written, or a masked slot held garbage"
        torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)
