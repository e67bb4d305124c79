"""Three configurations between the tiny ones and the benchmark's, against the plain implementation,
in float32 and bfloat16, all four ways of cutting, pages of 16 and of 64 tokens: head size 64 with a
group of 3 and an odd vocabulary (tied head); head size 128 with as many kv heads as query heads, a
width of 1000 and an intermediate width of 2744; and the Qwen2.5-0.5B sizes, two layers deep (group of
7, head size 64, vocabulary 151936).  They reach the kernels the tiny configurations do not (the
tcgen05 and TMA attention forms at head size 64, the streaming products at widths that are no power
of two) with other head counts and groups than the benchmark's."""

import numpy as np
import pytest

from tests import traces
from tests.conftest import cuda_or_skip
from tests.plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

BASE = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu"}
MEDIUM = {
    "group3_hd64_tied": dict(BASE, num_hidden_layers=3, hidden_size=768, num_attention_heads=12, num_key_value_heads=4,
                             head_dim=64, intermediate_size=2048, vocab_size=50257, rope_theta=10000.0,
                             rms_norm_eps=1e-5, max_position_embeddings=2048, tie_word_embeddings=True),
    "mha_hd128_odd_widths": dict(BASE, num_hidden_layers=2, hidden_size=1000, num_attention_heads=10,
                                 num_key_value_heads=10, head_dim=128, intermediate_size=2744, vocab_size=32003,
                                 rope_theta=500000.0, rms_norm_eps=1e-6, max_position_embeddings=4096,
                                 tie_word_embeddings=False),
    "qwen2.5_0.5b_widths": dict(BASE, num_hidden_layers=2, hidden_size=896, num_attention_heads=14,
                                num_key_value_heads=2, head_dim=64, intermediate_size=4864, vocab_size=151936,
                                rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=32768,
                                tie_word_embeddings=True),
}


@pytest.mark.parametrize("name", sorted(MEDIUM))
def test_medium_sizes_all_cuttings(name, tmp_path):
    from sllm_b200.engine import Engine, build_model
    from sllm_b200.weights import write_random_model
    dev = cuda_or_skip()
    cfg = MEDIUM[name]
    d = str(tmp_path / "model")
    write_random_model(d, cfg, 5 + sorted(MEDIUM).index(name), std=0.03, bias_std=0.2, gain_std=0.1)
    c, w = plain.load_model(d)
    rng = np.random.default_rng(17)
    reqs = {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate((150, 37, 260))}
    want = {r: plain.forward(ids, w, c) for r, ids in reqs.items()}
    spread = float(np.concatenate([v.ravel() for v in want.values()]).std())
    for dtype in ("float32", "bfloat16"):
        # bfloat16: bounds relative to the logits' spread, as for the benchmark's widths (measured here:
        # rms error 0.6 % of the spread, largest single error 5 %)
        tol = dict(rtol=1e-4, atol=1e-4) if dtype == "float32" else dict(rtol=2e-2, atol=0.08 * spread)
        model, _ = build_model(d, dtype, dev)
        for ps in ((8,) if dtype == "float32" else (16, 64)):
            for mode in ("whole", "tail_decode", "portions", "mixed"):
                tr = getattr(traces, mode)(reqs)
                # the mixed cutting uses pages again: there the freed ones are filled with NaN, which a
                # kernel that read a page its request does not hold would carry into the logits
                eng = Engine(model, page_size=ps, num_pages=-(-tr.max_tokens // ps), max_requests=4,
                             poison_freed=mode == "mixed")
                out = traces.replay_engine(tr, eng)
                traces.compare(tr, out, want, what=f"{name}/{dtype}/{mode}/pages of {ps}", **tol)
                if dtype == "bfloat16":
                    sq = [(out[st["step"]][i] - want[r][p]) ** 2 for st in tr.steps for i, (r, p) in enumerate(st["expect"])]
                    assert float(np.sqrt(np.mean(sq))) <= 0.02 * spread
                assert not eng.cache.requests


OTHER_HEADS = {
    "mha_hd48": dict(BASE, num_hidden_layers=2, hidden_size=336, num_attention_heads=7, num_key_value_heads=7, head_dim=48,
                     intermediate_size=1000, vocab_size=1003, rope_theta=10000.0, rms_norm_eps=1e-5,
                     max_position_embeddings=1024, tie_word_embeddings=True),
    "group3_hd80": dict(BASE, num_hidden_layers=2, hidden_size=400, num_attention_heads=6, num_key_value_heads=2, head_dim=80,
                        intermediate_size=1112, vocab_size=777, rope_theta=10000.0, rms_norm_eps=1e-6,
                        max_position_embeddings=1024, tie_word_embeddings=False),
    "group2_hd256": dict(BASE, num_hidden_layers=2, hidden_size=512, num_attention_heads=2, num_key_value_heads=1, head_dim=256,
                         intermediate_size=1024, vocab_size=2000, rope_theta=10000.0, rms_norm_eps=1e-6,
                         max_position_embeddings=1024, tie_word_embeddings=False),
}


@pytest.mark.parametrize("name", sorted(OTHER_HEADS))
def test_head_sizes_the_tensor_core_forms_do_not_take(name, tmp_path):
    """Head sizes 48, 80 and 256 in bfloat16 go to the CUDA-core attention kernel; whole and cut, against
    the plain implementation.  A head larger than any kernel takes is refused when the model is built."""
    from sllm_b200.engine import Engine, build_model
    from sllm_b200.weights import write_random_model
    dev = cuda_or_skip()
    cfg = OTHER_HEADS[name]
    d = str(tmp_path / "model")
    write_random_model(d, cfg, 31, std=0.03, bias_std=0.2, gain_std=0.1)
    c, w = plain.load_model(d)
    rng = np.random.default_rng(19)
    reqs = {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate((90, 37, 140))}
    want = {r: plain.forward(ids, w, c) for r, ids in reqs.items()}
    spread = float(np.concatenate([v.ravel() for v in want.values()]).std())
    for dtype in ("float32", "bfloat16"):
        tol = dict(rtol=1e-4, atol=1e-4) if dtype == "float32" else dict(rtol=2e-2, atol=0.08 * spread)
        model, _ = build_model(d, dtype, dev)
        for mode in ("whole", "portions", "mixed"):
            tr = getattr(traces, mode)(reqs)
            eng = Engine(model, page_size=16, num_pages=tr.max_tokens // 16, max_requests=4)
            out = traces.replay_engine(tr, eng)
            traces.compare(tr, out, want, what=f"{name}/{dtype}/{mode}", **tol)
    if name == "group2_hd256":
        big = dict(cfg, head_dim=272, hidden_size=544)
        d2 = str(tmp_path / "big")
        with pytest.raises(ValueError, match="head_dim=272"):     # already when its parts are made to name its tensors
            write_random_model(d2, big, 32, std=0.03)
            build_model(d2, "bfloat16", dev)


ODD_WIDTHS = {
    # rows of 200 and 180 bytes: no 16-byte alignment for the vector loads and TMA boxes of the fast forms
    "h100_i90_v777": dict(BASE, num_hidden_layers=2, hidden_size=100, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
                          intermediate_size=90, vocab_size=777, rope_theta=10000.0, rms_norm_eps=1e-6,
                          max_position_embeddings=512, tie_word_embeddings=False),
    "h36_i52_v130": dict(BASE, num_hidden_layers=3, hidden_size=36, num_attention_heads=2, num_key_value_heads=2, head_dim=16,
                         intermediate_size=52, vocab_size=130, rope_theta=1000000.0, rms_norm_eps=1e-5,
                         max_position_embeddings=512, tie_word_embeddings=True),
    "h250_i1000_v5003": dict(BASE, num_hidden_layers=2, hidden_size=250, num_attention_heads=7, num_key_value_heads=1, head_dim=64,
                             intermediate_size=1000, vocab_size=5003, rope_theta=10000.0, rms_norm_eps=1e-6,
                             max_position_embeddings=512, tie_word_embeddings=False),
}


@pytest.mark.parametrize("name", sorted(ODD_WIDTHS))
def test_widths_that_are_multiples_of_nothing(name, tmp_path):
    """A hidden size, an intermediate size and a vocabulary that are multiples of neither 8 nor 16: every
    kernel takes them or hands them to a form that does; whole and cut, both dtypes, against the plain
    implementation."""
    from sllm_b200.engine import Engine, build_model
    from sllm_b200.weights import write_random_model
    dev = cuda_or_skip()
    cfg = ODD_WIDTHS[name]
    d = str(tmp_path / "model")
    write_random_model(d, cfg, 41, std=0.05, bias_std=0.2, gain_std=0.1)
    c, w = plain.load_model(d)
    rng = np.random.default_rng(23)
    reqs = {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate((70, 9, 150))}
    want = {r: plain.forward(ids, w, c) for r, ids in reqs.items()}
    spread = float(np.concatenate([v.ravel() for v in want.values()]).std())
    for dtype in ("float32", "bfloat16"):
        tol = dict(rtol=1e-4, atol=1e-4) if dtype == "float32" else dict(rtol=2e-2, atol=0.08 * spread)
        model, _ = build_model(d, dtype, dev)
        for mode in ("whole", "tail_decode", "portions", "mixed"):
            tr = getattr(traces, mode)(reqs)
            eng = Engine(model, page_size=16, num_pages=tr.max_tokens // 16, max_requests=4)
            out = traces.replay_engine(tr, eng)
            traces.compare(tr, out, want, what=f"{name}/{dtype}/{mode}", **tol)


def test_portions_of_a_long_prompt_beside_decoded_tokens(tmp_path):
    """A prompt of 2,700 tokens fed in portions of 150 while another request decodes: from 2,048 tokens of
    context on, the few row tiles of a portion are cut over the context and merged, in the same step
    in which the decode form writes the other request's rows.  The logits at the portions' ends, at
    the decoded tokens and after the prompt, against the plain implementation."""
    from sllm_b200.engine import Engine, StepEntry, build_model
    from sllm_b200.weights import write_random_model
    dev = cuda_or_skip()
    cfg = dict(BASE, num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
               intermediate_size=512, vocab_size=1000, rope_theta=10000.0, rms_norm_eps=1e-6,
               max_position_embeddings=4096, tie_word_embeddings=True)
    d = str(tmp_path / "model")
    write_random_model(d, cfg, 51, std=0.04, bias_std=0.2, gain_std=0.1)
    c, w = plain.load_model(d)
    rng = np.random.default_rng(29)
    long_ids = rng.integers(0, cfg["vocab_size"], 2700).tolist()
    short_ids = rng.integers(0, cfg["vocab_size"], 40).tolist()
    want_long, want_short = plain.forward(long_ids, w, c), plain.forward(short_ids, w, c)
    spread = float(want_long.std())
    model, _ = build_model(d, "bfloat16", dev)
    eng = Engine(model, page_size=16, num_pages=(2700 + 64) // 16 + 4, max_requests=2)
    eng.step([StepEntry("s", short_ids[:20], [])])
    at, worst = 20, 0.0
    for start in range(0, 2700, 150):
        entries = [StepEntry("l", long_ids[start:start + 150], [149])]
        if at < 40:
            entries.append(StepEntry("s", [short_ids[at]], [0]))
        got = eng.step(entries).float().cpu().numpy()
        err = np.abs(got[0] - want_long[start + 149]).max()
        if at < 40:
            err = max(err, np.abs(got[1] - want_short[at]).max())
            at += 1
        worst = max(worst, float(err))
    assert worst <= 0.08 * spread, (worst, spread)
    eng.finish("l"), eng.finish("s")
    eng.cache.check()


def test_a_long_request_decodes_beside_prompt_portions(tmp_path):
    """The other way round: a request with 2,600 tokens of context decodes token by token while a second prompt
    comes in portions of 150.  The decode form cuts the long context into ranges in those mixed steps too, and its
    merge kernel leaves the portion's rows (the prefill form's, written after it) alone.  The logits of both, every
    step, against the plain implementation."""
    from sllm_b200 import ops
    from sllm_b200.engine import Engine, StepEntry, build_model
    from sllm_b200.weights import write_random_model
    dev = cuda_or_skip()
    cfg = dict(BASE, num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
               intermediate_size=512, vocab_size=1000, rope_theta=10000.0, rms_norm_eps=1e-6,
               max_position_embeddings=4096, tie_word_embeddings=True)
    d = str(tmp_path / "model")
    write_random_model(d, cfg, 52, std=0.04, bias_std=0.2, gain_std=0.1)
    c, w = plain.load_model(d)
    rng = np.random.default_rng(30)
    long_ids = rng.integers(0, cfg["vocab_size"], 2612).tolist()
    prompt = rng.integers(0, cfg["vocab_size"], 600).tolist()
    want_long, want_prompt = plain.forward(long_ids, w, c), plain.forward(prompt, w, c)
    spread = float(want_long.std())
    assert ops.choose_splits(1, 2, 2600, 3) > 1                     # what the decode form picks for the long request
    model, _ = build_model(d, "bfloat16", dev)
    eng = Engine(model, page_size=16, num_pages=(2612 + 600) // 16 + 8, max_requests=2)
    for start in range(0, 2600, 650):
        eng.step([StepEntry("l", long_ids[start:start + 650], [])])
    worst = 0.0
    for k in range(12):
        entries = [StepEntry("l", [long_ids[2600 + k]], [0])]
        if k % 3 == 0:                                               # every third step brings a portion of the prompt
            j = (k // 3) * 150
            entries.append(StepEntry("p", prompt[j:j + 150], [0, 149]))
        got = eng.step(entries).float().cpu().numpy()
        err = np.abs(got[0] - want_long[2600 + k]).max()
        if k % 3 == 0:
            err = max(err, np.abs(got[1] - want_prompt[j]).max(), np.abs(got[2] - want_prompt[j + 149]).max())
        worst = max(worst, float(err))
    ops.check_tcgen05_status()
    assert worst <= 0.08 * spread, (worst, spread)
    eng.finish("l"), eng.finish("p")
    eng.cache.check()


@pytest.mark.parametrize("live", [12, 40, 64])
def test_many_live_requests_decode_through_the_graphs(live, tmp_path):
    """12, 40 and 64 requests decode together: the captured steps of 12, 48 and 64 rows (the products of
    9..32 and of 33..64 rows, padding rows beside live ones), which the replay tests with their four live
    requests never reach.  float32: the plain implementation's tokens.  bfloat16: every token is the maximum
    of the plain logits of the engine's own sequence up to the bfloat16 path's tolerance."""
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    from sllm_b200.weights import write_random_model
    dev = cuda_or_skip()
    cfg = MEDIUM["group3_hd64_tied"]
    d = str(tmp_path / "model")
    write_random_model(d, cfg, 5, std=0.03, bias_std=0.2, gain_std=0.1)
    c, w = plain.load_model(d)
    rng = np.random.default_rng(live)
    prompts = [rng.integers(0, cfg["vocab_size"], int(n)).tolist() for n in rng.integers(3, 40, live)]
    new = 6
    want = [plain.generate(p, new, w, c) for p in prompts]
    for dtype in ("float32", "bfloat16"):
        llm = LLM(d, dtype=dtype, device=dev, block_size=16, num_pages=live * 4, max_num_seqs=live, chunk_size=64,
                  max_batch_tokens=live * 40, max_model_len=64)
        res = llm.generate(prompts, SamplingParams(max_new=new))
        rows = {k[0] for k, g in llm.engine.graphs.graphs.items() if g.graph is not None}
        assert {12: 12, 40: 48, 64: 64}[live] in rows, rows
        llm.engine.cache.check()
        if dtype == "float32":
            assert [r.ids for r in res] == want
            continue
        same = 0
        for p, r, x in zip(prompts, res, want):
            assert len(r.ids) == new
            logits = plain.forward(p + r.ids, w, c)
            spread = float(logits.std())
            for i, tok in enumerate(r.ids):
                row = logits[len(p) + i - 1]
                assert row[tok] >= row.max() - 0.16 * spread, (live, len(p), i)     # twice the bound on one value
            same += r.ids == x
        assert same >= live * 0.7            # and most sequences are the float32 ones outright
