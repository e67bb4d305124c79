"""Engine logic without a GPU: the step function, the cache and the batch layout,
with the PyTorch statements of the operations in the kernels' place, compared
with the plain implementation."""

import numpy as np
import pytest
import torch

from sllm_b200.engine import Engine, StepEntry, build_model
from tests.plain import qwen2_plain as plain


def _engine(model_dir, page, num_pages=64, max_requests=4):
    model, _ = build_model(model_dir, "float32", "cpu")
    return Engine(model, page_size=page, num_pages=num_pages, max_requests=max_requests)


def test_whole_prompt_matches_plain(tiny, cpu_ops):
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    rng = np.random.default_rng(5)
    ids = rng.integers(0, cfg["vocab_size"], 33).tolist()
    want = plain.forward(ids, w, cfg)
    eng = _engine(model_dir, page)
    got = eng.step([StepEntry("a", ids, list(range(len(ids))))]).numpy()
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)


def test_cuttings_match_plain(tiny, cpu_ops):
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    rng = np.random.default_rng(6)
    seqs = {k: rng.integers(0, cfg["vocab_size"], n).tolist() for k, n in (("a", 40), ("b", 23), ("c", 57))}
    want = {k: plain.forward(v, w, cfg) for k, v in seqs.items()}
    eng = _engine(model_dir, page, num_pages=sum(-(-len(v) // page) for v in seqs.values()))
    done = {k: 0 for k in seqs}
    cuts = [7, 2, 13, 1, 5, 2, 9, 3]
    i = 0
    while any(done[k] < len(seqs[k]) for k in seqs):
        entries, keys = [], []
        for k in seqs:
            if done[k] >= len(seqs[k]):
                continue
            n = min(cuts[i % len(cuts)], len(seqs[k]) - done[k])
            i += 1
            entries.append(StepEntry(k, seqs[k][done[k]:done[k] + n], list(range(n))))
            keys.append((k, done[k], n))
        got = eng.step(entries).numpy()
        r = 0
        for k, start, n in keys:
            np.testing.assert_allclose(got[r:r + n], want[k][start:start + n], rtol=1e-4, atol=1e-5)
            r += n
            done[k] += n
    for k in seqs:
        eng.finish(k)
    eng.cache.check()
    assert all(g.pool.used_count == 0 for g in eng.cache.groups)


def _requests(cfg, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate(lengths)}


@pytest.mark.parametrize("mode", ["whole", "tail_decode", "portions", "mixed"])
def test_trace_modes_on_cpu(tiny, cpu_ops, mode):
    """The four ways of cutting, through the engine with the CPU stand-in kernels."""
    from tests import traces
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    reqs = _requests(cfg, (50, 37, 64, 45, 41, 58), 11)
    want = {r: plain.forward(ids, w, cfg) for r, ids in reqs.items()}
    tr = getattr(traces, mode)(reqs)
    model, _ = build_model(model_dir, "float32", "cpu")
    eng = Engine(model, page_size=page, num_pages=tr.max_tokens // page, max_requests=4)
    out = traces.replay_engine(tr, eng)
    traces.compare(tr, out, want, rtol=1e-4, atol=1e-5, what=f"{name}/{mode}")
    eng.cache.check()
    assert not eng.cache.requests
    if mode == "mixed":
        assert eng.cache.reuse_count > 0, "the pool was meant to be so small that pages are used again"


def test_generate_on_cpu_matches_plain(tiny, cpu_ops):
    """Greedy and temperature generation through the entry point (scheduler, engine,
    sampler) with the CPU stand-in kernels, against the plain implementation."""
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (5, 17, 33, 1)]
    model, _ = build_model(model_dir, "float32", "cpu")
    for policy, pages in (("reserve", 64), ("on_demand", 9 if page == 16 else 17)):
        llm = LLM(model=model, block_size=page, num_pages=pages, max_num_seqs=3, chunk_size=24,
                  max_batch_tokens=40, policy=policy)
        res = llm.generate(prompts, SamplingParams(max_new=8))
        for p, r in zip(prompts, res):
            assert r.ids == plain.generate(p, 8, w, cfg) and r.finish_reason == "length"
        res = llm.generate(prompts[:2], SamplingParams(max_new=6, temperature=0.8, seed=7))
        for p, r in zip(prompts, res):
            assert r.ids == plain.generate(p, 6, w, cfg, temperature=0.8, seed=7)
        llm.engine.cache.check()
        assert not llm.engine.cache.requests


def test_one_packer_describes_both_kinds_of_step(tiny, cpu_ops):
    """A step launched kernel by kernel and a step replayed from a graph are described by the same
    packer: the live rows agree field by field, and the rows that pad a graph's batch have no context,
    no page to write to and the spare state slot."""
    from sllm_b200.engine.batch import BatchLayout, pack
    name, model_dir, page = tiny
    cfg, _ = plain.load_model(model_dir)
    eng = _engine(model_dir, page)
    reqs = _requests(cfg, (page + 3, 2 * page, 5), 3)
    eng.step([StepEntry(k, v, []) for k, v in reqs.items()])
    entries = [StepEntry(k, [7 + i], [0]) for i, k in enumerate(reqs)]
    totals = [len(v) + 1 for v in reqs.values()]
    for e, t in zip(entries, totals):
        eng.cache.reserve(e.req_id, t)
    G = len(eng.cache.groups)
    exact = BatchLayout(3, 3, 3, [3] * G)
    padded = BatchLayout(6, 6, 6, [9] * G, extras={"temps": 6})
    a = np.full(exact.total, 99, np.int32)
    b = np.full(padded.total, 99, np.int32)
    pack(exact, a, eng.cache, entries, totals)
    pack(padded, b, eng.cache, entries, totals)
    for key in BatchLayout.FIELDS + tuple(f"slot_mapping{g}" for g in range(G)):
        n = len(exact.sec(a, key))
        np.testing.assert_array_equal(exact.sec(a, key), padded.sec(b, key)[:n], err_msg=key)
    for g in range(G):
        np.testing.assert_array_equal(exact.sec(a, f"block_tables{g}").reshape(3, 3),
                                      padded.sec(b, f"block_tables{g}").reshape(6, 9)[:3, :3])
        assert (padded.sec(b, f"block_tables{g}").reshape(6, 9)[3:] == -1).all()
        assert (padded.sec(b, f"slot_mapping{g}")[3:] == -1).all()
    assert padded.sec(b, "ctx_len")[3:].tolist() == [0, 0, 0]
    assert padded.sec(b, "state_slots")[3:].tolist() == [eng.cache.padding_slot] * 3
    assert padded.sec(b, "q_start").tolist() == list(range(7))
    assert padded.sec(b, "logit_rows").tolist() == list(range(6))
    assert (padded.sec(b, "temps") == 99).all()                 # a caller's own section is left alone
    # token ids that come from the device are left for the caller
    pack(padded, b, eng.cache, entries, totals, tokens_from_host=False)
    assert padded.sec(b, "token_ids").tolist() == [0] * 6
    with pytest.raises(ValueError):
        pack(BatchLayout(4, 3, 3, [3] * G), a.copy(), eng.cache, entries, totals)


def test_a_step_is_chained_only_if_the_pages_of_all_its_requests_are_there(tiny, cpu_ops):
    """Two requests reach a page's edge in the same step and one page is free: each alone could take
    it, both cannot.  The step must not be queued behind the one in flight (the scheduler, which can
    preempt, decides instead)."""
    from types import SimpleNamespace
    name, model_dir, page = tiny
    cfg, _ = plain.load_model(model_dir)
    eng = _engine(model_dir, page, num_pages=3, max_requests=2)
    reqs = _requests(cfg, (page, page), 4)
    eng.step([StepEntry(k, v, []) for k, v in reqs.items()])
    assert eng.cache.groups[0].pool.free_count == 1
    graphs = eng.graphs
    entries = [StepEntry(k, [0], [0]) for k in reqs]
    key = (graphs.batch_bucket(2), graphs.bucket(page + 1), False)
    graphs.graphs[key] = SimpleNamespace(graph=object())        # as if captured
    assert all(eng.cache.can_reserve(e.req_id, page + 1) for e in entries)
    assert not graphs.can_chain(entries)
    assert graphs.can_chain(entries[:1]) is False               # no graph of one row
    graphs.graphs[(1, key[1], False)] = SimpleNamespace(graph=object())
    assert graphs.can_chain(entries[:1])
    eng.cache.check()
