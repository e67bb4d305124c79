"""The engine on the GPU beyond replay: generation through the entry point, long
decoding, the first tokens of a sequence, each part alone, and a toy mixer with
state of its own that is registered, built and stepped from this file alone."""

import json
import os

import numpy as np
import pytest
import torch

from tests.conftest import TINY, cuda_or_skip, make_model_dir
from tests.plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu
TOL = {"float32": dict(rtol=1e-4, atol=2e-5), "bfloat16": dict(rtol=2e-2, atol=2e-2)}


def _prompts(cfg, lengths, seed=2):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]


@pytest.mark.parametrize("policy", ["reserve", "on_demand"])
def test_greedy_generation_float32_equals_plain(tiny, policy):
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    dev = cuda_or_skip()
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    # on_demand: three requests fill the four pages; the first to need one more while
    # decoding finds none free and the youngest is preempted
    prompts = _prompts(cfg, (5, 17, 33, 1) if policy == "reserve" else (page - 2, page - 1, 2 * page - 2, 1))
    pages = 64 if policy == "reserve" else 4
    llm = LLM(model_dir, dtype="float32", device=dev, block_size=page, num_pages=pages, max_num_seqs=3,
              chunk_size=24, max_batch_tokens=40, policy=policy)
    res = llm.generate(prompts, SamplingParams(max_new=8))
    for p, r in zip(prompts, res):
        assert r.ids == plain.generate(p, 8, w, cfg) and r.finish_reason == "length"
    if policy == "on_demand":
        assert llm.scheduler.num_preemptions > 0, "the pool was meant to force a preemption"
    # temperature sampling with the request's own generator reproduces the plain sampler
    res = llm.generate(prompts[:3], SamplingParams(max_new=16, temperature=0.8, seed=7))
    for p, r in zip(prompts, res):
        assert r.ids == plain.generate(p, 16, w, cfg, temperature=0.8, seed=7)
    # top-k, top-p and the repetition penalty, each alone and together (decode steps with filters run
    # from the captured graph; rows with a penalty are sampled outside it)
    for kw in (dict(top_k=5), dict(top_p=0.7), dict(repetition_penalty=1.3), dict(top_k=7, top_p=0.9, repetition_penalty=1.2),
               dict(temperature=0.0, repetition_penalty=1.5)):
        kw = {"temperature": 0.9, **kw}
        res = llm.generate(prompts[:3], SamplingParams(max_new=12, seed=1, **kw))
        for p, r in zip(prompts, res):
            assert r.ids == plain.generate(p, 12, w, cfg, seed=1, **kw), kw
    # a stop id ends a request and is not part of the output
    first = plain.generate(prompts[0], 3, w, cfg)
    (r,) = llm.generate(prompts[:1], SamplingParams(max_new=8, stop_ids=(first[2],)))
    assert r.finish_reason == "stop" and r.ids == first[:first.index(first[2])]
    llm.engine.cache.check()
    assert not llm.engine.cache.requests


def test_greedy_generation_bfloat16_stays_within_rounding(tiny):
    """In bfloat16 a near-tie may fall the other way, so each chosen token is checked
    against the plain logits of the engine's own sequence: it must be the maximum up to
    the tolerance of the bfloat16 path."""
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    dev = cuda_or_skip()
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    prompts = _prompts(cfg, (5, 17, 33))
    llm = LLM(model_dir, dtype="bfloat16", device=dev, block_size=page, num_pages=64, max_num_seqs=3, chunk_size=24)
    for p, r in zip(prompts, llm.generate(prompts, SamplingParams(max_new=12))):
        seq = p + r.ids
        logits = plain.forward(seq, w, cfg)
        for i, tok in enumerate(r.ids):
            row = logits[len(p) + i - 1]
            assert row[tok] >= row.max() - 2 * (TOL["bfloat16"]["atol"] + TOL["bfloat16"]["rtol"] * abs(row.max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(tiny, dtype):
    """Three prompt tokens, then one token a step up to the model's position limit; and
    the first positions of a sequence each as a step of their own."""
    from sllm_b200.engine import Engine, StepEntry, build_model
    dev = cuda_or_skip()
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    n = cfg["max_position_embeddings"]
    ids = _prompts(cfg, (n,), seed=4)[0]
    want = plain.forward(ids, w, cfg)
    model, _ = build_model(model_dir, dtype, dev)
    eng = Engine(model, page_size=page, num_pages=-(-n // page) + 2, max_requests=2)
    got = [eng.step([StepEntry("a", ids[:3], [0, 1, 2])]).cpu().numpy()]
    for p in range(3, n):
        got.append(eng.step([StepEntry("a", ids[p:p + 1], [0])]).cpu().numpy())
    got = np.concatenate(got)
    np.testing.assert_allclose(got, want, **TOL[dtype])
    with pytest.raises(ValueError, match="exceed"):
        eng.step([StepEntry("a", [0], [0])])                     # past the position limit
    # the first tokens, one at a time, beside the long request
    got = np.concatenate([eng.step([StepEntry("b", ids[p:p + 1], [0])]).cpu().numpy() for p in range(4)])
    np.testing.assert_allclose(got, want[:4], **TOL[dtype])


def test_step_refuses_bad_entries(tiny):
    from sllm_b200.cache import OutOfPages
    from sllm_b200.engine import Engine, StepEntry, build_model
    dev = cuda_or_skip()
    name, model_dir, page = tiny
    model, _ = build_model(model_dir, "float32", dev)
    eng = Engine(model, page_size=page, num_pages=2, max_requests=2)
    with pytest.raises(OutOfPages):
        eng.step([StepEntry("a", [1] * (2 * page + 1), [0])])
    assert not eng.cache.requests and eng.cache.groups[0].pool.used_count == 0      # nothing was taken
    with pytest.raises(ValueError, match="vocabulary"):
        eng.step([StepEntry("a", [10 ** 6], [0])])
    with pytest.raises(ValueError, match="twice"):
        eng.step([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])])
    with pytest.raises(ValueError, match="outside"):
        eng.step([StepEntry("a", [1, 2], [2])])
    assert eng.step([StepEntry("a", [1, 2], [])]).shape == (0, model.plan.vocab_size)   # nothing wanted


# ---- each part alone, at sizes that are not the tiny models' -------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parts_alone(dtype):
    from sllm_b200.cache import CacheManager
    from sllm_b200.config import PartSpec
    from sllm_b200.engine.engine import Engine
    from sllm_b200.parts import FEED_FORWARDS, MIXERS, NORMS, POSITIONS, LayerCache
    dev = cuda_or_skip()
    H, nq, nkv, hd, I, eps, theta, rot = 72, 6, 2, 48, 200, 3e-6, 5e4, 24
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    rng = np.random.default_rng(0)
    kw = dict(dtype=dtype, device=dev)

    def t(a):
        return torch.from_numpy(np.asarray(a, dtype=np.float32))

    def r(a):
        return a.astype(np.float32) if dtype == torch.float32 else t(a).bfloat16().float().numpy()

    # norm, with the fused addition
    norm = NORMS.build(PartSpec("rmsnorm", {"size": H, "eps": eps}), **kw)
    gain = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    norm.bind(lambda n: t(gain))
    res, delta = rng.standard_normal((9, H)).astype(np.float32), rng.standard_normal((9, H)).astype(np.float32)
    total = res + delta
    res_d = t(res).clone().to(dev)
    got = norm.add_norm(res_d, t(delta).to(dev))
    np.testing.assert_allclose(res_d.cpu().numpy(), total, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(got.float().cpu().numpy(), plain.rms_norm(total, gain, eps), **tol)

    # position encoding: the table is cos/sin of float64 angles
    pos = POSITIONS.build(PartSpec("rotary", {"theta": theta, "rotary_dim": rot, "max_positions": 300}), **kw)
    cos, sin = plain.rotary_tables(theta, np.arange(300), rot)
    np.testing.assert_allclose(pos.table[:, 0].cpu().numpy(), cos[:, :rot // 2], rtol=0, atol=1e-7)
    np.testing.assert_allclose(pos.table[:, 1].cpu().numpy(), sin[:, :rot // 2], rtol=0, atol=1e-7)

    # feed-forward
    ffn = FEED_FORWARDS.build(PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}), **kw)
    w = {"mlp.gate_proj.weight": r(0.2 * rng.standard_normal((I, H))), "mlp.up_proj.weight": r(0.2 * rng.standard_normal((I, H))),
         "mlp.down_proj.weight": r(0.2 * rng.standard_normal((H, I)))}
    ffn.bind(lambda n: t(w[f"mlp.{n}"]))
    x = r(rng.standard_normal((11, H)))
    got = ffn.forward(t(x).to(dev).to(dtype), None)
    np.testing.assert_allclose(got.float().cpu().numpy(), plain.swiglu(x, {f".{k}": v for k, v in w.items()}, ""),
                               **{k: v * 4 for k, v in tol.items()})

    # mixer: attention over a paged cache, partial rotary, one request in two portions
    mixer = MIXERS.build(PartSpec("attention", {"hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": hd,
                                                "qkv_bias": True, "scale": hd ** -0.5, "window": None}), **kw)
    aw = {}
    for n_, rows in (("q", nq * hd), ("k", nkv * hd), ("v", nkv * hd)):
        aw[f"x.self_attn.{n_}_proj.weight"] = r(0.2 * rng.standard_normal((rows, H)))
        aw[f"x.self_attn.{n_}_proj.bias"] = (0.3 * rng.standard_normal(rows)).astype(np.float32)
    aw["x.self_attn.o_proj.weight"] = r(0.2 * rng.standard_normal((H, nq * hd)))
    mixer.bind(lambda n: t(aw[f"x.self_attn.{n}"]))
    S = 37
    xs = r(rng.standard_normal((S, H)))
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": hd}
    want = plain.attention_mixer(xs, aw, "x", cfg, cos[:S], sin[:S])

    class _M:            # the least a model must offer the engine: cache needs, sizes, device
        def __init__(self):
            self.device, self.dtype = torch.device(dev), dtype
            self.plan = type("P", (), {"vocab_size": 10, "max_positions": 300})()

        def cache_needs(self):
            return [("own", mixer.cache_need())]
    eng = Engine(_M(), page_size=8, num_pages=8, max_requests=1)
    from sllm_b200.engine import StepEntry
    outs = []
    for lo, hi in ((0, 20), (20, 22), (22, S)):
        ctx = eng.prepare([StepEntry("a", [0] * (hi - lo), [])])
        outs.append(mixer.forward(t(xs[lo:hi]).to(dev).to(dtype), ctx, eng.layer_caches[0], pos).float().cpu().numpy())
        eng.cache.commit("a", hi)
    np.testing.assert_allclose(np.concatenate(outs), want, **{k: v * 4 for k, v in tol.items()})


# ---- a toy mixer with state of its own ---------------------------------------------------------

def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """A mixer defined here, with a fixed-size state per request instead of keys and values:
    s_t = decay * s_{t-1} + x_t W_in ; y_t = s_t W_out.  It is registered under a new kind,
    stands in every second layer of a new architecture beside attention layers, gets a
    state slot from the cache manager, and is stepped in portions.  No file of the package
    is touched."""
    from sllm_b200.config import (Architecture, ModelPlan, PartSpec, RunEntry, pre_norm_layer, register_architecture,
                                  unregister_architecture)
    from sllm_b200.engine import Engine, StepEntry, build_model
    from sllm_b200.models.qwen2 import Qwen2Config
    from sllm_b200.models.qwen2 import plan as qwen2_plan
    from sllm_b200.parts import MIXERS, Mixer, SlotState, TensorSpec
    from sllm_b200.weights import write_random_model
    dev = cuda_or_skip()
    D, DECAY = 12, 0.9

    @MIXERS.register("toy_decay_state", replace=True)
    class ToyStateMixer(Mixer):
        def __init__(self, params, **kw):
            super().__init__(params, **kw)
            self.h, self.d, self.decay = params["hidden_size"], params["state_dim"], params["decay"]

        def cache_need(self):
            return SlotState((self.d,))

        def tensor_specs(self):
            return [TensorSpec("w_in.weight", (self.d, self.h)), TensorSpec("w_out.weight", (self.h, self.d))]

        def bind(self, fetch):
            self.w_in, self.w_out = self._f32(fetch("w_in.weight")), self._f32(fetch("w_out.weight"))

        def forward(self, x, step, cache, position, write_cache=True):
            u = x.float() @ self.w_in.t()                       # [T, d]
            out = torch.empty_like(u)
            t0 = 0
            for s, n in enumerate(step.q_lens):                 # each request's tokens in order
                slot = int(step.state_slots[s])
                st = cache.state[slot]
                for i in range(n):
                    st = self.decay * st + u[t0 + i]
                    out[t0 + i] = st
                cache.state[slot] = st
                t0 += n
            return out @ self.w_out.t()

    def toy_plan(cfg):
        base = qwen2_plan(cfg)
        toy = PartSpec("toy_decay_state", {"hidden_size": cfg.hidden_size, "state_dim": D, "decay": DECAY})
        layers = tuple(pre_norm_layer(l.prefix, toy if i % 2 else l.part("mixer"), l.part("ffn"), l.part("mixer_norm"),
                                      mixer_name="toy" if i % 2 else l.parts["mixer"].name) for i, l in enumerate(base.layers))
        return ModelPlan(architecture="ToyStateLM", hidden_size=base.hidden_size, vocab_size=base.vocab_size,
                         max_positions=base.max_positions, embedding_name=base.embedding_name, layers=layers,
                         run_list=tuple(RunEntry(i) for i in range(len(layers))), final_norm=base.final_norm,
                         final_norm_name=base.final_norm_name, head_name=base.head_name, position=base.position)

    register_architecture(Architecture("ToyStateLM", Qwen2Config, toy_plan), replace=True)
    try:
        config, init, page = TINY["B"]
        config = dict(config, architectures=["ToyStateLM"], num_hidden_layers=4)
        model_dir = write_random_model(str(tmp_path / "toy"), config, 5, std=0.05, bias_std=0.2, gain_std=0.1)
        cfg, w = plain.load_model(model_dir)

        def plain_toy(ids):
            h = plain.embed(ids, w["model.embed_tokens.weight"])
            cos, sin = plain.rotary_tables(cfg["rope_theta"], np.arange(len(ids)), cfg["head_dim"])
            for i in range(cfg["num_hidden_layers"]):
                p = f"model.layers.{i}"
                x = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])
                if i % 2:
                    u = x @ w[f"{p}.toy.w_in.weight"].T
                    st, ys = np.zeros(D, np.float32), []
                    for row in u:
                        st = DECAY * st + row
                        ys.append(st.copy())
                    h = h + np.stack(ys) @ w[f"{p}.toy.w_out.weight"].T
                else:
                    h = h + plain.attention_mixer(x, w, p, cfg, cos, sin)
                x = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
                h = h + plain.swiglu(x, w, p)
            h = plain.rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
            return h @ w["lm_head.weight"].T

        model, _ = build_model(model_dir, "float32", dev)
        assert [type(l.mixer).__name__ for l in model.layers] == ["Attention", "ToyStateMixer"] * 2
        eng = Engine(model, page_size=page, num_pages=20, max_requests=3)
        assert len(eng.cache.groups) == 1 and sorted(eng.cache.state_runs) == [1, 3]
        seqs = {"a": _prompts(cfg, (30,), 1)[0], "b": _prompts(cfg, (19,), 2)[0]}
        want = {k: plain_toy(v) for k, v in seqs.items()}
        done = {"a": 0, "b": 0}
        for cuts in ((7, 3), (2, 1), (11, 9), (1, 1), (9, 5)):
            entries, keys = [], []
            for k, n in zip("ab", cuts):
                n = min(n, len(seqs[k]) - done[k])
                if n:
                    entries.append(StepEntry(k, seqs[k][done[k]:done[k] + n], list(range(n))))
                    keys.append((k, done[k], n))
            got = eng.step(entries).cpu().numpy()
            r0 = 0
            for k, lo, n in keys:
                np.testing.assert_allclose(got[r0:r0 + n], want[k][lo:lo + n], rtol=1e-4, atol=2e-5)
                r0 += n
                done[k] += n
        # a finished request's slot is zeroed for the next one
        eng.finish("a")
        got = eng.step([StepEntry("c", seqs["a"][:5], [4])]).cpu().numpy()
        np.testing.assert_allclose(got[0], want["a"][4], rtol=1e-4, atol=2e-5)
    finally:
        unregister_architecture("ToyStateLM")
        MIXERS.unregister("toy_decay_state")


def test_pipelined_decode_equals_unpipelined(tiny):
    """Decode steps queued one ahead of the host (token ids chained on the device) give exactly the
    tokens of the step-by-step path: greedy and sampled, with stop ids that end requests while a
    step computed for them is already queued, and with requests joining and leaving."""
    from sllm_b200.engine import build_model
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    dev = cuda_or_skip()
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    model, _ = build_model(model_dir, "float32", dev)
    prompts = _prompts(cfg, (5, 17, 33, 9, 2), seed=12)
    first = plain.generate(prompts[1], 6, w, cfg)
    params = [SamplingParams(max_new=20), SamplingParams(max_new=30, stop_ids=(first[5],)),
              SamplingParams(max_new=11, temperature=0.7, seed=3), SamplingParams(max_new=25, temperature=1.1, seed=4),
              SamplingParams(max_new=7)]
    outs = []
    for pipelined in (False, True):
        llm = LLM(model=model, block_size=page, num_pages=64, max_num_seqs=3, chunk_size=24, pipeline_decode=pipelined)
        res = llm.generate(prompts, params)
        outs.append([(r.ids, r.finish_reason) for r in res])
        llm.engine.cache.check()
        assert not llm.engine.cache.requests and llm._inflight is None
    assert outs[0] == outs[1]
    assert outs[0][0][0] == plain.generate(prompts[0], 20, w, cfg)
    assert outs[0][1] == (first[:first.index(first[5])], "stop")     # ends at the stop id's first appearance
    assert outs[0][2][0] == plain.generate(prompts[2], 11, w, cfg, temperature=0.7, seed=3)


def test_chained_decode_steps_across_a_context_bucket(tmp_path):
    """A decode step queued behind the one in flight takes its token ids from the graph THAT step ran
    on.  When the longest context crosses a bucket of the graphs (256, 512, ...) the two steps run on
    different graphs; with every graph captured ahead (`warmup`) or left from an earlier call, the new
    graph's own output buffer holds stale ids.  Prompts of 250, 251 and 509 tokens decode across 256 and
    512 with the graphs warmed up, greedy and sampled, twice on one `LLM`: the tokens are the plain
    implementation's (serving/executor.py:378-393: each decode step consumes the token the step before
    produced)."""
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    dev = cuda_or_skip()
    config, init, page = TINY["B"]
    model_dir = make_model_dir(tmp_path, config, init, max_position_embeddings=1024)
    cfg, w = plain.load_model(model_dir)
    llm = LLM(model_dir, dtype="float32", device=dev, block_size=page, num_pages=3 * 1024 // page, max_num_seqs=3,
              chunk_size=128, max_batch_tokens=640, pipeline_decode=True)
    assert llm.warmup() >= 9                        # 1..3 requests x buckets 256, 512, 1024
    prompts = _prompts(cfg, (250, 251, 509), seed=41)
    for round_ in range(2):
        for kw in (dict(), dict(temperature=0.8, seed=7)):
            want = [plain.generate(p, 12, w, cfg, **kw) for p in prompts]
            # the two short ones together cross 256; the long one alone and all three together cross 512
            for group in ((0, 1), (2,), (0, 1, 2)):
                res = llm.generate([prompts[i] for i in group], SamplingParams(max_new=12, **kw))
                for i, r in zip(group, res):
                    assert r.ids == want[i], (round_, kw, group, i)
    llm.engine.cache.check()
    assert not llm.engine.cache.requests and llm._inflight is None
    buckets = {k[1] for k, g in llm.engine.graphs.graphs.items() if g.turn or g.graph is not None}
    assert {256, 512, 1024} <= buckets


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_graphs_pad_the_batch_to_a_captured_size(tiny, dtype):
    """Five and seven live requests run on the graphs of six and eight rows: the padding rows write
    nothing, and the live rows' tokens are those of each request alone."""
    from sllm_b200.engine import build_model
    from sllm_b200.engine.graphs import DecodeGraphs
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    dev = cuda_or_skip()
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    assert [DecodeGraphs.batch_bucket(n) for n in (1, 4, 5, 7, 9, 13, 17, 33)] == [1, 4, 6, 8, 12, 16, 24, 48]
    model, _ = build_model(model_dir, dtype, dev)
    prompts = _prompts(cfg, (5, 9, 14, 3, 21, 8, 11), seed=33)
    llm = LLM(model=model, block_size=page, num_pages=96, max_num_seqs=7, chunk_size=64)
    # requests end at different times: 7 live, then 5, then fewer
    params = [SamplingParams(max_new=n) for n in (12, 12, 12, 12, 12, 4, 4)]
    res = llm.generate(prompts, params)
    sizes = sorted({k[0] for k in llm.engine.graphs.graphs})
    assert 8 in sizes and 6 in sizes and 7 not in sizes and 5 not in sizes
    llm.engine.cache.check()
    for p, sp, r in zip(prompts, params, res):
        want = plain.generate(p, sp.max_new, w, cfg)
        if dtype == "float32":
            assert r.ids == want
        else:
            # a near-tie may fall the other way: every token must be the maximum of the plain logits of
            # the engine's own sequence up to the bfloat16 path's tolerance
            assert len(r.ids) == sp.max_new
            logits = plain.forward(p + r.ids, w, cfg)
            for i, tok in enumerate(r.ids):
                row = logits[len(p) + i - 1]
                assert row[tok] >= row.max() - 2 * (TOL["bfloat16"]["atol"] + TOL["bfloat16"]["rtol"] * abs(row.max()))


@pytest.mark.parametrize("policy", ["reserve", "on_demand"])
@pytest.mark.parametrize("pipelined", [False, True])
def test_random_arrivals_aborts_and_a_small_pool(tiny, policy, pipelined):
    """Requests arrive at random steps, some are aborted while they wait, are being prefilled or have a
    decode step in flight, the pool is small enough for pages to be used again (and, on demand, for
    preemptions): every request that ends has the plain implementation's tokens, greedy or sampled
    with its own seed, and no page or slot is lost."""
    from sllm_b200.engine import build_model
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    dev = cuda_or_skip()
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    model, _ = build_model(model_dir, "float32", dev)
    rng = np.random.default_rng(41 + pipelined)
    n = 14
    prompts = [rng.integers(0, cfg["vocab_size"], int(rng.integers(1, 40))).tolist() for _ in range(n)]
    params = []
    for i in range(n):
        kw = dict(max_new=int(rng.integers(1, 20)))
        if i % 3 == 1:
            kw.update(temperature=0.9, seed=100 + i)
        params.append(SamplingParams(**kw))
    llm = LLM(model=model, block_size=page, num_pages=-(-60 // page) + 2, max_num_seqs=3, chunk_size=8, max_batch_tokens=24,
              policy=policy, pipeline_decode=pipelined)
    reqs, aborted, nxt, steps = {}, set(), 0, 0
    while nxt < n or llm.scheduler.has_work:
        if nxt < n and rng.random() < 0.5:
            reqs[nxt] = llm.add_request(prompts[nxt], params[nxt], req_id=nxt)
            nxt += 1
        live = [i for i, r in reqs.items() if r.status != "finished" and i not in aborted]
        if live and rng.random() < 0.07:
            victim = int(rng.choice(live))
            assert llm.abort(victim)
            aborted.add(victim)
        if llm.scheduler.has_work:
            llm.step()
        steps += 1
        assert steps < 3000, "the run does not end"
    llm.drain()
    llm.engine.cache.check()
    assert not llm.engine.cache.requests
    assert len(aborted) >= 1 and len(aborted) < n
    for i, r in reqs.items():
        if i in aborted:
            continue
        sp = params[i]
        want = plain.generate(prompts[i], sp.max_new, w, cfg, temperature=sp.temperature or 0.0, seed=sp.seed)
        assert r.output == want, f"request {i} ({policy}, pipelined={pipelined})"


def test_graph_capture_survives_garbage_of_earlier_engines(tiny):
    """Engines made and dropped one after the other, with the collector set to run all the time: the
    capture of a decode graph must not be invalidated by the collection of an earlier engine's graphs
    and buffers in the middle of it."""
    import gc
    from sllm_b200.engine import build_model
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    dev = cuda_or_skip()
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    model, _ = build_model(model_dir, "float32", dev)
    prompts = _prompts(cfg, (7, 12), seed=21)
    want = [plain.generate(p, 6, w, cfg) for p in prompts]
    old = gc.get_threshold()
    gc.set_threshold(1, 1, 1)
    try:
        for _ in range(4):
            llm = LLM(model=model, block_size=page, num_pages=32, max_num_seqs=2)
            res = llm.generate(prompts, SamplingParams(max_new=6))
            assert [r.ids for r in res] == want
            assert llm.engine.graphs.graphs, "the decode steps ran without a graph"
            del llm, res
    finally:
        gc.set_threshold(*old)


def test_toy_routed_feed_forward_and_learned_positions(tmp_path):
    """Two more parts defined here and nowhere in the package: a feed-forward that routes each
    token to one of four small experts (router logits and their softmax in float32), and a position
    encoding that is a learned table added to the embeddings (the attention then rotates nothing).
    Registered, given tensors by the random-weights writer, built through the registry, stepped in
    portions and one token at a time, and compared with a plain numpy statement of the same model."""
    from sllm_b200.config import (Architecture, ModelPlan, PartSpec, RunEntry, pre_norm_layer, register_architecture,
                                  unregister_architecture)
    from sllm_b200.engine import Engine, StepEntry, build_model
    from sllm_b200.models.qwen2 import Qwen2Config
    from sllm_b200.models.qwen2 import plan as qwen2_plan
    from sllm_b200.parts import FEED_FORWARDS, POSITIONS, FeedForward, PositionEncoding, TensorSpec
    from sllm_b200.weights import write_random_model
    dev = cuda_or_skip()
    E, D = 4, 24

    @FEED_FORWARDS.register("toy_routed", replace=True)
    class ToyRouted(FeedForward):
        def __init__(self, params, **kw):
            super().__init__(params, **kw)
            self.h = params["hidden_size"]

        def tensor_specs(self):
            specs = [TensorSpec("router.weight", (E, self.h))]
            for e in range(E):
                specs += [TensorSpec(f"experts.{e}.w_in.weight", (D, self.h)), TensorSpec(f"experts.{e}.w_out.weight", (self.h, D))]
            return specs

        def bind(self, fetch):
            self.router = self._f32(fetch("router.weight"))
            self.w_in = torch.stack([self._f32(fetch(f"experts.{e}.w_in.weight")) for e in range(E)])
            self.w_out = torch.stack([self._f32(fetch(f"experts.{e}.w_out.weight")) for e in range(E)])

        def forward(self, x, step):
            xf = x.float()
            probs = torch.softmax(xf @ self.router.t(), dim=-1)                # float32 router
            top = probs.argmax(-1)
            hid = torch.relu(torch.einsum("th,tdh->td", xf, self.w_in[top]))
            return torch.einsum("td,thd->th", hid, self.w_out[top]) * probs.gather(1, top[:, None])

    @POSITIONS.register("toy_learned_abs", replace=True)
    class LearnedPositions(PositionEncoding):
        def tensor_specs(self):
            return [TensorSpec("weight", (self.params["max_positions"], self.params["hidden_size"]), role="embedding")]

        def bind(self, fetch):
            self.weight = self._f32(fetch("weight"))

        def on_embedding(self, residual, step):
            residual += self.weight[step.positions.long()]

    def toy_plan(cfg):
        base = qwen2_plan(cfg)
        routed = PartSpec("toy_routed", {"hidden_size": cfg.hidden_size})
        layers = tuple(pre_norm_layer(l.prefix, l.part("mixer"), routed if i % 2 else l.part("ffn"), l.part("mixer_norm"),
                                      ffn_name="moe" if i % 2 else l.parts["ffn"].name) for i, l in enumerate(base.layers))
        pos = PartSpec("toy_learned_abs", {"max_positions": cfg.max_position_embeddings, "hidden_size": cfg.hidden_size})
        return ModelPlan(architecture="ToyRoutedLM", hidden_size=base.hidden_size, vocab_size=base.vocab_size,
                         max_positions=base.max_positions, embedding_name=base.embedding_name, layers=layers,
                         run_list=tuple(RunEntry(i) for i in range(len(layers))), final_norm=base.final_norm,
                         final_norm_name=base.final_norm_name, head_name=base.head_name, position=pos,
                         position_name="model.pos_embed")

    register_architecture(Architecture("ToyRoutedLM", Qwen2Config, toy_plan), replace=True)
    try:
        config, init, page = TINY["A"]
        config = dict(config, architectures=["ToyRoutedLM"], num_hidden_layers=4)
        model_dir = write_random_model(str(tmp_path / "toy"), config, 6, std=0.08, bias_std=0.2, gain_std=0.1)
        cfg, w = plain.load_model(model_dir)
        nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

        def plain_toy(ids):
            s = len(ids)
            h = plain.embed(ids, w["model.embed_tokens.weight"]) + w["model.pos_embed.weight"][:s]
            for i in range(cfg["num_hidden_layers"]):
                p = f"model.layers.{i}"
                x = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])
                a = f"{p}.self_attn"
                q = plain.linear(x, w[f"{a}.q_proj.weight"], w[f"{a}.q_proj.bias"]).reshape(s, nq, hd).transpose(1, 0, 2)
                k = plain.linear(x, w[f"{a}.k_proj.weight"], w[f"{a}.k_proj.bias"]).reshape(s, nkv, hd).transpose(1, 0, 2)
                v = plain.linear(x, w[f"{a}.v_proj.weight"], w[f"{a}.v_proj.bias"]).reshape(s, nkv, hd).transpose(1, 0, 2)
                k, v = np.repeat(k, nq // nkv, axis=0), np.repeat(v, nq // nkv, axis=0)
                o = plain.causal_attention(q, k, v, hd ** -0.5).transpose(1, 0, 2).reshape(s, nq * hd)
                h = h + plain.linear(o, w[f"{a}.o_proj.weight"])
                x = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
                if i % 2:
                    logits = x @ w[f"{p}.moe.router.weight"].T
                    pr = np.exp(logits - logits.max(-1, keepdims=True))
                    pr = pr / pr.sum(-1, keepdims=True)
                    top = pr.argmax(-1)
                    out = np.zeros_like(x)
                    for t in range(s):
                        e = top[t]
                        hid = np.maximum(x[t] @ w[f"{p}.moe.experts.{e}.w_in.weight"].T, 0)
                        out[t] = hid @ w[f"{p}.moe.experts.{e}.w_out.weight"].T * pr[t, e]
                    h = h + out
                else:
                    h = h + plain.swiglu(x, w, p)
            h = plain.rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
            return h @ w["model.embed_tokens.weight"].T

        model, _ = build_model(model_dir, "float32", dev)
        assert [type(l.parts["ffn"]).__name__ for l in model.layers] == ["SwiGLU", "ToyRouted"] * 2
        assert type(model.position).__name__ == "LearnedPositions"
        eng = Engine(model, page_size=page, num_pages=12, max_requests=2)
        ids = _prompts(cfg, (45,), 5)[0]
        want = plain_toy(ids)
        got, p0 = [], 0
        for n in (11, 2, 1, 17, 1, 1, 12):
            got.append(eng.step([StepEntry("a", ids[p0:p0 + n], list(range(n)))]).cpu().numpy())
            p0 += n
        np.testing.assert_allclose(np.concatenate(got), want, rtol=1e-4, atol=2e-5)
    finally:
        unregister_architecture("ToyRoutedLM")
        FEED_FORWARDS.unregister("toy_routed")
        POSITIONS.unregister("toy_learned_abs")


def test_run_list_names_a_layer_twice_and_borrows_a_cache(tmp_path):
    """The order in which layers run is data: here layer 0 runs twice (each run with a cache of its
    own) and the last run of layer 1 reads the keys and values that layer 1's first run wrote,
    writing none itself.  Compared with a plain numpy statement, in portions and token by token."""
    from sllm_b200.config import Architecture, ModelPlan, RunEntry, register_architecture, unregister_architecture
    from sllm_b200.engine import Engine, StepEntry, build_model
    from sllm_b200.models.qwen2 import Qwen2Config
    from sllm_b200.models.qwen2 import plan as qwen2_plan
    from sllm_b200.weights import write_random_model
    dev = cuda_or_skip()
    RUNS = (RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(1, cache_from=1))

    def loop_plan(cfg):
        b = qwen2_plan(cfg)
        return ModelPlan(architecture="ToyLoopLM", hidden_size=b.hidden_size, vocab_size=b.vocab_size,
                         max_positions=b.max_positions, embedding_name=b.embedding_name, layers=b.layers,
                         run_list=RUNS, final_norm=b.final_norm, final_norm_name=b.final_norm_name,
                         head_name=b.head_name, position=b.position)

    register_architecture(Architecture("ToyLoopLM", Qwen2Config, loop_plan), replace=True)
    try:
        config, init, page = TINY["B"]
        config = dict(config, architectures=["ToyLoopLM"], num_hidden_layers=2)
        model_dir = write_random_model(str(tmp_path / "loop"), config, 9, std=0.05, bias_std=0.2, gain_std=0.1)
        cfg, w = plain.load_model(model_dir)
        nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

        def plain_loop(ids):
            s = len(ids)
            h = plain.embed(ids, w["model.embed_tokens.weight"])
            cos, sin = plain.rotary_tables(cfg["rope_theta"], np.arange(s), hd)
            kv_of_run = {}
            for run, e in enumerate(RUNS):
                p = f"model.layers.{e.layer}"
                a = f"{p}.self_attn"
                x = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])
                q = plain.linear(x, w[f"{a}.q_proj.weight"], w[f"{a}.q_proj.bias"]).reshape(s, nq, hd).transpose(1, 0, 2)
                q = plain.apply_rotary(q, cos, sin)
                if e.cache_from is None:
                    k = plain.linear(x, w[f"{a}.k_proj.weight"], w[f"{a}.k_proj.bias"]).reshape(s, nkv, hd).transpose(1, 0, 2)
                    v = plain.linear(x, w[f"{a}.v_proj.weight"], w[f"{a}.v_proj.bias"]).reshape(s, nkv, hd).transpose(1, 0, 2)
                    kv_of_run[run] = (plain.apply_rotary(k, cos, sin), v)
                k, v = kv_of_run[run if e.cache_from is None else e.cache_from]
                o = plain.causal_attention(q, np.repeat(k, nq // nkv, axis=0), np.repeat(v, nq // nkv, axis=0), hd ** -0.5)
                h = h + plain.linear(o.transpose(1, 0, 2).reshape(s, nq * hd), w[f"{a}.o_proj.weight"])
                x = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
                h = h + plain.swiglu(x, w, p)
            h = plain.rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
            return h @ w["lm_head.weight"].T

        for dtype, tol in (("float32", dict(rtol=1e-4, atol=2e-5)), ("bfloat16", dict(rtol=2e-2, atol=2e-2))):
            model, _ = build_model(model_dir, dtype, dev)
            eng = Engine(model, page_size=page, num_pages=16, max_requests=2)
            # three caching runs share one group; the borrowing run has the cache of run 1
            assert eng.cache.groups[0].runs == [0, 1, 2]
            assert eng.layer_caches[3].k.data_ptr() == eng.layer_caches[1].k.data_ptr()
            ids = _prompts(cfg, (40,), 6)[0]
            want = plain_loop(ids)
            got, p0 = [], 0
            for n in (13, 2, 1, 1, 20, 3):
                got.append(eng.step([StepEntry("a", ids[p0:p0 + n], list(range(n)))]).cpu().numpy())
                p0 += n
            np.testing.assert_allclose(np.concatenate(got), want, **tol)
    finally:
        unregister_architecture("ToyLoopLM")


def test_replayed_graphs_keep_the_status_word_checked(tmp_path):
    """Kernels fed by TMA report a wait that ran out through a status word; a decode step replayed from
    a graph launches them without passing through their wrappers, and must still be counted so that
    the word is read."""
    from sllm_b200 import ops
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    from sllm_b200.weights import write_random_model
    dev = cuda_or_skip()
    cfg = {"architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 2,
           "num_key_value_heads": 1, "head_dim": 64, "intermediate_size": 256, "vocab_size": 300, "rope_theta": 10000.0,
           "rms_norm_eps": 1e-6, "max_position_embeddings": 256, "tie_word_embeddings": True}
    d = write_random_model(str(tmp_path / "m"), cfg, 5, std=0.05)
    llm = LLM(d, dtype="bfloat16", device=dev, block_size=16, num_pages=32, max_num_seqs=2)
    ops.check_tcgen05_status()
    assert ops.status_word_launches() == 0
    rid = llm.add_request([1, 2, 3, 4, 5], SamplingParams(max_new=40))
    llm.step()                                          # the prompt
    llm.step()                                          # first decode step: run eagerly, then captured; the next is queued
    ops.check_tcgen05_status()
    assert ops.status_word_launches() == 0
    for _ in range(4):
        llm.step()                                      # each queues one replay
    assert ops.status_word_launches() >= 4 * cfg["num_hidden_layers"]
    ops.check_tcgen05_status()                          # reads the word: nothing gave up
    assert ops.status_word_launches() == 0
    llm.abort(getattr(rid, "req_id", rid))
    llm.drain()


@pytest.mark.parametrize("policy", ["reserve", "on_demand"])
def test_repetition_penalty_through_graphs_preemption_and_one_token_prompts(tiny, policy):
    """The penalty reads the engine's table of seen ids: rows are zeroed at admission (a slot is
    used again, a preempted request starts over), prompts of one token go straight to a captured
    decode step, penalised and plain requests share steps."""
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    dev = cuda_or_skip()
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    rng = np.random.default_rng(11)
    lengths = (1, page - 1, 2 * page - 2, 1, 7, page + 3)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]
    params = [SamplingParams(max_new=10, temperature=0.0 if i % 3 == 0 else 0.8, seed=i,
                             repetition_penalty=None if i == 2 else 1.0 + 0.25 * (i + 1), top_k=6 if i == 4 else None)
              for i in range(len(prompts))]
    llm = LLM(model_dir, dtype="float32", device=dev, block_size=page, num_pages=64 if policy == "reserve" else 5,
              max_num_seqs=3, chunk_size=24, max_batch_tokens=40, policy=policy)
    for round_ in range(2):                                    # the second round takes slots the first one used
        res = llm.generate(prompts, params)
        for p, q, r in zip(prompts, params, res):
            want = plain.generate(p, q.max_new, w, cfg, temperature=q.temperature, seed=q.seed, top_k=q.top_k,
                                  repetition_penalty=q.repetition_penalty)
            assert r.ids == want, (round_, len(p), q)
    if policy == "on_demand":
        assert llm.scheduler.num_preemptions > 0, "the pool was meant to force a preemption"
    assert any(key[2] for key in llm.engine.graphs.graphs), "decode steps with a penalty were meant to run from a graph"
    llm.engine.cache.check()


def test_warmup_captures_the_graphs_ahead(tiny):
    """`LLM.warmup` captures decode graphs from padding rows only; generation afterwards finds them
    (no step of those shapes runs launch by launch), gives the plain implementation's tokens, and the
    cache was not touched by the warm-up."""
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    dev = cuda_or_skip()
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    llm = LLM(model_dir, dtype="float32", device=dev, block_size=page, num_pages=64, max_num_seqs=3, chunk_size=24,
              max_batch_tokens=40)
    made = llm.warmup()
    graphs = llm.engine.graphs.graphs
    assert made == len(graphs) >= 3 and all(g.graph is not None for g in graphs.values())
    assert llm.warmup() == 0                                    # nothing left to capture
    llm.engine.cache.check()
    assert not llm.engine.cache.requests and all(g.pool.used_count == 0 for g in llm.engine.cache.groups)
    prompts = _prompts(cfg, (5, 17, 33))
    res = llm.generate(prompts, SamplingParams(max_new=8))
    for p, r in zip(prompts, res):
        assert r.ids == plain.generate(p, 8, w, cfg)
    assert len(llm.engine.graphs.graphs) == made                # every decode step found its graph
    assert llm.warmup(batch_sizes=[2], contexts=[64], penalised=True) == 1
    res = llm.generate(prompts[:2], SamplingParams(max_new=6, temperature=0.7, seed=3, repetition_penalty=1.4))
    for p, r in zip(prompts, res):
        assert r.ids == plain.generate(p, 6, w, cfg, temperature=0.7, seed=3, repetition_penalty=1.4)
