"""A whole architecture defined in this file and launched through the command line, with no edit to
the package: a block arrangement with FOUR norms of two kinds around its mixer and feed-forward
("sandwich": pre and post norms), a block without a feed-forward, a norm kind of its own
(mean-subtracting, with a bias), a recipe whose ``arch:`` is the toy's alias, and the geometry read
from the recipe by the architecture's own hook.  `python -m sllm_b200.serving.main <recipe> --mode
run --random-weights SEED` must print the greedy tokens of a plain numpy statement of the same model.

Runs twice: with the PyTorch stand-ins for the kernels (no GPU), and on the GPU with the real ones.

Below it, a second toy architecture: layers whose attention has a window beside layers without one (two cache
groups; pages given back while a request runs, and used again), replayed in all four cuttings.
"""

import os

import numpy as np
import pytest
import torch

from tests.conftest import cuda_or_skip
from tests.plain import qwen2_plain as plain

RECIPE = """
name: toy-sandwich
model_id: toy/sandwich
arch: toy-sandwich
dtype: float32
text:
  tie_word_embeddings: false
  hidden_size: 48
  num_layers: 3
  full_attention: {num_heads: 3, num_kv_heads: 1, head_dim: 16, rope: {theta: 5000.0}}
  mlp: {intermediate_size: 80}
  vocab_size: 200
  max_position_embeddings: 96
  rms_norm_eps: 1.0e-5
memory:
  kv_device_bytes: 1048576
defaults: {max_new: 6, max_num_seqs: 2, block_size: 8, chunk_size: 16}
"""
LN_EPS = 1e-5


def _register():
    from sllm_b200.config import (Architecture, LayerSpec, ModelPlan, PartEntry, PartSpec, RunEntry,
                                  register_architecture)
    from sllm_b200.models import qwen2
    from sllm_b200.parts import BLOCKS, NORMS, Norm, TensorSpec

    @NORMS.register("toy_layernorm", replace=True)
    class ToyLayerNorm(Norm):
        """(x - mean) / sqrt(var + eps) * weight + bias, in float32."""

        def __init__(self, params, **kw):
            super().__init__(params, **kw)
            self.size, self.eps = int(params["size"]), float(params["eps"])

        def tensor_specs(self):
            return [TensorSpec("weight", (self.size,), role="gain"), TensorSpec("bias", (self.size,), role="bias")]

        def bind(self, fetch):
            self.weight, self.bias = self._f32(fetch("weight")), self._f32(fetch("bias"))

        def norm(self, x):
            x = x.float()
            if x.dim() == 3:                      # a stack of partial sums from a k-split product
                x = x.sum(0)
            mu = x.mean(-1, keepdim=True)
            var = ((x - mu) ** 2).mean(-1, keepdim=True)
            return (x - mu) / torch.sqrt(var + self.eps) * self.weight + self.bias

    @BLOCKS.register("toy_sandwich", replace=True)
    class Sandwich:
        """h += post1(mixer(pre1(h))); h += post2(ffn(pre2(h))): six parts, four of them norms."""

        def __init__(self, parts):
            self.p = parts
            assert set(parts) == {"pre1", "mixer", "post1", "pre2", "ffn", "post2"}

        def cache_need(self):
            return self.p["mixer"].cache_need()

        def forward(self, residual, delta, step, cache, position, write_cache=True):
            p = self.p
            x = p["pre1"].add_norm(residual, delta)
            residual += p["post1"].norm(p["mixer"].forward(x, step, cache, position, write_cache))
            x = p["pre2"].add_norm(residual, None)
            return p["post2"].norm(p["ffn"].forward(x, step))

    @BLOCKS.register("toy_mixer_only", replace=True)
    class MixerOnly:
        """h += mixer(norm(h)): a layer without a feed-forward."""

        def __init__(self, parts):
            self.p = parts
            assert set(parts) == {"norm", "mixer"}

        def cache_need(self):
            return self.p["mixer"].cache_need()

        def forward(self, residual, delta, step, cache, position, write_cache=True):
            x = self.p["norm"].add_norm(residual, delta)
            return self.p["mixer"].forward(x, step, cache, position, write_cache)

    def toy_plan(cfg):
        base = qwen2.plan(cfg)
        first = base.layers[0]
        rms, mixer, ffn = first.part("mixer_norm"), first.part("mixer"), first.part("ffn")
        ln = PartSpec("toy_layernorm", {"size": cfg.hidden_size, "eps": LN_EPS})
        layers = []
        for i in range(cfg.num_hidden_layers):
            prefix = f"model.layers.{i}"
            if i % 2 == 0:
                layers.append(LayerSpec(prefix=prefix, block="toy_sandwich", parts={
                    "pre1": PartEntry("norm", rms, "input_layernorm"), "mixer": PartEntry("mixer", mixer, "self_attn"),
                    "post1": PartEntry("norm", ln, "post_mixer_norm"), "pre2": PartEntry("norm", rms, "pre_ffn_norm"),
                    "ffn": PartEntry("feed_forward", ffn, "mlp"), "post2": PartEntry("norm", ln, "post_ffn_norm")}))
            else:
                layers.append(LayerSpec(prefix=prefix, block="toy_mixer_only", parts={
                    "norm": PartEntry("norm", rms, "input_layernorm"), "mixer": PartEntry("mixer", mixer, "self_attn")}))
        return ModelPlan(architecture="ToySandwichLM", hidden_size=base.hidden_size, vocab_size=base.vocab_size,
                         max_positions=base.max_positions, embedding_name=base.embedding_name, layers=tuple(layers),
                         run_list=tuple(RunEntry(i) for i in range(len(layers))), final_norm=base.final_norm,
                         final_norm_name=base.final_norm_name, head_name=base.head_name, position=base.position)

    register_architecture(Architecture(
        "ToySandwichLM", qwen2.Qwen2Config, toy_plan, aliases=("toy-sandwich",),
        config_from_recipe=lambda t: dict(qwen2.config_from_recipe(t), architectures=["ToySandwichLM"])), replace=True)


def _unregister():
    from sllm_b200.config import unregister_architecture
    from sllm_b200.parts import BLOCKS, NORMS
    unregister_architecture("ToySandwichLM")
    NORMS.unregister("toy_layernorm")
    BLOCKS.unregister("toy_sandwich")
    BLOCKS.unregister("toy_mixer_only")


def _layernorm(x, w, b):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return ((x - mu) / np.sqrt(var + LN_EPS) * w + b).astype(np.float32)


def _plain_logits(ids, w, cfg):
    h = plain.embed(np.asarray(ids), w["model.embed_tokens.weight"])
    cos, sin = plain.rotary_tables(cfg["rope_theta"], np.arange(len(ids)), cfg["head_dim"])
    eps = cfg["rms_norm_eps"]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        x = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], eps)
        a = plain.attention_mixer(x, w, p, cfg, cos, sin)
        if i % 2 == 0:
            h = h + _layernorm(a, w[f"{p}.post_mixer_norm.weight"], w[f"{p}.post_mixer_norm.bias"])
            x = plain.rms_norm(h, w[f"{p}.pre_ffn_norm.weight"], eps)
            h = h + _layernorm(plain.swiglu(x, w, p), w[f"{p}.post_ffn_norm.weight"], w[f"{p}.post_ffn_norm.bias"])
        else:
            h = h + a
    h = plain.rms_norm(h, w["model.norm.weight"], eps)
    return h @ w["lm_head.weight"].T


def _run(tmp_path, capsys, extra=()):
    from sllm_b200.config.recipe import Recipe
    from sllm_b200.serving import main as cli
    from sllm_b200.weights import write_random_model
    _register()
    try:
        path = os.path.join(str(tmp_path), "toy-sandwich.yaml")
        with open(path, "w") as f:
            f.write(RECIPE)
        # plan mode describes the model from its own cache needs: two kinds of blocks, one cache group
        assert cli.main([path]) == 0
        out = capsys.readouterr().out
        assert "ToySandwichLM: 3 layers in 3 runs" in out and "3 runs x 1 kv heads of 16" in out and "1048576 bytes" in out
        prompt = [5, 17, 3, 150, 42, 7, 99, 120, 8, 61, 33]
        assert cli.main([path, "--mode", "run", "--random-weights", "4", "--prompt-ids", ",".join(map(str, prompt)),
                         "--log-level", "ERROR", *extra]) == 0
        got = [int(t) for t in capsys.readouterr().out.strip().split(",")]
        # the same folder again from the seed (main.py writes it with std 0.02 and bias_std 0.1), read by the plain code
        folder = write_random_model(os.path.join(str(tmp_path), "again"), Recipe.from_yaml(path).config_json(), 4,
                                    std=0.02, bias_std=0.1)
        cfg, w = plain.load_model(folder)
        assert any(k.endswith("post_ffn_norm.bias") for k in w) and "model.layers.1.mlp.gate_proj.weight" not in w
        ids, want = list(prompt), []
        for _ in range(6):
            want.append(int(np.argmax(_plain_logits(ids, w, cfg)[-1])))
            ids.append(want[-1])
        assert got == want
    finally:
        _unregister()


def test_toy_architecture_through_the_command_line_with_stand_in_kernels(tmp_path, capsys, cpu_ops, monkeypatch):
    import sllm_b200.engine.llm as llm_mod
    real = llm_mod.LLM
    monkeypatch.setattr(llm_mod, "LLM", lambda model_dir, **kw: real(model_dir, **dict(kw, device="cpu")))
    _run(tmp_path, capsys)


@pytest.mark.gpu
def test_toy_architecture_through_the_command_line(tmp_path, capsys):
    cuda_or_skip()
    _run(tmp_path, capsys)


# ---- layers with a window beside layers without: two cache groups, pages given back and used again ------------------

WINDOW = 20
# heads of 64, so that the TMA-fed decode kernel meets the window and the holes it leaves in the block tables
HD64 = ({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 192, "num_attention_heads": 6,
         "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 272, "vocab_size": 500, "rope_theta": 10000.0,
         "rms_norm_eps": 1e-6, "max_position_embeddings": 256, "tie_word_embeddings": True, "hidden_act": "silu"},
        {"std": 0.05}, 16)


def _register_windowed():
    from sllm_b200.config import Architecture, ModelPlan, PartSpec, RunEntry, pre_norm_layer, register_architecture
    from sllm_b200.models import qwen2

    def plan(cfg):
        base = qwen2.plan(cfg)
        layers = []
        for i, l in enumerate(base.layers):
            mixer = l.part("mixer")
            if i % 2:                               # every second layer only ever reads the last WINDOW keys
                mixer = PartSpec(mixer.kind, dict(mixer.params, window=WINDOW))
            layers.append(pre_norm_layer(l.prefix, mixer, l.part("ffn"), l.part("mixer_norm")))
        return ModelPlan(architecture="ToyWindowLM", hidden_size=base.hidden_size, vocab_size=base.vocab_size,
                         max_positions=base.max_positions, embedding_name=base.embedding_name, layers=tuple(layers),
                         run_list=tuple(RunEntry(i) for i in range(len(layers))), final_norm=base.final_norm,
                         final_norm_name=base.final_norm_name, head_name=base.head_name, position=base.position)

    register_architecture(Architecture("ToyWindowLM", qwen2.Qwen2Config, plan), replace=True)


def _plain_windowed(ids, w, cfg):
    h = plain.embed(np.asarray(ids), w["model.embed_tokens.weight"])
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    s = len(ids)
    cos, sin = plain.rotary_tables(cfg["rope_theta"], np.arange(s), hd)
    for i in range(cfg["num_hidden_layers"]):
        p, a = f"model.layers.{i}", f"model.layers.{i}.self_attn"
        x = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])
        q, k, v = (plain.linear(x, w[f"{a}.{n}_proj.weight"], w[f"{a}.{n}_proj.bias"]).reshape(s, heads, hd).transpose(1, 0, 2)
                   for n, heads in (("q", nq), ("k", nkv), ("v", nkv)))
        q, k = plain.apply_rotary(q, cos, sin), plain.apply_rotary(k, cos, sin)
        o = plain.causal_attention(q, np.repeat(k, nq // nkv, axis=0), np.repeat(v, nq // nkv, axis=0), hd ** -0.5,
                                   window=WINDOW if i % 2 else None)
        h = h + plain.linear(o.transpose(1, 0, 2).reshape(s, nq * hd), w[f"{a}.o_proj.weight"])
        x = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        h = h + plain.swiglu(x, w, p)
    h = plain.rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return (h @ head.T).astype(np.float32)


def _run_windowed(tmp_path, dev, dtypes, configs):
    """Every cutting of the requests through a model whose odd layers have a window: those layers form a cache
    group of their own, give the pages the window has passed back while a request still runs, and read block tables
    with holes.  The pools are sized for the trace's peak, so pages given back are used again."""
    from sllm_b200.config import unregister_architecture
    from sllm_b200.engine import Engine, build_model
    from sllm_b200.weights import write_random_model
    from tests import traces
    from tests.conftest import TINY
    _register_windowed()
    try:
        for which in configs:
            config, init, page = TINY[which] if which in TINY else HD64
            config = dict(config, architectures=["ToyWindowLM"], num_hidden_layers=4)
            d = write_random_model(os.path.join(str(tmp_path), f"win{which}"), config, 21, std=init["std"], bias_std=0.2, gain_std=0.1)
            cfg, w = plain.load_model(d)
            rng = np.random.default_rng(3)
            top = cfg["max_position_embeddings"]
            reqs = {f"r{i}": rng.integers(0, cfg["vocab_size"], min(n, top)).tolist() for i, n in enumerate((70, 37, 100, 45, 64, 90))}
            want = {r: _plain_windowed(ids, w, cfg) for r, ids in reqs.items()}
            for dtype in dtypes:
                tol = dict(rtol=1e-4, atol=2e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)
                model, _ = build_model(d, dtype, dev)
                for mode in ("whole", "tail_decode", "portions", "mixed"):
                    tr = getattr(traces, mode)(reqs)
                    eng = Engine(model, page_size=page, num_pages=tr.max_tokens // page, max_requests=4, poison_freed=True)
                    assert [g.need.window for g in eng.cache.groups] == [None, WINDOW] and [len(g.runs) for g in eng.cache.groups] == [2, 2]
                    out = traces.replay_engine(tr, eng)
                    traces.compare(tr, out, want, what=f"windowed {which}/{dtype}/{mode}", **tol)
                    eng.cache.check()
                    assert not eng.cache.requests and all(g.pool.used_count == 0 for g in eng.cache.groups)
                    if mode in ("tail_decode", "mixed"):
                        assert eng.cache.reuse_count > 0, "pages the window gave back were meant to be used again"
                if dtype == "float32" and dev != "cpu":
                    # generation through the entry point: decode steps from captured graphs over both cache groups,
                    # with so few pages that only the window's giving back lets all requests finish
                    from sllm_b200.engine.llm import LLM
                    from sllm_b200.sampling import SamplingParams
                    prompts = [ids[:n] for ids, n in zip(reqs.values(), (9, 30, 17))]
                    new = min(40, top - 31)
                    llm = LLM(model=model, block_size=page, num_pages=3 * (-(-(30 + new) // page)) + 1, max_num_seqs=3, chunk_size=16,
                              max_batch_tokens=64, policy="on_demand")
                    res = llm.generate(prompts, SamplingParams(max_new=new))
                    for pr, r in zip(prompts, res):
                        ids, out = list(pr), []
                        for _ in range(new):
                            out.append(int(np.argmax(_plain_windowed(ids, w, cfg)[-1])))
                            ids.append(out[-1])
                        assert r.ids == out, (which, len(pr))
                    assert any(g.graph is not None for g in llm.engine.graphs.graphs.values())
                    llm.engine.cache.check()
    finally:
        unregister_architecture("ToyWindowLM")


def test_windowed_layers_beside_full_ones_with_stand_in_kernels(tmp_path, cpu_ops):
    _run_windowed(tmp_path, "cpu", ("float32",), ("A",))


@pytest.mark.gpu
def test_windowed_layers_beside_full_ones(tmp_path):
    _run_windowed(tmp_path, cuda_or_skip(), ("float32", "bfloat16"), ("A", "B", "hd64"))
