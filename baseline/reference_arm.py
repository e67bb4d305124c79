"""The reference arm of the benchmark: skfine24/sLLM's own device-resident decode, unmodified,
timed on the same metric and sizes as this engine's arm.

The reference is a source tree that is run in place (it has no setup.py; pip cannot install
it).  This module finds a copy of it (``baseline/_ref``, else ``$SLLM_REF_PATH``), builds its
CUDA library with its own script (``kernels/cuda/build.sh`` with ``NVCC_ARCH=sm_100``: plain SIMT
kernels and cuBLAS, nothing specific to one GPU generation), and drives its stock decode path the
way its own benchmark does (bench/gpu_decode_timing.py:94-116): ``ref.incremental.prefill`` in
numpy on the host, ``DeviceWeightTable(weights, recipe, dtype="bf16")`` once, one
``DeviceDecodeState`` per sequence on that table (tests/test_gpu_decode.py:298-324), and
``DeviceDecodeState.step`` for every token of every sequence.  The reference decodes one token of
one sequence per call and mirrors the new keys and values into the host cache after every step;
a batch of B sequences is B such calls.  Nothing of this package is imported here.

What differs from this engine's arm, and is said in the record's ``config``: the prompt is one
sequence of uniform random ids whose host cache is copied to all B sequences (the numpy prefill of
a 7B-size model takes minutes per prompt), and time is wall clock around the steps (the
reference's step synchronises the device itself and has host work inside that cannot be timed
apart without changing it).
"""

from __future__ import annotations

import copy
import os
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))


class Unavailable(RuntimeError):
    """The reference cannot be run here; the message is the one-line reason."""


def find_tree() -> str:
    for cand in (os.path.join(HERE, "_ref"), os.environ.get("SLLM_REF_PATH")):
        if cand and os.path.isfile(os.path.join(cand, "kernels", "cuda", "kernels.cu")):
            return os.path.abspath(cand)
    raise Unavailable("no copy of skfine24/sLLM under baseline/_ref or $SLLM_REF_PATH")


def ensure_library(tree: str, say) -> str:
    """The reference's ``sllm_gpu.so``, built with its own script if it is not there yet.  A tree
    that cannot be written to is copied to a temporary folder first.  Returns the tree to import from."""
    so = os.path.join(tree, "kernels", "cuda", "sllm_gpu.so")
    if os.path.isfile(so):
        return tree
    if not os.access(os.path.join(tree, "kernels", "cuda"), os.W_OK):
        dst = os.path.join(tempfile.mkdtemp(prefix="sllm_ref_"), "sLLM")
        shutil.copytree(tree, dst)
        for root, dirs, files in os.walk(dst):
            for n in dirs + files:
                os.chmod(os.path.join(root, n), 0o755)
        tree = dst
    say(f"building the reference's CUDA library ({tree}/kernels/cuda/build.sh, NVCC_ARCH=sm_100)")
    env = dict(os.environ, NVCC_ARCH="sm_100")
    if not shutil.which("nvcc") and os.path.isfile("/usr/local/cuda/bin/nvcc"):
        env["NVCC"] = "/usr/local/cuda/bin/nvcc"
    r = subprocess.run(["bash", os.path.join(tree, "kernels", "cuda", "build.sh")], env=env, capture_output=True, text=True)
    if r.returncode != 0 or not os.path.isfile(os.path.join(tree, "kernels", "cuda", "sllm_gpu.so")):
        raise Unavailable("the reference's kernels/cuda/build.sh failed: " + (r.stderr or r.stdout).strip().splitlines()[-1][:200])
    return tree


def recipe_dict(cfg: dict) -> dict:
    """A config.json of this architecture as the reference's recipe (recipes/schema.py)."""
    L = cfg["num_hidden_layers"]
    return {
        "model_id": "bench/qwen2-sizes", "arch": "qwen2", "dtype": "bfloat16",
        "text": {
            "prefix": "model", "tie_word_embeddings": cfg["tie_word_embeddings"],
            "hidden_size": cfg["hidden_size"], "num_layers": L, "layer_types": ["full_attention"] * L,
            "full_attention": {"kernel": "standard_gqa", "num_heads": cfg["num_attention_heads"],
                               "num_kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                               "output_gate": False,
                               "rope": {"type": "default", "theta": cfg["rope_theta"], "partial_rotary_factor": 1.0}},
            "mlp": {"type": "dense", "intermediate_size": cfg["intermediate_size"], "hidden_act": "silu"},
            "vocab_size": cfg["vocab_size"], "max_position_embeddings": cfg["max_position_embeddings"],
            "rms_norm_eps": cfg["rms_norm_eps"],
        },
        "mtp": {"enabled": False}, "vision": {"enabled": False}, "tp": {"size": 1},
    }


def random_weights(cfg: dict, seed: int, std: float, share_layers: bool, say):
    """float32 host tensors under the checkpoint's names: matrices and biases N(0, std), gains 1.
    ``share_layers``: every layer's names point at the first layer's arrays (host memory is short);
    the device table still holds one buffer per layer, so the decode step reads as many bytes."""
    import numpy as np
    rng = np.random.default_rng(seed)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nk = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]

    def n(*shape):
        a = rng.standard_normal(shape, dtype=np.float32)
        a *= np.float32(std)
        return a

    w = {"model.embed_tokens.weight": n(V, H), "model.norm.weight": np.ones(H, np.float32)}
    if not cfg["tie_word_embeddings"]:
        w["lm_head.weight"] = n(V, H)
    first = None
    for i in range(cfg["num_hidden_layers"]):
        if first is None or not share_layers:
            layer = {"input_layernorm.weight": np.ones(H, np.float32), "post_attention_layernorm.weight": np.ones(H, np.float32),
                     "self_attn.o_proj.weight": n(H, nq), "mlp.gate_proj.weight": n(I, H), "mlp.up_proj.weight": n(I, H),
                     "mlp.down_proj.weight": n(H, I)}
            for name, rows in (("q", nq), ("k", nk), ("v", nk)):
                layer[f"self_attn.{name}_proj.weight"] = n(rows, H)
                layer[f"self_attn.{name}_proj.bias"] = n(rows)
            first = first or layer
            if i % 4 == 3:
                say(f"host weights: layer {i + 1} of {cfg['num_hidden_layers']}")
        else:
            layer = first
        for k, v in layer.items():
            w[f"model.layers.{i}.{k}"] = v
    return w


def run(cfg: dict, *, batch: int, context: int, steps: int, warmup: int, repeats: int = 1, std: float = 0.02, seed: int = 0,
        time_limit_s: float = 1500.0, clock_sampler=None,
        say=lambda m: print(f"[reference arm] {m}", file=sys.stderr, flush=True)) -> dict:
    """Time ``steps`` decode steps of ``batch`` sequences, ``repeats`` times in a row after ``warmup`` untimed
    steps, the last region's contexts ending at ``context``, through the reference's device-resident path in
    bfloat16; the median region is the result (fewer regions are run if the time at hand ends first).
    ``clock_sampler``: an object with ``start()`` and ``stop()`` that samples the GPU's clocks meanwhile.
    Returns the fields of the benchmark's record that are measured here.  Raises `Unavailable` with the reason."""
    import numpy as np
    t_start = time.perf_counter()
    tree = ensure_library(find_tree(), say)
    sys.path.insert(0, tree)
    try:
        from kernels import _sllm_cuda as ck
        from kernels.device_decode import DeviceDecodeState, DeviceWeightTable
        from recipes.schema import Recipe
        from ref import incremental as inc
    except Exception as exc:                       # a missing dependency of the reference (yaml, ...)
        raise Unavailable(f"importing the reference failed: {type(exc).__name__}: {exc}") from exc
    if ck.device_count() < 1:
        raise Unavailable("the reference's library sees no CUDA device")
    recipe = Recipe.from_dict(recipe_dict(cfg))

    try:
        import psutil
        avail = psutil.virtual_memory().available
    except Exception:
        avail = 0
    params = 4 * (cfg["num_hidden_layers"] * (cfg["hidden_size"] * (2 * cfg["num_attention_heads"] * cfg["head_dim"]
                  + 2 * cfg["num_key_value_heads"] * cfg["head_dim"] + 3 * cfg["intermediate_size"]))
                  + 2 * cfg["vocab_size"] * cfg["hidden_size"])
    share = avail < 2.5 * params
    say(f"host memory available {avail / 2**30:.0f} GiB, float32 weights {params / 2**30:.0f} GiB"
        + (": one layer's tensors shared by all layers" if share else ""))
    t0 = time.perf_counter()
    weights = random_weights(cfg, seed, std, share, say)
    t_weights = time.perf_counter() - t0

    # the prompt: long enough that the timed steps end at `context`; shortened only if the numpy prefill
    # would not fit the time this arm has (estimated from a short one)
    prompt_len = context - (warmup + repeats * steps)
    rng = np.random.default_rng(seed + 1)
    probe_len = min(128, prompt_len)
    t0 = time.perf_counter()
    inc.prefill(rng.integers(0, cfg["vocab_size"], probe_len).tolist(), weights, recipe)
    t_probe = time.perf_counter() - t0
    left = time_limit_s - (time.perf_counter() - t_start) - 240.0       # the upload and the steps need their share
    estimate = t_probe * (prompt_len / probe_len) * 1.5                 # attention grows faster than linearly
    say(f"numpy prefill of {probe_len} tokens: {t_probe:.1f} s; estimate for {prompt_len}: {estimate:.0f} s, {left:.0f} s at hand")
    shortened = False
    if estimate > left:
        prompt_len = max(16, int(prompt_len * left / estimate) // 16 * 16)
        shortened = True
        say(f"prompt shortened to {prompt_len} tokens")
    prompt = rng.integers(0, cfg["vocab_size"], prompt_len).tolist()
    t0 = time.perf_counter()
    cache0, logits0 = inc.prefill(prompt, weights, recipe)
    t_prefill = time.perf_counter() - t0
    first_id = int(np.argmax(logits0[0, -1]))
    del logits0
    say(f"numpy prefill of {prompt_len} tokens: {t_prefill:.1f} s")

    t0 = time.perf_counter()
    try:
        table = DeviceWeightTable(weights, recipe, dtype="bf16")
    except Exception as exc:
        raise Unavailable(f"DeviceWeightTable: {type(exc).__name__}: {exc}") from exc
    say(f"weights on the device ({table.total_bytes / 1e9:.1f} GB) in {time.perf_counter() - t0:.1f} s")
    states = []
    try:
        # one check of the device path against the reference's own numpy step, as its benchmark prints
        check_cache = copy.deepcopy(cache0)
        want = inc.decode_step(check_cache, weights, recipe, first_id)
        del check_cache
        for _ in range(batch):
            states.append(DeviceDecodeState(table, copy.deepcopy(cache0), recipe))
        ids = [first_id] * batch
        got = None

        def one_step():
            nonlocal got
            for b, st in enumerate(states):
                logits = st.step(ids[b])
                if got is None:
                    got = logits.copy()
                ids[b] = int(np.argmax(logits))

        for _ in range(warmup):
            one_step()
        agree = {"max_abs_diff_vs_numpy": float(np.max(np.abs(got - want))), "same_argmax": bool(np.argmax(got) == np.argmax(want))}
        ck.sync()
        if clock_sampler is not None:
            clock_sampler.start()
        walls = []
        for r in range(repeats):
            t0 = time.perf_counter()
            for _ in range(steps):
                one_step()
            ck.sync()
            walls.append(time.perf_counter() - t0)
            if time.perf_counter() - t_start + 1.5 * walls[-1] + 30.0 > time_limit_s:
                say(f"time at hand ends: {len(walls)} of {repeats} regions timed")
                break
        clocks = clock_sampler.stop() if clock_sampler is not None else None
        wall = sorted(walls)[len(walls) // 2]
        # batch 1 on the same table: the first sequence alone
        b1_steps = max(4, steps // 2)
        solo = states[0]
        tok = ids[0]
        t1 = time.perf_counter()
        for _ in range(b1_steps):
            tok = int(np.argmax(solo.step(tok)))
        ck.sync()
        wall_b1 = time.perf_counter() - t1
    finally:
        for st in states:
            st.free()
        table.free()
    L, V = cfg["num_hidden_layers"], cfg["vocab_size"]
    nk = cfg["num_key_value_heads"] * cfg["head_dim"]
    # per sequence and step the reference uploads cos|sin of the position and reads back the logits and the
    # new key and value rows of every layer (kernels/device_decode.py:283-284, 327-329)
    h2d = batch * 2 * cfg["head_dim"] * 4
    d2h = batch * (V * 4 + 2 * L * nk * 4)
    return {
        "ms_per_step": wall * 1e3 / steps, "tok_s": batch * steps / wall, "prompt_len": prompt_len, "shortened": shortened,
        "ms_min": min(walls) * 1e3 / steps, "ms_max": max(walls) * 1e3 / steps, "repeats": len(walls), "clocks": clocks,
        "h2d": h2d, "d2h": d2h, "decode_b1": b1_steps / wall_b1, "agree": agree,
        "prefill": {"value": round(prompt_len / t_prefill, 1), "tokens": prompt_len, "ms": round(t_prefill * 1e3, 1),
                    "where": "host numpy (the reference has no device prefill)"},
        "host_weights_s": round(t_weights, 1), "shared_layers": share, "tree": tree,
        "launches_per_step": batch * (L * 11 + 3),      # kernels/device_decode.py:15-19: 11 device ops a layer
    }
