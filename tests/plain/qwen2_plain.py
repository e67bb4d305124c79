"""Plain, slow, whole-sequence implementation of the Qwen2.5 dense architecture.

This is the oracle that the engine is compared with.  It is written from the
formulas of the reference project's numpy model code (each function cites the
file and lines it restates) and shares no code with the product package: it has
its own safetensors reader, no cache, no batching, one function per part, and
recomputes the whole sequence for every question asked of it.

Everything is numpy.  Like the reference, activations are float32, the rotary
tables are float64 (so rotated q/k and the q.k product are float64 until the
scores are cast back to float32 before the softmax).
"""

from __future__ import annotations

import json
import struct

import numpy as np


# --------------------------------------------------------------------------
# model folder
# --------------------------------------------------------------------------

def read_config(model_dir: str) -> dict:
    """config.json of a model folder, with the defaults the architecture gives.

    Keys and defaults follow recipes/schema.py:349-372, 426-431 (hidden size,
    layers, heads, kv heads, optional head_dim, eps default 1e-6, tie flag
    default false) restated on config.json's own key names.
    """
    with open(f"{model_dir}/config.json") as f:
        c = json.load(f)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    c.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    c.setdefault("rms_norm_eps", 1e-6)
    c.setdefault("tie_word_embeddings", False)
    c.setdefault("partial_rotary_factor", 1.0)
    return c


_NP_DTYPES = {"F32": np.float32, "F16": np.float16, "F64": np.float64,
              "I32": np.int32, "I64": np.int64}


def read_safetensors(path: str) -> dict:
    """All tensors of one safetensors file as float32 (integers stay integers).

    Format as loaders/safetensors_reader.py:82-139 describes it: 8-byte
    little-endian header length, a JSON header of name -> dtype/shape/
    data_offsets, then the raw bytes.  BF16 is widened by placing the 16 bits
    in the top half of a float32 (loaders/fp8.py:58-64).
    """
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = blob[lo:hi]
        if meta["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32)
        else:
            arr = np.frombuffer(raw, dtype=_NP_DTYPES[meta["dtype"]])
            if arr.dtype.kind == "f":
                arr = arr.astype(np.float32)
        out[name] = arr.reshape(meta["shape"]).copy()
    return out


def load_model(model_dir: str):
    return read_config(model_dir), read_safetensors(f"{model_dir}/model.safetensors")


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def embed(ids, table):
    """h0[t] = embed_tokens.weight[id_t] as float32 (ref/standard.py:95-96)."""
    return table[np.asarray(ids, dtype=np.int64)].astype(np.float32)


def rms_norm(x, weight, eps):
    """y = x * (mean(x^2) + eps)^-1/2 * w, plain w (ref/standard.py:25-31)."""
    xf = x.astype(np.float32)
    var = (xf * xf).mean(-1, keepdims=True)
    out = xf * (var + np.float32(eps)) ** -0.5
    return (out * weight.astype(np.float32)).astype(np.float32)


def linear(x, w, bias=None):
    """x @ w.T (+ bias); w is (out, in) (ref/qwen3_5.py:59-64)."""
    out = x @ w.T
    if bias is not None:
        out = out + bias
    return out


def rotary_tables(theta, positions, rotary_dim):
    """cos/sin of pos * theta^(-2j/rot), j < rot/2, doubled along the last axis,
    float64 (ref/qwen3_5.py:343-352)."""
    inv_freq = 1.0 / (theta ** (np.arange(0, rotary_dim, 2, dtype=np.float64) / rotary_dim))
    freqs = np.asarray(positions, dtype=np.float64)[:, None] * inv_freq[None, :]
    emb = np.concatenate((freqs, freqs), axis=-1)
    return np.cos(emb), np.sin(emb)


def rotate_half(x):
    """concat(-x[half:], x[:half]) (ref/qwen3_5.py:337-340)."""
    h = x.shape[-1] // 2
    return np.concatenate((-x[..., h:], x[..., :h]), axis=-1)


def apply_rotary(x, cos, sin):
    """x: (heads, S, hd).  First rot dims rotated, the rest passed through
    (ref/qwen3_5.py:355-370)."""
    rot = cos.shape[-1]
    xr, xp = x[..., :rot], x[..., rot:]
    out = xr * cos[None] + rotate_half(xr) * sin[None]
    return np.concatenate((out, xp), axis=-1)


def causal_attention(q, k, v, scale, window=None):
    """q,k,v: (heads, S, hd) with k,v already repeated.  Scores times scale,
    keys after the query masked to -inf, cast to float32, softmax with the row
    maximum subtracted, then probs @ v (ref/qwen3_5.py:373-390).

    `window` (keys older than window-1 positions masked too) is not part of the
    reference's architecture; it exists for the kernel tests of the window
    option and is None for every model test.
    """
    s = q.shape[1]
    scores = np.matmul(q, np.swapaxes(k, -1, -2)) * np.float32(scale)
    i = np.arange(s)[:, None]
    j = np.arange(s)[None, :]
    mask = j > i
    if window is not None:
        mask = mask | (j <= i - window)
    scores = np.where(mask[None], np.float32("-inf"), scores).astype(np.float32)
    scores = scores - scores.max(-1, keepdims=True)
    probs = np.exp(scores)
    probs = probs / probs.sum(-1, keepdims=True)
    return np.matmul(probs, v)


def attention_mixer(x, w, prefix, cfg, cos, sin):
    """GQA attention with q/k/v bias (by presence), no o bias: project, split
    heads, rotate q and k, repeat k/v per group (q head h reads kv head
    h // (nq/nkv)), attend, merge heads, o_proj (ref/standard.py:34-72)."""
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    s = x.shape[0]
    a = f"{prefix}.self_attn"
    q = linear(x, w[f"{a}.q_proj.weight"], w.get(f"{a}.q_proj.bias")).reshape(s, nq, hd)
    k = linear(x, w[f"{a}.k_proj.weight"], w.get(f"{a}.k_proj.bias")).reshape(s, nkv, hd)
    v = linear(x, w[f"{a}.v_proj.weight"], w.get(f"{a}.v_proj.bias")).reshape(s, nkv, hd)
    q, k, v = (np.transpose(t, (1, 0, 2)) for t in (q, k, v))
    q = apply_rotary(q, cos, sin)
    k = apply_rotary(k, cos, sin)
    rep = nq // nkv
    if rep > 1:
        k = np.repeat(k, rep, axis=0)
        v = np.repeat(v, rep, axis=0)
    o = causal_attention(q, k, v, hd ** -0.5)
    o = np.transpose(o, (1, 0, 2)).reshape(s, nq * hd)
    return linear(o, w[f"{a}.o_proj.weight"]).astype(np.float32)


def silu(x):
    """x / (1 + exp(-x)) (ref/qwen3_5.py:28-29)."""
    return x * (1.0 / (1.0 + np.exp(-x)))


def swiglu(x, w, prefix):
    """down(silu(gate(x)) * up(x)), no biases (ref/qwen3_5.py:444-451)."""
    m = f"{prefix}.mlp"
    g = linear(x, w[f"{m}.gate_proj.weight"])
    u = linear(x, w[f"{m}.up_proj.weight"])
    return linear(silu(g) * u, w[f"{m}.down_proj.weight"]).astype(np.float32)


def block(h, w, prefix, cfg, cos, sin):
    """Pre-norm block: h += attn(norm(h)); h += mlp(norm(h))
    (ref/standard.py:102-129)."""
    eps = cfg["rms_norm_eps"]
    x = rms_norm(h, w[f"{prefix}.input_layernorm.weight"], eps)
    h = h + attention_mixer(x, w, prefix, cfg, cos, sin)
    x = rms_norm(h, w[f"{prefix}.post_attention_layernorm.weight"], eps)
    return h + swiglu(x, w, prefix)


def forward(ids, w, cfg):
    """Logits (S, V) float32 of one whole sequence, positions 0..S-1
    (ref/standard.py:79-134)."""
    ids = np.asarray(ids, dtype=np.int64)
    h = embed(ids, w["model.embed_tokens.weight"])
    rot = int(cfg["head_dim"] * cfg.get("partial_rotary_factor", 1.0))
    cos, sin = rotary_tables(cfg["rope_theta"], np.arange(len(ids)), rot)
    for i in range(cfg["num_hidden_layers"]):
        h = block(h, w, f"model.layers.{i}", cfg, cos, sin)
    h = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return (h @ head.T).astype(np.float32)


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------

def greedy(logits) -> int:
    """First maximum (runtime/sampler.py:8-9)."""
    return int(np.argmax(logits))


def apply_repetition_penalty(logits, seen_ids, penalty):
    """Seen ids: positive logits divided, negative multiplied by the penalty;
    a copy; ids outside the vocabulary ignored (runtime/sampler.py:12-33)."""
    out = np.asarray(logits, dtype=np.float64).copy()
    if penalty is None or penalty <= 0 or penalty == 1.0 or seen_ids is None:
        return out
    ids = np.asarray(seen_ids, dtype=np.int64)
    ids = ids[(ids >= 0) & (ids < out.size)]
    if ids.size:
        vals = out[ids]
        out[ids] = np.where(vals < 0, vals * penalty, vals / penalty)
    return out


def sample(logits, temperature=1.0, top_k=None, top_p=None, u=None) -> int:
    """float64 softmax of logits/temperature, top-k then top-p filtering with
    renormalisation, inverse CDF at the uniform `u`; temperature <= 0 is greedy
    (runtime/sampler.py:36-88).  The caller draws `u = rng.random()`, one per
    sampled token (runtime/sampler.py:86)."""
    logits = np.asarray(logits, dtype=np.float64)
    if temperature is None or temperature <= 0:
        return greedy(logits)
    logits = logits / temperature
    probs = np.exp(logits - logits.max())
    probs = probs / probs.sum()
    if top_k is not None:
        k = min(int(top_k), probs.size)
        if k <= 0:
            raise ValueError("top_k must be >= 1")
        keep = np.argsort(probs)[-k:]
        mask = np.zeros(probs.shape, dtype=bool)
        mask[keep] = True
        probs = np.where(mask, probs, 0.0)
        if probs.sum() > 0:
            probs = probs / probs.sum()
    if top_p is not None:
        order = np.argsort(probs)[::-1]
        cum = np.cumsum(probs[order])
        cutoff = int(np.searchsorted(cum, top_p) + 1)
        mask = np.zeros(probs.shape, dtype=bool)
        mask[order[:cutoff]] = True
        probs = np.where(mask, probs, 0.0)
    total = probs.sum()
    if total <= 0 or not np.isfinite(total):
        return greedy(logits)
    probs = probs / total
    idx = int(np.searchsorted(np.cumsum(probs), u))
    return min(idx, probs.size - 1)


def generate(prompt, max_new, w, cfg, temperature=0.0, seed=None, stop_ids=(), top_k=None, top_p=None,
             repetition_penalty=None):
    """Token-by-token generation by recomputing the whole sequence each time:
    sample from the last row (after the repetition penalty over every id so far), a
    stop id ends the request and is not appended, the context limit ends it too
    (serving/executor.py:366-393)."""
    ids = list(prompt)
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(max_new):
        logits = forward(ids, w, cfg)[-1]
        if repetition_penalty is not None and repetition_penalty != 1.0:      # serving/executor.py:430-433
            logits = apply_repetition_penalty(logits, ids, repetition_penalty)
        if temperature and temperature > 0:
            nxt = sample(logits, temperature, top_k, top_p, u=rng.random())
        else:
            nxt = greedy(logits)
        if nxt in stop_ids:
            break
        ids.append(nxt)
        out.append(nxt)
        if len(ids) >= cfg["max_position_embeddings"]:
            break
    return out
