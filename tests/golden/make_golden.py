"""Makes tests/golden/qwen2_tiny_golden.npz: logits of the reference project's own
numpy model code (ref/standard.py `standard_model_forward`, and the cached path
ref/incremental.py `prefill`/`decode_step`) on two tiny random models.

Run once, where the reference's source tree can be imported:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/sLLM

The test `tests/test_plain.py::test_plain_matches_reference_golden` regenerates the
same weights from `golden_weights` below and compares the plain implementation with
the stored logits, so the plain implementation is anchored on the reference's code
and not only on a reading of its formulas.  Only numbers are stored here: no code of
the reference.
"""

from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    # name: (config.json keys, seed, std, lengths)
    "A": (dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
               intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
               max_position_embeddings=128, tie_word_embeddings=True), 0, 0.05, (5, 33)),
    "B": (dict(num_hidden_layers=3, hidden_size=96, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
               intermediate_size=320, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
               max_position_embeddings=256, tie_word_embeddings=False), 1, 0.04, (9, 40)),
}


def golden_weights(cfg: dict, seed: int, std: float) -> dict:
    """float32 tensors under checkpoint names, drawn in a fixed order."""
    rng = np.random.default_rng(seed)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq = cfg["num_attention_heads"] * cfg["head_dim"]
    nk = cfg["num_key_value_heads"] * cfg["head_dim"]

    def n(*shape, s=std):
        return (s * rng.standard_normal(shape)).astype(np.float32)

    w = {"model.embed_tokens.weight": n(V, H)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        w[f"{p}.input_layernorm.weight"] = (1 + n(H, s=0.1)).astype(np.float32)
        w[f"{p}.post_attention_layernorm.weight"] = (1 + n(H, s=0.1)).astype(np.float32)
        for name, rows in (("q", nq), ("k", nk), ("v", nk)):
            w[f"{p}.self_attn.{name}_proj.weight"] = n(rows, H)
            w[f"{p}.self_attn.{name}_proj.bias"] = n(rows, s=6 * std)
        w[f"{p}.self_attn.o_proj.weight"] = n(H, nq)
        w[f"{p}.mlp.gate_proj.weight"] = n(I, H)
        w[f"{p}.mlp.up_proj.weight"] = n(I, H)
        w[f"{p}.mlp.down_proj.weight"] = n(H, I)
    w["model.norm.weight"] = (1 + n(H, s=0.1)).astype(np.float32)
    if not cfg["tie_word_embeddings"]:
        w["lm_head.weight"] = n(V, H)
    return w


def golden_ids(cfg: dict, seed: int, length: int) -> np.ndarray:
    return np.random.default_rng(1000 + seed + length).integers(0, cfg["vocab_size"], length)


def _recipe(cfg, Recipe):
    L = cfg["num_hidden_layers"]
    return Recipe.from_dict({
        "model_id": "tiny/golden", "arch": "qwen2", "dtype": "bfloat16",
        "text": {
            "prefix": "model", "tie_word_embeddings": cfg["tie_word_embeddings"],
            "hidden_size": cfg["hidden_size"], "num_layers": L, "layer_types": ["full_attention"] * L,
            "full_attention": {"kernel": "standard_gqa", "num_heads": cfg["num_attention_heads"],
                               "num_kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                               "output_gate": False,
                               "rope": {"type": "default", "theta": cfg["rope_theta"],
                                        "partial_rotary_factor": 1.0}},
            "mlp": {"type": "dense", "intermediate_size": cfg["intermediate_size"], "hidden_act": "silu"},
            "vocab_size": cfg["vocab_size"], "max_position_embeddings": cfg["max_position_embeddings"],
            "rms_norm_eps": cfg["rms_norm_eps"],
        },
        "mtp": {"enabled": False}, "vision": {"enabled": False}, "tp": {"size": 1},
    })


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from recipes.schema import Recipe
    from ref import incremental as inc
    from ref.standard import standard_model_forward
    out = {}
    for name, (cfg, seed, std, lengths) in CASES.items():
        recipe = _recipe(cfg, Recipe)
        w = golden_weights(cfg, seed, std)
        for n in lengths:
            ids = golden_ids(cfg, seed, n)
            logits = standard_model_forward(ids[None, :], w, recipe)[0]
            out[f"{name}_{n}_full"] = logits.astype(np.float32)
            # cached path: all but the last 3 tokens as the prompt, then token by token
            if n > 4:
                cache, pl = inc.prefill(ids[: n - 3], w, recipe)
                rows = [pl[0, -1]]
                for t in ids[n - 3: n]:
                    rows.append(inc.decode_step(cache, w, recipe, int(t)))
                out[f"{name}_{n}_cached"] = np.stack(rows).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "qwen2_tiny_golden.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SLLM_REF_PATH", ""))
