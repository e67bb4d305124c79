"""Qwen2.5 dense (``Qwen2ForCausalLM``): typed configuration and model plan.

The architecture as the reference's standard path computes it
(ref/standard.py:79-134): token embedding; per layer a pre-norm block of GQA
attention (q/k/v bias, no o bias, rotate-half rotary on q and k, causal, no
window) and a SwiGLU feed-forward, each behind an RMSNorm with plain gain;
a final RMSNorm; an output head that is its own matrix or the embedding table.

This file is all that names the architecture: it reads config.json's keys,
turns them into part specifications, and registers itself.  Tensor names are
the checkpoint's own (ref/standard.py:7-13).
"""

from __future__ import annotations

from dataclasses import dataclass

from ..config.errors import ConfigError
from ..config.fields import get_bool, get_float, get_int, get_str
from ..config.plan import ModelPlan, PartSpec, RunEntry, pre_norm_layer
from ..config.registry import Architecture, register_architecture

NAME = "Qwen2ForCausalLM"


@dataclass(frozen=True)
class Qwen2Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    partial_rotary_factor: float
    tie_word_embeddings: bool
    attention_bias: bool
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    architecture: str = NAME

    @property
    def rotary_dim(self) -> int:
        """floor(head_dim * partial_rotary_factor) (recipes/schema.py:479-481)."""
        return int(self.head_dim * self.partial_rotary_factor)

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen2Config":
        hidden = get_int(raw, "hidden_size")
        nq = get_int(raw, "num_attention_heads")
        nkv = get_int(raw, "num_key_value_heads", nq)
        # head_dim is optional and defaults to hidden // heads (recipes/schema.py:139-140)
        hd = get_int(raw, "head_dim", hidden // nq)
        cfg = cls(
            hidden_size=hidden,
            num_hidden_layers=get_int(raw, "num_hidden_layers"),
            num_attention_heads=nq,
            num_key_value_heads=nkv,
            head_dim=hd,
            intermediate_size=get_int(raw, "intermediate_size"),
            vocab_size=get_int(raw, "vocab_size"),
            max_position_embeddings=get_int(raw, "max_position_embeddings"),
            rms_norm_eps=get_float(raw, "rms_norm_eps", 1e-6),        # recipes/schema.py:428
            rope_theta=get_float(raw, "rope_theta"),                   # no silent default
            partial_rotary_factor=get_float(raw, "partial_rotary_factor", 1.0),
            tie_word_embeddings=get_bool(raw, "tie_word_embeddings", False),  # recipes/schema.py:431
            attention_bias=get_bool(raw, "attention_bias", True),
            hidden_act=get_str(raw, "hidden_act", "silu"),
            torch_dtype=get_str(raw, "torch_dtype", "bfloat16"),
        )
        if nq % nkv:
            raise ConfigError(f"config.json: num_attention_heads={nq} must be a multiple of "
                              f"num_key_value_heads={nkv}")
        if cfg.hidden_act != "silu":                                   # recipes/schema.py:147
            raise ConfigError(f"config.json: hidden_act={cfg.hidden_act!r}; only 'silu' exists in this architecture")
        if not 0.0 < cfg.partial_rotary_factor <= 1.0:
            raise ConfigError("config.json: partial_rotary_factor must lie in (0, 1]")
        if cfg.rotary_dim < 2 or cfg.rotary_dim % 2:
            raise ConfigError(f"config.json: head_dim*partial_rotary_factor={cfg.rotary_dim} must be even and >= 2")
        if raw.get("use_sliding_window"):
            raise ConfigError("config.json: use_sliding_window=true: the architecture's reference path has no "
                              "window; refusing rather than ignoring it")
        if raw.get("rope_scaling") is not None:
            raise ConfigError("config.json: rope_scaling is set; only the default rotary type exists here")
        return cfg

    def to_dict(self) -> dict:
        return {
            "architectures": [self.architecture], "model_type": "qwen2",
            "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "partial_rotary_factor": self.partial_rotary_factor,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias, "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype, "use_sliding_window": False,
            "rope_scaling": None,
        }


def plan(cfg: Qwen2Config) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    position = PartSpec("rotary", {
        "theta": cfg.rope_theta, "rotary_dim": cfg.rotary_dim,
        "max_positions": cfg.max_position_embeddings,
    })
    mixer = PartSpec("attention", {
        "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
        "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
        "qkv_bias": cfg.attention_bias, "out_bias": False,
        "scale": cfg.head_dim ** -0.5,      # ref/standard.py:70
        "window": None,
    })
    ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size,
                              "intermediate_size": cfg.intermediate_size})
    layers = tuple(
        pre_norm_layer(f"model.layers.{i}", mixer, ffn, norm)
        for i in range(cfg.num_hidden_layers))
    p = ModelPlan(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding_name="model.embed_tokens.weight",
        layers=layers,
        run_list=tuple(RunEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm,
        final_norm_name="model.norm",
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        position=position,
        # a tied model may still carry a copy of the head; the embedding is used whenever the flag is set
        # (kernels/device_decode.py:127-128)
        ignored_names=("lm_head.weight",) if cfg.tie_word_embeddings else (),
    )
    p.validate()
    return p


def config_from_recipe(t: dict) -> dict:
    """config.json keys from a recipe's inline geometry, under the reference's key names
    (recipes/schema.py:357-431, 128-133, 86, 159-161): ``hidden_size``, ``num_layers``,
    ``full_attention.{num_heads, num_kv_heads, head_dim, rope.{theta, partial_rotary_factor}}``,
    ``mlp.{intermediate_size, hidden_act}``, ``vocab_size``, ``max_position_embeddings``,
    ``rms_norm_eps``, ``tie_word_embeddings``.  A missing key raises KeyError naming it."""
    fa, mlp = t["full_attention"], t["mlp"]
    cfg = {
        "architectures": [NAME], "model_type": "qwen2",
        "hidden_size": t["hidden_size"], "num_hidden_layers": t["num_layers"],
        "num_attention_heads": fa["num_heads"], "num_key_value_heads": fa["num_kv_heads"],
        "intermediate_size": mlp["intermediate_size"], "hidden_act": mlp.get("hidden_act", "silu"),
        "vocab_size": t["vocab_size"], "max_position_embeddings": t["max_position_embeddings"],
        "rms_norm_eps": float(t.get("rms_norm_eps", 1e-6)),
        "rope_theta": float(fa["rope"]["theta"]),
        "partial_rotary_factor": float(fa["rope"].get("partial_rotary_factor", 1.0)),
        "tie_word_embeddings": bool(t.get("tie_word_embeddings", False)),
    }
    if "head_dim" in fa:
        cfg["head_dim"] = fa["head_dim"]
    return cfg


register_architecture(Architecture(name=NAME, config_cls=Qwen2Config, plan=plan, aliases=("qwen2",),
                                   config_from_recipe=config_from_recipe), replace=True)
