"""Recipes: a YAML file that names a model and how to launch it.

A subset of the reference's recipe schema (recipes/schema.py:298-469;
recipes/Qwen2.5-Coder-0.5B.yaml): ``model_id``, ``arch``, ``dtype``,
``paths.local_dir``, ``memory.kv_utilization``, ``defaults`` (``max_new``,
``max_num_seqs``, ``max_model_len``, ``block_size``, ``chunk_size``).  The model's
geometry is read from the folder's config.json; a recipe may carry it inline under
``text`` (the reference's key names) for the random-weights mode, where no folder
exists yet.  Precedence of settings: command line > recipe ``defaults`` >
built-in (serving/main.py:287-308).
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field

from .errors import ConfigError

KNOWN_ARCHS = ("qwen2",)
KNOWN_DTYPES = ("bfloat16", "float32")


@dataclass
class Recipe:
    name: str
    model_id: str
    arch: str
    dtype: str
    local_dir: str | None
    kv_utilization: float
    defaults: dict = field(default_factory=dict)
    text: dict | None = None
    path: str | None = None

    @classmethod
    def from_dict(cls, raw: dict, path: str | None = None) -> "Recipe":
        if not isinstance(raw, dict):
            raise ConfigError("recipe: expected a mapping at the top level")

        def need(key):
            if key not in raw:
                raise ConfigError(f"recipe: required key {key!r} is missing")
            return raw[key]

        arch = str(need("arch"))
        if arch not in KNOWN_ARCHS:
            raise ConfigError(f"recipe: arch {arch!r} is not served by this engine; known: {list(KNOWN_ARCHS)}")
        dtype = str(raw.get("dtype", "bfloat16"))
        if dtype not in KNOWN_DTYPES:
            raise ConfigError(f"recipe: dtype {dtype!r}; known: {list(KNOWN_DTYPES)}")
        tp = (raw.get("tp") or {}).get("size", 1)
        if tp != 1:
            raise ConfigError(f"recipe: tp.size={tp}; this engine runs on one GPU")
        mem = raw.get("memory") or {}
        util = float(mem.get("kv_utilization", (raw.get("defaults") or {}).get("kv_utilization", 0.9)))
        if not 0.0 < util <= 1.0:
            raise ConfigError("recipe: memory.kv_utilization must lie in (0, 1]")
        local = (raw.get("paths") or {}).get("local_dir")
        defaults = dict(raw.get("defaults") or {})
        for k in ("max_new", "max_num_seqs", "max_model_len", "block_size", "chunk_size"):
            if k in defaults and (isinstance(defaults[k], bool) or not isinstance(defaults[k], int) or defaults[k] < 1):
                raise ConfigError(f"recipe: defaults.{k} must be a positive integer, got {defaults[k]!r}")
        text = raw.get("text")
        if text is not None and not isinstance(text, dict):
            raise ConfigError("recipe: text must be a mapping")
        return cls(name=str(raw.get("name") or need("model_id")), model_id=str(need("model_id")), arch=arch,
                   dtype=dtype, local_dir=os.path.expanduser(local) if local else None, kv_utilization=util,
                   defaults=defaults, text=text, path=path)

    @classmethod
    def from_yaml(cls, path: str) -> "Recipe":
        import yaml
        try:
            with open(path) as f:
                raw = yaml.safe_load(f)
        except FileNotFoundError:
            raise ConfigError(f"recipe {path}: not found") from None
        except yaml.YAMLError as e:
            raise ConfigError(f"recipe {path}: not valid YAML ({e})") from None
        return cls.from_dict(raw, path)

    def config_json(self) -> dict:
        """config.json keys from the inline geometry (the reference's ``text`` keys:
        recipes/schema.py:357-431, 128-133, 86, 159-161)."""
        t = self.text
        if not t:
            raise ConfigError(f"recipe {self.name}: no inline geometry under 'text'")
        try:
            fa, mlp = t["full_attention"], t["mlp"]
            cfg = {
                "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
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
        except KeyError as e:
            raise ConfigError(f"recipe {self.name}: inline geometry lacks key {e.args[0]!r}") from None
        return cfg


def resolve_recipe(name_or_path: str, recipes_dir: str) -> Recipe:
    """A path, or a name under the recipes folder (serving/main.py:51-58)."""
    for cand in (name_or_path, os.path.join(recipes_dir, name_or_path),
                 os.path.join(recipes_dir, name_or_path + ".yaml")):
        if os.path.isfile(cand):
            return Recipe.from_yaml(cand)
    raise ConfigError(f"recipe {name_or_path!r} not found (looked in {recipes_dir})")
