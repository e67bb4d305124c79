"""Recipes: a YAML file that names a model and how to launch it.

A subset of the reference's recipe schema (recipes/schema.py:298-469;
recipes/Qwen2.5-Coder-0.5B.yaml): ``model_id``, ``arch``, ``dtype``,
``paths.local_dir``, ``memory.kv_utilization`` and ``memory.kv_device_bytes``
(recipes/schema.py:236-277), ``defaults`` (``max_new``, ``max_num_seqs``,
``max_model_len``, ``block_size``, ``chunk_size``).  ``arch`` is any name or alias the
architecture registry knows; nothing here names one.  The model's geometry is read from
the folder's config.json; a recipe may carry it inline under ``text`` for the
random-weights mode, where no folder exists yet: the architecture itself turns that
mapping into config.json keys (`Architecture.config_from_recipe`).  Precedence of
settings: command line > recipe ``defaults`` > built-in (serving/main.py:287-308).
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field

from .errors import ConfigError

KNOWN_DTYPES = ("bfloat16", "float32")


@dataclass
class Recipe:
    name: str
    model_id: str
    arch: str
    dtype: str
    local_dir: str | None
    kv_utilization: float
    kv_device_bytes: int | None = None     # the cache's budget in bytes (None: what the device has left, times the utilisation)
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
        from .. import models  # noqa: F401  (the architectures this package ships register themselves)
        from .registry import get_architecture, known_architectures
        try:
            get_architecture(arch)
        except ConfigError:
            raise ConfigError(f"recipe: arch {arch!r} is not served by this engine; known: {known_architectures()} "
                              f"and their aliases") from None
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
        if mem.get("kv_placement", "device") != "device":
            raise ConfigError(f"recipe: memory.kv_placement={mem['kv_placement']!r}; this engine keeps the cache on the device")
        kv_bytes = mem.get("kv_device_bytes")
        if kv_bytes is not None and (isinstance(kv_bytes, bool) or not isinstance(kv_bytes, int) or kv_bytes < 1):
            raise ConfigError(f"recipe: memory.kv_device_bytes must be a positive integer, got {kv_bytes!r}")
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
                   kv_device_bytes=kv_bytes, defaults=defaults, text=text, path=path)

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

    def architecture(self):
        from .registry import get_architecture
        return get_architecture(self.arch)

    def config_json(self) -> dict:
        """config.json keys from the inline geometry under ``text``, as the recipe's architecture reads it."""
        if not self.text:
            raise ConfigError(f"recipe {self.name}: no inline geometry under 'text'")
        arch = self.architecture()
        if arch.config_from_recipe is None:
            raise ConfigError(f"recipe {self.name}: architecture {arch.name!r} reads no inline geometry; give a model folder")
        try:
            cfg = dict(arch.config_from_recipe(self.text))
        except KeyError as e:
            raise ConfigError(f"recipe {self.name}: inline geometry lacks key {e.args[0]!r}") from None
        cfg.setdefault("architectures", [arch.name])
        return cfg


def resolve_recipe(name_or_path: str, recipes_dir: str) -> Recipe:
    """A path, or a name under the recipes folder (serving/main.py:51-58)."""
    for cand in (name_or_path, os.path.join(recipes_dir, name_or_path),
                 os.path.join(recipes_dir, name_or_path + ".yaml")):
        if os.path.isfile(cand):
            return Recipe.from_yaml(cand)
    raise ConfigError(f"recipe {name_or_path!r} not found (looked in {recipes_dir})")
