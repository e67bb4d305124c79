"""One registry from an architecture's name (config.json ``architectures[0]``)
to its typed configuration class and its plan function.

The reference picks its engine by an if-chain over ``recipe.arch``
(serving/main.py:196-247) and a list of known names (recipes/schema.py:28);
here a name maps to data, and a new architecture registers itself without a
change to this file.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable

from .errors import ConfigError
from .plan import ModelPlan


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type                       # has classmethod from_dict(dict)
    plan: Callable[[object], ModelPlan]    # typed config -> plan
    random_init: Callable | None = None    # (config, plan) -> per-tensor init rules; None: defaults
    aliases: tuple[str, ...] = ()          # short names a recipe's ``arch:`` may use
    # a recipe's inline geometry (its ``text`` mapping) -> config.json keys, for the random-weights mode
    # where no model folder exists yet; None: the architecture cannot be described inline
    config_from_recipe: Callable[[dict], dict] | None = None


_ARCHITECTURES: dict[str, Architecture] = {}
_ALIASES: dict[str, str] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch
    for a in arch.aliases:
        _ALIASES[a] = arch.name


def unregister_architecture(name: str) -> None:
    arch = _ARCHITECTURES.pop(name, None)
    if arch:
        for a in arch.aliases:
            _ALIASES.pop(a, None)


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    name = _ALIASES.get(name, name)
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture {name!r}; known: {known_architectures()}") from None


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path) as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: not found") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return raw


def architecture_of(raw: dict) -> Architecture:
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: key 'architectures' must be a non-empty list of names")
    return get_architecture(archs[0])


def load_config(model_dir: str):
    """(architecture, typed config) of a model folder."""
    raw = read_config_json(model_dir)
    arch = architecture_of(raw)
    return arch, arch.config_cls.from_dict(raw)
