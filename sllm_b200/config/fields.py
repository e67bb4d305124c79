"""Typed readers of config.json keys.  Each names the key in its error, in the
manner of the reference's recipe schema (recipes/schema.py:34-44)."""

from __future__ import annotations

from .errors import ConfigError

_MISSING = object()


def _get(raw: dict, key: str, default):
    if key in raw and raw[key] is not None:
        return raw[key]
    if default is _MISSING:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    return default


def get_int(raw: dict, key: str, default=_MISSING, *, minimum: int = 1) -> int:
    v = _get(raw, key, default)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: key {key!r} must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: key {key!r} must be >= {minimum}, got {v}")
    return v


def get_float(raw: dict, key: str, default=_MISSING, *, positive: bool = True) -> float:
    v = _get(raw, key, default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: key {key!r} must be a number, got {v!r}")
    v = float(v)
    if positive and not v > 0:
        raise ConfigError(f"config.json: key {key!r} must be > 0, got {v}")
    return v


def get_bool(raw: dict, key: str, default=_MISSING) -> bool:
    v = _get(raw, key, default)
    if not isinstance(v, bool):
        raise ConfigError(f"config.json: key {key!r} must be true or false, got {v!r}")
    return v


def get_str(raw: dict, key: str, default=_MISSING) -> str:
    v = _get(raw, key, default)
    if not isinstance(v, str):
        raise ConfigError(f"config.json: key {key!r} must be a string, got {v!r}")
    return v
