"""Architectures.  Importing this package registers each of them."""
from . import qwen2  # noqa: F401
from .causal_lm import CausalLM

__all__ = ["CausalLM", "qwen2"]
