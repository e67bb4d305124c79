"""From a model folder to a model on the device: config.json chooses the
architecture through the registry, the plan builds the parts, the loader binds
the folder's tensors by name."""

from __future__ import annotations

import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..config.registry import load_config
from ..models.causal_lm import CausalLM
from ..weights.loader import load_into

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {name!r}") from None


def build_model(model_dir: str, dtype="bfloat16", device="cuda:0", *, progress=None):
    """(model, typed config) of the folder, weights bound."""
    arch, cfg = load_config(model_dir)
    model = CausalLM(arch.plan(cfg), dtype=parse_dtype(dtype), device=device)
    load_into(model, model_dir, progress=progress)
    return model, cfg
