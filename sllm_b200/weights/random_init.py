"""Random-weights mode: a model folder (config.json + model.safetensors) from a
configuration and a seed, for any registered architecture.

The reference's tiny fixture draws matrices N(0,1)*0.1, q/k/v biases *0.3 and
gains of one from ``default_rng(3)`` (serving/dev_model.py:158-185).  Here the
tensors are those the model itself says it expects, drawn in that order from
``numpy.random.default_rng(seed)``: matrices, biases and the embedding
N(0, std), gains 1 + N(0, gain_std).  Stored in bfloat16 unless asked otherwise
(values are rounded once, at writing; every reader then sees the same numbers).
"""

from __future__ import annotations

import json
import os

import numpy as np
import torch

from ..config.registry import architecture_of
from .safetensors_io import write_safetensors

_STORAGE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def random_tensors(specs, seed: int, *, std: float = 0.02, bias_std: float | None = None,
                   gain_std: float = 0.0, storage: str = "bfloat16", include_optional: bool = True) -> dict:
    rng = np.random.default_rng(seed)
    bias_std = std if bias_std is None else bias_std
    dt = _STORAGE[storage]
    out = {}
    for s in specs:
        if s.optional and not include_optional:
            continue
        if s.role == "gain":
            a = 1.0 + gain_std * rng.standard_normal(s.shape, dtype=np.float32) if gain_std else np.ones(s.shape, np.float32)
        elif s.role == "bias":
            a = bias_std * rng.standard_normal(s.shape, dtype=np.float32)
        else:
            a = std * rng.standard_normal(s.shape, dtype=np.float32)
        out[s.name] = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dt)
    return out


def write_random_model(model_dir: str, config: dict, seed: int, *, std: float = 0.02,
                       bias_std: float | None = None, gain_std: float = 0.0,
                       storage: str = "bfloat16", include_optional: bool = True) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a dict with
    config.json's keys, ``architectures`` included).  Returns the folder."""
    from ..models.causal_lm import CausalLM
    arch = architecture_of(config)
    cfg = arch.config_cls.from_dict(config)
    model = CausalLM(arch.plan(cfg), dtype=torch.float32, device="cpu")
    tensors = random_tensors(model.tensor_specs(), seed, std=std, bias_std=bias_std, gain_std=gain_std,
                             storage=storage, include_optional=include_optional)
    os.makedirs(model_dir, exist_ok=True)
    raw = dict(config)
    raw.setdefault("torch_dtype", storage)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(raw, f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed})
    return model_dir
