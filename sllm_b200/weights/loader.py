"""Bind a model folder's tensors to a model by name.

The reference looks each tensor up in a flat dict and finds a missing one as a
bare KeyError in mid-forward (ref/standard.py:95-134; loaders/weights.py:44-108).
Here the model states what it expects (name, shape, whether optional), the folder
states what it has, and every disagreement is reported at once in one
`WeightError`: missing names, unexpected names and wrong shapes.
"""

from __future__ import annotations

import json
import os
import warnings
from typing import Iterable

import torch

from ..parts.base import TensorSpec
from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """The folder's tensors do not fit the model.  Lists all faults at once."""

    def __init__(self, model_dir: str, missing=(), unexpected=(), wrong_shape=(), other=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)      # (name, expected, found)
        self.other = list(other)
        lines = [f"weights in {model_dir} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, exp, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name}: expected {tuple(exp)}, found {tuple(got)}")
        lines.extend(f"  {o}" for o in self.other)
        super().__init__("\n".join(lines))


class TensorSource:
    """All tensors of a model folder: ``model.safetensors``, or the shards that
    ``model.safetensors.index.json`` names, or every ``*.safetensors`` sorted."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        if os.path.isfile(index):
            with open(index) as f:
                shards = sorted(set(json.load(f)["weight_map"].values()))
        elif os.path.isfile(single):
            shards = ["model.safetensors"]
        else:
            shards = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors")) \
                if os.path.isdir(model_dir) else []
        if not shards:
            raise WeightError(model_dir, other=["no *.safetensors file found"])
        self.files = []
        self.where: dict[str, SafetensorsFile] = {}
        for s in shards:
            try:
                f = SafetensorsFile(os.path.join(model_dir, s))
            except (SafetensorsError, OSError) as e:
                raise WeightError(model_dir, other=[str(e)]) from None
            self.files.append(f)
            for n in f.names():
                self.where[n] = f

    def names(self) -> list[str]:
        return list(self.where)

    def shape_of(self, name: str):
        return self.where[name].shape_of(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self.where[name].tensor(name)


def check(source: TensorSource, specs: Iterable[TensorSpec], *, ignore: Iterable[str] = ()) -> None:
    """Raise one WeightError naming every missing, unexpected and mis-shaped tensor."""
    specs = list(specs)
    have = set(source.names())
    want = {s.name: s for s in specs}
    missing = [s.name for s in specs if not s.optional and s.name not in have]
    unexpected = sorted(have - set(want) - set(ignore))
    wrong = [(n, want[n].shape, source.shape_of(n)) for n in want
             if n in have and tuple(source.shape_of(n)) != tuple(want[n].shape)]
    other = []
    # optional tensors that belong together must come together
    groups: dict[str, list[TensorSpec]] = {}
    for s in specs:
        if s.optional and s.together:
            groups.setdefault(s.together, []).append(s)
    for key, members in groups.items():
        present = [m.name for m in members if m.name in have]
        if present and len(present) != len(members):
            absent = [m.name for m in members if m.name not in have]
            other.append(f"incomplete optional set {key}: has {present}, lacks {absent}")
    if missing or unexpected or wrong or other:
        raise WeightError(source.model_dir, missing, unexpected, wrong, other)


def load_into(model, model_dir: str, *, progress=None) -> None:
    """Check the folder against ``model.tensor_specs()`` and bind every tensor."""
    source = TensorSource(model_dir)
    specs = model.tensor_specs()
    ignored = list(model.ignored_tensor_names())
    check(source, specs, ignore=ignored)
    have = set(source.names())
    unused = sorted(have & set(ignored))
    if unused:
        warnings.warn(f"{model_dir}: {', '.join(unused)} is in the checkpoint and not used by this model "
                      f"(a tied output head reads the embedding table)", stacklevel=2)
    total = sum(1 for s in specs if s.name in have)
    done = 0

    def fetch(name: str):
        nonlocal done
        if name not in have:
            return None
        done += 1
        if progress and (done in (1, total) or done % 200 == 0):
            progress(done, total)
        return source.tensor(name)

    model.bind(fetch)
