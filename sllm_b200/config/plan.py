"""The description of a model as data: which parts stand in which layer, under
which tensor names, and in which order the layers run.

An architecture turns its typed configuration into a `ModelPlan`; the generic
model class builds itself from the plan alone.  Nothing here names a concrete
architecture.  Every size and constant a part needs travels in its
`PartSpec.params`, taken from the configuration.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind and the parameters it is built with."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class PartEntry:
    """One part of a layer: the registry its kind is looked up in (``"mixer"``,
    ``"feed_forward"`` or ``"norm"``), what it is built with, and the tensor-name prefix
    below the layer's under which its tensors lie (empty: directly under the layer's)."""
    family: str
    spec: PartSpec
    name: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement and the parts it arranges, by role.

    Which roles there are is the block kind's business: the pre-norm block asks for
    ``mixer``, ``ffn``, ``mixer_norm`` and ``ffn_norm`` (see `pre_norm_layer`); another
    arrangement may ask for four norms of different kinds, or for no feed-forward.
    `prefix` is the layer's tensor-name prefix (``model.layers.3``).  Layers of one
    model may differ in every field.
    """
    prefix: str
    parts: dict[str, PartEntry]
    block: str = "pre_norm"

    def part(self, role: str) -> PartSpec:
        return self.parts[role].spec


def pre_norm_layer(prefix: str, mixer: PartSpec, ffn: PartSpec, norm: PartSpec, *, ffn_norm: PartSpec | None = None,
                   block: str = "pre_norm", mixer_name: str = "self_attn", ffn_name: str = "mlp",
                   mixer_norm_name: str = "input_layernorm", ffn_norm_name: str = "post_attention_layernorm") -> LayerSpec:
    """The common layer: a mixer and a feed-forward, each behind a norm of its own."""
    return LayerSpec(prefix=prefix, block=block, parts={
        "mixer_norm": PartEntry("norm", norm, mixer_norm_name),
        "mixer": PartEntry("mixer", mixer, mixer_name),
        "ffn_norm": PartEntry("norm", ffn_norm or norm, ffn_norm_name),
        "ffn": PartEntry("feed_forward", ffn, ffn_name),
    })


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run list: run layer `layer` here.

    `cache_from` is None when the run owns a cache of its own, or the index of
    an earlier entry of the run list whose cache this run reads (it then writes
    none).  A layer may be named by several entries; each owns its cache unless
    it borrows one.
    """
    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding_name: str
    layers: tuple[LayerSpec, ...]
    run_list: tuple[RunEntry, ...]
    final_norm: PartSpec
    final_norm_name: str
    head_name: str | None          # None: the head is the embedding table (tied)
    position: PartSpec | None      # the position encoding the mixers share
    position_name: str | None = None   # prefix of the position encoding's own tensors, if it has any
    ignored_names: tuple[str, ...] = ()  # tensors a checkpoint may carry that the model does not use (said once, in a warning)

    def validate(self) -> None:
        from .errors import ConfigError
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for i, layer in enumerate(self.layers):
            for role, e in layer.parts.items():
                if e.family not in ("mixer", "feed_forward", "norm"):
                    raise ConfigError(f"layers[{i}].parts[{role!r}]: unknown family {e.family!r} "
                                      f"(mixer, feed_forward or norm)")
        for i, e in enumerate(self.run_list):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"run_list[{i}] names layer {e.layer}, "
                                  f"the model has {len(self.layers)}")
            if e.cache_from is not None:
                if not 0 <= e.cache_from < i:
                    raise ConfigError(f"run_list[{i}].cache_from={e.cache_from} must name an earlier entry")
                if self.run_list[e.cache_from].cache_from is not None:
                    raise ConfigError(f"run_list[{i}].cache_from={e.cache_from} names an entry that borrows too")
