"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a `PartSpec` (kind + parameters), states which tensors it
wants under which relative names, binds them, and computes.  No part knows
which model or layer it stands in.  Kinds are registered by name, so a test or
another architecture can add a mixer, feed-forward, norm, position encoding or
block arrangement without a change to these files.

Interfaces (all tensors are torch tensors on the engine's device):

``Norm``            ``add_norm(residual, delta) -> normed``: ``residual`` is the
                    float32 stream ``[T, H]``; if ``delta`` is given it is added
                    into ``residual`` in place first; the normed copy comes back
                    in the compute dtype.
``PositionEncoding`` owns what encodes positions: tables the mixers apply (rotary), or
                    ``on_embedding(residual, step)`` for encodings added to the input.
``Mixer``           ``forward(x, step, cache, position, write_cache) -> delta``:
                    ``x`` normed ``[T, H]``; ``step`` the batch description
                    (`StepContext`); ``cache`` the run's `LayerCache` (paged
                    keys/values, or per-request state slots, or None);
                    returns the ``[T, H]`` term to add to the residual stream.
                    ``cache_need()`` says what it wants of the cache manager.
``FeedForward``     ``forward(x, step) -> delta``.
                    A mixer or feed-forward whose class sets ``accepts_residual = True``
                    is also given ``residual=`` (the float32 stream) and may add its
                    term into it in place and return None.
``Block``           built from the dict of the layer's parts by role;
                    ``forward(residual, delta, step, cache, position, write_cache) -> delta``:
                    arranges norms, mixer and feed-forward around the residual stream; the
                    last term is handed on un-added, so that the next norm fuses
                    the addition.  ``cache_need()`` says what the layer wants of the
                    cache manager.  A block that sets ``accepts_next_norm = True`` is also
                    given ``next_norm=`` (the first norm of the layer that runs next) and may
                    hand on an `OwedNorm` made for it; it then exposes its own first norm as
                    ``first_norm``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

import torch


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part expects.  ``role`` drives random initialisation
    (matrix, bias, gain, embedding); optional tensors that only make sense
    together share a ``together`` key."""
    name: str
    shape: tuple
    role: str = "matrix"
    optional: bool = False
    together: str | None = None

    def prefixed(self, prefix: str) -> "TensorSpec":
        name = f"{prefix}.{self.name}" if prefix else self.name
        tg = f"{prefix}.{self.together}" if (prefix and self.together) else self.together
        return TensorSpec(name, self.shape, self.role, self.optional, tg)


# ---- what a mixer may ask of the cache manager ------------------------------

@dataclass(frozen=True)
class PagedKV:
    """Keys and values per token, in pages.  ``window``: only the last
    ``window`` positions are ever read again (None: all)."""
    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class SlotState:
    """A fixed-size float32 state per request, zeroed when the request starts."""
    shape: tuple


# ---- the batch a step runs --------------------------------------------------

@dataclass
class GroupView:
    """Per cache group: where this step's tokens go and what each request reads."""
    page_size: int
    block_tables: torch.Tensor      # int32 [S, max_pages]; -1 where no page is held
    slot_mapping: torch.Tensor      # int32 [T]; page*page_size+offset of each new token


@dataclass
class StepContext:
    """One batch: T tokens of S requests, each request's tokens consecutive.

    A request's portion may be any number of tokens (a prompt portion, or one
    decoded token); ``ctx_len`` counts its tokens in the cache after this step,
    so its portion covers positions ``ctx_len - q_len .. ctx_len - 1``.
    """
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor         # int32 [T]
    positions: torch.Tensor         # int32 [T]
    seq_of_token: torch.Tensor      # int32 [T]  batch-local request index
    q_start: torch.Tensor           # int32 [S+1] first token of each request, cumulative
    ctx_len: torch.Tensor           # int32 [S]
    state_slots: torch.Tensor       # int32 [S]  per-request state slot
    logit_rows: torch.Tensor        # int32 [R]  rows of the batch whose logits are wanted
    groups: list[GroupView]
    # host copies, for launch shapes
    q_lens: list[int] = field(default_factory=list)
    ctx_lens: list[int] = field(default_factory=list)
    max_q_len: int = 0
    max_ctx_len: int = 0
    attn_tiles: dict = field(default_factory=dict)   # scratch for ops: per-(group, rows) tile lists
    is_graph_replay: bool = False


@dataclass
class LayerCache:
    """What one run of a layer owns in the cache."""
    group: int | None = None            # index into StepContext.groups (paged)
    k: torch.Tensor | None = None       # [num_pages, nkv, page_size, hd]
    v: torch.Tensor | None = None
    state: torch.Tensor | None = None   # [num_slots, *shape] float32


# ---- a norm whose division is still owed --------------------------------------------

@dataclass
class OwedNorm:
    """What a norm would have returned, with the division by the root mean square still to do.

    A product that completes the residual stream can, in its own epilogue, write the next norm's input
    as ``x = compute_dtype(stream * gain)`` together with partial sums of squares of the stream's rows
    (``scale``, an `ops.RowScale`); the part that consumes the normed activations multiplies the rows of
    ITS product by the reciprocal root mean square, which is the same thing:
    W (x g / rms) = (W (x g)) / rms.  A decode step then needs no kernel for that norm.

    The protocol is optional on every side.  A mixer or feed-forward whose class sets
    ``accepts_next_norm = True`` is handed ``next_norm=`` (the `Norm` that will read the stream next, or None)
    and may return an `OwedNorm` made for it instead of None or a term; a norm offers itself through
    `Norm.as_rms()`.  A consumer that cannot take one calls `plain()`, which runs the norm as a kernel of
    its own on the (complete) stream."""
    x: torch.Tensor
    scale: object                       # ops.RowScale
    norm: "Norm"                        # the norm this stands for
    residual: torch.Tensor              # the stream it was made from

    def plain(self) -> torch.Tensor:
        return self.norm.add_norm(self.residual, None)


# ---- registries ---------------------------------------------------------------

class Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: dict[str, Callable] = {}

    def register(self, kind: str, *, replace: bool = False):
        def deco(cls):
            if kind in self._kinds and not replace:
                raise ValueError(f"{self.what} kind {kind!r} is already registered")
            self._kinds[kind] = cls
            return cls
        return deco

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def kinds(self) -> list[str]:
        return sorted(self._kinds)

    def get(self, kind: str):
        try:
            return self._kinds[kind]
        except KeyError:
            raise ValueError(f"unknown {self.what} kind {kind!r}; known: {self.kinds()}") from None

    def build(self, spec, **kw):
        return self.get(spec.kind)(spec.params, **kw)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block")


class Part:
    """Base of every part.  ``dtype`` is the compute dtype (bfloat16 or
    float32); matrices are held in it, gains and biases in float32."""

    def __init__(self, params: dict, *, dtype: torch.dtype, device):
        self.params = dict(params)
        self.dtype = dtype
        self.device = torch.device(device)

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def bind(self, fetch: Callable[[str], torch.Tensor | None]) -> None:
        """``fetch(relative_name)`` gives the stored CPU tensor or None."""

    # helpers ------------------------------------------------------------------
    def _matrix(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def _f32(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return 0


class Mixer(Part):
    def cache_need(self):
        return None

    def forward(self, x, step: StepContext, cache: LayerCache | None, position, write_cache: bool = True):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, step: StepContext):
        raise NotImplementedError


class Norm(Part):
    def add_norm(self, residual, delta):
        raise NotImplementedError

    def as_rms(self):
        """``(gain float32 [H], eps)`` if this norm is y = x * rsqrt(mean(x^2) + eps) * gain, so that a
        product's epilogue may prepare its input (`OwedNorm`); None otherwise."""
        return None


class PositionEncoding(Part):
    """Owns what encodes positions.  Mixers receive the object (rotary encodings expose ``table``
    and ``rotary_dim``, which the attention mixer applies to queries and keys); an encoding that
    acts on the input instead overrides `on_embedding`."""

    def on_embedding(self, residual, step: StepContext) -> None:
        """Called once per step on the float32 stream right after the embedding lookup."""
