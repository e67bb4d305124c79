"""The parts the Qwen2.5 dense architecture is made of: RMSNorm, rotate-half
rotary tables, GQA attention over the paged cache, SwiGLU, and the pre-norm
block.  Each takes its sizes and constants as parameters; none names a model.

All arithmetic runs in the hand-written kernels behind `sllm_b200.ops`.
"""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, FeedForward,
                   LayerCache, Mixer, Norm, OwedNorm, PagedKV, Part, PositionEncoding,
                   StepContext, TensorSpec)


class Linear:
    """y = x W^T (+ b); W is (out, in) row-major as checkpoints store it
    (ref/qwen3_5.py:59-64).  The matrix is held in the compute dtype, the bias
    in float32."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None):
        self.weight = weight
        self.bias = bias

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype, allow_partials: bool = False) -> torch.Tensor:
        """``allow_partials``: the caller's consumer adds a stack ``[parts, T, N]`` of float32
        partial sums (the fused add + norm and the rotary kernel do), so a product of few
        rows may split its k dimension over more SMs."""
        return ops.linear(x, self.weight, self.bias, out_dtype, allow_partials)

    def into(self, x: torch.Tensor, residual: torch.Tensor | None, next_norm=None):
        """The layer's term for the residual stream: added into ``residual`` in place where a
        kernel does that (returns None), else returned for the next norm to add.  Where the kernel
        that completes the stream can also prepare the input of ``next_norm`` (the norm that reads the
        stream next), that input comes back as an `OwedNorm`."""
        if residual is not None and ops.can_accumulate(x, self.weight):
            rms = next_norm.as_rms() if next_norm is not None else None
            if rms is not None and ops.can_accumulate_norm(x, self.weight):
                xg, scale = ops.linear_accumulate_norm(x, self.weight, self.bias, residual, *rms)
                return OwedNorm(xg, scale, next_norm, residual)
            ops.linear_accumulate(x, self.weight, self.bias, residual)
            return None
        return ops.linear(x, self.weight, self.bias, torch.float32, True)

    def nbytes(self) -> int:
        n = self.weight.numel() * self.weight.element_size()
        if self.bias is not None:
            n += self.bias.numel() * 4
        return n


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """y = x * (mean(x^2) + eps)^-1/2 * w with plain gain w, computed in float32
    on the float32 residual stream (ref/standard.py:25-31).  Fused with the
    addition that precedes it, as the reference's device path does
    (kernels/cuda/kernels.cu:791-839)."""

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec("weight", (self.size,), role="gain")]

    def bind(self, fetch):
        self.weight = self._f32(fetch("weight"))

    def add_norm(self, residual, delta):
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.dtype)

    def as_rms(self):
        return (self.weight, self.eps) if self.dtype == torch.bfloat16 else None

    def weight_bytes(self):
        return self.size * 4


@POSITIONS.register("rotary")
class Rotary(PositionEncoding):
    """Rotate-half rotary encoding over the first ``rotary_dim`` dims of a head:
    angle(pos, j) = pos * theta^(-2j/rot), j < rot/2 (ref/qwen3_5.py:343-352).
    The table of cos and sin is computed once in float64 and stored in float32,
    ``[max_positions, rot/2]`` each."""

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.theta = float(params["theta"])
        self.rotary_dim = int(params["rotary_dim"])
        self.max_positions = int(params["max_positions"])
        half = self.rotary_dim // 2
        inv_freq = 1.0 / (self.theta ** (np.arange(0, self.rotary_dim, 2, dtype=np.float64) / self.rotary_dim))
        ang = np.arange(self.max_positions, dtype=np.float64)[:, None] * inv_freq[None, :]
        table = np.stack([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)   # [P, 2, half]
        assert table.shape == (self.max_positions, 2, half)
        self.table = torch.from_numpy(table).to(self.device).contiguous()


@MIXERS.register("attention")
class Attention(Mixer):
    """Grouped-query attention over a paged cache.

    q = xWq^T+bq, k, v likewise (biases optional); q and k rotated; k (after
    bias and rotation) and v (after bias) written to the cache before any read;
    query head h reads kv head h // (nq/nkv); scores scaled, causal (and an
    optional window), softmax in float32; heads merged; o_proj without bias
    unless asked (ref/standard.py:34-72; cache content ref/incremental.py:135-139).
    q|k|v are one matrix, as the reference's device path fuses them
    (kernels/device_decode.py:84-87).
    """

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nq = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.out_bias = bool(p.get("out_bias", False))
        self.scale = float(p.get("scale", self.hd ** -0.5))
        self.window = p.get("window")
        self.names = p.get("names", ("q_proj", "k_proj", "v_proj", "o_proj"))
        if self.nq % self.nkv:
            raise ValueError(f"attention: {self.nq} query heads are no multiple of {self.nkv} kv heads")
        if not 1 <= self.hd <= self.MAX_HEAD_DIM:
            # said when the model is built, not at the first step: the attention kernels keep a head in
            # registers and shared memory (tensor-core forms 16..128, the CUDA-core form up to 256)
            raise ValueError(f"attention: head_dim={self.hd} is outside 1..{self.MAX_HEAD_DIM}, the largest head the "
                             f"attention kernels take")
        self.qkv = None
        self.out = None

    def cache_need(self):
        return PagedKV(self.nkv, self.hd, self.window)

    def tensor_specs(self):
        nq, nk, h = self.nq * self.hd, self.nkv * self.hd, self.hidden
        qn, kn, vn, on = self.names
        specs = [TensorSpec(f"{qn}.weight", (nq, h)), TensorSpec(f"{kn}.weight", (nk, h)),
                 TensorSpec(f"{vn}.weight", (nk, h)), TensorSpec(f"{on}.weight", (h, nq))]
        if self.qkv_bias:
            # present or absent as a set, decided by the checkpoint (ref/standard.py:114-116)
            specs += [TensorSpec(f"{n}.bias", (s,), role="bias", optional=True, together="qkv_bias")
                      for n, s in ((qn, nq), (kn, nk), (vn, nk))]
        if self.out_bias:
            specs.append(TensorSpec(f"{on}.bias", (h,), role="bias"))
        return specs

    def bind(self, fetch):
        qn, kn, vn, on = self.names
        w = torch.cat([fetch(f"{n}.weight") for n in (qn, kn, vn)], dim=0)
        bias = None
        if self.qkv_bias and fetch(f"{qn}.bias") is not None:
            bias = self._f32(torch.cat([fetch(f"{n}.bias").float() for n in (qn, kn, vn)]))
        self.qkv = Linear(self._matrix(w))
        self.qkv_b = bias                       # added in the rotary kernel, before rotation
        ob = self._f32(fetch(f"{on}.bias")) if self.out_bias else None
        self.out = Linear(self._matrix(fetch(f"{on}.weight")), ob)

    accepts_residual = True
    accepts_next_norm = True
    MAX_HEAD_DIM = 256

    def forward(self, x, step: StepContext, cache: LayerCache, position, write_cache=True, residual=None, next_norm=None):
        g = step.groups[cache.group]
        table = getattr(position, "table", None)           # an encoding without a rotary table: no rotation
        rot = getattr(position, "rotary_dim", 0) if table is not None else 0
        slots = g.slot_mapping if write_cache else None
        owed = x if isinstance(x, OwedNorm) else None
        fused = owed is not None and ops.qkv_rope_supports(owed.x, self.qkv.weight, table, rot, self.nq, self.nkv, self.hd, cache.k)
        if owed is not None and not fused and not ops.linear_scaled_supports(owed.x, self.qkv.weight):
            x, owed = owed.plain(), None
        if owed is not None and fused:
            q = ops.linear_rope_kv_write(owed.x, self.qkv.weight, self.qkv_b, step.positions, table, rot,
                                         self.nq, self.nkv, self.hd, slots, cache.k, cache.v, scale=owed.scale)
        elif owed is not None:
            # a prompt portion: the product pays the owed division in its epilogue, the rotary kernel follows
            qkv = ops.linear(owed.x, self.qkv.weight, None, torch.float32, scale=owed.scale)
            q = ops.rope_kv_write(qkv, self.qkv_b, step.positions, table, rot, self.nq, self.nkv, self.hd,
                                  slots, cache.k, cache.v, self.dtype)
        elif ops.qkv_rope_supports(x, self.qkv.weight, table, rot, self.nq, self.nkv, self.hd, cache.k):
            # few tokens: bias, rotation and the cache write happen as the product's rows leave their CTA
            q = ops.linear_rope_kv_write(x, self.qkv.weight, self.qkv_b, step.positions, table, rot,
                                         self.nq, self.nkv, self.hd, slots, cache.k, cache.v)
        else:
            qkv = self.qkv(x, torch.float32, True)            # [T, (nq+2nkv)*hd] float32, maybe in parts
            q = ops.rope_kv_write(qkv, self.qkv_b, step.positions, table, rot, self.nq, self.nkv, self.hd,
                                  slots, cache.k, cache.v, self.dtype)
        o = ops.paged_attention(q, cache.k, cache.v, step, cache.group,
                                self.nq, self.nkv, self.hd, self.scale, self.window)
        return self.out.into(o, residual, next_norm)

    def weight_bytes(self):
        return self.qkv.nbytes() + self.out.nbytes() + (self.qkv_b.numel() * 4 if self.qkv_b is not None else 0)


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """down(silu(gate(x)) * up(x)), silu(z) = z/(1+e^-z), no biases
    (ref/qwen3_5.py:28-29, 444-451).  gate and up are one matrix
    (kernels/device_decode.py:93-95); their rows alternate in blocks of
    ``interleave`` so that a tile of the product holds a gate row and its up
    row together and the activation can be applied where the tile is made."""

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.names = params.get("names", ("gate_proj", "up_proj", "down_proj"))
        self.interleave = 8 if self.inter % 8 == 0 else self.inter
        self.gate_up = None
        self.down = None

    def tensor_specs(self):
        g, u, d = self.names
        return [TensorSpec(f"{g}.weight", (self.inter, self.hidden)),
                TensorSpec(f"{u}.weight", (self.inter, self.hidden)),
                TensorSpec(f"{d}.weight", (self.hidden, self.inter))]

    def bind(self, fetch):
        g, u, d = self.names
        b = self.interleave
        wg = fetch(f"{g}.weight").reshape(self.inter // b, b, self.hidden)
        wu = fetch(f"{u}.weight").reshape(self.inter // b, b, self.hidden)
        gu = torch.stack([wg, wu], dim=1).reshape(2 * self.inter, self.hidden)
        self.gate_up = Linear(self._matrix(gu))
        self.down = Linear(self._matrix(fetch(f"{d}.weight")))

    accepts_residual = True
    accepts_next_norm = True

    def forward(self, x, step, residual=None, next_norm=None):
        if isinstance(x, OwedNorm):
            if ops.silu_scaled_supports(x.x, self.gate_up.weight, self.interleave, self.dtype):
                act = ops.linear_silu_mul(x.x, self.gate_up.weight, self.interleave, self.dtype, scale=x.scale)
                return self.down.into(act, residual, next_norm)
            x = x.plain()
        act = ops.linear_silu_mul(x, self.gate_up.weight, self.interleave, self.dtype)   # [T, I]
        return self.down.into(act, residual, next_norm)

    def weight_bytes(self):
        return self.gate_up.nbytes() + self.down.nbytes()


@BLOCKS.register("pre_norm")
class PreNormBlock:
    """h += mixer(norm1(h)); h += ffn(norm2(h)) (ref/standard.py:102-129).  The
    addition of each term is done by the norm that follows it, so the block
    takes the pending term of the layer before and hands its own on."""

    ROLES = ("mixer", "ffn", "mixer_norm", "ffn_norm")

    def __init__(self, parts: dict):
        if set(parts) != set(self.ROLES):
            raise ValueError(f"the pre-norm block arranges {self.ROLES}; the layer names {sorted(parts)}")
        self.mixer, self.ffn = parts["mixer"], parts["ffn"]
        self.mixer_norm, self.ffn_norm = parts["mixer_norm"], parts["ffn_norm"]

    def cache_need(self):
        return self.mixer.cache_need()

    accepts_next_norm = True

    @property
    def first_norm(self):
        return self.mixer_norm

    @staticmethod
    def _call(part, *args, residual, next_norm):
        """A part is told what it says it understands: the stream to add into, the norm that reads it next."""
        kw = {}
        if getattr(part, "accepts_residual", False):
            kw["residual"] = residual
            if getattr(part, "accepts_next_norm", False):
                kw["next_norm"] = next_norm       # (only a part that completes the stream itself can prepare it)
        return part.forward(*args, **kw)

    def _normed(self, norm, residual, delta):
        """The input of the part behind ``norm``: an `OwedNorm` made for this very norm as it is (a part
        that cannot take it asks for the plain form itself), anything else through the norm's kernel."""
        if isinstance(delta, OwedNorm):
            return delta if delta.norm is norm else norm.add_norm(residual, None)
        return norm.add_norm(residual, delta)

    def forward(self, residual, delta, step, cache, position, write_cache=True, next_norm=None):
        x = self._normed(self.mixer_norm, residual, delta)
        if isinstance(x, OwedNorm) and not getattr(self.mixer, "accepts_next_norm", False):
            x = x.plain()
        d = self._call(self.mixer, x, step, cache, position, write_cache, residual=residual, next_norm=self.ffn_norm)
        x = self._normed(self.ffn_norm, residual, d)
        if isinstance(x, OwedNorm) and not getattr(self.ffn, "accepts_next_norm", False):
            x = x.plain()
        return self._call(self.ffn, x, step, residual=residual, next_norm=next_norm)
