"""The generic causal language model: embedding, a run list of blocks built from
a `ModelPlan`, a final norm and an output head.  It knows no architecture; the
plan decides which parts stand where and in which order they run.
"""

from __future__ import annotations

import torch

from .. import ops
from ..config.plan import ModelPlan
from ..parts import standard as _standard  # noqa: F401  (registers the standard parts)
from ..parts.base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS,
                          LayerCache, OwedNorm, StepContext, TensorSpec)


FAMILIES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS}


class Layer:
    """The parts a `LayerSpec` names, built, and the block that arranges them.  The block receives
    them by role and says what the layer wants of the cache manager."""

    def __init__(self, spec, *, dtype, device):
        self.spec = spec
        self.parts = {role: FAMILIES[e.family].build(e.spec, dtype=dtype, device=device) for role, e in spec.parts.items()}
        self.block = BLOCKS.get(spec.block)(self.parts)

    @property
    def mixer(self):
        return self.parts.get("mixer")

    def cache_need(self):
        return self.block.cache_need()

    def named_parts(self):
        s = self.spec
        return [(f"{s.prefix}.{e.name}" if e.name else s.prefix, self.parts[role]) for role, e in s.parts.items()]


class CausalLM:
    def __init__(self, plan: ModelPlan, *, dtype: torch.dtype, device):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype must be bfloat16 or float32, got {dtype}")
        plan.validate()
        self.plan = plan
        self.dtype = dtype
        self.device = torch.device(device)
        kw = dict(dtype=dtype, device=self.device)
        self.layers = [Layer(s, **kw) for s in plan.layers]
        self.final_norm = NORMS.build(plan.final_norm, **kw)
        self.position = POSITIONS.build(plan.position, **kw) if plan.position is not None else None
        self.embedding = None      # [V, H] compute dtype
        self.head = None           # [V, H] compute dtype (the embedding itself when tied)

    # ---- weights ---------------------------------------------------------------
    def _named_parts(self):
        out = []
        for layer in self.layers:
            out.extend(layer.named_parts())
        out.append((self.plan.final_norm_name, self.final_norm))
        if self.position is not None and self.plan.position_name:
            out.append((self.plan.position_name, self.position))
        return out

    def tensor_specs(self) -> list[TensorSpec]:
        p = self.plan
        specs = [TensorSpec(p.embedding_name, (p.vocab_size, p.hidden_size), role="embedding")]
        for prefix, part in self._named_parts():
            specs.extend(s.prefixed(prefix) for s in part.tensor_specs())
        if p.head_name is not None:
            specs.append(TensorSpec(p.head_name, (p.vocab_size, p.hidden_size), role="matrix"))
        return specs

    def ignored_tensor_names(self):
        """Tensors a checkpoint may carry that this model does not use (the plan names them)."""
        return list(self.plan.ignored_names)

    def bind(self, fetch) -> None:
        p = self.plan
        self.embedding = fetch(p.embedding_name).to(device=self.device, dtype=self.dtype).contiguous()
        for prefix, part in self._named_parts():
            part.bind(lambda rel, _p=prefix: fetch(f"{_p}.{rel}"))
        if p.head_name is None:
            self.head = self.embedding
        else:
            self.head = fetch(p.head_name).to(device=self.device, dtype=self.dtype).contiguous()

    def weight_bytes(self) -> int:
        """Bytes of every tensor a decode step reads once (the head counts once
        more when it is the embedding table: the step reads it whole as the head
        and only single rows of it as the embedding)."""
        n = self.head.numel() * self.head.element_size()
        for _, part in self._named_parts():
            n += part.weight_bytes()
        return n

    # ---- cache needs ----------------------------------------------------------------
    def cache_needs(self):
        """One entry per run of the run list: the mixer's need, or the index of
        the run whose cache it borrows."""
        out = []
        for e in self.plan.run_list:
            if e.cache_from is not None:
                out.append(("borrow", e.cache_from))
            else:
                out.append(("own", self.layers[e.layer].cache_need()))
        return out

    # ---- forward ------------------------------------------------------------------
    def forward(self, step: StepContext, caches: list[LayerCache]) -> torch.Tensor:
        """Run the batch's tokens through every entry of the run list and return
        float32 logits ``[R, V]`` at ``step.logit_rows``."""
        residual = ops.embed_gather(self.embedding, step.token_ids)       # [T, H] float32
        if self.position is not None:
            self.position.on_embedding(residual, step)
        delta = None
        runs = self.plan.run_list
        for i, e in enumerate(runs):
            block = self.layers[e.layer].block
            kw = {}
            if getattr(block, "accepts_next_norm", False) and i + 1 < len(runs):
                # the norm that reads the stream next: this block's last product may prepare its input
                kw["next_norm"] = getattr(self.layers[runs[i + 1].layer].block, "first_norm", None)
            delta = block.forward(residual, delta, step, caches[i], self.position, write_cache=e.cache_from is None, **kw)
        if isinstance(delta, OwedNorm):          # (a block handed one on although nothing asked: take the stream as it is)
            delta = None
        if step.logit_rows.numel() == 0:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=self.device)
        res_rows = ops.gather_rows(residual, step.logit_rows)
        delta_rows = ops.gather_rows(delta, step.logit_rows) if delta is not None else None
        x = self.final_norm.add_norm(res_rows, delta_rows)
        return ops.linear(x, self.head, None, torch.float32)
