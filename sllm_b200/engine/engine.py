"""The step function: one batch of (request, its next tokens) through the model,
from the cache, returning logits at the wanted places.

The reference runs every scheduled action as a forward of its own and treats
prompt chunks after the first as bookkeeping (serving/executor.py:1041-1080).
Here a step is one forward over all tokens it is given: prompt portions of any
length beside single decoded tokens, each request's keys and values written to
its pages before attention reads them.  Generation, the scheduler and trace
replay all go through `Engine.step`.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pools import OutOfPages
from ..parts.base import StepContext
from .batch import BatchLayout, context, pack, pages_missing


@dataclass
class StepEntry:
    req_id: object
    tokens: list
    want: list = field(default_factory=list)     # places among `tokens` whose logits are wanted


class ContextOverflow(ValueError):
    """A request would grow past the model's position limit."""


class Engine:
    def __init__(self, model, *, page_size: int = 16, num_pages: int, max_requests: int = 8,
                 max_model_len: int | None = None, poison_freed: bool | None = None):
        """``poison_freed``: the cache manager's debugging aid (pages that go back to the pool are filled
        with NaN); None reads ``SLLM_POISON_FREED_PAGES=1`` from the environment."""
        self.model = model
        self.device = model.device
        if poison_freed is None:
            poison_freed = os.environ.get("SLLM_POISON_FREED_PAGES", "0") == "1"
        self.cache = CacheManager(model.cache_needs(), page_size=page_size, num_pages=num_pages,
                                  max_requests=max_requests, poison_freed=poison_freed)
        self.layer_caches = self.cache.allocate_storage(model.dtype, self.device)
        self.vocab_size = model.plan.vocab_size
        self.max_positions = min(max_model_len or model.plan.max_positions, model.plan.max_positions)
        self._pin = self.device.type == "cuda"
        self.steps_run = 0
        self._graphs = None
        self._seen = None
        self.h2d_bytes = 0          # bytes of step descriptions copied to the device so far (measurement)
        self.d2h_bytes = 0          # bytes of sampled ids copied back from captured steps so far

    # ---- requests ------------------------------------------------------------------
    def is_live(self, req_id) -> bool:
        return req_id in self.cache.requests

    def num_tokens(self, req_id) -> int:
        return self.cache.requests[req_id].num_tokens

    def seen_table(self) -> torch.Tensor:
        """uint8 ``[state slots + 1, vocabulary]``: the ids each live request has consumed, for the
        repetition penalty (a row per state slot, the last for padding rows).  Made when first asked for
        (all zeros, so a request whose first step asks for it starts with an empty row); from then
        on the cache manager zeroes a request's row at its admission."""
        if self._seen is None:
            self._seen = torch.zeros((self.cache.max_requests + 1, self.vocab_size), dtype=torch.uint8, device=self.device)
            self.cache.register_slot_table("seen_ids", self._seen)      # a request's row is zeroed at its admission
        return self._seen

    def finish(self, req_id) -> None:
        """The request is over: its pages and its slot go back."""
        self.cache.free_request(req_id)

    # ---- one step --------------------------------------------------------------------
    def prepare(self, entries) -> StepContext:
        """Reserve pages for the step's tokens and describe the batch on the device.
        Raises `OutOfPages` or `ContextOverflow` with nothing changed."""
        entries = list(entries)
        if not entries:
            raise ValueError("a step needs at least one entry")
        cache = self.cache
        seen = set()
        totals = []
        new_requests = 0
        for e in entries:
            if e.req_id in seen:
                raise ValueError(f"request {e.req_id!r} stands twice in one step")
            seen.add(e.req_id)
            n = len(e.tokens)
            if n < 1:
                raise ValueError(f"request {e.req_id!r}: an entry needs at least one token")
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.req_id!r}: wanted place {w} is outside its {n} tokens")
            if n == 1:
                bad = not 0 <= int(e.tokens[0]) < self.vocab_size
            else:               # (a prompt portion: one pass in numpy, not a loop over its tokens)
                ids = np.asarray(e.tokens)
                bad = bool(ids.min() < 0 or ids.max() >= self.vocab_size)
            if bad:
                t = next(t for t in e.tokens if not 0 <= int(t) < self.vocab_size)
                raise ValueError(f"request {e.req_id!r}: token id {t} is outside the vocabulary")
            req = cache.requests.get(e.req_id)
            have = req.num_tokens if req else 0
            if req is None:
                new_requests += 1
            if have + n > self.max_positions:
                raise ContextOverflow(f"request {e.req_id!r}: {have}+{n} tokens exceed max positions "
                                      f"{self.max_positions}")
            totals.append(have + n)
        # all or nothing: count what every group has to give before taking any
        if new_requests > cache.slots.free_count:
            raise OutOfPages(f"{new_requests} new requests, {cache.slots.free_count} state slots free")
        for gi, need in enumerate(pages_missing(cache, entries, totals)):
            pool = cache.groups[gi].pool
            if need > pool.free_count:
                raise OutOfPages(f"step needs {need} pages in group {gi}, {pool.free_count} free of {pool.capacity}")
        for e, tot in zip(entries, totals):
            if e.req_id not in cache.requests:
                cache.add_request(e.req_id)
            cache.reserve(e.req_id, tot)

        # ---- the description: packed into one pinned buffer, one copy --------------------
        q_lens = [len(e.tokens) for e in entries]
        layout = BatchLayout(sum(q_lens), len(entries), sum(len(e.want) for e in entries),
                             [max(len(cache.requests[e.req_id].tables[gi]) for e in entries)
                              for gi in range(len(cache.groups))])
        host = torch.empty(layout.total, dtype=torch.int32, pin_memory=self._pin)
        pack(layout, host.numpy(), cache, entries, totals)
        dev = host.to(self.device, non_blocking=True)
        self.h2d_bytes += host.numel() * host.element_size()
        return context(layout, dev, cache.page_size, q_lens, totals)

    def step(self, entries) -> torch.Tensor:
        """Run the entries as one batch.  Returns float32 logits ``[R, V]`` on the
        device, R the number of wanted places, in the order of the entries and of
        each entry's ``want``."""
        entries = list(entries)
        return self.run(self.prepare(entries), entries)

    def run(self, ctx: StepContext, entries) -> torch.Tensor:
        """The device part of a step prepared by `prepare`."""
        logits = self.model.forward(ctx, self.layer_caches)
        for e, tot in zip(entries, ctx.ctx_lens):
            self.cache.commit(e.req_id, tot)
        self.steps_run += 1
        if self.device.type == "cuda":
            from .. import ops
            ops.check_tcgen05_status()      # reads a status word only if such a kernel ran in this step
        return logits

    # ---- decoding through a captured graph -------------------------------------------------
    @property
    def graphs(self):
        """CUDA graphs of the decode step (forward and sampling kernel), one per batch size and
        context bucket: the first step of a kind runs eagerly on the graph's static buffers and is
        then captured; later ones copy the batch description into those buffers and replay."""
        from .graphs import DecodeGraphs
        if self._graphs is None:
            self._graphs = DecodeGraphs(self)
        return self._graphs
