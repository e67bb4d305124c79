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

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pools import OutOfPages
from ..parts.base import GroupView, StepContext


@dataclass
class StepEntry:
    req_id: object
    tokens: list
    want: list = field(default_factory=list)     # places among `tokens` whose logits are wanted


class ContextOverflow(ValueError):
    """A request would grow past the model's position limit."""


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class Engine:
    def __init__(self, model, *, page_size: int = 16, num_pages: int, max_requests: int = 8,
                 max_model_len: int | None = None):
        self.model = model
        self.device = model.device
        self.cache = CacheManager(model.cache_needs(), page_size=page_size, num_pages=num_pages,
                                  max_requests=max_requests)
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
            for t in e.tokens:
                if not 0 <= int(t) < self.vocab_size:
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
        for gi, g in enumerate(cache.groups):
            need = 0
            for e, tot in zip(entries, totals):
                req = cache.requests.get(e.req_id)
                need += max(0, cache.pages_for(tot) - (len(req.tables[gi]) if req else 0))
            if need > g.pool.free_count:
                raise OutOfPages(f"step needs {need} pages in group {gi}, {g.pool.free_count} free "
                                 f"of {g.pool.capacity}")
        for e, tot in zip(entries, totals):
            if e.req_id not in cache.requests:
                cache.add_request(e.req_id)
            cache.reserve(e.req_id, tot)

        # ---- host arrays, packed into one buffer, one copy --------------------------
        S = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        T = sum(q_lens)
        ps = cache.page_size
        R = sum(len(e.want) for e in entries)
        max_pages = [max(len(cache.requests[e.req_id].tables[gi]) for e in entries)
                     for gi in range(len(cache.groups))]
        sizes = {"token_ids": T, "positions": T, "seq_of_token": T, "q_start": S + 1, "ctx_len": S,
                 "state_slots": S, "logit_rows": R}
        for gi, mp in enumerate(max_pages):
            sizes[f"slot_mapping{gi}"] = T
            sizes[f"block_tables{gi}"] = S * mp
        offs = {}
        total = 0
        for k, n in sizes.items():
            offs[k] = total
            total += _pad4(max(n, 1))
        host = torch.empty(total, dtype=torch.int32, pin_memory=self._pin)
        h = host.numpy()
        h.fill(-1)

        def sec(k):
            return h[offs[k]: offs[k] + sizes[k]]

        tok, pos, sot = sec("token_ids"), sec("positions"), sec("seq_of_token")
        q_start, ctx_len, slots, rows = sec("q_start"), sec("ctx_len"), sec("state_slots"), sec("logit_rows")
        t0 = 0
        r0 = 0
        q_start[0] = 0
        for si, (e, tot) in enumerate(zip(entries, totals)):
            n = q_lens[si]
            req = cache.requests[e.req_id]
            tok[t0:t0 + n] = np.asarray(e.tokens, dtype=np.int32)
            pos[t0:t0 + n] = np.arange(tot - n, tot, dtype=np.int32)
            sot[t0:t0 + n] = si
            q_start[si + 1] = t0 + n
            ctx_len[si] = tot
            slots[si] = req.slot
            for w in e.want:
                rows[r0] = t0 + w
                r0 += 1
            for gi, mp in enumerate(max_pages):
                table = np.asarray(req.tables[gi], dtype=np.int32)
                bt = sec(f"block_tables{gi}").reshape(S, mp)
                bt[si, :len(table)] = table
                p = np.arange(tot - n, tot, dtype=np.int64)
                pages = table[p // ps]
                if (pages < 0).any():
                    raise RuntimeError(f"request {e.req_id!r}: a token would be written to a page given back")
                sec(f"slot_mapping{gi}")[t0:t0 + n] = (pages.astype(np.int64) * ps + p % ps).astype(np.int32)
            t0 += n
        dev = host.to(self.device, non_blocking=True)
        self.h2d_bytes += host.numel() * host.element_size()

        def dsec(k):
            return dev[offs[k]: offs[k] + sizes[k]]

        groups = [GroupView(ps, dsec(f"block_tables{gi}").view(S, mp), dsec(f"slot_mapping{gi}"))
                  for gi, mp in enumerate(max_pages)]
        return StepContext(
            num_tokens=T, num_seqs=S, token_ids=dsec("token_ids"), positions=dsec("positions"),
            seq_of_token=dsec("seq_of_token"), q_start=dsec("q_start"), ctx_len=dsec("ctx_len"),
            state_slots=dsec("state_slots"), logit_rows=dsec("logit_rows"), groups=groups,
            q_lens=q_lens, ctx_lens=[int(t) for t in totals], max_q_len=max(q_lens),
            max_ctx_len=int(max(totals)))

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

    def decode_graph_step(self, entries, temperatures, uniforms, device_timer=None):
        """One decode step (every entry brings one token and wants its logits) through a graph.
        Returns the sampled ids (int32 tensor on the host)."""
        return self.graphs.step(list(entries), temperatures, uniforms, device_timer)
