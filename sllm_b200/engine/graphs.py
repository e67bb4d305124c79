"""CUDA graphs of the decode step.

A decode step launches eight kernels per layer; launched one by one from Python
they cost more host time than the device needs to run them.  The step's shape is
fixed by the number of requests alone (one token each), so its forward and the
sampling kernel are captured once per (batch size, context bucket) and replayed:
the host fills one pinned buffer with the batch description (token ids, positions,
slots, block tables, temperatures, uniforms), copies it to the graph's static device
buffer and launches the graph.  Kernels read lengths and tables from device memory,
so nothing about a request's context is baked into the graph except the bucket that
decides how many ways the attention kernel splits the context.

A capture costs tens of milliseconds, so batch sizes are rounded up to a few sizes
(`DecodeGraphs.batch_bucket`) and the rows beyond the live requests are padding: token 0
at position 0 with no context, no page to write to (slot -1: the rotary kernel skips the
write, the attention kernels find no key) and the cache's spare state slot; what the
padding rows sample is dropped.  A decode step is bound by reading the weights, which the
padding does not add to.
"""

from __future__ import annotations

import gc

import numpy as np
import torch

from .. import ops
from ..parts.base import GroupView, StepContext


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class _Graph:
    def __init__(self, engine, B: int, bucket: int, penalised: bool = False):
        """``B``: rows of the captured step (live requests plus padding).  ``penalised``: the step also
        records its tokens in the engine's table of seen ids and applies the rows' repetition
        penalties before it samples."""
        self.penalised = bool(penalised)
        if self.penalised:
            engine.seen_table()                      # made here, never inside a capture
        cache = engine.cache
        self.B = B
        ps = cache.page_size
        self.cap_pages = -(-engine.max_positions // ps)
        G = len(cache.groups)
        sizes = {"token_ids": B, "positions": B, "seq_of_token": B, "q_start": B + 1, "ctx_len": B,
                 "state_slots": B, "logit_rows": B, "temps": B, "uniforms": 2 * B, "top_k": B, "top_p": B, "penalty": B}
        for gi in range(G):
            sizes[f"slot_mapping{gi}"] = B
            sizes[f"block_tables{gi}"] = B * self.cap_pages
        self.offs, total = {}, 0
        for k, n in sizes.items():
            self.offs[k] = (total, n)
            total += _pad4(n)
        # two host staging buffers: a step may be filled while the copy of the one before is still queued
        pin = engine.device.type == "cuda"
        self.hosts = [torch.zeros(total, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self.ids_host = [torch.zeros(B, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self.ids_ready = [torch.cuda.Event() if pin else None for _ in range(2)]
        self.turn = 0
        self.host = self.hosts[0]
        self.h = self.host.numpy()
        self.dev = torch.zeros(total, dtype=torch.int32, device=engine.device)
        # what never changes in a decode step
        for hb in self.hosts:
            self.h = hb.numpy()
            self._hsec("seq_of_token")[:] = np.arange(B)
            self._hsec("q_start")[:] = np.arange(B + 1)
            self._hsec("logit_rows")[:] = np.arange(B)
            for gi in range(G):
                self._hsec(f"block_tables{gi}")[:] = -1
        self.h = self.host.numpy()
        groups = [GroupView(ps, self._dsec(f"block_tables{gi}").view(B, self.cap_pages), self._dsec(f"slot_mapping{gi}"))
                  for gi in range(G)]
        self.ctx = StepContext(
            num_tokens=B, num_seqs=B, token_ids=self._dsec("token_ids"), positions=self._dsec("positions"),
            seq_of_token=self._dsec("seq_of_token"), q_start=self._dsec("q_start"), ctx_len=self._dsec("ctx_len"),
            state_slots=self._dsec("state_slots"), logit_rows=self._dsec("logit_rows"), groups=groups,
            q_lens=[1] * B, ctx_lens=[bucket] * B, max_q_len=1, max_ctx_len=bucket, is_graph_replay=True)
        self.temps = self._dsec("temps").view(torch.float32)
        self.uniforms = self._dsec("uniforms").view(torch.float64)
        self.top_k = self._dsec("top_k")
        self.top_p = self._dsec("top_p").view(torch.float32)
        self.penalty = self._dsec("penalty").view(torch.float32)
        self.graph = None
        self.ids = None
        self.launches = 0
        self.reporting = 0

    def run(self, engine):
        """The step's kernels on the static buffers: what is run once eagerly and then captured."""
        if self.penalised:
            ops.mark_seen(engine.seen_table(), self.ctx)
        logits = engine.model.forward(self.ctx, engine.layer_caches)
        if self.penalised:
            ops.penalty_from_seen_(logits, engine.seen_table(), self.ctx, self.penalty)
        self.ids = ops.sample_rows(logits, self.temps, self.uniforms, self.top_k, self.top_p)

    def _hsec(self, k):
        o, n = self.offs[k]
        return self.h[o:o + n]

    def _dsec(self, k):
        o, n = self.offs[k]
        return self.dev[o:o + n]

    def fill(self, engine, entries, totals, temperatures, uniforms, tokens_on_device: bool = False, top_k=None, top_p=None,
             penalties=None):
        """Describe the step in the next host buffer and queue its copy to the device.  With
        ``tokens_on_device`` the token ids are not the host's to give: they are the ids the graph's
        previous replay sampled, copied on the device."""
        self.turn ^= 1
        self.host = self.hosts[self.turn]
        self.h = self.host.numpy()
        cache = engine.cache
        ps = cache.page_size
        B = self.B
        tok, pos, ctx, slots = (self._hsec(k) for k in ("token_ids", "positions", "ctx_len", "state_slots"))
        n = len(entries)
        for i, (e, tot) in enumerate(zip(entries, totals)):
            req = cache.requests[e.req_id]
            tok[i] = e.tokens[0] if not tokens_on_device else 0
            pos[i] = tot - 1
            ctx[i] = tot
            slots[i] = req.slot
            for gi in range(len(cache.groups)):
                table = req.tables[gi]
                bt = self._hsec(f"block_tables{gi}")
                row = bt[i * self.cap_pages:(i + 1) * self.cap_pages]
                m = len(table)
                row[:m] = table
                row[m:] = -1
                page = table[(tot - 1) // ps]
                if page < 0:
                    raise RuntimeError(f"request {e.req_id!r}: a token would be written to a page given back")
                self._hsec(f"slot_mapping{gi}")[i] = page * ps + (tot - 1) % ps
        if n < B:                                    # padding rows: no context, nothing written, the spare state slot
            tok[n:] = 0
            pos[n:] = 0
            ctx[n:] = 0
            slots[n:] = cache.padding_slot
            for gi in range(len(cache.groups)):
                self._hsec(f"block_tables{gi}")[n * self.cap_pages:] = -1
                self._hsec(f"slot_mapping{gi}")[n:] = -1
        t_host, u_host = self._hsec("temps").view(np.float32), self._hsec("uniforms").view(np.float64)
        t_host[:n] = temperatures
        u_host[:n] = uniforms
        t_host[n:] = 0.0
        u_host[n:] = 0.0
        k_host, p_host = self._hsec("top_k"), self._hsec("top_p").view(np.float32)
        k_host[:] = 0                                # no filter unless the step names one
        p_host[:] = -1.0
        if top_k is not None:
            k_host[:n] = top_k
        if top_p is not None:
            p_host[:n] = top_p
        pen_host = self._hsec("penalty").view(np.float32)
        pen_host[:] = 1.0
        if penalties is not None:
            pen_host[:n] = penalties
        self.dev.copy_(self.host, non_blocking=True)
        if tokens_on_device:
            self._dsec("token_ids").copy_(self.ids)          # after the host's copy, before the replay


class Launched:
    """A decode step that has been queued on the device and whose ids have not been read yet."""

    def __init__(self, graph, turn, ids_now=None, n=None):
        self.graph, self.turn, self.ids_now, self.n = graph, turn, ids_now, n


class DecodeGraphs:
    def __init__(self, engine):
        self.engine = engine
        self.graphs: dict[tuple, _Graph] = {}

    @staticmethod
    def bucket(max_ctx: int) -> int:
        b = 256
        while b < max_ctx:
            b *= 2
        return b

    @staticmethod
    def batch_bucket(n: int) -> int:
        """Rows of the graph that serves ``n`` requests: n up to 4, then 6, 8, 12, 16, 24, 32, ...
        (at most a third of the rows are padding)."""
        if n <= 4:
            return n
        b = 4
        while True:
            for c in (b + b // 2, 2 * b):
                if c >= n:
                    return c
            b *= 2

    def step(self, entries, temperatures, uniforms, device_timer=None):
        """Launch and read one decode step (see `launch`, `read`)."""
        h = self.launch(entries, temperatures, uniforms, device_timer=device_timer)
        return torch.tensor(self.read(h), dtype=torch.int32)

    def can_chain(self, entries, penalised: bool = False) -> bool:
        """Whether a step for these requests, one token further each, can be queued behind the
        step in flight with its token ids taken from that step's samples on the device: the same
        requests in the same order, a graph already captured for their number and context bucket,
        and pages at hand."""
        eng, cache = self.engine, self.engine.cache
        totals = []
        for e in entries:
            req = cache.requests.get(e.req_id)
            if req is None or req.num_tokens + 1 > eng.max_positions:
                return False
            totals.append(req.num_tokens + 1)
        gr = self.graphs.get((self.batch_bucket(len(entries)), self.bucket(max(totals)), bool(penalised)))
        if gr is None or gr.graph is None:
            return False
        return all(cache.can_reserve(e.req_id, t) for e, t in zip(entries, totals))

    def _capture(self, gr: _Graph) -> torch.Tensor:
        """Run the step that `gr`'s static buffers describe once, launch by launch, then capture the same
        launches as a graph.  Returns the ids the eager run sampled."""
        eng = self.engine
        before = ops.launches["own"]
        gr.run(eng)
        gr.launches = ops.launches["own"] - before
        eager_ids = gr.ids
        graph = torch.cuda.CUDAGraph()
        # Nothing may free device memory or destroy a graph while the capture runs: a collection
        # of garbage (an engine dropped earlier, say) in the middle of it would invalidate it.
        # (torch's graph context collects once before it begins; here the collector stays off.)
        gc_was_on = gc.isenabled()
        gc.disable()
        reporting = ops.status_word_launches()
        try:
            with torch.cuda.graph(graph):
                gr.run(eng)
        finally:
            if gc_was_on:
                gc.enable()
        ops.launches["own"] -= gr.launches          # capturing launched nothing
        gr.reporting = ops.status_word_launches() - reporting      # kernels of the graph that report through the status word
        ops.note_status_word_launches(-gr.reporting)
        gr.graph = graph
        return eager_ids

    def warmup(self, batch_sizes, contexts, penalised: bool = False) -> int:
        """Capture the graphs for these numbers of requests and context lengths ahead of the first
        request (a capture costs tens of milliseconds, which the first step of each shape pays
        otherwise).  The captured step is made of padding rows only: it reads no page and writes
        none.  Returns how many graphs were captured."""
        eng = self.engine
        made = 0
        for rows in sorted({self.batch_bucket(int(n)) for n in batch_sizes}):
            for bucket in sorted({self.bucket(min(int(c), eng.max_positions)) for c in contexts}):
                key = (rows, bucket, bool(penalised))
                if key in self.graphs and self.graphs[key].graph is not None:
                    continue
                gr = self.graphs[key] = _Graph(eng, *key)
                gr.fill(eng, [], [], np.zeros(0, np.float32), np.zeros(0, np.float64))
                self._capture(gr)
                made += 1
        torch.cuda.synchronize(eng.device)
        return made

    def launch(self, entries, temperatures, uniforms, device_timer=None, tokens_on_device: bool = False,
               top_k=None, top_p=None, penalties=None) -> Launched:
        """Queue one decode step: reserve pages, describe the batch, replay the graph, queue the copy
        of the sampled ids to pinned host memory.  Does not wait for the device, except the first
        time a (batch size, context bucket) is seen: that step runs eagerly and is then captured."""
        eng = self.engine
        cache = eng.cache
        totals = []
        for e in entries:
            if len(e.tokens) != 1:
                raise ValueError("a graph decode step takes one token per request")
            req = cache.requests.get(e.req_id)
            if req is None:
                raise ValueError(f"request {e.req_id!r} is not live; its prompt runs through step()")
            tot = req.num_tokens + 1
            if tot > eng.max_positions:
                from .engine import ContextOverflow
                raise ContextOverflow(f"request {e.req_id!r}: {tot} tokens exceed max positions {eng.max_positions}")
            if not tokens_on_device and not 0 <= int(e.tokens[0]) < eng.vocab_size:
                raise ValueError(f"request {e.req_id!r}: token id {e.tokens[0]} is outside the vocabulary")
            totals.append(tot)
        # pages: all or nothing
        for gi, g in enumerate(cache.groups):
            need = sum(max(0, cache.pages_for(t) - len(cache.requests[e.req_id].tables[gi]))
                       for e, t in zip(entries, totals))
            if need > g.pool.free_count:
                from ..cache.pools import OutOfPages
                raise OutOfPages(f"step needs {need} pages in group {gi}, {g.pool.free_count} free")
        for e, t in zip(entries, totals):
            cache.reserve(e.req_id, t)
        key = (self.batch_bucket(len(entries)), self.bucket(max(totals)), penalties is not None)
        gr = self.graphs.get(key)
        if gr is None:
            gr = self.graphs[key] = _Graph(eng, *key)
        if tokens_on_device and gr.graph is None:
            raise RuntimeError("a chained step needs a captured graph (see can_chain)")
        gr.fill(eng, entries, totals, temperatures, uniforms, tokens_on_device, top_k, top_p, penalties)
        eng.h2d_bytes += gr.host.numel() * gr.host.element_size()
        eng.d2h_bytes += gr.ids_host[0].numel() * gr.ids_host[0].element_size()
        if device_timer is not None:
            device_timer.start()
        ids_now = None
        if gr.graph is None:
            # first use: run eagerly on the static buffers (this step's result), then capture
            ids_now = self._capture(gr).cpu().tolist()[:len(entries)]
            # the graph's own output buffer must hold this step's ids for a step chained behind it
            gr.ids[:len(ids_now)].copy_(torch.tensor(ids_now, dtype=torch.int32, device=eng.device))
        else:
            gr.graph.replay()
            ops.launches["own"] += gr.launches
            ops.note_status_word_launches(gr.reporting)
            gr.ids_host[gr.turn].copy_(gr.ids, non_blocking=True)
            gr.ids_ready[gr.turn].record()
        if device_timer is not None:
            device_timer.stop()
        for e, t in zip(entries, totals):
            cache.commit(e.req_id, t)
        eng.steps_run += 1
        return Launched(gr, gr.turn, ids_now, len(entries))

    def read(self, h: Launched) -> list:
        """The ids a launched step sampled (waits for that step, not for any queued behind it)."""
        if h.ids_now is not None:
            out = h.ids_now
        else:
            h.graph.ids_ready[h.turn].synchronize()
            out = h.graph.ids_host[h.turn].tolist()[:h.n]
        if self.engine.steps_run % 64 == 0:
            ops.check_tcgen05_status()      # a wait that ran out inside a TMA-fed kernel, if any
        return out
