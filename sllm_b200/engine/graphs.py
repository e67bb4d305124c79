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
from .batch import BatchLayout, context, pack, pages_missing


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
        cap_pages = -(-engine.max_positions // cache.page_size)
        # the step's description (every row brings one token and wants its logits) and, behind it, what the
        # sampling kernel reads
        self.layout = BatchLayout(B, B, B, [cap_pages] * len(cache.groups),
                                  extras={"temps": B, "uniforms": 2 * B, "top_k": B, "top_p": B, "penalty": B})
        total = self.layout.total
        # two host staging buffers: a step may be filled while the copy of the one before is still queued
        pin = engine.device.type == "cuda"
        self.hosts = [torch.zeros(total, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self.ids_host = [torch.zeros(B, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self.ids_ready = [torch.cuda.Event() if pin else None for _ in range(2)]
        self.turn = 0
        self.host = self.hosts[0]
        self.dev = torch.zeros(total, dtype=torch.int32, device=engine.device)
        # launch shapes come from the bucket, not from the requests: every context up to it replays this graph
        self.ctx = context(self.layout, self.dev, cache.page_size, [1] * B, [bucket] * B, is_graph_replay=True)
        sec = self.layout.sec
        self.temps = sec(self.dev, "temps").view(torch.float32)
        self.uniforms = sec(self.dev, "uniforms").view(torch.float64)
        self.top_k = sec(self.dev, "top_k")
        self.top_p = sec(self.dev, "top_p").view(torch.float32)
        self.penalty = sec(self.dev, "penalty").view(torch.float32)
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

    def fill(self, engine, entries, totals, temperatures, uniforms, ids_from=None, top_k=None, top_p=None,
             penalties=None):
        """Describe the step in the next host buffer and queue its copy to the device.  ``ids_from``:
        the token ids are not the host's to give; they are what the step before sampled, an int32
        tensor on the device (one id per entry, in the entries' order), copied on the device."""
        self.turn ^= 1
        self.host = self.hosts[self.turn]
        h = self.host.numpy()
        n = len(entries)
        pack(self.layout, h, engine.cache, entries, totals, tokens_from_host=ids_from is None)
        sec = self.layout.sec
        t_host, u_host = sec(h, "temps").view(np.float32), sec(h, "uniforms").view(np.float64)
        t_host[:n] = temperatures
        u_host[:n] = uniforms
        t_host[n:] = 0.0
        u_host[n:] = 0.0
        k_host, p_host = sec(h, "top_k"), sec(h, "top_p").view(np.float32)
        k_host[:] = 0                                # no filter unless the step names one
        p_host[:] = -1.0
        if top_k is not None:
            k_host[:n] = top_k
        if top_p is not None:
            p_host[:n] = top_p
        pen_host = sec(h, "penalty").view(np.float32)
        pen_host[:] = 1.0
        if penalties is not None:
            pen_host[:n] = penalties
        self.dev.copy_(self.host, non_blocking=True)
        if ids_from is not None:
            sec(self.dev, "token_ids")[:n].copy_(ids_from[:n])      # after the host's copy, before the replay


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

    def can_chain(self, entries, penalised: bool = False) -> bool:
        """Whether a step for these requests, one token further each, can be queued behind the
        step in flight with its token ids taken from that step's samples on the device: the
        requests are live, a graph is already captured for their number and context bucket (it
        need not be the graph in flight: the ids are copied from that one's output), and the
        pools hold the pages all of them need together."""
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
        return all(need <= g.pool.free_count for need, g in zip(pages_missing(cache, entries, totals), cache.groups))

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

    def launch(self, entries, temperatures, uniforms, device_timer=None, after: Launched | None = None,
               top_k=None, top_p=None, penalties=None) -> Launched:
        """Queue one decode step: reserve pages, describe the batch, replay the graph, queue the copy
        of the sampled ids to pinned host memory.  Does not wait for the device, except the first
        time a (batch size, context bucket) is seen: that step runs eagerly and is then captured.

        ``after``: the step in flight for the same requests in the same order.  The new step's token
        ids are then the ids THAT step sampled, copied on the device from the output buffer of the
        graph it ran on (which is another graph than this step's when the longest context has just
        crossed a bucket), and the entries' own tokens are not looked at."""
        tokens_on_device = after is not None
        if tokens_on_device and after.n != len(entries):
            raise ValueError("a chained step serves the requests of the step in flight, in their order")
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
        for gi, (need, g) in enumerate(zip(pages_missing(cache, entries, totals), cache.groups)):
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
        gr.fill(eng, entries, totals, temperatures, uniforms, after.graph.ids if tokens_on_device else None, top_k, top_p,
                penalties)
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
