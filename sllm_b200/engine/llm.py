"""The Python entry point: a model folder in, generated token ids out.

The reference's entry points work on text through its own tokenizer
(``InferenceEngine.complete/chat``, serving/executor.py:536-754) and run each
sequence's forward on its own (``BatchedInferenceEngine.step``,
serving/executor.py:1034-1082).  This engine's interface is token ids; every step
is one batched forward through `Engine.step`, and sampling runs on the device.
Option names follow the reference where it has them: ``max_new``, ``temperature``,
``top_k``, ``top_p``, ``seed``, ``repetition_penalty`` (serving/executor.py:334-345),
``block_size``/``chunk_size``/``max_num_seqs`` (runtime/scheduler.py:62-69; recipe
``defaults``), ``kv_utilization`` (recipes/schema.py:255).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..sampling import Sampler, SamplingParams
from .engine import Engine, StepEntry
from .loading import build_model, parse_dtype
from .scheduler import Scheduler


@dataclass
class GenerationResult:
    req_id: object
    prompt: list
    ids: list                  # generated token ids (a stop id is not among them)
    finish_reason: str         # "stop" | "length" | "abort"
    preemptions: int = 0


def plan_num_pages(model, page_size: int, *, kv_utilization: float = 0.9, kv_bytes: int | None = None,
                   cap_tokens: int | None = None) -> int:
    """Pages that fit the device memory left after the weights, times the utilisation
    (runtime/placement.py:48-51: budget * utilisation // (bytes per token * block size)),
    or an explicit budget in bytes; never more than ``cap_tokens`` worth."""
    from ..cache.manager import CacheManager
    probe = CacheManager(model.cache_needs(), page_size=page_size, num_pages=0, max_requests=1)
    item = 2 if model.dtype == torch.bfloat16 else 4
    per_token = max(probe.bytes_per_token(item), 1)
    if kv_bytes is None:
        free, _ = torch.cuda.mem_get_info(model.device)
        kv_bytes = int(free * kv_utilization)
    pages = kv_bytes // (per_token * page_size)
    if cap_tokens is not None:
        pages = min(pages, -(-cap_tokens // page_size))
    return max(int(pages), 1)


ROW_TILE = 256       # rows of a tile of the prompt-portion products (a pair of CTAs of `gemm_pair.cu`)


class LLM:
    def __init__(self, model_dir: str | None = None, *, model=None, dtype="bfloat16", device="cuda:0",
                 block_size: int = 16, num_pages: int | None = None, kv_utilization: float = 0.9,
                 kv_bytes: int | None = None, max_num_seqs: int = 8, max_batch_tokens: int = 2048,
                 chunk_size: int = 512, max_model_len: int | None = None, policy: str = "reserve",
                 cuda_graphs: bool = True, pipeline_decode: bool = True, progress=None, row_tile: int | None = None):
        """``row_tile``: see `Scheduler` (None: the prompt-portion kernels' 256 rows for a bfloat16 model, off in
        float32; 0: off)."""
        if (model_dir is None) == (model is None):
            raise ValueError("give a model folder or a built model")
        if model is None:
            model, _ = build_model(model_dir, parse_dtype(dtype), device, progress=progress)
        self.model = model
        self.max_model_len = min(max_model_len or model.plan.max_positions, model.plan.max_positions)
        if num_pages is None:
            num_pages = plan_num_pages(model, block_size, kv_utilization=kv_utilization, kv_bytes=kv_bytes,
                                       cap_tokens=max_num_seqs * self.max_model_len + block_size * max_num_seqs)
        self.engine = Engine(model, page_size=block_size, num_pages=num_pages, max_requests=max_num_seqs,
                             max_model_len=self.max_model_len)
        self.scheduler = Scheduler(self.engine.cache, max_positions=self.max_model_len, max_num_seqs=max_num_seqs,
                                   max_batch_tokens=max_batch_tokens, chunk_size=chunk_size, policy=policy,
                                   row_tile=ROW_TILE if (row_tile is None and model.dtype == torch.bfloat16) else int(row_tile or 0))
        self.sampler = Sampler(model.device)
        self.cuda_graphs = bool(cuda_graphs) and model.device.type == "cuda"
        self.pipeline_decode = self.cuda_graphs and bool(pipeline_decode)
        self._inflight = None
        self._next_id = 0
        self.steps = 0

    # ---- request-level interface ---------------------------------------------------------
    def add_request(self, prompt_token_ids, params: SamplingParams | None = None, req_id=None):
        if req_id is None:
            req_id = self._next_id
            self._next_id += 1
        return self.scheduler.add(req_id, prompt_token_ids, params or SamplingParams())

    def warmup(self, batch_sizes=None, contexts=None, penalised: bool = False) -> int:
        """Capture the decode graphs ahead of the first request: for every number of requests up to
        ``max_num_seqs`` (or those given) and every context bucket up to the model length (or those
        that hold the given lengths).  Returns the number of graphs captured; 0 without CUDA graphs."""
        if not self.cuda_graphs:
            return 0
        if batch_sizes is None:
            batch_sizes = range(1, self.scheduler.max_num_seqs + 1)
        if contexts is None:
            contexts, c = [], 256                     # the buckets: powers of two from 256 up to the model length
            while True:
                contexts.append(min(c, self.max_model_len))
                if c >= self.max_model_len:
                    break
                c *= 2
        return self.engine.graphs.warmup(batch_sizes, contexts, penalised)

    def abort(self, req_id) -> bool:
        return self.scheduler.abort(req_id)

    def step(self, device_timer=None):
        """Schedule, run and sample one step.  Returns (finished requests, new tokens by request).
        ``device_timer``: an object whose ``start()``/``stop()`` are called around the part of
        the step that runs on the device (measurement only).

        Pure decode steps run from a CUDA graph and are pipelined: while the device runs one, the
        next is already queued behind it with its token ids taken on the device from the first
        one's samples, and only then does the host wait for the first one's ids.  The host's
        scheduling and bookkeeping thus overlap the device's work.  The queued step assumes that
        no request stops; one that does (a stop id) has a token computed in vain, which is dropped.
        """
        sched = self.scheduler
        if self._inflight is None:
            plan = sched.schedule()
            if not plan:
                if sched.has_work:
                    # serving/executor.py:1094-1099: requests remain but nothing can be scheduled
                    raise RuntimeError("scheduler stalled: requests remain but none can be scheduled "
                                       "(the cache cannot hold the next one)")
                return [], {}
            entries = [StepEntry(p.req.req_id, p.req.token_slice(p.start, p.count),
                                 [p.count - 1] if p.sample else []) for p in plan]
            rows = [(p.req.params, p.req.rng, None) for p in plan if p.sample]
            # repetition penalties come from the engine's table of seen ids, which every step that
            # holds a penalised request keeps up to date (its prompt portions included)
            track = any(p.req.params.penalised for p in plan)
            penalties = self.sampler.penalties([p.req.params for p in plan if p.sample]) if track else None
            if not (self.cuda_graphs and all(p.count == 1 and p.sample for p in plan)):
                ctx = self.engine.prepare(entries)
                if device_timer is not None:
                    device_timer.start()
                if track:
                    seen = self.engine.seen_table()
                    ops.mark_seen(seen, ctx)
                logits = self.engine.run(ctx, entries)
                if penalties is not None and logits.shape[0]:
                    pen = torch.from_numpy(penalties)
                    ops.penalty_from_seen_(logits, seen, ctx, (pen.pin_memory() if self.sampler._pin else pen).to(
                        logits.device, non_blocking=True))
                ids = self.sampler.sample(logits, rows, device_timer=device_timer)
                sampled = {p.req.req_id: t for p, t in zip((p for p in plan if p.sample), ids)}
                finished = sched.update(plan, sampled)
                self.steps += 1
                return finished, sampled
            # a pure decode step: replayed from a captured graph, sampling included
            temps, unis, top_k, top_p = self.sampler.host_inputs(rows)
            handle = self.engine.graphs.launch(entries, temps, unis, device_timer=device_timer, top_k=top_k, top_p=top_p,
                                               penalties=penalties)
            self._inflight = (plan, handle)
        plan, handle = self._inflight
        self._inflight = self._chain(plan, handle, device_timer)
        ids = self.engine.graphs.read(handle)
        sampled = {p.req.req_id: int(t) for p, t in zip(plan, ids) if p.req.status == "running"}
        finished = sched.update(plan, sampled)
        self.steps += 1
        return finished, sampled

    def _chain(self, plan, handle, device_timer):
        """Queue the decode step after ``plan``'s (in flight as ``handle``) behind it, if nothing can
        change who runs: no request waits for admission, none of the plan's requests ends by length
        with this token, and the graph and the pages are there.  The queued step consumes the ids
        ``handle``'s step samples (serving/executor.py:378-393: every decode step is fed the token
        the one before produced).  Returns (next plan, handle) or None."""
        sched = self.scheduler
        if not self.pipeline_decode or sched.waiting or len(plan) != len(sched.running):
            return None
        for p in plan:
            r = p.req
            if (r.status != "running" or len(r.output) + 1 >= r.params.max_new
                    or r.num_tokens + 1 >= sched.max_positions):
                return None
        entries = [StepEntry(p.req.req_id, [0], [0]) for p in plan]
        penalties = self.sampler.penalties([p.req.params for p in plan])
        if not self.engine.graphs.can_chain(entries, penalties is not None):
            return None
        rows = [(p.req.params, p.req.rng, None) for p in plan]
        temps, unis, top_k, top_p = self.sampler.host_inputs(rows)
        queued = self.engine.graphs.launch(entries, temps, unis, device_timer=device_timer, after=handle,
                                           top_k=top_k, top_p=top_p, penalties=penalties)
        from .scheduler import Planned
        nxt = [Planned(p.req, p.start + 1, 1, True) for p in plan]
        return nxt, queued

    def drain(self) -> None:
        """Wait for a decode step still queued on the device and drop its result (its requests
        have all ended)."""
        if self._inflight is not None:
            plan, handle = self._inflight
            self._inflight = None
            self.engine.graphs.read(handle)
            if any(p.req.status == "running" for p in plan):
                raise RuntimeError("a decode step in flight was dropped while its requests still run")

    # ---- batch interface -------------------------------------------------------------------
    def generate(self, prompt_token_ids, params=None) -> list[GenerationResult]:
        """Generate for each prompt (a list of token ids).  ``params``: one
        `SamplingParams` for all, or one per prompt.  Results in the prompts' order."""
        prompts = list(prompt_token_ids)
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while any(r.status != "finished" for r in reqs):
            self.step()
        if not self.scheduler.has_work:
            self.drain()
        return [GenerationResult(r.req_id, r.prompt, list(r.output), r.finish_reason, r.preemptions) for r in reqs]
