"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.  Pure bookkeeping over the cache manager; it runs no
arithmetic and needs no device.

After the reference's scheduler (runtime/scheduler.py:61-188): a FIFO of waiting
requests; admission while a running slot and pages are free, requests that do not
fit being skipped and kept in order (backfill, scheduler.py:117-136); prompt
portions of at most ``chunk_size``; one token per decoding request; a finished
or aborted request gives everything back at once.  Beyond it: a budget of tokens
per step (decoding requests first, what is left to prompt portions in order), and
a second page policy.

When pages run out
------------------
``policy="reserve"`` (the reference's, scheduler.py:168-180): a request is admitted
only if pages for ``prompt + max_new`` tokens are free, and takes them all at
admission; pages cannot run out later; a request that does not fit waits; one that
could never fit is refused when it is added.

``policy="on_demand"``: pages are taken as tokens arrive.  If a decoding request
needs a page and none is free, the youngest running request is preempted: its pages
go back, it returns to the head of the waiting queue with the tokens it has already
produced, and its prompt plus those tokens are computed again when it is readmitted
(recompute; nothing is swapped out).  A prompt portion that finds too few pages is
shortened to what fits, or waits a step.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams


@dataclass
class Request:
    req_id: object
    prompt: list
    params: SamplingParams
    output: list = field(default_factory=list)
    num_computed: int = 0              # tokens whose keys and values lie in the cache
    status: str = "waiting"            # waiting | running | finished
    finish_reason: str | None = None   # stop | length | abort
    preemptions: int = 0
    rng: np.random.Generator | None = None

    @property
    def tokens(self) -> list:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    def token_slice(self, start: int, count: int) -> list:
        """``tokens[start:start+count]`` without building the whole list (a decode step asks for
        the last token of thousands)."""
        n = len(self.prompt)
        if start >= n:
            return self.output[start - n:start - n + count]
        if start + count <= n:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.output[:start + count - n]

    @property
    def pending(self) -> int:
        return len(self.prompt) + len(self.output) - self.num_computed


@dataclass
class Planned:
    """One entry of a step: run ``count`` tokens of ``req`` from ``start``; ``sample``
    says that the portion reaches the request's last token, whose logits pick the next."""
    req: Request
    start: int
    count: int
    sample: bool


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_positions: int, max_num_seqs: int = 8,
                 max_batch_tokens: int = 2048, chunk_size: int = 512, policy: str = "reserve",
                 row_tile: int = 0, row_tile_slack: int | None = None):
        """``row_tile`` (0: off): the rows the kernels of a prompt portion work in.  A step of a few tokens more than
        a multiple of it pays for a whole tile more (512 prompt tokens beside 31 decoded ones: three tiles of 256 rows
        for 543 tokens), so a step that is at most ``row_tile_slack`` tokens over a multiple (by default half a tile:
        it saves more rows of padding than it puts off) gives those tokens of a prompt portion back to the next step."""
        if min(max_num_seqs, max_batch_tokens, chunk_size) < 1:
            raise ValueError("sizes must be >= 1")                 # runtime/scheduler.py:70-71
        if policy not in ("reserve", "on_demand"):
            raise ValueError("policy must be 'reserve' or 'on_demand'")
        self.cache = cache
        self.max_positions = max_positions
        self.max_num_seqs = max_num_seqs
        self.max_batch_tokens = max_batch_tokens
        self.chunk_size = chunk_size
        self.policy = policy
        self.row_tile = max(0, int(row_tile))
        self.row_tile_slack = self.row_tile // 2 if row_tile_slack is None else max(0, int(row_tile_slack))
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []       # in order of admission
        self.done: list[Request] = []
        self.num_preemptions = 0

    # ---- public --------------------------------------------------------------------
    def add(self, req_id, prompt, params: SamplingParams) -> Request:
        if any(r.req_id == req_id for r in self.waiting) or any(r.req_id == req_id for r in self.running):
            raise ValueError(f"request {req_id!r} already registered")       # runtime/scheduler.py:84-85
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        if len(prompt) + params.max_new > self.max_positions:               # serving/executor.py:931-934
            raise ValueError(f"prompt ({len(prompt)}) + max_new ({params.max_new}) exceeds the model's "
                             f"{self.max_positions} positions")
        if not self.cache.fits_at_all(len(prompt) + params.max_new):
            raise ValueError(f"request {req_id!r} needs more pages than the whole pool has")
        req = Request(req_id, prompt, params, rng=np.random.default_rng(params.seed))
        self.waiting.append(req)
        return req

    def abort(self, req_id) -> bool:
        """Cancel a request wherever it is (runtime/scheduler.py:100-115)."""
        for r in self.running:
            if r.req_id == req_id:
                self._finish(r, "abort")
                return True
        for r in list(self.waiting):
            if r.req_id == req_id:
                self.waiting.remove(r)
                r.status, r.finish_reason = "finished", "abort"
                self.done.append(r)
                return True
        return False

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def schedule(self) -> list[Planned]:
        """Decide the next step: which requests run how many tokens."""
        budget = self.max_batch_tokens
        plan: list[Planned] = []
        planned_ids = set()
        # decoding requests first, then prompt portions, each in order of admission
        for decoding in (True, False):
            for r in list(self.running):
                if r.status != "running" or r.req_id in planned_ids or (r.pending == 1) != decoding:
                    continue
                if budget <= 0:
                    break
                n = 1 if decoding else min(r.pending, self.chunk_size, budget)
                n = self._take_pages(r, n, plan, planned_ids)
                if n <= 0:
                    continue
                plan.append(Planned(r, r.num_computed, n, r.num_computed + n == r.num_tokens))
                planned_ids.add(r.req_id)
                budget -= n
        # admission (pump): skip what does not fit, keep its place
        skipped = []
        while self.waiting and len(self.running) < self.max_num_seqs and budget > 0:
            r = self.waiting.popleft()
            n = min(r.pending, self.chunk_size, budget)
            if self.policy == "on_demand" and self.cache.groups:
                # start with the pages there are; the rest of the prompt follows as they come free
                n = min(n, min(g.pool.free_count for g in self.cache.groups) * self.cache.page_size)
            total = len(r.prompt) + r.params.max_new if self.policy == "reserve" else r.num_computed + n
            if n <= 0 or not self.cache.can_reserve(r.req_id, total):
                skipped.append(r)
                continue
            self.cache.add_request(r.req_id)
            self.cache.reserve(r.req_id, total)
            r.status = "running"
            self.running.append(r)
            plan.append(Planned(r, r.num_computed, n, r.num_computed + n == r.num_tokens))
            planned_ids.add(r.req_id)
            budget -= n
        self.waiting.extendleft(reversed(skipped))
        self._trim_to_row_tiles(plan)
        return plan

    def _trim_to_row_tiles(self, plan: list[Planned]) -> None:
        """See ``row_tile``: the last prompt portion of the plan that can spare them loses the tokens that would open
        another tile of rows (its pages stay reserved; the tokens come with the next step)."""
        if not self.row_tile:
            return
        total = sum(p.count for p in plan)
        over = total % self.row_tile
        if total < self.row_tile or over == 0 or over > self.row_tile_slack:
            return
        for p in reversed(plan):
            if p.count > over and p.req.pending > 1:       # a prompt portion (a decoding request has one pending token)
                p.count -= over
                p.sample = False                            # it no longer reaches the prompt's last token
                return

    def update(self, plan, sampled: dict) -> list[Request]:
        """After the step ran: ``sampled`` maps each request whose portion reached its
        last token to the token picked.  Returns the requests that finished."""
        finished = []
        for p in plan:
            r = p.req
            if r.status != "running":
                continue
            r.num_computed += p.count
            if self.cache.requests[r.req_id].num_tokens < r.num_computed:   # the engine may be a queued step ahead
                self.cache.commit(r.req_id, r.num_computed)
            if not p.sample:
                continue
            tok = int(sampled[r.req_id])
            if tok in r.params.stop_ids:                       # not appended (serving/executor.py:384-386)
                self._finish(r, "stop")
            else:
                r.output.append(tok)
                if len(r.output) >= r.params.max_new or r.num_tokens >= self.max_positions:
                    self._finish(r, "length")                  # serving/executor.py:388-389
            if r.status == "finished":
                finished.append(r)
        return finished

    # ---- internals -------------------------------------------------------------------
    def _take_pages(self, r: Request, n: int, plan, planned_ids) -> int:
        """Reserve pages for ``n`` more tokens of a running request; returns how many
        tokens it may run (0: wait)."""
        cache = self.cache
        if cache.can_reserve(r.req_id, r.num_computed + n):
            cache.reserve(r.req_id, r.num_computed + n)
            return n
        if self.policy == "reserve":
            raise RuntimeError(f"request {r.req_id!r} was admitted with its pages reserved and lacks them")
        if n > 1:
            # a prompt portion: shorten it to the pages there are
            held = min(len(t) for t in cache.requests[r.req_id].tables) if cache.groups else 0
            free = min(g.pool.free_count for g in cache.groups) if cache.groups else 0
            n = min(n, (held + free) * cache.page_size - r.num_computed)
            if n > 0:
                cache.reserve(r.req_id, r.num_computed + n)
            return max(n, 0)
        # a decoding request: make room by preempting the youngest running request,
        # which may be this one
        while not cache.can_reserve(r.req_id, r.num_computed + 1):
            live = [v for v in self.running if v.status == "running"]
            v = live[-1]
            if v is r:
                if len(live) == 1:
                    raise RuntimeError(f"request {r.req_id!r} cannot get a page although it runs alone")
                self._preempt(r)
                return 0
            for p in [p for p in plan if p.req is v]:
                plan.remove(p)
                planned_ids.discard(v.req_id)
            self._preempt(v)
        cache.reserve(r.req_id, r.num_computed + 1)
        return 1

    def _preempt(self, r: Request) -> None:
        self.cache.free_request(r.req_id)
        self.running.remove(r)
        r.num_computed = 0
        r.status = "waiting"
        r.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(r)

    def _finish(self, r: Request, reason: str) -> None:
        if r.status == "finished":
            return
        self.cache.free_request(r.req_id)
        self.running.remove(r)
        r.status, r.finish_reason = "finished", reason
        self.done.append(r)
