"""The cache manager: keys and values in pages with a block table per request,
one pool per group of layers with the same need, and slots for per-request
state of fixed size.

The reference pairs a page allocator with a state-slot allocator per sequence
(runtime/blocks.py:114-179) but backs no tensors with it (runtime/blocks.py:1-7;
its device cache is contiguous and doubles, kernels/device_decode.py:220-263).
Here the pages are the storage.  Runs of the run list whose mixers ask for the
same thing (kv heads, head size, window) form a group: one pool, one block
table per request, one page id meaning the same page in every layer of the
group.  A group with a window gives pages back as soon as the window has passed
them; everything a request holds goes back when it ends.

Bookkeeping needs no device; `allocate_storage` creates the tensors.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..parts.base import LayerCache, PagedKV, SlotState
from .pools import OutOfPages, PagePool, SlotPool


RUN_TOKENS = 64      # the attention kernels' key tile: its pages are one copy when their ids are consecutive


@dataclass
class CacheGroup:
    need: PagedKV
    runs: list[int]
    pool: PagePool


@dataclass
class RequestCache:
    req_id: object
    slot: int
    num_tokens: int = 0                       # tokens committed to the cache
    tables: list[list[int]] = field(default_factory=list)   # per group: page ids, -1 once released


class CacheManager:
    def __init__(self, needs, *, page_size: int, num_pages, max_requests: int, poison_freed: bool = False):
        """``needs``: per run ``("own", PagedKV|SlotState|None)`` or ``("borrow", run)``
        (`CausalLM.cache_needs`).  ``num_pages``: pages per group (an int for all
        groups, or one per group).  ``poison_freed`` (a debugging aid, off by default): a page
        that goes back to its pool is filled with NaN in every layer and zeroed again when it is
        handed out, so that a read of a page the reader no longer holds shows in the logits."""
        self.poison_freed = bool(poison_freed)
        if page_size < 1:
            raise ValueError("page_size must be >= 1")
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        # one state slot beyond the requests': rows that pad a batch to a captured size use it
        self.padding_slot = self.max_requests
        self.needs = list(needs)
        self.groups: list[CacheGroup] = []
        self.run_group: dict[int, int] = {}        # run -> group (owning runs)
        self.state_runs: dict[int, SlotState] = {}
        by_need: dict[PagedKV, int] = {}
        for run, (how, what) in enumerate(self.needs):
            if how == "borrow":
                continue
            if isinstance(what, PagedKV):
                if what not in by_need:
                    by_need[what] = len(self.groups)
                    self.groups.append(CacheGroup(what, [], None))
                g = by_need[what]
                self.groups[g].runs.append(run)
                self.run_group[run] = g
            elif isinstance(what, SlotState):
                self.state_runs[run] = what
            elif what is not None:
                raise TypeError(f"run {run}: unknown cache need {what!r}")
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(self.groups)
        if len(num_pages) != len(self.groups):
            raise ValueError(f"num_pages names {len(num_pages)} groups, the model has {len(self.groups)}")
        # ids are best held in runs of a 64-key tile's pages (see pools.py)
        for g, n in zip(self.groups, num_pages):
            g.pool = PagePool(n, run=max(1, RUN_TOKENS // self.page_size))
        self.slots = SlotPool(self.max_requests)
        self.requests: dict[object, RequestCache] = {}
        self.kv_storage = []       # per group: tensor [runs, 2, pages, nkv, page_size, hd]
        self.state_storage = {}    # run -> tensor [slots, *shape]
        self.slot_tables = {}      # name -> tensor [slots, ...] of per-request state that others own (`register_slot_table`)
        self.reuse_count = 0       # pages handed out that had been held before
        self._ever_used = [set() for _ in self.groups]

    # ---- arithmetic -------------------------------------------------------------
    def pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size) if tokens > 0 else 0

    def _first_needed_page(self, g: CacheGroup, committed: int) -> int:
        """First page a query at position ``committed`` (the next one) still reads."""
        if g.need.window is None:
            return 0
        return max(0, committed - g.need.window + 1) // self.page_size

    def _extra_pages(self, req: RequestCache | None, total_tokens: int) -> list[int]:
        out = []
        for gi, g in enumerate(self.groups):
            have = len(req.tables[gi]) if req else 0
            out.append(max(0, self.pages_for(total_tokens) - have))
        return out

    def can_reserve(self, req_id, total_tokens: int) -> bool:
        req = self.requests.get(req_id)
        if req is None and not self.slots.free_count:
            return False
        extra = self._extra_pages(req, total_tokens)
        return all(e <= g.pool.free_count for e, g in zip(extra, self.groups))

    def fits_at_all(self, total_tokens: int) -> bool:
        """Could a request of this many tokens ever be held, with the pools empty?"""
        n = self.pages_for(total_tokens)
        for g in self.groups:
            need = n if g.need.window is None else min(n, self.pages_for(g.need.window) + 1)
            if need > g.pool.capacity:
                return False
        return True

    # ---- life of a request -----------------------------------------------------------
    def add_request(self, req_id) -> RequestCache:
        if req_id in self.requests:
            raise ValueError(f"request {req_id!r} is already live")
        slot = self.slots.allocate(req_id)
        req = RequestCache(req_id, slot, 0, [[] for _ in self.groups])
        self.requests[req_id] = req
        for t in (*self.state_storage.values(), *self.slot_tables.values()):
            t[slot].zero_()
        return req

    def register_slot_table(self, name: str, table) -> None:
        """Per-request state of fixed size that lives outside the model (the sampler's table of
        seen ids): one row per state slot and one for padding rows; a request's row is zeroed when
        it is admitted, like the mixers' own state."""
        if table.shape[0] != self.max_requests + 1:
            raise ValueError(f"slot table {name!r} has {table.shape[0]} rows, the cache has {self.max_requests} + 1 slots")
        self.slot_tables[name] = table

    def reserve(self, req_id, total_tokens: int) -> None:
        """Grow the request's tables to hold ``total_tokens``.  Takes all pages
        or none: `OutOfPages` leaves every pool as it was."""
        req = self.requests[req_id]
        extra = self._extra_pages(req, total_tokens)
        if not any(extra):          # (most decode steps: the token lands in a page the request holds)
            return
        for e, g in zip(extra, self.groups):
            if e > g.pool.free_count:
                raise OutOfPages(f"request {req_id!r} needs {e} more pages for {total_tokens} tokens, "
                                 f"{g.pool.free_count} free of {g.pool.capacity}")
        for gi, (e, g) in enumerate(zip(extra, self.groups)):
            tail = req.tables[gi][-1] if req.tables[gi] and req.tables[gi][-1] >= 0 else None
            ids = g.pool.allocate(req_id, e, after=tail)
            self.reuse_count += sum(1 for p in ids if p in self._ever_used[gi])
            self._ever_used[gi].update(ids)
            req.tables[gi].extend(ids)
            if self.poison_freed:
                self._fill_pages(gi, ids, 0.0)

    def commit(self, req_id, total_tokens: int) -> None:
        """``total_tokens`` of the request now lie in the cache.  Pages that a
        window has passed go back to their pool."""
        req = self.requests[req_id]
        if total_tokens < req.num_tokens:
            raise ValueError("a request's token count cannot shrink")
        if any(self.pages_for(total_tokens) > len(t) for t in req.tables):
            raise ValueError(f"request {req_id!r}: {total_tokens} tokens committed beyond its reserved pages")
        req.num_tokens = total_tokens
        for gi, g in enumerate(self.groups):
            if g.need.window is None:
                continue
            first = self._first_needed_page(g, total_tokens)
            table = req.tables[gi]
            gone = [table[i] for i in range(min(first, len(table))) if table[i] >= 0]
            if gone:
                g.pool.free(req_id, gone)
                if self.poison_freed:
                    self._fill_pages(gi, gone, float("nan"))
                for i in range(min(first, len(table))):
                    table[i] = -1

    def free_request(self, req_id) -> None:
        req = self.requests.get(req_id)
        if req is None:
            raise KeyError(f"request {req_id!r} is not live")
        # free before forgetting: an ownership error must not lose the table
        for gi, g in enumerate(self.groups):
            held = [p for p in req.tables[gi] if p >= 0]
            g.pool.free(req_id, held)
            if self.poison_freed:
                self._fill_pages(gi, held, float("nan"))
        self.slots.free(req_id, req.slot)
        del self.requests[req_id]

    def _fill_pages(self, group: int, pages, value: float) -> None:
        """Keys and values of ``pages`` in every run of the group (nothing before `allocate_storage`)."""
        if pages and group < len(self.kv_storage):
            import torch
            idx = torch.as_tensor(list(pages), dtype=torch.long, device=self.kv_storage[group].device)
            self.kv_storage[group].index_fill_(2, idx, value)

    def slot_of_token(self, req_id, group: int, position: int) -> int:
        """Flat slot (page * page_size + offset) of a token position."""
        page = self.requests[req_id].tables[group][position // self.page_size]
        if page < 0:
            raise ValueError(f"request {req_id!r}: position {position} lies in a page already given back")
        return page * self.page_size + position % self.page_size

    def check(self) -> None:
        """No page lost, held twice or free while listed in a table."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            listed = []
            for req in self.requests.values():
                listed.extend(p for p in req.tables[gi] if p >= 0)
            assert len(listed) == len(set(listed)), "a page stands in two tables"
            assert set(listed) == set(g.pool._owner), "tables and pool disagree"
            for req in self.requests.values():
                for p in req.tables[gi]:
                    assert p < 0 or g.pool.owner_of(p) == req.req_id
        self.slots.check()

    # ---- storage -----------------------------------------------------------------------
    def bytes_per_token(self, itemsize: int) -> int:
        """Sum over caching runs of 2 * kv heads * head size * itemsize
        (runtime/memory_planner.py:12-15)."""
        return sum(len(g.runs) * 2 * g.need.num_kv_heads * g.need.head_dim * itemsize for g in self.groups)

    def state_bytes_per_request(self) -> int:
        """Bytes of fixed-size float32 state each request holds in the mixers' slots (tables that others
        register with `register_slot_table` are theirs to count)."""
        total = 0
        for s in self.state_runs.values():
            n = 4
            for d in s.shape:
                n *= int(d)
            total += n
        return total

    def describe(self) -> list[str]:
        """One line per cache group and one for the state slots: what the model asks of the cache."""
        lines = []
        for gi, g in enumerate(self.groups):
            w = "all keys" if g.need.window is None else f"a window of {g.need.window}"
            lines.append(f"group {gi}: {len(g.runs)} runs x {g.need.num_kv_heads} kv heads of {g.need.head_dim}, {w}")
        if self.state_runs:
            lines.append(f"state slots: {len(self.state_runs)} runs, {self.state_bytes_per_request()} bytes per request")
        return lines

    def allocate_storage(self, dtype, device) -> list[LayerCache]:
        """Create the page and state tensors; returns one `LayerCache` per run."""
        import torch
        self.kv_storage = []
        for g in self.groups:
            shape = (len(g.runs), 2, max(g.pool.capacity, 1), g.need.num_kv_heads, self.page_size, g.need.head_dim)
            # with the debugging aid on, pages nobody holds are NaN from the start
            fill = float("nan") if self.poison_freed else 0.0
            self.kv_storage.append(torch.full(shape, fill, dtype=dtype, device=device))
        self.state_storage = {
            run: torch.zeros((self.max_requests + 1,) + tuple(s.shape), dtype=torch.float32, device=device)
            for run, s in self.state_runs.items()}
        caches: list[LayerCache] = []
        for run, (how, what) in enumerate(self.needs):
            src = what if how == "borrow" else run
            if src in self.run_group:
                gi = self.run_group[src]
                i = self.groups[gi].runs.index(src)
                caches.append(LayerCache(group=gi, k=self.kv_storage[gi][i, 0], v=self.kv_storage[gi][i, 1]))
            elif src in self.state_runs:
                caches.append(LayerCache(state=self.state_storage[src]))
            else:
                caches.append(LayerCache())
        return caches
