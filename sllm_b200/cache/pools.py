"""Allocators of page ids and state slots, with ownership checks.

Behaviour after the reference's bookkeeping (runtime/blocks.py:31-111): ids
``0..capacity-1``; the lowest free id is given out first; an allocation that does
not fit raises and takes nothing; a free validates every id (held by that owner,
not listed twice) before it changes anything.

Beyond the reference: a pool may be told that ids are best held in RUNS (aligned
groups of ``run`` consecutive ids).  The attention kernels fetch a 64-key tile whose
pages have consecutive ids as one box instead of one per page, so a request's table
should read p, p+1, p+2, ... even when many requests grow by a page at a time.  An
owner that names its last page gets the next id if that is free and lies in the same
group; otherwise the first page of the lowest wholly free group; only when no group
is wholly free the lowest free id of all.  Nothing is set aside: the rest of a group
stays free, and is simply the last choice of everybody else.  With ``run`` = 1 this
is "lowest free id first".
"""

from __future__ import annotations

import heapq


class OutOfPages(Exception):
    """The pool cannot give what was asked.  Nothing was taken."""


class PagePool:
    def __init__(self, capacity: int, run: int = 1):
        if capacity < 0:
            raise ValueError("capacity must be >= 0")
        if run < 1:
            raise ValueError("run must be >= 1")
        self.capacity = int(capacity)
        self.run = int(run)
        self._free = set(range(self.capacity))
        self._heap = list(range(self.capacity))       # free ids, a valid min-heap; may hold ids no longer free
        self._owner: dict[int, object] = {}
        groups = -(-self.capacity // self.run) if self.capacity else 0
        self._group_size = [min(self.run, self.capacity - g * self.run) for g in range(groups)]
        self._group_free = list(self._group_size)     # free ids per group
        self._whole = list(range(groups))             # wholly free groups, a min-heap; may hold groups no longer whole

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.capacity - len(self._free)

    def _take(self, p: int, owner) -> int:
        self._free.remove(p)
        self._group_free[p // self.run] -= 1
        self._owner[p] = owner
        return p

    def _lowest_free(self) -> int:
        while self._heap[0] not in self._free:
            heapq.heappop(self._heap)
        return self._heap[0]                          # stays in the heap: `_take` makes it stale, a later call pops it

    def _lowest_whole_group(self):
        while self._whole:
            g = self._whole[0]
            if self._group_free[g] == self._group_size[g]:
                return g
            heapq.heappop(self._whole)
        return None

    def allocate(self, owner, count: int, after: int | None = None) -> list[int]:
        """``count`` ids for ``owner``.  ``after``: the id the owner holds last (its table's tail), so that the
        new ones continue its run where they can."""
        if count < 0:
            raise ValueError("count must be >= 0")
        if count > len(self._free):
            raise OutOfPages(f"need {count} pages, {len(self._free)} free of {self.capacity}")
        ids = []
        for _ in range(count):
            nxt = None if after is None else after + 1
            if self.run > 1 and nxt is not None and nxt % self.run != 0 and nxt in self._free:
                p = nxt                                # the owner's group goes on
            else:
                g = self._lowest_whole_group() if self.run > 1 else None
                p = g * self.run if g is not None else self._lowest_free()
            ids.append(self._take(p, owner))
            after = p
        return ids

    def free(self, owner, ids) -> None:
        ids = list(ids)
        seen = set()
        for p in ids:
            if p in seen:
                raise ValueError(f"page {p} listed twice")
            seen.add(p)
            if p not in self._owner or self._owner[p] != owner:
                raise ValueError(f"page {p} is not held by {owner!r}")
        for p in ids:
            del self._owner[p]
            self._free.add(p)
            heapq.heappush(self._heap, p)
            g = p // self.run
            self._group_free[g] += 1
            if self._group_free[g] == self._group_size[g]:
                heapq.heappush(self._whole, g)
        if len(self._heap) > 4 * self.capacity + 16:  # stale entries do not pile up
            self._heap = sorted(self._free)
            self._whole = [g for g in range(len(self._group_size)) if self._group_free[g] == self._group_size[g]]

    def owner_of(self, page: int):
        return self._owner.get(page)

    def owned(self, owner) -> list[int]:
        return sorted(p for p, o in self._owner.items() if o == owner)

    def check(self) -> None:
        """Every id is free or held, never both, never lost; the group counts agree."""
        free = self._free
        held = set(self._owner)
        assert not (free & held), f"pages both free and held: {sorted(free & held)}"
        assert free | held == set(range(self.capacity)), "a page was lost"
        assert free <= set(self._heap), "a free page is missing from the heap"
        for g, n in enumerate(self._group_free):
            lo = g * self.run
            assert n == sum(1 for p in range(lo, lo + self._group_size[g]) if p in free), f"group {g}: free count off"
            assert n < self._group_size[g] or g in self._whole, f"group {g} is wholly free and not listed"


class SlotPool:
    """One fixed-size state slot per request (runtime/blocks.py:80-111)."""

    def __init__(self, capacity: int):
        if capacity < 0:
            raise ValueError("capacity must be >= 0")
        self.capacity = int(capacity)
        self._free = list(range(self.capacity))
        self._owner: dict[int, object] = {}

    @property
    def free_count(self) -> int:
        return len(self._free)

    def allocate(self, owner) -> int:
        if not self._free:
            raise OutOfPages("no state slot left")
        s = heapq.heappop(self._free)
        self._owner[s] = owner
        return s

    def free(self, owner, slot: int) -> None:
        if slot not in self._owner or self._owner[slot] != owner:
            raise ValueError(f"state slot {slot} is not held by {owner!r}")
        del self._owner[slot]
        heapq.heappush(self._free, slot)

    def check(self) -> None:
        free = set(self._free)
        assert len(free) == len(self._free)
        assert not (free & set(self._owner))
        assert free | set(self._owner) == set(range(self.capacity))
