"""Allocators of page ids and state slots, with ownership checks.

Behaviour after the reference's bookkeeping (runtime/blocks.py:31-111): ids
``0..capacity-1``; the lowest free id is given out first (a min-heap); an
allocation that does not fit raises and takes nothing; a free validates every
id (held by that owner, not listed twice) before it changes anything.
"""

from __future__ import annotations

import heapq


class OutOfPages(Exception):
    """The pool cannot give what was asked.  Nothing was taken."""


class PagePool:
    def __init__(self, capacity: int):
        if capacity < 0:
            raise ValueError("capacity must be >= 0")
        self.capacity = int(capacity)
        self._free = list(range(self.capacity))       # a valid min-heap
        self._owner: dict[int, object] = {}

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.capacity - len(self._free)

    def allocate(self, owner, count: int) -> list[int]:
        if count < 0:
            raise ValueError("count must be >= 0")
        if count > len(self._free):
            raise OutOfPages(f"need {count} pages, {len(self._free)} free of {self.capacity}")
        ids = [heapq.heappop(self._free) for _ in range(count)]
        for p in ids:
            self._owner[p] = owner
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
            heapq.heappush(self._free, p)

    def owner_of(self, page: int):
        return self._owner.get(page)

    def owned(self, owner) -> list[int]:
        return sorted(p for p, o in self._owner.items() if o == owner)

    def check(self) -> None:
        """Every id is free or held, never both, never lost."""
        free = set(self._free)
        assert len(free) == len(self._free), "a page is in the free list twice"
        held = set(self._owner)
        assert not (free & held), f"pages both free and held: {sorted(free & held)}"
        assert free | held == set(range(self.capacity)), "a page was lost"


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
