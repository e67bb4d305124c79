"""The cache manager without a device: no page lost, held twice or freed twice, under
random orders of requests; windows give pages back; state slots."""

import random

import pytest

from sllm_b200.cache import CacheManager, OutOfPages, PagePool, SlotPool
from sllm_b200.parts import PagedKV, SlotState


def test_page_pool_lowest_first_and_ownership():
    p = PagePool(6)
    assert p.allocate("a", 3) == [0, 1, 2] and p.allocate("b", 2) == [3, 4]
    with pytest.raises(OutOfPages):
        p.allocate("c", 2)
    assert p.free_count == 1                                 # a failed allocation takes nothing
    with pytest.raises(ValueError, match="not held"):
        p.free("b", [0])
    with pytest.raises(ValueError, match="twice"):
        p.free("a", [1, 1])
    with pytest.raises(ValueError):
        p.free("a", [0, 3])                                  # validated before anything is freed
    assert p.owned("a") == [0, 1, 2]
    p.free("a", [1])
    with pytest.raises(ValueError, match="not held"):
        p.free("a", [1])                                     # freed twice
    assert p.allocate("c", 2) == [1, 5]                      # lowest ids first
    p.check()


def test_page_pool_hands_out_runs():
    """A pool told that ids are best held in runs of 4: owners that grow by a page at a time, in turn,
    each get consecutive ids inside aligned groups; when no group is wholly free the rest of other owners'
    groups is used, lowest id first; the books stay right throughout."""
    p = PagePool(24, run=4)
    tails = {}
    for _ in range(4):                                       # three owners, four rounds of one page each
        for o in "abc":
            (tails[o],) = p.allocate(o, 1, after=tails.get(o))
            p.check()
    assert p.owned("a") == [0, 1, 2, 3] and p.owned("b") == [4, 5, 6, 7] and p.owned("c") == [8, 9, 10, 11]
    # a group ends: the next one is the lowest wholly free group, not the id after the tail
    assert p.allocate("a", 1, after=3) == [12]
    assert p.allocate("b", 6, after=7) == [16, 17, 18, 19, 20, 21]      # whole groups first, in order
    # no wholly free group is left (12 is a's, 20..21 b's): c takes the lowest free ids, whoever's group they are in
    assert p.allocate("c", 2, after=11) == [13, 14]
    assert p.allocate("a", 1, after=12) == [15]              # a's own group, what is left of it
    p.free("b", [16, 17, 18, 19])
    assert p.allocate("c", 1, after=14) == [16]              # a group came back whole
    with pytest.raises(OutOfPages):
        p.allocate("c", 6, after=16)
    p.check()
    assert p.free_count == 5
    # without a tail, or with runs of one, it is "lowest free id first"
    q = PagePool(6, run=1)
    assert q.allocate("a", 2, after=4) == [0, 1]


def test_requests_that_grow_in_turn_hold_runs_of_pages():
    """Eight requests decoding side by side, a page each every few steps: every request's table is made of
    aligned runs of 64 tokens' pages (what the attention kernels fetch as one copy), not of every eighth id."""
    m = _manager(num_pages=8 * 24, page=16, window=None, max_requests=8, layers=1)
    for r in range(8):
        m.add_request(r)
        m.reserve(r, 40 + r)                                  # prompts of different lengths: 3 pages each
        m.commit(r, 40 + r)
    for n in range(48, 360, 8):                              # then they grow together
        for r in range(8):
            m.reserve(r, n)
            m.commit(r, n)
        m.check()
    for r in range(8):
        t = m.requests[r].tables[0]
        assert len(t) == 22
        runs = sum(1 for i in range(0, len(t) - 3, 4) if t[i] % 4 == 0 and t[i:i + 4] == list(range(t[i], t[i] + 4)))
        assert runs == 5, (r, t)                             # every whole group of four is one run


def test_slot_pool():
    s = SlotPool(2)
    assert s.allocate("a") == 0 and s.allocate("b") == 1
    with pytest.raises(OutOfPages):
        s.allocate("c")
    with pytest.raises(ValueError):
        s.free("a", 1)
    s.free("a", 0)
    assert s.allocate("c") == 0
    s.check()


def _manager(num_pages=12, page=4, window=None, max_requests=4, layers=3):
    needs = [("own", PagedKV(2, 16, window)) for _ in range(layers)]
    return CacheManager(needs, page_size=page, num_pages=num_pages, max_requests=max_requests)


def test_reserve_commit_free():
    m = _manager()
    assert len(m.groups) == 1 and m.groups[0].runs == [0, 1, 2]
    assert m.bytes_per_token(2) == 3 * 2 * 2 * 16 * 2
    m.add_request("a")
    m.reserve("a", 9)
    assert m.requests["a"].tables[0] == [0, 1, 2]
    m.reserve("a", 9)                                        # no more pages for the same count
    assert m.groups[0].pool.used_count == 3
    with pytest.raises(ValueError, match="beyond"):
        m.commit("a", 13)
    m.commit("a", 9)
    assert m.slot_of_token("a", 0, 6) == 1 * 4 + 2
    with pytest.raises(ValueError, match="already live"):
        m.add_request("a")
    m.add_request("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 40)
    assert m.requests["b"].tables[0] == [] and m.groups[0].pool.used_count == 3   # all or nothing
    assert not m.can_reserve("b", 40) and m.can_reserve("b", 36)
    m.free_request("a")
    with pytest.raises(KeyError):
        m.free_request("a")
    m.free_request("b")
    m.check()
    assert m.groups[0].pool.free_count == 12 and m.slots.free_count == 4


def test_groups_by_need_and_borrowed_cache():
    needs = [("own", PagedKV(2, 16)), ("own", PagedKV(2, 16, 8)), ("own", PagedKV(2, 16)), ("borrow", 0),
             ("own", SlotState((3, 5))), ("own", None)]
    m = CacheManager(needs, page_size=4, num_pages=[10, 6], max_requests=2)
    assert [g.runs for g in m.groups] == [[0, 2], [1]]
    m.add_request("a")
    m.reserve("a", 20)
    assert len(m.requests["a"].tables[0]) == 5 and len(m.requests["a"].tables[1]) == 5
    m.commit("a", 20)                          # the window group has let go of what lies behind it
    assert m.requests["a"].tables[1][:3] == [-1, -1, -1] and m.groups[1].pool.used_count == 2
    assert m.groups[0].pool.used_count == 5
    import torch
    caches = m.allocate_storage(torch.float32, "cpu")
    assert caches[3].k.data_ptr() == caches[0].k.data_ptr() and caches[3].group == 0
    assert caches[1].group == 1 and caches[4].state.shape == (2 + 1, 3, 5) and caches[5].k is None     # one spare slot for padding rows


def test_window_gives_pages_back():
    m = _manager(num_pages=6, page=4, window=6, layers=1)
    m.add_request("a")
    total = 0
    for n in (5, 3, 1, 1, 7, 2, 1, 1, 1, 4):
        total += n
        m.reserve("a", total)
        m.commit("a", total)
        m.check()
        first_needed = max(0, total - 6 + 1) // 4
        table = m.requests["a"].tables[0]
        assert all(p == -1 for p in table[:first_needed]) and all(p >= 0 for p in table[first_needed:])
        if first_needed:
            with pytest.raises(ValueError, match="given back"):
                m.slot_of_token("a", 0, 0)
    assert total == 26 and m.groups[0].pool.used_count <= 3     # 26 tokens would need 7 pages without the window
    assert m.reuse_count > 0
    m.free_request("a")
    m.check()
    assert m.groups[0].pool.free_count == 6


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 10])
def test_random_orders_keep_the_books(seed, window):
    rng = random.Random(seed)
    m = _manager(num_pages=20, page=4, window=window, max_requests=5, layers=2)
    live = {}
    next_id = 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            m.add_request(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.8 and live:
            r = rng.choice(list(live))
            n = live[r] + rng.choice([1, 1, 1, 2, 5, 9])
            if m.can_reserve(r, n):
                m.reserve(r, n)
                m.commit(r, n)
                live[r] = n
            else:
                before = m.groups[0].pool.free_count
                with pytest.raises(OutOfPages):
                    m.reserve(r, n)
                assert m.groups[0].pool.free_count == before
        elif live:
            r = rng.choice(list(live))
            m.free_request(r)
            del live[r]
        m.check()
        held = sum(sum(1 for p in m.requests[r].tables[0] if p >= 0) for r in live)
        assert held == m.groups[0].pool.used_count
    for r in list(live):
        m.free_request(r)
    m.check()
    assert m.groups[0].pool.free_count == 20 and m.slots.free_count == 5


def test_slot_tables_of_others_are_zeroed_at_admission():
    """Per-request state that lives outside the model (the sampler's seen ids) registers with the
    cache manager: one row per state slot and one for padding; a row is zeroed when a request takes
    the slot, and only then."""
    import torch
    cm = CacheManager([("own", PagedKV(2, 16, None))], page_size=4, num_pages=8, max_requests=2)
    with pytest.raises(ValueError):
        cm.register_slot_table("seen", torch.ones(2, 5))
    table = torch.ones(3, 5)
    cm.register_slot_table("seen", table)
    a = cm.add_request("a")
    assert table[a.slot].sum() == 0 and table.sum() == 10
    table[a.slot] = 7
    b = cm.add_request("b")
    assert table[b.slot].sum() == 0 and table[a.slot].sum() == 35
    cm.free_request("a")
    assert table[a.slot].sum() == 35                       # giving the slot back changes nothing
    c = cm.add_request("c")
    assert c.slot == a.slot and table[c.slot].sum() == 0


def test_freed_pages_are_poisoned_and_fresh_ones_zeroed_when_asked():
    """The debugging aid: a page that goes back to its pool (at the request's end, or when a window has
    passed it) holds NaN in every layer of its group; a page handed out holds zeros."""
    import torch
    needs = [("own", PagedKV(2, 4, None)), ("own", PagedKV(2, 4, None)), ("own", PagedKV(1, 4, 8))]
    cm = CacheManager(needs, page_size=4, num_pages=6, max_requests=2, poison_freed=True)
    cm.allocate_storage(torch.float32, "cpu")
    assert all(bool(t.isnan().all()) for t in cm.kv_storage)
    cm.add_request("a")
    cm.reserve("a", 10)
    held = cm.requests["a"].tables[0]
    assert bool((cm.kv_storage[0][:, :, held] == 0).all())
    others = [p for p in range(6) if p not in held]
    assert bool(cm.kv_storage[0][:, :, others].isnan().all())
    cm.kv_storage[1][:, :, cm.requests["a"].tables[1]] = 1.0
    cm.commit("a", 10)                                            # window 8: position 10 reads from 3 on; page 0 stays
    cm.reserve("a", 14)
    cm.commit("a", 14)                                            # reads from 7 on: page 0 has gone back
    t1 = cm.requests["a"].tables[1]
    assert t1[0] == -1 and bool(cm.kv_storage[1][:, :, 0].isnan().all()) and bool((cm.kv_storage[1][:, :, t1[1]] == 1).all())
    cm.free_request("a")
    assert all(bool(t.isnan().all()) for t in cm.kv_storage)
    cm.check()
    # off by default: nothing is filled
    cm = CacheManager(needs, page_size=4, num_pages=6, max_requests=2)
    cm.allocate_storage(torch.float32, "cpu")
    cm.add_request("a")
    cm.reserve("a", 5)
    cm.free_request("a")
    assert all(bool((t == 0).all()) for t in cm.kv_storage)
