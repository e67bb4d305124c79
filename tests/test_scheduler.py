"""The scheduler's decisions, with the executor emulated (no device): admission,
order, the token budget, portions, prefill to decode, finishing, abort, and what
happens when pages run out under each policy."""

import pytest

from sllm_b200.cache import CacheManager
from sllm_b200.engine.scheduler import Scheduler
from sllm_b200.parts import PagedKV
from sllm_b200.sampling import SamplingParams


def make(num_pages=64, page=4, **kw):
    cache = CacheManager([("own", PagedKV(1, 16))], page_size=page, num_pages=num_pages,
                         max_requests=kw.get("max_num_seqs", 8))
    kw.setdefault("max_positions", 512)
    return Scheduler(cache, **kw), cache


def run(s, token=lambda r: 1, max_steps=10_000):
    """Emulate execution: every sampled token is `token(request)`.  Returns the step log."""
    log = []
    while s.has_work:
        plan = s.schedule()
        assert plan, "stalled"
        log.append([(p.req.req_id, p.start, p.count, p.sample) for p in plan])
        s.update(plan, {p.req.req_id: token(p.req) for p in plan if p.sample})
        s.cache.check()
        assert len(log) < max_steps
    return log


def test_portions_and_prefill_to_decode():
    s, cache = make(chunk_size=8, max_batch_tokens=100)
    s.add("a", list(range(20)), SamplingParams(max_new=3))
    log = run(s)
    assert [e[0][1:] for e in log] == [(0, 8, False), (8, 8, False), (16, 4, True), (20, 1, True), (21, 1, True)]
    (r,) = s.done
    assert r.output == [1, 1, 1] and r.finish_reason == "length"
    assert cache.groups[0].pool.used_count == 0 and cache.slots.free_count == 8


def test_budget_serves_decodes_first_then_prompts_in_order():
    s, _ = make(chunk_size=16, max_batch_tokens=12, max_num_seqs=4)
    s.add("a", [0] * 4, SamplingParams(max_new=50))
    plan = s.schedule()
    s.update(plan, {"a": 1})                       # a is decoding now
    s.add("b", [0] * 30, SamplingParams(max_new=2))
    s.add("c", [0] * 30, SamplingParams(max_new=2))
    plan = s.schedule()
    assert [(p.req.req_id, p.count) for p in plan] == [("a", 1), ("b", 11)]     # 12 tokens in all
    s.update(plan, {"a": 1})
    plan = s.schedule()
    assert [(p.req.req_id, p.count) for p in plan] == [("a", 1), ("b", 11)]
    s.update(plan, {"a": 1})
    plan = s.schedule()
    assert [(p.req.req_id, p.start, p.count, p.sample) for p in plan] == [("a", 6, 1, True), ("b", 22, 8, True), ("c", 0, 3, False)]


def test_concurrency_cap_fifo_and_continuous_admission():
    s, _ = make(max_num_seqs=2, chunk_size=64)
    for i, n in enumerate((5, 6, 7)):
        s.add(i, [0] * n, SamplingParams(max_new=2 + i))
    log = run(s)
    assert [e[0] for e in log[0]] == [0, 1]
    first_with_2 = next(i for i, st in enumerate(log) if any(e[0] == 2 for e in st))
    assert all(any(e[0] == 0 for e in st) for st in log[:first_with_2])           # 2 enters when 0 has left
    assert [r.req_id for r in s.done] == [0, 1, 2]


def test_reserve_policy_blocks_backfills_and_never_preempts():
    s, cache = make(num_pages=10, page=4, chunk_size=64, policy="reserve")
    s.add("big", [0] * 20, SamplingParams(max_new=12))       # 8 pages
    s.add("huge", [0] * 30, SamplingParams(max_new=6))        # 9 pages: does not fit beside big
    s.add("small", [0] * 3, SamplingParams(max_new=4))        # 2 pages: backfills past huge
    plan = s.schedule()
    assert [p.req.req_id for p in plan] == ["big", "small"]
    assert [r.req_id for r in s.waiting] == ["huge"]
    assert cache.groups[0].pool.used_count == 10              # worst case taken at admission
    log = run(s)
    assert s.num_preemptions == 0
    assert [r.req_id for r in s.done][-1] == "huge"
    with pytest.raises(ValueError, match="whole pool"):
        s.add("never", [0] * 40, SamplingParams(max_new=8))


def test_on_demand_preempts_the_youngest_and_recomputes():
    s, cache = make(num_pages=6, page=4, chunk_size=64, policy="on_demand", max_num_seqs=3)
    s.add("old", [0] * 7, SamplingParams(max_new=10))
    s.add("young", [0] * 7, SamplingParams(max_new=10))
    counter = {"old": 100, "young": 200}

    def token(r):
        counter[r.req_id] += 1
        return counter[r.req_id]
    log = run(s, token)
    assert s.num_preemptions >= 1
    young = next(r for r in s.done if r.req_id == "young")
    old = next(r for r in s.done if r.req_id == "old")
    assert old.preemptions == 0 and young.preemptions >= 1
    assert old.output == list(range(101, 111)) and young.output == list(range(201, 211))   # nothing lost or repeated
    # after preemption the request came back with prompt + the tokens it had produced, from position 0
    again = [e for st in log for e in st if e[0] == "young" and e[1] == 0]
    assert len(again) == 1 + young.preemptions and again[-1][2] > 7
    assert cache.groups[0].pool.used_count == 0


def test_on_demand_shortens_a_prompt_portion_to_the_pages_there_are():
    s, cache = make(num_pages=5, page=4, chunk_size=64, policy="on_demand", max_num_seqs=2)
    s.add("a", [0] * 6, SamplingParams(max_new=1))
    s.add("b", [0] * 18, SamplingParams(max_new=1))
    plan = s.schedule()
    # a takes 2 pages; b starts with the 3 that are left, 12 of its 18 tokens
    assert [(p.req.req_id, p.count, p.sample) for p in plan] == [("a", 6, True), ("b", 12, False)]
    s.update(plan, {"a": 1})
    plan = s.schedule()                        # a has finished and freed its pages
    assert [(p.req.req_id, p.start, p.count, p.sample) for p in plan] == [("b", 12, 6, True)]
    s.update(plan, {"b": 1})
    assert sorted(r.req_id for r in s.done) == ["a", "b"] and not s.has_work


def test_stop_token_is_not_appended_and_context_limit_ends():
    s, _ = make()
    s.add("a", [5, 6], SamplingParams(max_new=10, stop_ids=(9,)))
    toks = iter([3, 4, 9, 7])
    run(s, lambda r: next(toks))
    assert s.done[0].output == [3, 4] and s.done[0].finish_reason == "stop"
    s, _ = make(max_positions=8)
    with pytest.raises(ValueError, match="exceeds"):
        s.add("b", [0] * 6, SamplingParams(max_new=3))
    s.add("b", [0] * 6, SamplingParams(max_new=2))
    run(s)
    assert len(s.done[0].tokens) == 8


def test_abort_and_duplicates():
    s, cache = make(max_num_seqs=1)
    s.add("a", [0] * 5, SamplingParams(max_new=5))
    s.add("b", [0] * 5, SamplingParams(max_new=5))
    with pytest.raises(ValueError, match="already"):
        s.add("a", [1], SamplingParams())
    with pytest.raises(ValueError, match="at least one"):
        s.add("c", [], SamplingParams())
    s.update(s.schedule(), {"a": 1})
    assert s.abort("b") and s.abort("a") and not s.abort("zzz")
    assert not s.has_work and cache.groups[0].pool.used_count == 0
    assert {r.req_id: r.finish_reason for r in s.done} == {"a": "abort", "b": "abort"}


def test_a_step_a_few_tokens_over_a_tile_of_rows_gives_them_back():
    """With ``row_tile`` set (the prompt-portion kernels work in tiles of that many rows), a step that is a few
    tokens over a multiple of the tile shortens a prompt portion by them: the portion no longer samples, the
    tokens come with the next step, nothing is lost; steps under a tile, on a multiple, or further over than the
    slack stay as they are."""
    s, cache = make(num_pages=400, chunk_size=32, max_batch_tokens=100, max_num_seqs=8, row_tile=16, row_tile_slack=4)
    for i in range(3):                                   # three requests that will be decoding
        s.add(f"d{i}", [0] * 2, SamplingParams(max_new=200))
    plan = s.schedule()
    assert sum(p.count for p in plan) == 6               # under a tile: untouched
    s.update(plan, {p.req.req_id: 1 for p in plan if p.sample})
    s.add("p", [0] * 70, SamplingParams(max_new=2))
    plan = s.schedule()                                  # 3 decoded tokens + a portion of 32 = 35 = 2 tiles + 3
    assert [(p.req.req_id, p.count, p.sample) for p in plan] == [("d0", 1, True), ("d1", 1, True), ("d2", 1, True), ("p", 29, False)]
    s.update(plan, {p.req.req_id: 1 for p in plan if p.sample})
    plan = s.schedule()                                  # the portion goes on where it stopped
    assert (plan[-1].req.req_id, plan[-1].start, plan[-1].count) == ("p", 29, 29)
    s.update(plan, {p.req.req_id: 1 for p in plan if p.sample})
    plan = s.schedule()                                  # 3 + the last 12 = 15: under a tile, and the portion samples
    assert (plan[-1].start, plan[-1].count, plan[-1].sample) == (58, 12, True)
    s.update(plan, {p.req.req_id: 1 for p in plan if p.sample})
    # further over than the slack: 3 + 32 + ... a second prompt of 25 tokens: 3 + 1 + 25 = 29 = a tile + 13
    s.add("q", [0] * 25, SamplingParams(max_new=2))
    plan = s.schedule()
    assert sum(p.count for p in plan) == 29 and plan[-1].count == 25 and plan[-1].sample
    log = run(s)
    assert not s.has_work and all(r.finish_reason == "length" for r in s.done)
    assert {r.req_id: len(r.output) for r in s.done} == {"d0": 200, "d1": 200, "d2": 200, "p": 2, "q": 2}
    assert cache.groups[0].pool.used_count == 0


def test_the_last_portion_of_a_prompt_that_is_trimmed_samples_a_step_later():
    s, _ = make(num_pages=400, chunk_size=64, max_batch_tokens=100, row_tile=16, row_tile_slack=8)
    s.add("a", [0] * 35, SamplingParams(max_new=1))      # 35 = 2 tiles + 3
    log = run(s)
    assert [e[0][1:] for e in log] == [(0, 32, False), (32, 3, True)]
