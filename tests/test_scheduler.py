"""The scheduler's decisions, with the real cache manager and no GPU: order within a step,
the token budget, portions, admission, finishing, and what happens when pages run out."""

import random

import pytest

from yalis_b200.cache.manager import CacheManager, PageGroup
from yalis_b200.engine.scheduler import FINISHED, RUNNING, WAITING, Request, Scheduler
from yalis_b200.sampling.sampler import GREEDY


def make(pages=64, page=4, slots=4, budget=16, chunk=None, max_context=None):
    m = CacheManager(slots, [PageGroup("kv_all", page, pages, None, 256)])
    return m, Scheduler(m, max_tokens_per_step=budget, prefill_chunk=chunk, max_context=max_context)


def run(sched, manager, next_token=lambda r: 7, max_steps=10_000):
    """Drive the scheduler without a model; returns the per-step plans as tuples."""
    log = []
    for _ in range(max_steps):
        if not sched.has_work():
            return log
        plan = sched.plan()
        log.append(plan)
        sched.update(plan, [next_token(e.request) for e in plan.entries if e.samples])
        manager.check()
    raise AssertionError("the scheduler did not finish")


def shape(plan):
    return [(e.request.id, e.start, e.count, e.samples) for e in plan.entries]


def test_whole_prompt_then_decode_until_length():
    m, s = make()
    r = Request("a", [1, 2, 3, 4, 5], 3, GREEDY)
    s.add(r)
    log = run(s, m)
    assert [shape(p) for p in log] == [[("a", 0, 5, True)], [("a", 5, 1, True)], [("a", 6, 1, True)]]
    assert r.output == [7, 7, 7] and r.finish_reason == "length" and r.state == FINISHED
    assert m.free_pages("kv_all") == 64 and m.free_slots() == 4     # everything given back


def test_portions_under_chunk_and_budget():
    m, s = make(budget=10, chunk=6)
    s.add(Request("a", list(range(14)), 1, GREEDY))
    s.add(Request("b", list(range(9)), 1, GREEDY))
    log = run(s, m)
    assert shape(log[0]) == [("a", 0, 6, False), ("b", 0, 4, False)]          # chunk caps a, budget caps b
    assert shape(log[1]) == [("a", 6, 6, False), ("b", 4, 4, False)]          # older request first
    # a last single token is scheduled like a decode: first
    assert shape(log[2]) == [("b", 8, 1, True), ("a", 12, 2, True)]
    assert all(p.n_tokens <= 10 for p in log)


def test_decodes_come_before_portions_and_admissions():
    m, s = make(budget=8, chunk=8)
    s.add(Request("a", [1, 2, 3], 4, GREEDY))
    run_one = s.plan(); s.update(run_one, [7])
    s.add(Request("b", list(range(20)), 2, GREEDY))
    plan = s.plan()
    assert shape(plan) == [("a", 3, 1, True), ("b", 0, 7, False)]             # decode first, rest of the budget to b


def test_eos_finishes_and_frees_within_the_update():
    m, s = make(slots=1)
    a = Request("a", [1, 2, 3], 10, GREEDY, eos_id=9)
    b = Request("b", [4, 5], 2, GREEDY)
    s.add(a); s.add(b)
    p = s.plan()
    assert shape(p) == [("a", 0, 3, True)]                                    # one slot: b waits
    done = s.update(p, [9])
    assert done == [a] and a.finish_reason == "eos" and a.output == [9]
    assert shape(s.plan()) == [("b", 0, 2, True)]                             # admitted in the very next plan


def test_context_limit_clamps_new_tokens_and_refuses_long_prompts():
    m, s = make(max_context=8)
    r = Request("a", [1] * 6, 50, GREEDY)
    s.add(r)
    assert r.max_new_tokens == 3                                              # 6 + 3 - 1 tokens held at most
    with pytest.raises(ValueError):
        s.add(Request("b", [1] * 9, 1, GREEDY))
    with pytest.raises(ValueError):
        s.add(Request("c", [], 1, GREEDY))
    run(s, m)
    assert len(r.output) == 3 and m.length(0) == 0


def test_decode_out_of_pages_preempts_the_youngest():
    # 6 pages of 4. a: 8 tokens (2 pages), b: 8 tokens (2 pages), c: 7 tokens (2 pages): pool full.
    m, s = make(pages=6, page=4, slots=4, budget=64)
    a, b, c = (Request(n, [1] * k, 6, GREEDY) for n, k in (("a", 8), ("b", 8), ("c", 7)))
    for r in (a, b, c):
        s.add(r)
    p = s.plan(); s.update(p, [7, 7, 7])
    assert m.free_pages("kv_all") == 0
    p = s.plan()
    # a and b need a third page each; c (the youngest) gives way and its two pages serve both
    assert [r.id for r in p.preempted] == ["c"] and shape(p) == [("a", 8, 1, True), ("b", 8, 1, True)]
    assert c.state == WAITING and c.computed == 0 and c.slot is None and c.preemptions == 1
    assert list(s.waiting)[0] is c                                            # back at the head of the queue
    assert c not in [e.request for e in p.entries]                            # and not readmitted in the same step
    s.update(p, [7, 7])
    log = run(s, m)
    assert all(r.finish_reason == "length" and len(r.output) == 6 for r in (a, b, c))
    # a preempted request is recomputed from all its tokens, its outputs kept
    readmit = [e for pl in log for e in pl.entries if e.request is c and e.start == 0][0]
    assert readmit.count == len(c.prompt) + 1


def test_request_that_can_never_fit_fails_alone():
    m, s = make(pages=2, page=4, slots=2, budget=64)
    big = Request("big", [1] * 8, 5, GREEDY)          # fills the pool, cannot decode its 9th token
    s.add(big)
    log = run(s, m)
    assert big.finish_reason == "out_of_pages" and big.state == FINISHED
    assert log[-1].failed == [big] and m.free_pages("kv_all") == 2
    # a prompt larger than the whole pool is prefilled in what fits, then fails the same way
    m, s = make(pages=2, page=4, slots=2, budget=64)
    huge = Request("huge", [1] * 20, 1, GREEDY)
    s.add(huge)
    run(s, m)
    assert huge.finish_reason == "out_of_pages" and m.free_pages("kv_all") == 2


def test_portion_shrinks_to_the_free_pages():
    m, s = make(pages=5, page=4, slots=2, budget=64)
    a = Request("a", [1] * 12, 8, GREEDY)             # 3 pages
    s.add(a)
    p = s.plan(); s.update(p, [7])
    b = Request("b", [1] * 20, 1, GREEDY)             # wants 5 pages, 2 are free
    s.add(b)
    p = s.plan()
    assert shape(p) == [("a", 12, 1, True), ("b", 0, 4, False)]               # a's decode took a page; one page left for b
    s.update(p, [7])
    assert m.free_pages("kv_all") == 0


@pytest.mark.parametrize("seed", range(5))
def test_random_load_always_finishes_and_frees(seed):
    rng = random.Random(seed)
    page = rng.choice([1, 4, 16])
    pages = rng.choice([24, 40])
    m, s = make(pages=pages, page=page, slots=rng.choice([2, 4]), budget=rng.choice([8, 32]),
                chunk=rng.choice([None, 5]), max_context=200)
    reqs = [Request(i, [1] * rng.randint(1, 60), rng.randint(1, 20), GREEDY, eos_id=3) for i in range(12)]
    for r in reqs:
        s.add(r)
    run(s, m, next_token=lambda r: rng.choice([3, 5, 5, 5, 5, 5, 5, 5]))
    for r in reqs:
        assert r.state == FINISHED and r.finish_reason in ("length", "eos", "out_of_pages")
        if r.finish_reason == "length":
            assert len(r.output) == r.max_new_tokens
        if r.finish_reason == "eos":
            assert r.output[-1] == 3 and 3 not in r.output[:-1]
    assert m.free_pages("kv_all") == pages and not s.running and not s.waiting
