"""The scheduler's decisions, on the host-side allocator alone (no GPU)."""
import random

import pytest

from sandyrt_b200.cache.pages import BlockAllocator, CacheLayout
from sandyrt_b200.engine.scheduler import Request, RequestRefused, RequestState, Scheduler
from sandyrt_b200.parts.base import PagedKVSpec


def _sched(pages=16, page_size=16, max_requests=4, **kw):
    layout = CacheLayout.from_specs([PagedKVSpec(2, 16)] * 2, page_size)
    alloc = BlockAllocator(layout, [pages], max_requests)
    kw.setdefault("max_live", max_requests)
    return Scheduler(alloc, **kw), alloc


def _run(sched, alloc, token_of=lambda req: 7, max_steps=10_000):
    """Drive plan/complete until idle; returns the list of plans."""
    plans = []
    while sched.has_work():
        plan = sched.plan()
        assert plan.portions, "a step with live requests must move something"
        assert plan.n_tokens <= sched.max_step_tokens
        for p in plan.portions:                       # what a step may hold
            assert p.count >= 1 and p.start == p.request.computed
            assert alloc.length(p.request.rid) == p.start
            assert len(alloc.block_list(p.request.rid, 0)) * alloc.page_size >= p.start + p.count
        sampled = {p.request.rid: token_of(p.request) for p in plan.portions if p.samples}
        sched.complete(plan, sampled)
        alloc.check()
        plans.append(plan)
        assert len(plans) < max_steps
    return plans


def test_refusals():
    sched, _ = _sched(pages=4, max_positions=128)
    with pytest.raises(RequestRefused, match="empty"):
        sched.add(Request("a", [], 4))
    with pytest.raises(RequestRefused, match="max_tokens"):
        sched.add(Request("a", [1], -1))
    with pytest.raises(RequestRefused, match="positions"):
        sched.add(Request("a", [1] * 129, 4))
    with pytest.raises(RequestRefused, match="pool has 4"):
        sched.add(Request("a", [1] * 60, 10))         # grows to 69 tokens = 5 pages


def test_max_tokens_zero_finishes_without_a_step():
    sched, _ = _sched()
    r = Request("a", [1, 2, 3], 0)
    sched.add(r)
    assert r.state is RequestState.FINISHED and r.finish_reason == "length" and not sched.has_work()


def test_prompt_is_cut_under_the_budget_and_decodes_go_first():
    sched, alloc = _sched(pages=32, max_step_tokens=24, prefill_chunk=16)
    a, b = Request("a", list(range(40)), 3), Request("b", list(range(10)), 5)
    sched.add(a); sched.add(b)
    p1 = sched.plan()
    assert [(p.request.rid, p.start, p.count, p.samples) for p in p1.portions] == \
        [("a", 0, 16, False), ("b", 0, 8, False)]     # chunk limit 16, then what is left of 24
    sched.complete(p1, {})
    p2 = sched.plan()
    assert [(p.request.rid, p.start, p.count, p.samples) for p in p2.portions] == \
        [("a", 16, 16, False), ("b", 8, 2, True)]
    sched.complete(p2, {"b": 5})
    p3 = sched.plan()                                  # b decodes first, a gets the rest of its prompt
    assert [(p.request.rid, p.start, p.count, p.samples) for p in p3.portions] == \
        [("b", 10, 1, True), ("a", 32, 8, True)]
    sched.complete(p3, {"a": 1, "b": 2})
    assert a.output == [1] and b.output == [5, 2]


def test_finish_reasons_and_freeing():
    sched, alloc = _sched(max_positions=20)
    stop = Request("s", [1, 2, 3], 10, stop_ids=frozenset([99]))
    length = Request("l", [1, 2, 3], 4)
    ctx = Request("c", [1] * 18, 10)                  # runs into the model's 20 positions
    for r in (stop, length, ctx):
        sched.add(r)
    tokens = {"s": iter([5, 99, 6]), "l": iter(range(10, 20)), "c": iter(range(30, 50))}
    _run(sched, alloc, token_of=lambda req: next(tokens[req.rid]))
    assert (stop.output, stop.finish_reason) == ([5, 99], "stop")        # the stop token is kept
    assert (length.output, length.finish_reason) == ([10, 11, 12, 13], "length")
    assert ctx.finish_reason == "length" and len(ctx.prompt) + len(ctx.output) == 21
    assert alloc.free_pages() == 16 and alloc.free_slots() == 4 and not alloc.live()


def test_admission_is_first_come_first_served_and_bounded():
    sched, alloc = _sched(pages=64, max_requests=2)
    reqs = [Request(i, [1] * 5, 3) for i in range(5)]
    for r in reqs:
        sched.add(r)
    plan = sched.plan()
    assert [p.request.rid for p in plan.portions] == [0, 1]              # two slots only
    sched.complete(plan, {0: 1, 1: 1})
    order = []
    while sched.has_work():
        plan = sched.plan()
        order += [p.request.rid for p in plan.portions if p.start == 0]
        sched.complete(plan, {p.request.rid: 1 for p in plan.portions if p.samples})
    assert order == [2, 3, 4]
    assert all(r.finish_reason == "length" for r in reqs)


def test_out_of_pages_preempts_the_newest_and_recomputes_it():
    # 6 pages of 4 tokens.  Two requests of 8 prompt tokens fill 4 pages; decoding grows both
    # until the pool is empty; then the newer one must give way and is recomputed later.
    sched, alloc = _sched(pages=6, page_size=4, max_requests=4)
    a, b = Request("a", [1] * 8, 12), Request("b", [2] * 8, 12)
    sched.add(a); sched.add(b)
    counter = iter(range(100, 1000))
    plans = _run(sched, alloc, token_of=lambda req: next(counter))
    assert b.preemptions >= 1 and a.preemptions == 0
    assert sched.stats["preemptions"] == b.preemptions
    assert len(a.output) == 12 and len(b.output) == 12
    # after its preemption b came back with prompt + output so far as one portion from 0
    back = [p for plan in plans for p in plan.portions if p.request is b and p.start == 0]
    assert len(back) == 1 + b.preemptions and back[-1].count > 8
    # the preempted request was not scheduled in the step that preempted it
    for plan in plans:
        for r in plan.preempted:
            assert all(p.request is not r for p in plan.portions)
    assert alloc.free_pages() == 6


def test_stuck_prompts_do_not_deadlock():
    # Two long prompts admitted together cannot both finish their prompt in 8 pages.
    sched, alloc = _sched(pages=8, page_size=4, max_requests=4, prefill_chunk=8, max_step_tokens=16)
    a, b = Request("a", [1] * 24, 2), Request("b", [2] * 24, 2)
    sched.add(a); sched.add(b)
    _run(sched, alloc)
    assert a.finish_reason == b.finish_reason == "length"
    assert len(a.output) == 2 and len(b.output) == 2


@pytest.mark.parametrize("seed", range(6))
def test_random_load_always_drains(seed):
    rng = random.Random(seed)
    sched, alloc = _sched(pages=rng.choice([8, 12, 24]), page_size=rng.choice([4, 8]), max_requests=rng.choice([2, 4]),
                          prefill_chunk=rng.choice([3, 8, 64]), max_step_tokens=rng.choice([8, 32]), max_positions=64)
    reqs = []
    for i in range(12):
        n, m = rng.randint(1, 30), rng.randint(1, 20)
        r = Request(i, [rng.randrange(50) for _ in range(n)], m, stop_ids=frozenset([3]))
        try:
            sched.add(r)
            reqs.append(r)
        except RequestRefused:
            pass
    _run(sched, alloc, token_of=lambda req: rng.randrange(50))
    for r in reqs:
        assert r.state is RequestState.FINISHED and r.finish_reason in ("stop", "length")
        assert 1 <= len(r.output) <= r.max_tokens
        if r.finish_reason == "stop":
            assert r.output[-1] == 3 and 3 not in r.output[:-1]
    assert alloc.free_pages() == alloc.pools[0].num_pages and not alloc.live()
