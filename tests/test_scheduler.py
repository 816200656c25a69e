"""The scheduler's decisions, on the CPU, against the cache manager's bookkeeping.  The model
is faked: the token after a sequence is a fixed function of that sequence, so any schedule
must produce the same tokens."""
import pytest

from litellmengine_b200.cache import CacheManager, OutOfPages, PagedNeed
from litellmengine_b200.engine.request import RequestStatus
from litellmengine_b200.engine.scheduler import Scheduler


def fake_next(ids):
    return (sum((i + 1) * t for i, t in enumerate(ids)) * 31 + len(ids)) % 97


def make(pages, page=4, slots=4, budget=16, chunk=None, window=None, longest=None):
    cache = CacheManager([PagedNeed(1, 16, window)], page_size=page, max_total_tokens=pages * page, max_slots=slots,
                         max_request_tokens=longest)
    return cache, Scheduler(cache, max_tokens_per_step=budget, chunk=chunk)


def run_step(cache, sched):
    """What the engine does around a step, minus the GPU."""
    plan = sched.schedule()
    for p in plan:
        r = p.request
        assert cache.length(r.slot) == r.cached_len
        cache.ensure(r.slot, r.cached_len + p.num_tokens)
    sampled = []
    for p in plan:
        r = p.request
        cache.commit(r.slot, r.cached_len + p.num_tokens)
        if p.samples:
            sampled.append(fake_next(r.input_ids))
    done = sched.update(plan, sampled)
    cache.check_invariants()
    return plan, done


def run_all(cache, sched, limit=500):
    steps = []
    while sched.has_work():
        steps.append(run_step(cache, sched)[0])
        assert len(steps) < limit
    return steps


def expected(prompt, n, eos=-1):
    ids, new = list(prompt), []
    for _ in range(n):
        t = fake_next(ids)
        ids.append(t)
        new.append(t)
        if t == eos:
            break
    return new


def test_budget_portions_and_decode_first():
    cache, s = make(pages=32, budget=8, chunk=6)
    a = s.add(list(range(1, 11)), 3)          # 10 prompt tokens
    b = s.add(list(range(20, 25)), 3)         # 5
    p1, _ = run_step(cache, s)
    assert [(p.request.request_id, p.num_tokens, p.samples) for p in p1] == [(0, 6, False), (1, 2, False)]
    p2, _ = run_step(cache, s)                # a: 4 left (ends its prompt), b: 3 left
    assert [(p.request.request_id, p.num_tokens, p.samples) for p in p2] == [(0, 4, True), (1, 3, True)]
    p3, _ = run_step(cache, s)                # both decode: one token each
    assert [(p.request.request_id, p.num_tokens, p.samples) for p in p3] == [(0, 1, True), (1, 1, True)]
    c = s.add(list(range(30, 50)), 2)         # arrives while others decode: decoders go first
    p4, done = run_step(cache, s)
    assert [(p.request.request_id, p.num_tokens) for p in p4] == [(0, 1), (1, 1), (2, 6)]
    assert {r.request_id for r in done} == {0, 1}
    run_all(cache, s)
    assert a.generated_ids == expected(range(1, 11), 3) and b.generated_ids == expected(range(20, 25), 3)
    assert c.generated_ids == expected(range(30, 50), 2)
    assert all(g.pool.free_count == g.pool.num_pages for g in cache.groups) and cache.free_slots == 4


def test_first_come_first_served_without_overtaking():
    cache, s = make(pages=6, budget=64)       # 24 tokens of cache
    big = s.add(list(range(1, 21)), 2)        # 20 tokens: 5 pages
    big2 = s.add(list(range(1, 17)), 2)       # 16 tokens: does not fit beside big
    small = s.add([1, 2], 2)                  # would fit, but must not overtake big2
    p1, _ = run_step(cache, s)
    assert [p.request.request_id for p in p1] == [0]
    assert big2.status is RequestStatus.WAITING and small.status is RequestStatus.WAITING
    run_all(cache, s)
    assert [r.generated_ids for r in (big, big2, small)] == [expected(range(1, 21), 2), expected(range(1, 17), 2),
                                                            expected([1, 2], 2)]


def test_finish_rules():
    cache, s = make(pages=16)
    z = s.add([5, 6], 0)
    assert z.finished and z.finish_reason == "length" and not s.has_work()
    free = expected([3, 4, 5], 6)
    r = s.add([3, 4, 5], 6, eos_token_id=free[2])
    run_all(cache, s)
    assert r.generated_ids == free[:free.index(free[2]) + 1] and r.finish_reason == "eos"   # eos is kept
    assert r.cached_len == len(r.input_ids) - 1           # the last sampled token is never run
    r2 = s.add([3, 4, 5], 4)
    run_all(cache, s)
    assert r2.generated_ids == free[:4] and r2.finish_reason == "length"
    with pytest.raises(ValueError):
        s.add([], 3)
    with pytest.raises(ValueError):
        s.add([1], 3, temperature=-1.0)


def test_a_request_that_can_never_fit_is_refused_at_add():
    cache, s = make(pages=4)                  # 16 tokens
    with pytest.raises(OutOfPages, match="at most 16"):
        s.add(list(range(10)), 8)             # 10 + 7 cached tokens
    ok = s.add(list(range(10)), 7)            # 10 + 6 = 16
    run_all(cache, s)
    assert ok.generated_ids == expected(range(10), 7)


def test_pages_run_out_latest_request_is_preempted_and_recomputed():
    cache, s = make(pages=6, budget=64)       # 24 tokens
    a = s.add(list(range(1, 9)), 12)          # 8 prompt -> up to 19 cached: 5 pages
    b = s.add(list(range(11, 19)), 12)        # same; both start (2 + 2 pages), then collide
    steps = run_all(cache, s)
    assert s.num_preemptions >= 1 and b.preemptions >= 1 and a.preemptions == 0     # the later one yields
    assert a.generated_ids == expected(range(1, 9), 12) and b.generated_ids == expected(range(11, 19), 12)
    # after the preemption b was recomputed from its first token, prompt and generated together
    redo = [p for plan in steps for p in plan if p.request is b and p.num_tokens > 8]
    assert redo, "b must come back with more than its prompt to recompute"
    assert all(g.pool.free_count == g.pool.num_pages for g in cache.groups)


def test_same_adds_same_schedule():
    def trace():
        cache, s = make(pages=7, budget=12, chunk=5)
        for i in range(5):
            s.add(list(range(i + 1, i + 8)), 6)
        return [[(p.request.request_id, p.num_tokens, p.samples) for p in plan] for plan in run_all(cache, s)]
    assert trace() == trace()


def test_window_group_lets_long_requests_share_few_pages():
    cache, s = make(pages=6, page=4, budget=8, chunk=4, window=6, longest=64)   # 24 tokens of pages
    a = s.add(list(range(1, 30)), 20)         # 48 cached tokens through 6 pages
    with pytest.raises(OutOfPages):
        s.add(list(range(1, 40)), 200)        # beyond the per-request limit even with a window
    run_all(cache, s)
    assert a.generated_ids == expected(range(1, 30), 20)
    cache, s = make(pages=6, page=4, budget=8, chunk=4, window=None, longest=64)
    with pytest.raises(OutOfPages, match="at most 24"):
        s.add(list(range(1, 30)), 20)         # without a window the pool is the limit


# ---- tokens read one step late --------------------------------------------------------------
def run_pipelined(cache, sched, limit=2000):
    """The engine's pipelined loop, minus the GPU: a step is launched (`advance`) before the
    tokens of the step before it are read (`deliver`).  The fake device knows every token, so
    a portion that ends with a pending token is checked to be exactly the next one."""
    in_flight, steps = None, 0
    device_ids = {}                                       # request id -> ids as the device has seen them
    while sched.has_work() or in_flight:
        plan = sched.schedule()
        launched = None
        if plan:
            sampled = []
            for p in plan:
                r = p.request
                assert cache.length(r.slot) == r.cached_len
                cache.ensure(r.slot, r.cached_len + p.num_tokens)
                cache.commit(r.slot, r.cached_len + p.num_tokens)
                end = r.cached_len + p.num_tokens
                assert end <= len(r.input_ids) + r.pending
                if end > len(r.input_ids):                # the last token comes from the step before
                    assert r.pending == 1 and in_flight is not None
                    prev_plan, prev_sampled = in_flight
                    owners = [q.request for q in prev_plan if q.samples]
                    assert owners[r.feedback_index] is r
                if p.samples:                             # the device holds every token sampled so far
                    ids = device_ids.setdefault(r.request_id, list(r.input_ids[:r.prompt_len]))
                    assert ids[:len(r.input_ids)] == r.input_ids and len(ids) == end
                    ids.append(fake_next(ids))
                    sampled.append(ids[-1])
            sched.advance(plan)
            launched = (plan, sampled)
        if in_flight:
            sched.deliver(*in_flight)
        in_flight = launched
        cache.check_invariants()
        steps += 1
        assert steps < limit
    return steps


@pytest.mark.parametrize("pages,budget,chunk", [(64, 16, None), (12, 8, 5), (9, 16, 3)])
def test_reading_tokens_one_step_late_gives_the_same_tokens(pages, budget, chunk):
    cache, s = make(pages=pages, budget=budget, chunk=chunk, slots=3)
    prompts = [[3, 1, 4, 1, 5, 9, 2], [6, 5], [3, 5, 8, 9, 7, 9, 3, 2, 3, 8, 4], [1], [2, 7, 1, 8]]
    news = [6, 9, 4, 1, 7]
    reqs = [s.add(p, n) for p, n in zip(prompts, news)]
    run_pipelined(cache, s)
    for r, p, n in zip(reqs, prompts, news):
        assert r.finished and r.generated_ids == expected(p, n) and r.pending == 0, (r.generated_ids, expected(p, n))
    assert cache.groups[0].pool.free_count == pages and cache.free_slots == 3


def test_a_request_awaiting_its_last_token_is_not_scheduled_again():
    cache, s = make(pages=16)
    a = s.add([5, 6, 7], 2)
    plan = s.schedule()
    s.advance(plan)                                        # prompt launched: first token pending
    assert a.pending == 1 and a.remain_len == 1 and a.extend_len == 1
    plan2 = s.schedule()
    assert [(p.request, p.num_tokens, p.samples) for p in plan2] == [(a, 1, True)]
    s.advance(plan2)
    s.deliver(plan, [11])
    assert a.pending == 1 and a.remain_len == 0           # its second and last token is on its way
    assert s.schedule() == []                              # nothing to launch, and no OutOfPages either
    s.deliver(plan2, [12])
    assert a.finished and a.generated_ids == [11, 12] and not s.has_work()


def test_end_of_sequence_found_one_step_late_drops_the_extra_token():
    cache, s = make(pages=16)
    a = s.add([5, 6, 7], 10, eos_token_id=42)
    b = s.add([1, 2], 10)
    p1 = s.schedule(); s.advance(p1)
    p2 = s.schedule(); s.advance(p2)                       # both decode on, their first tokens unread
    got = s.deliver(p1, [42, 9])                           # a's first token was its end of sequence
    assert [(r.request_id, t) for r, t in got] == [(a.request_id, 42), (b.request_id, 9)]
    assert a.finished and a.finish_reason == "eos" and a.slot == -1
    p3 = s.schedule()                                      # a is gone from the plan
    assert [p.request for p in p3] == [b]
    s.advance(p3)
    got = s.deliver(p2, [77, 10])                          # 77 was sampled for a after its end: dropped
    assert [(r.request_id, t) for r, t in got] == [(b.request_id, 10)]
    assert a.generated_ids == [42] and b.generated_ids == [9, 10]
    cache.check_invariants()
