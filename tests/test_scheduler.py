"""The scheduler's decisions, without a GPU: the cache manager only keeps accounts."""

import pytest

from mini_llm_stack_b200.cache.manager import CacheManager
from mini_llm_stack_b200.engine.request import FINISHED, Request
from mini_llm_stack_b200.engine.scheduler import Scheduler, SchedulerError
from mini_llm_stack_b200.parts.base import PagedKV


def make(num_blocks=8, block_size=4, max_batch=4, budget=16, chunk=8, max_seq_len=64,
         specs=(PagedKV(2, 16),)):
    cache = CacheManager(list(specs), num_blocks, block_size, max_batch, max_seq_len,
                         allocate=False)
    return Scheduler(cache, max_batch, budget, chunk, max_seq_len), cache


def run(sched, token=lambda req: 100 + len(req.generated), max_steps=1000, log=None):
    """Drive the scheduler with a stand-in for the model: returns the plans."""
    plans = []
    while sched.has_work():
        plan = sched.plan()
        plans.append(plan)
        if log is not None:
            log.append([(p.request.req_id, p.n_tokens, p.wants_logits) for p in plan.entries])
        sched.cache.check()
        for p in plan.entries:                     # what the step function does
            sched.cache.commit(p.request.req_id, p.n_tokens)
        sched.complete(plan, {p.request.req_id: token(p.request) for p in plan.entries
                              if p.wants_logits})
        assert len(plans) < max_steps
    return plans


def test_prompt_is_cut_under_chunk_and_budget_then_decodes():
    s, _ = make(num_blocks=16, budget=12, chunk=8)
    a = Request(0, list(range(19)), max_new_tokens=3)
    s.add(a)
    log = []
    run(s, log=log)
    assert log == [[(0, 8, False)], [(0, 8, False)], [(0, 3, True)], [(0, 1, True)], [(0, 1, True)]]
    assert a.state == FINISHED and a.generated == [100, 101, 102]
    assert s.cache.num_free_pages() == 16


def test_decodes_come_first_and_share_the_step_with_portions():
    s, _ = make(num_blocks=32, budget=10, chunk=8)
    a = Request(0, [1, 2, 3], max_new_tokens=4)
    s.add(a)
    p0 = s.plan()
    s.cache.commit(0, 3)
    s.complete(p0, {0: 9})
    b = Request(1, list(range(20)), max_new_tokens=2)
    c = Request(2, list(range(5)), max_new_tokens=2)
    s.add(b)
    s.add(c)
    p1 = s.plan()
    got = [(p.request.req_id, p.n_tokens, p.wants_logits) for p in p1.entries]
    # a decodes (1 token), b gets a portion of 8, c the last token of the budget
    assert got == [(0, 1, True), (1, 8, False), (2, 1, False)]
    assert p1.n_tokens == 10 and [r.req_id for r in p1.admitted] == [1, 2]


def test_fcfs_admission_stops_at_the_first_that_does_not_fit():
    # serve/engine.py:190-198: no skipping over the head of the line
    s, cache = make(num_blocks=6, block_size=4, budget=64, chunk=64)
    big = Request(0, list(range(20)), max_new_tokens=2)       # needs 6 pages for 21 tokens
    small = Request(1, [1, 2], max_new_tokens=2)
    blocker = Request(2, list(range(6)), max_new_tokens=10)
    s.add(blocker)
    p0 = s.plan()
    s.cache.commit(2, 6)
    s.complete(p0, {2: 5})
    s.add(big)
    s.add(small)
    plan = s.plan()
    assert [p.request.req_id for p in plan.entries] == [2]     # big does not fit, small waits
    assert list(s.waiting) == [big, small]


def test_max_batch_limits_running():
    s, _ = make(num_blocks=32, max_batch=2)
    for i in range(4):
        s.add(Request(i, [1, 2, 3], max_new_tokens=2))
    plan = s.plan()
    assert len(plan.entries) == 2 and len(s.running) == 2 and len(s.waiting) == 2
    run(s)
    assert [r.req_id for r in s.finished] == [0, 1, 2, 3]


def test_finish_rules():
    s, _ = make(num_blocks=16, max_seq_len=12)
    a = Request(0, [1, 2, 3], max_new_tokens=50, eos_token=7)
    b = Request(1, [1, 2, 3], max_new_tokens=50)
    c = Request(2, [1, 2, 3], max_new_tokens=2)
    for r in (a, b, c):
        s.add(r)
    run(s, token=lambda req: 7 if (req.req_id == 0 and len(req.generated) == 2) else 1)
    assert a.generated == [1, 1, 7]                 # eos is kept (serve/engine.py:220)
    assert len(b.tokens) == 12                      # stops at max_seq_len (:221)
    assert len(c.generated) == 2                    # max_new_tokens (:219)


def test_out_of_pages_preempts_the_newest_and_recomputes():
    # 6 requests of 5 + 6 tokens in 8 pages of 4 (the reference's few-pages test,
    # tests/test_serving.py:164-179): all must finish with 6 tokens
    s, cache = make(num_blocks=8, block_size=4, max_batch=6, budget=64, chunk=64)
    reqs = [Request(i, [i + 1] * 5, max_new_tokens=6) for i in range(6)]
    for r in reqs:
        s.add(r)
    log = []
    plans = run(s, log=log)
    assert all(len(r.generated) == 6 for r in reqs)
    assert len(plans) > 6 and s.preemptions > 0
    victims = [v for p in plans for v in p.preempted]
    assert victims and all(v.preemptions >= 1 for v in victims)
    # a victim is the newest running request and goes to the front of the line
    first = next(p for p in plans if p.preempted)
    assert first.preempted[0].req_id == max(
        x.request.req_id for x in first.entries + [type("P", (), {"request": first.preempted[0]})])
    # after re-admission the whole token list is run again in one portion
    v = victims[0]
    redo = [e for step in log for e in step if e[0] == v.req_id and e[1] > 1]
    assert len(redo) >= 2 and redo[-1][1] > 5
    assert cache.num_free_pages() == 8
    cache.check()


def test_preempted_request_keeps_its_tokens():
    s, cache = make(num_blocks=4, block_size=4, max_batch=2, budget=64, chunk=64)
    a = Request(0, [1] * 6, max_new_tokens=8)
    b = Request(1, [2] * 5, max_new_tokens=8)
    s.add(a)
    s.add(b)
    run(s)
    assert a.generated == [100 + i for i in range(8)]
    assert b.generated == [100 + i for i in range(8)]
    assert b.preemptions >= 1 and a.preemptions == 0


def test_requests_that_can_never_fit_are_refused_at_submit():
    s, _ = make(num_blocks=4, block_size=4, max_seq_len=64)
    with pytest.raises(SchedulerError, match="never fit"):
        s.add(Request(0, [1] * 10, max_new_tokens=10))
    with pytest.raises(SchedulerError, match="too long"):
        s.add(Request(1, [1] * 64, max_new_tokens=1))
    with pytest.raises(SchedulerError, match="at least one"):
        s.add(Request(2, [], max_new_tokens=1))
    s.add(Request(3, [1] * 10, max_new_tokens=6))            # 16 tokens = 4 pages: fits


def test_window_group_needs_fewer_pages_over_time():
    s, cache = make(num_blocks=6, block_size=4, budget=8, chunk=8, max_seq_len=64,
                    specs=(PagedKV(2, 16, window=6),))
    a = Request(0, list(range(20)), max_new_tokens=20)       # 40 tokens > 6 pages * 4
    s.add(a)
    run(s)
    assert len(a.generated) == 20 and cache.paged[0].pool.high_water <= 5
