"""The cache manager: pages, block tables, windows, state slots (CPU)."""

import random

import numpy as np
import pytest
import torch

from mini_llm_stack_b200.cache.manager import CacheError, CacheManager
from mini_llm_stack_b200.cache.page_pool import PagePool, PagePoolError
from mini_llm_stack_b200.cache.state_slots import SlotPoolError, StateSlotPool
from mini_llm_stack_b200.parts.base import FixedState, PagedKV

FULL = PagedKV(2, 16)
WIN = PagedKV(2, 16, window=10)


def _mgr(specs=(FULL, FULL), num_blocks=8, block_size=4, max_requests=4, max_seq_len=64,
         allocate=False):
    return CacheManager(list(specs), num_blocks, block_size, max_requests, max_seq_len,
                        allocate=allocate)


def test_page_accounting_like_the_reference():
    # tests/test_serving.py:22-33 of the reference: 8 pages of 4 tokens
    c = _mgr()
    assert c.can_hold(32) and not c.can_hold(33)
    assert c.admit("a") and c.reserve("a", 9)
    assert c.num_free_pages() == 5
    assert c.admit("b") and c.reserve("b", 4)
    assert c.num_free_pages() == 4
    c.free("a")
    assert c.num_free_pages() == 7
    c.free("b")
    assert c.num_free_pages() == 8
    c.check()


def test_a_page_is_claimed_only_at_its_boundary():
    # tests/test_serving.py:36-46 of the reference
    c = _mgr(num_blocks=4)
    c.admit(0)
    assert c.reserve(0, 3)
    c.commit(0, 3)
    assert c.reserve(0, 1) and len(c.pages_of(0)) == 1
    c.commit(0, 1)
    assert c.reserve(0, 1) and len(c.pages_of(0)) == 2
    c.admit(1)
    assert c.reserve(1, 8)
    c.commit(1, 8)
    before = c.pages_of(1)
    assert not c.reserve(1, 1)                   # no free page: nothing changes
    assert c.pages_of(1) == before and c.num_free_pages() == 0
    c.check()


def test_lifo_reuse_and_first_page_zero():
    c = _mgr()
    c.admit("a")
    c.reserve("a", 8)
    assert c.pages_of("a") == [0, 1]             # page 0 is handed out first
    c.admit("b")
    c.reserve("b", 4)
    assert c.pages_of("b") == [2]
    c.free("a")
    c.admit("c")
    c.reserve("c", 12)
    assert c.pages_of("c") == [0, 1, 3]          # freed pages are used again first
    c.check()


def test_reserve_is_all_groups_or_none():
    c = _mgr(specs=(FULL, WIN, FULL), num_blocks=3)
    c.admit("a")
    assert c.reserve("a", 12)
    c.admit("b")
    assert not c.reserve("b", 1)
    assert all(g.pool.num_free == 0 for g in c.paged)
    c.free("a")
    assert c.reserve("b", 1)
    c.check()


def test_groups_by_need_and_handles():
    specs = [FULL, WIN, FULL, FixedState((3, 5)), WIN, None]
    c = CacheManager(specs, 6, 4, 3, 32, device="cpu", kv_dtype=torch.float32)
    assert [g.members for g in c.paged] == [[0, 2], [1, 4]]
    assert [g.members for g in c.fixed] == [[3]]
    h = c.handles()
    assert [x.kind for x in h] == ["paged", "paged", "paged", "fixed", "paged", "none"]
    assert h[0].group == h[2].group == 0 and h[1].group == h[4].group == 1
    assert h[1].window == 10 and h[0].window is None
    assert h[0].k_pool.shape == (2, 6, 4, 16) and h[3].state.shape == (3, 3, 5)
    # members of a group have memory of their own
    assert h[0].k_pool.data_ptr() != h[2].k_pool.data_ptr()


def test_window_gives_pages_back_when_passed():
    c = _mgr(specs=(FULL, WIN), num_blocks=16, block_size=4, max_seq_len=64)
    c.admit("r")
    total = 0
    for n in (7, 9, 1, 1, 6, 1):
        assert c.reserve("r", n)
        c.commit("r", n)
        total += n
        full = c.pages_of("r", 0)
        win = c.pages_of("r", 1)
        assert len(full) == len(win) == c.pages_for(total)
        assert -1 not in full
        # keys < total - window + 1 are never read again; whole pages of them are gone
        dead = max(0, total - 10 + 1) // 4
        assert [p == -1 for p in win] == [i < dead for i in range(len(win))]
        c.check()
    assert c.paged[1].pool.num_held == len([p for p in c.pages_of("r", 1) if p >= 0])
    c.free("r")
    assert c.paged[0].pool.num_free == 16 and c.paged[1].pool.num_free == 16
    c.check()


def test_truncate_gives_whole_pages_back():
    c = _mgr(specs=(FULL, FULL), num_blocks=8, block_size=4)
    c.admit("r")
    assert c.reserve("r", 14)
    c.commit("r", 14)
    assert c.num_free_pages() == 4
    c.truncate("r", 14)                                   # nothing to do
    c.truncate("r", 9)                                    # pages 0..2 stay, page 3 goes back
    assert c.length("r") == 9 and c.pages_of("r", 0)[:3] == [0, 1, 2] and c.num_free_pages() == 5
    c.check()
    assert c.reserve("r", 4)                              # grows again from token 9, page 3 again
    c.commit("r", 4)
    assert c.pages_of("r", 0) == [0, 1, 2, 3]
    c.truncate("r", 0)
    assert c.length("r") == 0 and c.num_free_pages() == 8
    with pytest.raises(CacheError):
        c.truncate("r", 1)
    c.check()
    c.free("r")
    # a window that has let pages go cannot be cut back to where it would read them
    w = _mgr(specs=(FULL, WIN), num_blocks=16, block_size=4, max_seq_len=64)
    w.admit("r")
    assert w.reserve("r", 30)
    w.commit("r", 30)                                     # keys < 21 are gone: five pages
    w.truncate("r", 29)                                   # reads keys >= 20: all still there
    with pytest.raises(CacheError, match="window"):
        w.truncate("r", 20)
    w.check()
    # state of fixed size cannot go back either
    f = _mgr(specs=(FULL, FixedState((3,))), num_blocks=8, block_size=4)
    f.admit("r")
    assert f.reserve("r", 5)
    f.commit("r", 5)
    with pytest.raises(CacheError, match="fixed size"):
        f.truncate("r", 3)


def test_step_arrays():
    c = _mgr(num_blocks=8, block_size=4, max_seq_len=32)
    c.admit("a")
    c.admit("b")
    c.reserve("a", 6)
    c.commit("a", 6)
    c.reserve("b", 3)
    c.reserve("a", 1)
    arr = c.step_arrays([("b", 3), ("a", 1)])
    table, slots = arr[0]
    assert table.shape == (2, 8) and table.dtype == np.int32
    pa, pb = c.pages_of("a"), c.pages_of("b")
    assert list(table[0, :1]) == pb and list(table[1, :2]) == pa and table[0, 1] == -1
    assert list(slots) == [pb[0] * 4, pb[0] * 4 + 1, pb[0] * 4 + 2, pa[1] * 4 + 2]
    with pytest.raises(CacheError, match="no page reserved"):
        c.step_arrays([("a", 4)])


def test_slots_and_limits():
    c = _mgr(max_requests=2)
    assert c.admit(1) and c.admit(2) and not c.admit(3)
    assert not c.can_hold(1)
    with pytest.raises(CacheError, match="already"):
        c.admit(1)
    with pytest.raises(CacheError, match="block table"):
        c.reserve(1, 65)
    assert c.fits_at_all(32) and not c.fits_at_all(33)
    c.free(1)
    assert c.admit(3) and c.row(3) == 0          # the slot freed last comes first
    c.check()


def test_fixed_state_is_zeroed_when_claimed():
    c = CacheManager([FixedState((4,))], 1, 4, 2, 16, device="cpu")
    c.admit("a")
    c.fixed[0].state[0, c.row("a")] = 7.0
    c.free("a")
    c.admit("b")
    assert c.row("b") == 0 and float(c.fixed[0].state[0, 0].abs().sum()) == 0.0


def test_pool_errors():
    p = PagePool(3)
    got = p.take(2, "x")
    assert p.take(2, "y") is None and p.num_free == 1
    with pytest.raises(PagePoolError, match="belongs"):
        p.give(got, "y")
    p.give(got, "x")
    with pytest.raises(PagePoolError, match="twice"):
        p.give(got[:1], "x")
    with pytest.raises(PagePoolError, match="not in the pool"):
        p.give([9], "x")
    s = StateSlotPool(1)
    a = s.claim("x")
    assert s.claim("y") is None
    s.release(a, "x")
    with pytest.raises(SlotPoolError):
        s.release(a, "x")


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    specs = (FULL, WIN, FULL) if seed % 2 else (FULL,)
    c = _mgr(specs=specs, num_blocks=12, block_size=4, max_requests=5, max_seq_len=40)
    live, next_id = {}, 0
    for _ in range(600):
        act = rng.random()
        if act < 0.25 and len(live) < 5:
            if c.admit(next_id):
                live[next_id] = 0
            next_id += 1
        elif act < 0.8 and live:
            r = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 7])
            if live[r] + n <= 40:
                before = [g.pool.num_free for g in c.paged]
                if c.reserve(r, n):
                    c.commit(r, n)
                    live[r] += n
                    assert c.length(r) == live[r]
                else:
                    assert before == [g.pool.num_free for g in c.paged]
        elif act < 0.88 and live:
            r = rng.choice(list(live))
            n = rng.randint(0, live[r])
            try:
                c.truncate(r, n)
                live[r] = n
            except CacheError:
                assert any(g.spec.window for g in c.paged)    # only a window may refuse
        elif live:
            r = rng.choice(list(live))
            c.free(r)
            del live[r]
        c.check()
        for g in c.paged:
            held = sum(1 for r in live for p in c.pages_of(r, g.gid) if p >= 0)
            assert held == g.pool.num_held
            pages = [p for r in live for p in c.pages_of(r, g.gid) if p >= 0]
            assert len(pages) == len(set(pages))            # no page held twice
    for r in list(live):
        c.free(r)
    assert all(g.pool.num_free == 12 for g in c.paged) and c.slots.num_free == 5
