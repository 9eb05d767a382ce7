"""The cache manager on the CPU (bookkeeping only): no page lost, held twice or freed twice, under random orders."""

import random

import pytest

from ferrisinfer_b200.cache import NO_PAGE, CacheManager, PagePool
from ferrisinfer_b200.errors import CacheError, OutOfPages
from ferrisinfer_b200.parts import FixedState, PagedKV

FULL = PagedKV(2, 16, None)
WINDOW = PagedKV(2, 16, 10)


def manager(needs=(FULL, FULL), page_size=4, num_pages=8, max_requests=3):
    return CacheManager(list(needs), page_size, num_pages, max_requests)


def test_pool_hands_out_ascending_and_reuses_the_last_freed_first():
    pool = PagePool(4)
    assert pool.alloc(3) == [0, 1, 2]
    pool.release(1)
    assert pool.alloc(1) == [1]
    with pytest.raises(OutOfPages):
        pool.alloc(2)
    assert pool.num_free == 1  # the failed request took nothing
    pool.release(0)
    with pytest.raises(CacheError, match="twice"):
        pool.release(0)
    with pytest.raises(CacheError):
        pool.retain(0)
    pool.retain(2)
    assert pool.release(2) is False and pool.release(2) is True


def test_layers_with_the_same_need_share_a_group_and_different_needs_do_not():
    m = manager(needs=(FULL, WINDOW, FULL, None, FixedState((3,)), WINDOW))
    assert [g.members for g in m.groups] == [[0, 2], [1, 5]]
    assert m.layer_caches[3] is None and m.layer_caches[4].need == FixedState((3,))
    assert m.layer_caches[0].group == 0 and m.layer_caches[5].group == 1


def test_extend_commit_release_cycle():
    m = manager()
    m.admit("a")
    assert m.pages_needed("a", 9) == {0: 3}
    m.extend("a", 9)
    assert m.block_table("a", 0) == [0, 1, 2]
    assert m.slots_for("a", 0, 3, 3) == [3, 4, 5]
    m.commit("a", 9)
    m.extend("a", 12)  # still inside the third page
    assert m.block_table("a", 0) == [0, 1, 2]
    m.extend("a", 13)
    assert m.block_table("a", 0) == [0, 1, 2, 3]
    m.check_invariants()
    assert m.release("a") == 4
    assert m.free_pages() == {0: 8}
    with pytest.raises(CacheError, match="twice"):
        m.release("a")
    m.check_invariants()


def test_extend_takes_all_groups_or_nothing():
    m = CacheManager([FULL, WINDOW], 4, {0: 8, 1: 2}, 2)
    m.admit("a")
    with pytest.raises(OutOfPages, match="group 1"):
        m.extend("a", 12)
    assert m.free_pages() == {0: 8, 1: 2} and m.block_table("a", 0) == []
    m.check_invariants()


def test_window_group_gives_pages_back_once_the_window_has_passed_them():
    m = CacheManager([FULL, WINDOW], 4, 16, 2)
    m.admit("a")
    m.extend("a", 30)
    m.commit("a", 30)
    # the next query (position 30) reads keys 21..30: blocks 0..4 (positions 0..19) are behind the window
    assert m.block_table("a", 1)[:5] == [NO_PAGE] * 5 and NO_PAGE not in m.block_table("a", 1)[5:]
    assert NO_PAGE not in m.block_table("a", 0)
    assert m.groups[1].pool.num_used == 3 and m.groups[0].pool.num_used == 8
    m.check_invariants()
    m.extend("a", 31)
    assert m.pages_needed("a", 31) == {0: 0, 1: 0}
    with pytest.raises(CacheError, match="no page"):
        m.slots_for("a", 1, 5, 1)
    m.release("a")
    assert m.free_pages() == {0: 16, 1: 16}


def test_state_slots():
    m = manager(max_requests=2)
    a, b = m.admit("a").slot, m.admit("b").slot
    assert {a, b} == {0, 1}
    with pytest.raises(CacheError, match="slots"):
        m.admit("c")
    with pytest.raises(CacheError, match="already"):
        m.admit("a")
    m.release("a")
    assert m.admit("c").slot == a
    m.check_invariants()


def test_shrinking_and_unknown_requests_are_errors():
    m = manager()
    m.admit("a")
    m.extend("a", 5)
    m.commit("a", 5)
    with pytest.raises(CacheError):
        m.commit("a", 4)
    with pytest.raises(CacheError):
        m.extend("a", 3)
    with pytest.raises(CacheError, match="not admitted"):
        m.extend("nobody", 3)


@pytest.mark.parametrize("seed", range(12))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    page_size = rng.choice([1, 4, 16])
    needs = [FULL, PagedKV(2, 16, rng.choice([3, 10, 40])), FULL]
    m = CacheManager(needs, page_size, rng.choice([6, 20, 64]), max_requests=4)
    live, counter = {}, 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and m.num_free_slots:
            rid = f"r{counter}"
            counter += 1
            m.admit(rid)
            live[rid] = 0
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            new_total = live[rid] + rng.choice([1, 1, 1, 2, 7, 19])
            if m.can_extend(rid, new_total):
                m.extend(rid, new_total)
                # every position the step writes, and every position a query of the step reads, has a page
                for g in m.groups:
                    m.slots_for(rid, g.gid, live[rid], new_total - live[rid])
                    first_read = 0 if g.window is None else max(0, live[rid] - g.window + 1)
                    m.slots_for(rid, g.gid, first_read, new_total - first_read)
                m.commit(rid, new_total)
                live[rid] = new_total
            else:
                before = m.free_pages()
                with pytest.raises(OutOfPages):
                    m.extend(rid, new_total)
                assert m.free_pages() == before
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_invariants()
    for rid in list(live):
        m.release(rid)
    m.check_invariants()
    assert all(g.pool.num_used == 0 for g in m.groups) and m.num_free_slots == 4
