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


# ------------------------------------------------------------------------------------ prefix sharing
def sharing_manager(**kw):
    return CacheManager([FULL, FULL], 4, kw.pop("num_pages", 32), kw.pop("max_requests", 4), prefix_sharing=True, **kw)


def run_prompt(m, rid, prompt, upto=None):
    rc = m.admit(rid, prompt)
    total = len(prompt) if upto is None else upto
    m.extend(rid, total)
    m.commit(rid, total)
    return rc


def test_full_pages_of_a_common_prefix_are_shared_and_counted():
    m = sharing_manager()
    common = list(range(100, 110))  # two full pages of 4 and a half
    run_prompt(m, "a", common + [1, 2, 3])
    used = m.groups[0].pool.num_used
    rc = m.admit("b", common + [7, 8])
    assert rc.num_tokens == 8 and rc.shared_tokens == 8  # the two full pages; the third differs
    assert m.block_table("b", 0) == m.block_table("a", 0)[:2]
    assert [m.groups[0].pool.refcount(p) for p in m.block_table("b", 0)] == [2, 2]
    assert m.groups[0].pool.num_used == used  # nothing new was taken
    m.extend("b", 12)
    m.commit("b", 12)
    assert m.block_table("b", 0)[2] != m.block_table("a", 0)[2]  # the page that differs is private
    m.check_invariants()
    assert m.stats["shared_tokens"] == 8 and m.stats["shared_pages"] == 2 * len(m.groups)
    # the donor leaves first: its shared pages stay with the borrower and in the index
    freed = m.release("a")
    assert freed == 2 * len(m.groups) and m.groups[0].pool.refcount(m.block_table("b", 0)[0]) == 1
    rc = m.admit("c", common + [9])
    assert rc.num_tokens == 8
    m.release("b")
    m.release("c")
    m.check_invariants()
    assert m.groups[0].pool.num_used == 0 and not m.prefix.blocks and not m.prefix.by_page


def test_the_whole_prompt_is_never_shared_and_short_prefixes_are_not_worth_it():
    m = sharing_manager()
    prompt = list(range(8))
    run_prompt(m, "a", prompt)
    assert m.admit("same", list(prompt)).num_tokens == 4  # 8 tokens are two full pages, but one token must be computed
    assert m.admit("longer", prompt + [5]).num_tokens == 8
    strict = sharing_manager(min_prefix_share_tokens=12)
    run_prompt(strict, "a", prompt + [1, 2, 3, 4, 5])
    assert strict.admit("b", prompt + [9]).num_tokens == 0  # 8 common tokens < 12
    assert strict.admit("c", prompt + [1, 2, 3, 4, 9]).num_tokens == 12


def test_pages_are_shared_only_once_they_are_computed():
    m = sharing_manager()
    prompt = list(range(20))
    run_prompt(m, "a", prompt, upto=6)  # only the first page of a is complete
    assert m.admit("b", list(prompt)).num_tokens == 4
    m.extend("a", 20)
    m.commit("a", 20)
    assert m.admit("c", list(prompt)).num_tokens == 16


def test_generated_tokens_and_other_prompts_do_not_match():
    m = sharing_manager()
    run_prompt(m, "a", [1, 2, 3, 4, 5, 6, 7, 8, 9])
    assert m.admit("b", [1, 2, 3, 4, 5, 6, 7, 0, 9]).num_tokens == 4  # the second page differs in one token
    assert m.admit("c", [2, 2, 3, 4, 5, 6, 7, 8, 9]).num_tokens == 0  # a chain starts at the first page
    m.extend("a", 14)  # tokens beyond the prompt (generated) are not offered
    m.commit("a", 14)
    assert m.get("a").registered_blocks == 2


def test_sharing_is_off_where_a_page_does_not_mean_the_same_for_every_layer():
    assert CacheManager([FULL, WINDOW], 4, 8, 2, prefix_sharing=True).prefix is None
    assert CacheManager([FULL, FixedState((3,))], 4, 8, 2, prefix_sharing=True).prefix is None
    assert CacheManager([FULL], 4, 8, 2).prefix is None
    assert CacheManager([FULL], 4, 8, 2, prefix_sharing=True).prefix is not None


@pytest.mark.parametrize("keep", [False, True])
@pytest.mark.parametrize("seed", range(8))
def test_random_orders_with_shared_prefixes(seed, keep):
    rng = random.Random(seed)
    m = CacheManager([FULL, FULL], 4, 48 if not keep else 14, max_requests=5, prefix_sharing=True, keep_finished=keep)
    stems = [[rng.randrange(50) for _ in range(rng.choice([5, 9, 16]))] for _ in range(3)]
    live, counter = {}, 0
    for _ in range(300):
        action = rng.random()
        if action < 0.3 and m.num_free_slots:
            prompt = list(rng.choice(stems)) + [rng.randrange(50) for _ in range(rng.randrange(1, 6))]
            rid = f"r{counter}"
            counter += 1
            rc = m.admit(rid, prompt)
            assert rc.num_tokens % 4 == 0 and rc.num_tokens < len(prompt)
            live[rid] = [rc.num_tokens, len(prompt) + rng.randrange(0, 6)]
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            have, goal = live[rid]
            new_total = min(goal, have + rng.choice([1, 2, 5]))
            if new_total > have and m.can_extend(rid, new_total):
                m.extend(rid, new_total)
                m.commit(rid, new_total)
                live[rid][0] = new_total
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_invariants()
    for rid in list(live):
        m.release(rid)
    m.check_invariants()
    if keep:
        assert m.stats["revived_pages"] > 0 and m.stats["evicted_pages"] > 0
        assert all(g.pool.num_used == m.num_idle_blocks for g in m.groups) and m.free_pages() == {0: 14}
        kept = m.num_idle_blocks
        assert kept == len(m.prefix.blocks) and m.drop_idle() == kept  # with no request left, all that is indexed is idle
        m.check_invariants()
    assert all(g.pool.num_used == 0 for g in m.groups) and not m.prefix.blocks


def test_pages_of_a_finished_prompt_wait_for_the_next_request_that_begins_alike():
    m = sharing_manager(num_pages=8, keep_finished=True)
    common = list(range(100, 110))  # two full pages of 4 and a half
    run_prompt(m, "a", common + [1, 2, 3])  # 13 tokens: four pages, three of them full
    pages_a = list(m.block_table("a", 0))
    assert m.release("a") == len(m.groups)  # only the page that is not full goes back to the free list
    assert m.num_idle_blocks == 3 and m.groups[0].pool.num_used == 3 and m.free_pages() == {0: 8}
    m.check_invariants()
    rc = m.admit("b", common + [7, 8])
    assert rc.num_tokens == 8 and m.block_table("b", 0) == pages_a[:2]  # nothing is computed again
    assert m.num_idle_blocks == 1 and m.stats["revived_pages"] == 2 * len(m.groups)
    assert [m.groups[0].pool.refcount(p) for p in pages_a[:3]] == [2, 2, 1]
    m.check_invariants()
    m.extend("b", 12)
    m.commit("b", 12)
    m.release("b")
    # b's own third page ([108, 109, 7, 8]) is kept beside a's ([108, 109, 1, 2])
    assert m.num_idle_blocks == 4
    m.check_invariants()


def test_kept_pages_are_given_up_when_their_room_is_needed_ends_of_chains_first():
    m = sharing_manager(num_pages=6, keep_finished=True)
    old = list(range(12))
    run_prompt(m, "old", old + [50])        # three full pages and one more
    m.release("old")
    new = list(range(20, 28))
    run_prompt(m, "new", new + [51])        # two full pages and one more: the pool is full now (3 idle + 3)
    m.release("new")
    assert m.num_idle_blocks == 5 and m.groups[0].pool.num_free == 1 and m.free_pages() == {0: 6}
    # a request that needs three pages takes the free one and the two LAST pages of the older chain
    rc = m.admit("x", [90, 91, 92, 93, 94, 95, 96, 97, 98])
    assert rc.num_tokens == 0 and m.can_extend("x", 9)
    m.extend("x", 9)
    m.commit("x", 9)
    m.check_invariants()
    assert m.stats["evicted_pages"] == 2 * len(m.groups) and m.num_idle_blocks == 3
    assert m.admit("old again", old + [50]).num_tokens == 4   # the head of the older chain is still there
    assert m.admit("new again", new + [51]).num_tokens == 8   # the newer chain is whole
    assert m.num_idle_blocks == 0
    # nothing idle is left to give up: the next request that needs room is refused, and nothing changes
    m.admit("y", [1] * 9)
    assert not m.can_extend("y", 9)
    with pytest.raises(OutOfPages):
        m.extend("y", 9)
    m.check_invariants()
    for rid in ("x", "old again", "new again", "y"):
        m.release(rid)
    assert m.free_pages() == {0: 6}
    m.drop_idle()
    assert all(g.pool.num_used == 0 for g in m.groups) and not m.prefix.blocks and not m.prefix.by_page
    m.check_invariants()
