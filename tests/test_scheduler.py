"""The scheduler's decisions, on the CPU: the cache manager keeps books only and a stand-in 'model' picks tokens."""

import pytest

from ferrisinfer_b200.cache import CacheManager
from ferrisinfer_b200.engine.scheduler import FinishReason, Phase, Scheduler, SchedulerConfig
from ferrisinfer_b200.errors import SchedulerError
from ferrisinfer_b200.parts import PagedKV
from ferrisinfer_b200.sampling import SamplingParams

FULL = PagedKV(2, 16, None)


def make(num_pages=64, page_size=4, needs=(FULL,), cache_options=None, **cfg):
    config = SchedulerConfig(**{**dict(max_batch_size=4, max_prefill_chunk_tokens=8, max_prefill_batch_tokens=16,
                                       max_sequence_length=64, max_generated_tokens=32), **cfg})
    cache = CacheManager(list(needs), page_size, num_pages, config.max_batch_size, **(cache_options or {}))
    return Scheduler(config, cache), cache


def run_step(sched, cache, token=lambda seq: 1):
    """What the engine does around a step: extend the cache for every planned share, commit, sample."""
    plan = sched.schedule()
    sampled = {}
    for e in plan.entries:
        cache.extend(e.seq.request_id, e.start + e.count)  # must never run out: the plan promised pages
        cache.commit(e.seq.request_id, e.start + e.count)
        if e.samples:
            sampled[e.seq.request_id] = (token(e.seq), 0.5)
    done = sched.update(plan, sampled)
    cache.check_invariants()
    return plan, done


def greedy(n):
    return SamplingParams.greedy(max_new_tokens=n)


def test_a_prompt_is_cut_into_portions_across_steps():
    sched, cache = make()
    sched.submit("a", list(range(19)), greedy(2))
    shares = []
    while sched.has_unfinished():
        plan, _ = run_step(sched, cache)
        shares.append([(e.start, e.count, e.samples) for e in plan.entries])
    assert shares == [[(0, 8, False)], [(8, 8, False)], [(16, 3, True)], [(19, 1, True)]]
    seq = sched.finished["a"]
    assert seq.generated == [1, 1] and seq.finish_reason is FinishReason.MAX_NEW_TOKENS
    assert cache.free_pages() == {0: 64} and cache.num_free_slots == 4


def test_decoded_tokens_come_first_and_prompts_fill_the_rest_of_the_budget():
    sched, cache = make(max_prefill_batch_tokens=10)
    sched.submit("a", [1, 2, 3], greedy(8))
    run_step(sched, cache)  # a: whole prompt, samples
    sched.submit("b", list(range(30)), greedy(8))
    sched.submit("c", list(range(5)), greedy(8))
    plan, _ = run_step(sched, cache)
    assert [(e.seq.request_id, e.count) for e in plan.entries] == [("a", 1), ("b", 8), ("c", 1)]
    assert plan.num_tokens == 10
    plan, _ = run_step(sched, cache)
    assert [(e.seq.request_id, e.start, e.count) for e in plan.entries] == [("a", 4, 1), ("b", 8, 8), ("c", 1, 1)]


def test_batch_size_limits_live_requests():
    sched, cache = make(max_batch_size=2)
    for i in range(3):
        sched.submit(i, [1, 2], greedy(3))
    plan, _ = run_step(sched, cache)
    assert [e.seq.request_id for e in plan.entries] == [0, 1] and len(sched.waiting) == 1
    while sched.has_unfinished():
        run_step(sched, cache)
    assert sorted(sched.finished) == [0, 1, 2]


def test_any_of_several_stop_tokens_ends_a_request():
    sched, cache = make(max_generated_tokens=8, max_sequence_length=32)
    sched.submit("either", [1, 2], SamplingParams.greedy(max_new_tokens=8, stop_token_id=7, stop_token_ids=[9, 11]))
    sched.submit("only", [1, 2], SamplingParams.greedy(max_new_tokens=4, stop_token_ids=(5,)))
    counts = {}

    def token(seq):
        counts[seq.request_id] = counts.get(seq.request_id, 0) + 1
        if seq.request_id == "either":
            return 11 if counts["either"] == 3 else 2
        return 7  # not among this request's stop tokens

    while sched.has_unfinished():
        run_step(sched, cache, token)
    f = sched.finished
    assert f["either"].finish_reason is FinishReason.STOP_TOKEN and f["either"].generated == [2, 2, 11]
    assert f["only"].finish_reason is FinishReason.MAX_NEW_TOKENS and f["only"].generated == [7, 7, 7, 7]
    assert SamplingParams(stop_token_ids=[3]).stop_token_ids == (3,)


def test_finish_reasons():
    sched, cache = make(max_generated_tokens=3, max_sequence_length=12)
    sched.submit("stop", [1, 2], SamplingParams.greedy(max_new_tokens=8, stop_token_id=7))
    sched.submit("cap", [1, 2], greedy(30))  # the session's cap of 3 is smaller
    sched.submit("len", list(range(11)), greedy(3))
    sched.submit("none", [1, 2, 3], greedy(0))
    counts = {}

    def token(seq):
        counts[seq.request_id] = counts.get(seq.request_id, 0) + 1
        return 7 if (seq.request_id == "stop" and counts["stop"] == 2) else 1

    while sched.has_unfinished():
        run_step(sched, cache, token)
    f = sched.finished
    assert f["stop"].finish_reason is FinishReason.STOP_TOKEN and f["stop"].generated == [1, 7]
    assert f["cap"].finish_reason is FinishReason.SESSION_LIMIT and len(f["cap"].generated) == 3
    assert f["len"].finish_reason is FinishReason.SEQUENCE_LENGTH and len(f["len"].generated) == 1
    assert f["none"].finish_reason is FinishReason.MAX_NEW_TOKENS and f["none"].generated == []
    assert cache.free_pages() == {0: 64}


def test_refusals_at_submit():
    sched, cache = make(num_pages=4)
    with pytest.raises(SchedulerError, match="at least one"):
        sched.submit("e", [], greedy(1))
    with pytest.raises(SchedulerError, match="max_sequence_length"):
        sched.submit("l", list(range(65)), greedy(1))
    with pytest.raises(SchedulerError, match="never hold"):
        sched.submit("p", list(range(10)), greedy(20))  # 30 tokens need 8 pages of 4; the pool has 4
    sched.submit("ok", list(range(10)), greedy(6))
    with pytest.raises(SchedulerError, match="already"):
        sched.submit("ok", [1], greedy(1))


def test_nothing_is_admitted_and_portions_shrink_when_pages_are_short():
    sched, cache = make(num_pages=6, max_prefill_chunk_tokens=8, max_prefill_batch_tokens=32)
    sched.submit("a", list(range(8)), greedy(12))  # reaches 20 tokens: 5 of the 6 pages
    sched.submit("b", list(range(16)), greedy(2))
    log = []
    while sched.has_unfinished():
        plan, _ = run_step(sched, cache)
        log.append(([(e.seq.request_id, e.start, e.count) for e in plan.entries], [s.request_id for s in plan.preempted]))
    assert log[0] == ([("a", 0, 8), ("b", 0, 8)], [])  # 4 pages taken, 2 free
    # a's token takes one page; b's next portion of 8 would need two: it is cut at the page's edge
    assert log[1] == ([("a", 8, 1), ("b", 8, 4)], [])
    # no page is free: a decodes inside its page, b's portion shrinks to nothing
    assert log[2] == ([("a", 9, 1)], []) and log[3] == ([("a", 10, 1)], []) and log[4] == ([("a", 11, 1)], [])
    # a's next token needs a page: b, admitted last, is preempted, and is not re-admitted in the same step
    assert log[5] == ([("a", 12, 1)], ["b"])
    # b returns from position 0 only when its first portion fits
    assert log[6] == ([("a", 13, 1), ("b", 0, 8)], [])
    assert sched.finished["a"].generated == [1] * 12 and sched.finished["b"].generated == [1, 1]
    assert sched.finished["b"].preemptions >= 1 and sched.stats["preemptions"] == sched.finished["b"].preemptions
    assert cache.free_pages() == {0: 6}
    # while b waited for pages, nothing was admitted over it
    waiting_steps = [entries for entries, _ in log[7:] if all(rid == "a" for rid, _, _ in entries)]
    assert waiting_steps


def test_a_preempted_request_is_recomputed_as_one_prompt_and_keeps_its_tokens():
    sched, cache = make(num_pages=5, max_prefill_chunk_tokens=16, max_prefill_batch_tokens=32)
    sched.submit("a", list(range(7)), greedy(9))
    sched.submit("b", list(range(6)), greedy(9))
    log = []
    n = {"a": 0, "b": 0}

    def token(seq):
        n[seq.request_id] += 1
        return 10 * (1 if seq.request_id == "a" else 2) + n[seq.request_id]

    while sched.has_unfinished():
        plan, _ = run_step(sched, cache, token)
        log.append([(e.seq.request_id, e.start, e.count) for e in plan.entries])
    b = sched.finished["b"]
    assert b.preemptions >= 1
    assert sched.finished["a"].generated == [11 + i for i in range(9)]
    assert b.generated == [21 + i for i in range(9)]  # no token lost or sampled twice
    # after the preemption b comes back with its prompt AND what it had generated, from position 0
    restarts = [s for s in log for (rid, start, count) in s if rid == "b" and start == 0]
    assert len(restarts) == 1 + b.preemptions


def test_a_preempted_request_finds_its_own_pages_again_where_they_were_not_needed():
    """The scene of the test above with kept prompt pages: the preempted request's full pages wait in the cache, the
    request that needed room takes the last of them, and the rest is there when the preempted one comes back."""
    sched, cache = make(num_pages=6, max_prefill_chunk_tokens=8, max_prefill_batch_tokens=32,
                        cache_options=dict(prefix_sharing=True, keep_finished=True))
    sched.submit("a", list(range(8)), greedy(12))
    sched.submit("b", list(range(100, 116)), greedy(2))
    log = []
    while sched.has_unfinished():
        plan, _ = run_step(sched, cache)
        log.append(([(e.seq.request_id, e.start, e.count) for e in plan.entries], [s.request_id for s in plan.preempted]))
    assert log[5] == ([("a", 12, 1)], ["b"])  # as without kept pages: b had 12 tokens in three full pages
    # one of b's pages went to a; the other two still hold b's first 8 tokens, so no page is free for b's next
    # portion while a runs (without kept pages b would compute those 8 tokens again here)
    assert log[6] == ([("a", 13, 1)], [])
    after = [entries for entries, _ in log[6:] if any(rid == "b" for rid, _, _ in entries)]
    # a's last page took another of b's pages; b comes back at token 4, not 0, once a has ended
    assert after[0][-1][:2] == ("b", 4)
    b = sched.finished["b"]
    assert b.generated == [1, 1] and b.preemptions >= 1 and b.reused_prompt_tokens == 4
    assert sched.finished["a"].generated == [1] * 12
    # b was admitted and sent away again in every step in which its next portion did not fit: that does not count
    assert cache.stats["revived_pages"] == 1 and cache.stats["shared_tokens"] == 4 and cache.stats["evicted_pages"] >= 2
    assert cache.free_pages() == {0: 6} and not cache.requests
    cache.check_invariants()


def test_cancel_gives_everything_back():
    sched, cache = make()
    sched.submit("a", list(range(9)), greedy(5))
    sched.submit("b", list(range(9)), greedy(5))
    run_step(sched, cache)
    assert sched.cancel("a").finish_reason is FinishReason.CANCELLED
    assert sched.cancel("nobody") is None
    cache.check_invariants()
    while sched.has_unfinished():
        run_step(sched, cache)
    assert cache.free_pages() == {0: 64} and sched.finished["b"].finish_reason is FinishReason.MAX_NEW_TOKENS


@pytest.mark.parametrize("seed", range(6))
def test_random_load_never_overdraws_the_pool(seed):
    import random

    rng = random.Random(seed)
    window = PagedKV(2, 16, rng.choice([6, 20]))
    sched, cache = make(num_pages=rng.choice([12, 20]), page_size=rng.choice([2, 4]), needs=(FULL, window),
                        max_prefill_chunk_tokens=rng.choice([3, 8]), max_prefill_batch_tokens=rng.choice([6, 16]),
                        max_sequence_length=40, max_generated_tokens=16)
    submitted = 0
    for step in range(300):
        if submitted < 14 and rng.random() < 0.3:
            try:
                sched.submit(submitted, [1] * rng.randint(1, 25), greedy(rng.randint(0, 16)))
            except SchedulerError:
                pass
            submitted += 1
        if sched.has_unfinished():
            run_step(sched, cache, token=lambda seq: rng.randrange(5))
        elif submitted >= 14:
            break
    assert not sched.has_unfinished()
    assert all(g.pool.num_used == 0 for g in cache.groups) and cache.num_free_slots == 4
    for seq in sched.finished.values():
        assert seq.finish_reason is not None and len(seq.generated) <= seq.max_new_tokens


@pytest.mark.parametrize("seed", range(8))
def test_random_load_with_kept_prompt_pages(seed):
    """Prompts that begin alike, a pool that forces preemptions, pages of finished and preempted prompts kept until
    their room is needed: every request ends, nothing is lost, and what the scheduler promises the cache delivers
    (run_step extends without checking)."""
    import random

    rng = random.Random(100 + seed)
    sched, cache = make(num_pages=rng.choice([10, 14, 20]), page_size=rng.choice([2, 4]),
                        max_prefill_chunk_tokens=rng.choice([3, 8]), max_prefill_batch_tokens=rng.choice([6, 16]),
                        max_sequence_length=40, max_generated_tokens=12, min_prefix_share_tokens=rng.choice([0, 4]),
                        cache_options=dict(prefix_sharing=True, keep_finished=True,
                                           min_prefix_share_tokens=rng.choice([0, 4])))
    stems = [[rng.randrange(9) for _ in range(rng.choice([6, 11, 17]))] for _ in range(3)]
    submitted = 0
    for step in range(400):
        if submitted < 16 and rng.random() < 0.3:
            prompt = list(rng.choice(stems)) + [rng.randrange(9) for _ in range(rng.randint(1, 6))]
            try:
                sched.submit(submitted, prompt, greedy(rng.randint(0, 12)))
            except SchedulerError:
                pass
            submitted += 1
        if sched.has_unfinished():
            run_step(sched, cache, token=lambda seq: rng.randrange(5))
        elif submitted >= 16:
            break
    assert not sched.has_unfinished() and not cache.requests
    assert cache.free_pages() == {0: cache.groups[0].pool.num_pages} and cache.num_free_slots == 4
    assert cache.groups[0].pool.num_used == cache.num_idle_blocks
    assert cache.stats["revived_pages"] > 0
    for seq in sched.finished.values():
        assert seq.finish_reason is not None and len(seq.generated) <= seq.max_new_tokens
    cache.drop_idle()
    cache.check_invariants()
    assert cache.groups[0].pool.num_used == 0


def test_a_new_request_reuses_the_pages_of_a_live_request_with_the_same_beginning():
    config = SchedulerConfig(max_batch_size=4, max_prefill_chunk_tokens=8, max_prefill_batch_tokens=32,
                             max_sequence_length=64, max_generated_tokens=32, min_prefix_share_tokens=8)
    cache = CacheManager([FULL], 4, 64, 4, prefix_sharing=True, min_prefix_share_tokens=8)
    sched = Scheduler(config, cache)
    stem = list(range(100, 118))  # 18 tokens: four full pages and a half
    sched.submit("a", stem + [1, 2], greedy(4))
    for _ in range(3):
        run_step(sched, cache)  # a's prompt (20 tokens) is in the cache; it decodes
    sched.submit("b", stem + [5, 6, 7], greedy(2))
    plan, _ = run_step(sched, cache)
    shares = {e.seq.request_id: (e.start, e.count) for e in plan.entries}
    assert shares["b"] == (16, 5)  # four pages reused, the rest computed
    b = [s for s in sched.running if s.request_id == "b"][0]
    assert b.reused_prompt_tokens == 16 and cache.stats["shared_tokens"] == 16
    while sched.has_unfinished():
        run_step(sched, cache)
    assert sched.finished["b"].generated == [1, 1] and cache.free_pages() == {0: 64}
    assert not cache.prefix.blocks
