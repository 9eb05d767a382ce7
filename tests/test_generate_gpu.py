"""Generation through the Python entry point: greedy against the plain implementation, sampling with seeds,
preemption when pages run out, the command line."""

import json
import os
import subprocess
import sys

import pytest
import torch

import helpers
import plain_qwen2 as plain
from helpers import TINY

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROMPTS = {"A": (5, 9, 17), "B": (3, 11, 23, 40)}
SLACK = {"float32": 1e-4, "bfloat16": 3e-2}  # how far below the plain maximum a chosen logit may lie


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen")
    return {name: helpers.make_folder(root, TINY[name], seed=31 + i) for i, name in enumerate(("A", "B"))}


def _all_pages_are_back(engine):
    """No request holds a page: every page is on a free list, or is a page of a finished prompt that only the
    prefix index keeps (it counts as free, and a request that needs its room gets it)."""
    cache = engine.runner.cache
    cache.check_invariants()
    assert not cache.requests
    assert all(cache.free_pages()[g.gid] == g.pool.num_pages for g in cache.groups)
    assert all(g.pool.num_used == cache.num_idle_blocks for g in cache.groups)
    cache.drop_idle()
    assert all(g.pool.num_used == 0 for g in cache.groups)
    cache.check_invariants()


def _engine(folder, dtype, device=None, **kw):
    from ferrisinfer_b200 import SchedulerConfig
    from ferrisinfer_b200.engine.engine import Engine

    sched = SchedulerConfig(max_batch_size=4, max_prefill_chunk_tokens=8, max_prefill_batch_tokens=24,
                            max_sequence_length=256, max_generated_tokens=64)
    return Engine(folder, dtype=dtype, device=device, scheduler=kw.pop("scheduler", sched), **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_follows_the_plain_implementation(name, dtype, device, folders):
    from ferrisinfer_b200 import FinishReason, SamplingParams

    config, weights = helpers.read_folder(folders[name])
    prompts = [helpers.random_ids(config["vocab_size"], n, n) for n in PROMPTS[name]]
    engine = _engine(folders[name], dtype, device, page_size=4 if name == "A" else 8, num_pages=64)
    outs = engine.generate(prompts, SamplingParams.greedy(max_new_tokens=8))
    for prompt, out in zip(prompts, outs):
        ids = out.generated_token_ids()
        assert len(ids) == 8 and out.finish_reason is FinishReason.MAX_NEW_TOKENS and out.prompt_token_ids == prompt
        logits = plain.forward(config, weights, prompt + ids, torch.float64)
        for i, tok in enumerate(ids):
            row = logits[len(prompt) + i - 1]
            assert row[tok] >= row.max() - SLACK[dtype], (i, tok, int(row.argmax()))
        if dtype == "float32":
            assert ids == plain.generate_greedy(config, weights, prompt, 8, torch.float64)
            p0 = plain.greedy(logits[len(prompt) - 1].float().numpy())[1]
            assert abs(out.generated_tokens[0].probability - p0) < 1e-5
    engine.runner.cache.check_invariants()
    _all_pages_are_back(engine)


def test_stop_token_and_length_limits(device, folders):
    from ferrisinfer_b200 import FinishReason, SamplingParams, SchedulerConfig

    config, weights = helpers.read_folder(folders["A"])
    prompt = helpers.random_ids(256, 9, 4)
    greedy = plain.generate_greedy(config, weights, prompt, 6, torch.float64)
    engine = _engine(folders["A"], "float32", device, page_size=4, num_pages=64)
    out = engine.generate(prompt, SamplingParams.greedy(max_new_tokens=6, stop_token_id=greedy[2]))
    first_hit = greedy.index(greedy[2])
    assert out.generated_token_ids() == greedy[:first_hit + 1] and out.finish_reason is FinishReason.STOP_TOKEN
    out = engine.generate(prompt, SamplingParams.greedy(max_new_tokens=0))
    assert out.generated_token_ids() == [] and out.finish_reason is FinishReason.MAX_NEW_TOKENS
    short = SchedulerConfig(max_batch_size=2, max_sequence_length=12, max_generated_tokens=64)
    engine = _engine(folders["A"], "float32", device, page_size=4, num_pages=16, scheduler=short)
    out = engine.generate(prompt, SamplingParams.greedy(max_new_tokens=30))
    assert len(out.generated_token_ids()) == 3 and out.finish_reason is FinishReason.SEQUENCE_LENGTH


def test_sampling_is_seeded_and_does_not_depend_on_the_batch(device, folders):
    """Config B of the baseline: temperature 0.7 with a fixed seed.  In 32-bit a row's logits do not depend on
    what else is in the batch, and each request draws from its own generator."""
    from ferrisinfer_b200 import SamplingParams

    vocab = TINY["B"]["vocab_size"]
    prompts = [helpers.random_ids(vocab, n, n) for n in PROMPTS["B"]]
    params = [SamplingParams(temperature=0.7, top_k=0, top_p=1.0, seed=100 + i, max_new_tokens=12)
              for i in range(len(prompts))]
    engine = _engine(folders["B"], "float32", device, page_size=8, num_pages=64)
    together = [o.generated_token_ids() for o in engine.generate(prompts, params)]
    again = [o.generated_token_ids() for o in engine.generate(prompts, params)]
    alone = [engine.generate(p, sp).generated_token_ids() for p, sp in zip(prompts, params)]
    assert together == again == alone
    other = engine.generate(prompts[0], SamplingParams(temperature=0.7, top_k=0, top_p=1.0, seed=999, max_new_tokens=12))
    assert other.generated_token_ids() != together[0]
    chat = engine.generate(prompts[1], SamplingParams.chat_default(max_new_tokens=12))
    assert len(chat.generated_token_ids()) == 12 and all(0 < t.probability <= 1 for t in chat.generated_tokens)


def test_sampled_tokens_follow_the_plain_sampler(device, folders):
    """Teacher-forced: at each step the plain sampler, given the plain logits of the engine's prefix and the same
    generator state, picks the engine's token."""
    from ferrisinfer_b200 import SamplingParams

    config, weights = helpers.read_folder(folders["B"])
    prompt = helpers.random_ids(config["vocab_size"], 11, 5)
    sp = SamplingParams(temperature=0.7, top_k=0, top_p=1.0, seed=42, max_new_tokens=10)
    engine = _engine(folders["B"], "float32", device, page_size=8, num_pages=64)
    out = engine.generate(prompt, sp)
    ids = out.generated_token_ids()
    logits = plain.forward(config, weights, prompt + ids, torch.float32)
    rng = plain.XorShift64Star(42)
    agree = 0
    for i, tok in enumerate(ids):
        want, prob = plain.sample(logits[len(prompt) + i - 1].numpy(), 0.7, 0, 1.0, rng)
        agree += int(want == tok)
        if want == tok:
            assert abs(prob - out.generated_tokens[i].probability) < 1e-4
    assert agree >= len(ids) - 1, (ids, agree)  # a draw that lands within rounding of a boundary may differ


def test_preemption_when_pages_run_out_does_not_change_the_tokens(device, folders):
    from ferrisinfer_b200 import SamplingParams, SchedulerConfig

    vocab = TINY["A"]["vocab_size"]
    prompts = [helpers.random_ids(vocab, n, 50 + n) for n in (14, 11, 9)]
    params = [SamplingParams(temperature=0.8, top_k=0, top_p=1.0, seed=7 + i, max_new_tokens=20) for i in range(3)]
    sched = SchedulerConfig(max_batch_size=4, max_prefill_chunk_tokens=8, max_prefill_batch_tokens=24,
                            max_sequence_length=64, max_generated_tokens=32)
    roomy = _engine(folders["A"], "float32", device, page_size=4, num_pages=64, scheduler=sched)
    want = [o.generated_token_ids() for o in roomy.generate(prompts, params)]
    tight = _engine(folders["A"], "float32", device, page_size=4, num_pages=15, scheduler=sched)  # 60 tokens for three requests of ~31
    outs = tight.generate(prompts, params)
    assert tight.scheduler.stats["preemptions"] >= 1 and sum(o.preemptions for o in outs) >= 1
    assert [o.generated_token_ids() for o in outs] == want
    tight.runner.cache.check_invariants()
    _all_pages_are_back(tight)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_requests_that_begin_alike_share_pages_and_generate_the_same(dtype, device, folders):
    """Eight requests share a long beginning (the baseline's shared-prefix case, in small): with sharing the later
    ones compute only what differs, hold the donor's pages, and generate exactly what they generate without it."""
    from ferrisinfer_b200 import SamplingParams, SchedulerConfig

    vocab = TINY["A"]["vocab_size"]
    stem = helpers.random_ids(vocab, 50, 77)
    prompts = [stem + helpers.random_ids(vocab, 3 + i, 200 + i) for i in range(8)]
    params = SamplingParams.greedy(max_new_tokens=6)
    sched = SchedulerConfig(max_batch_size=8, max_prefill_chunk_tokens=16, max_prefill_batch_tokens=64,
                            max_sequence_length=128, max_generated_tokens=32, min_prefix_share_tokens=8)

    def run(sharing):
        engine = _engine(folders["A"], dtype, device, page_size=4, num_pages=256, scheduler=sched, prefix_sharing=sharing)
        first = engine.submit(prompts[0], params)
        while not engine.scheduler.running or engine.scheduler.running[0].num_computed < len(prompts[0]):
            engine.step()  # until the first request's prompt is in the cache
        rest = [engine.submit(p, params) for p in prompts[1:]]
        most_pages = 0
        while engine.has_unfinished():
            engine.step()
            most_pages = max(most_pages, engine.runner.cache.groups[0].pool.num_used)
            engine.runner.cache.check_invariants()
        outs = [engine.output_of(i) for i in [first] + rest]
        _all_pages_are_back(engine)
        return outs, most_pages, engine.runner.cache.stats

    shared, pages_shared, stats = run(True)
    alone, pages_alone, _ = run(False)
    assert [o.generated_token_ids() for o in shared] == [o.generated_token_ids() for o in alone]
    assert all(o.reused_prompt_tokens == 48 for o in shared[1:]) and shared[0].reused_prompt_tokens == 0
    assert stats["shared_tokens"] == 7 * 48 and pages_shared <= pages_alone - 60


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_later_request_finds_the_pages_of_a_finished_one(dtype, device, folders):
    """Requests one after the other with the same long beginning: the pages of the first one's prompt outlive it,
    the later ones compute only what differs and generate what they generate in an engine that keeps nothing;
    when other prompts need the room, the kept pages are given up and everything still comes out the same."""
    from ferrisinfer_b200 import SamplingParams, SchedulerConfig

    vocab = TINY["A"]["vocab_size"]
    stem = helpers.random_ids(vocab, 41, 5)
    prompts = [stem + helpers.random_ids(vocab, 2 + i, 300 + i) for i in range(3)]
    others = [helpers.random_ids(vocab, 44, 400 + i) for i in range(3)]
    params = SamplingParams.greedy(max_new_tokens=5)
    sched = SchedulerConfig(max_batch_size=4, max_prefill_chunk_tokens=16, max_prefill_batch_tokens=32,
                            max_sequence_length=128, max_generated_tokens=16, min_prefix_share_tokens=8)

    def run(keep):
        # 24 pages of 4: one request of ~50 tokens holds 13, so kept pages must make room for the others
        engine = _engine(folders["A"], dtype, device, page_size=4, num_pages=24, scheduler=sched, keep_finished_prefixes=keep)
        outs = []
        for p in prompts + others + prompts[:1]:
            rid = engine.submit(p, params)
            while engine.has_unfinished():
                engine.step()
                engine.runner.cache.check_invariants()
            outs.append(engine.output_of(rid))
        stats = dict(engine.runner.cache.stats)
        _all_pages_are_back(engine)
        return outs, stats

    kept, stats = run(True)
    plain, plain_stats = run(False)
    assert [o.generated_token_ids() for o in kept] == [o.generated_token_ids() for o in plain]
    assert [o.reused_prompt_tokens for o in kept[:3]] == [0, 40, 40] and all(o.reused_prompt_tokens == 0 for o in plain)
    assert stats["revived_pages"] >= 20 and stats["evicted_pages"] > 0 and plain_stats["revived_pages"] == 0


def test_abort_gives_pages_back(device, folders):
    from ferrisinfer_b200 import FinishReason, SamplingParams

    engine = _engine(folders["A"], "float32", device, page_size=4, num_pages=32)
    a = engine.submit(helpers.random_ids(256, 20, 1), SamplingParams.greedy(max_new_tokens=30))
    b = engine.submit(helpers.random_ids(256, 10, 2), SamplingParams.greedy(max_new_tokens=5))
    for _ in range(3):
        engine.step()
    assert engine.abort(a) and not engine.abort("nobody")
    while engine.has_unfinished():
        engine.step()
    assert engine.output_of(a).finish_reason is FinishReason.CANCELLED
    assert len(engine.output_of(b).generated_tokens) == 5
    _all_pages_are_back(engine)


def test_command_line(device, folders):
    def run(*args):
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ferrisinfer"), *args], capture_output=True,
                           text=True, timeout=600)
        return r.returncode, r.stdout, r.stderr

    code, out, _ = run("help")
    assert code == 0 and "generate-hf [ids] [tokens]" in out
    code, out, _ = run("inspect-hf", folders["B"])
    assert code == 0 and json.loads(out)["problems"] is None
    config, weights = helpers.read_folder(folders["B"])
    prompt = helpers.random_ids(config["vocab_size"], 7, 8)
    code, out, err = run("generate-hf", ",".join(map(str, prompt)), "5", "--model", folders["B"], "--dtype", "float32")
    assert code == 0, err
    line = [l for l in out.splitlines() if l.startswith("generated token ids:")][0]
    assert [int(t) for t in line.split(":")[1].split()] == plain.generate_greedy(config, weights, prompt, 5, torch.float64)
    code, out, err = run("profile-continuous-hf", "6", "--model", folders["B"])
    assert code == 0 and "preemptions" in out, err
    code, _, err = run("generate-hf", "1,2", "--model", os.path.join(folders["B"], "nowhere"))
    assert code == 1 and "error" in err
    code, _, _ = run("no-such-command")
    assert code == 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_a_step_ahead_changes_nothing_but_the_timing(dtype, device, folders):
    """While a decode step runs, the engine queues the next one with the tokens still on the device.  The
    outputs are those of the engine that waits for every step: greedy and seeded sampling, requests that end
    on a stop token with a step too many in flight, one cancelled on the way, new ones joining late."""
    from ferrisinfer_b200 import FinishReason, SamplingParams

    config, _ = helpers.read_folder(folders["B"])
    prompts = [helpers.random_ids(config["vocab_size"], n, 50 + n) for n in (4, 13, 22, 7)]

    def run(run_ahead, stops):
        engine = _engine(folders["B"], dtype, device, page_size=8, num_pages=64, run_ahead=run_ahead)
        params = [SamplingParams.greedy(max_new_tokens=20, stop_token_id=stops[0]),
                  SamplingParams(temperature=0.9, top_k=40, top_p=0.95, seed=7, max_new_tokens=20, stop_token_id=stops[1]),
                  SamplingParams.greedy(max_new_tokens=20),
                  SamplingParams(temperature=1.3, top_k=0, seed=11, max_new_tokens=9)]
        ids = [engine.submit(p, sp) for p, sp in zip(prompts[:3], params[:3])]
        seen, steps = {i: [] for i in ids}, 0
        while engine.has_unfinished():
            for o in engine.step():
                if o.token is not None:
                    seen.setdefault(o.request_id, []).append(o.token.token_id)
            steps += 1
            if steps == 9:
                assert engine.abort(ids[2])
            if steps == 12:
                ids.append(engine.submit(prompts[3], params[3]))
        outs = [engine.output_of(i) for i in ids]
        for i, o in zip(ids, outs):
            if o.finish_reason is not FinishReason.CANCELLED:
                assert seen[i] == o.generated_token_ids()
        engine.runner.cache.check_invariants()
        _all_pages_are_back(engine)
        return [(o.generated_token_ids(), o.finish_reason) for o in outs], engine.steps_run_ahead

    free, _ = run(False, (None, None))
    stops = (free[0][0][6], free[1][0][10])  # tokens that the first two requests do generate
    want, none_ahead = run(False, stops)
    got, ahead = run(True, stops)
    assert none_ahead == 0 and ahead >= 10
    assert want[0][1] is FinishReason.STOP_TOKEN and want[1][1] is FinishReason.STOP_TOKEN
    assert want[2][1] is FinishReason.CANCELLED
    assert got == want


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_requests_arriving_ending_and_preempted_at_random_with_a_step_in_flight(seed, device, folders):
    """Twelve requests arrive at random steps into a pool that is too small for them, some are cancelled on the way,
    some end on a stop token, greedy and seeded sampling mixed: what each request generates is what it generates
    alone in a roomy engine, with and without a step running ahead."""
    import random

    from ferrisinfer_b200 import FinishReason, SamplingParams, SchedulerConfig

    rng = random.Random(seed)
    vocab = TINY["A"]["vocab_size"]
    n = 12
    prompts = [helpers.random_ids(vocab, rng.randint(2, 30), 900 + 13 * seed + i) for i in range(n)]
    budgets = [rng.randint(1, 24) for _ in range(n)]
    sampled = [rng.random() < 0.5 for _ in range(n)]

    def params(i, stop=None):
        if sampled[i]:
            return SamplingParams(temperature=0.9, top_k=0, top_p=0.9, seed=100 + i, max_new_tokens=budgets[i], stop_token_id=stop)
        return SamplingParams.greedy(max_new_tokens=budgets[i], stop_token_id=stop)

    sched = SchedulerConfig(max_batch_size=5, max_prefill_chunk_tokens=8, max_prefill_batch_tokens=20,
                            max_sequence_length=64, max_generated_tokens=32)
    roomy = _engine(folders["A"], "float32", device, page_size=4, num_pages=256, scheduler=sched, run_ahead=False)
    alone = [roomy.generate(prompts[i], params(i)).generated_token_ids() for i in range(n)]
    stops = [alone[i][len(alone[i]) // 2] if (i % 3 == 0 and len(alone[i]) > 2) else None for i in range(n)]
    arrive = sorted(rng.randint(0, 14) for _ in range(n))
    cancel_at = {i: arrive[i] + rng.randint(2, 12) for i in range(n) if i % 4 == 1}

    def run(run_ahead):
        engine = _engine(folders["A"], "float32", device, page_size=4, num_pages=20, scheduler=sched, run_ahead=run_ahead)
        ids, step = {}, 0
        while len(ids) < n or engine.has_unfinished():
            for i in range(n):
                if i not in ids and arrive[i] <= step:
                    ids[i] = engine.submit(prompts[i], params(i, stops[i]))
            for i, at in cancel_at.items():
                if at == step and i in ids:
                    engine.abort(ids[i])
            engine.step()
            engine.runner.cache.check_invariants()
            step += 1
            assert step < 2000
        outs = {i: engine.output_of(ids[i]) for i in range(n)}
        _all_pages_are_back(engine)
        return outs, engine.scheduler.stats["preemptions"], engine.steps_run_ahead

    for run_ahead in (False, True):
        outs, preemptions, ahead = run(run_ahead)
        assert preemptions >= 1, "the pool is small enough to force a request out"
        assert (ahead > 0) == run_ahead
        for i in range(n):
            got, reason = outs[i].generated_token_ids(), outs[i].finish_reason
            if reason is FinishReason.CANCELLED:
                assert got == alone[i][:len(got)]
            elif stops[i] is not None:
                first = alone[i].index(stops[i])
                assert got == alone[i][:first + 1] and reason is FinishReason.STOP_TOKEN
            else:
                assert got == alone[i] and reason in (FinishReason.MAX_NEW_TOKENS, FinishReason.SESSION_LIMIT)
