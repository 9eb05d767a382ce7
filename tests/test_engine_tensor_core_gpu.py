"""The scheduler, prefix sharing, preemption and the step that runs ahead, over the tensor-core kernels.

The tiny configurations A and B have head sizes 16 and 32, so in bfloat16 they run the general attention kernel.
Here the same schedules run on configuration D (head size 64, pages of 16) and on a model with the layer sizes of
the smallest published size, in both precisions, with folders whose attention scores are spread out: the decode
kernel that rotates and writes the cache (and, when a step runs ahead, reads a token id that the host has not
seen), the merge of key ranges inside the output product, the q/k/v product with rotation in its epilogue, shared
pages of 16 tokens, and graphs filled up to a bucket.  Every token that the engine chooses is checked against the
plain implementation's logits for the engine's own prefix; logits of shared pages are compared directly.
"""

import random

import pytest
import torch

import helpers
import plain_qwen2 as plain
from helpers import TINY, TOL
from test_real_sizes_gpu import SIZES

pytestmark = pytest.mark.gpu

PAGE = 16
# D has a window from its second layer on, and pages of prompts are shared only where every layer keeps all keys:
# the tests of sharing run on D without its window
CONFIGS = {"D": TINY["D"], "D-no-window": dict(TINY["D"], use_sliding_window=False),
           "0.5B": dict(SIZES["0.5B"], vocab_size=1201)}
SHARING = ["D-no-window", "0.5B"]
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("tc-engine")
    return {name: helpers.make_folder(root, cfg, seed=51 + i, score_std=1.0 if name == "0.5B" else 1.8)
            for i, (name, cfg) in enumerate(CONFIGS.items())}


@pytest.fixture(scope="module")
def oracle(folders, device):
    """(config, weights on the device) per folder, and a function that gives the plain logits of a sequence."""
    loaded = {}
    for name, folder in folders.items():
        config, weights = helpers.read_folder(folder)
        loaded[name] = (config, {n: t.to(device) for n, t in weights.items()})

    def logits(name, ids):
        config, weights = loaded[name]
        return plain.forward(config, weights, ids, torch.float64).to("cpu", torch.float32)

    return logits


def _slack(dtype, rows: torch.Tensor) -> float:
    """How far below the plain maximum a chosen logit may lie: twice what the replay tests allow a logit to be off."""
    t = TOL[torch.float32 if dtype == "float32" else torch.bfloat16]
    spread = rows.std().item()
    return 2 * (t["atol"] * max(1.0, spread / 0.2) + t["rtol"] * rows.abs().max().item())


def _follows_plain(oracle, name, dtype, prompt, generated):
    """Every generated token is (within rounding) the plain implementation's greedy choice for the same prefix."""
    rows = oracle(name, prompt + generated)[len(prompt) - 1:len(prompt) + len(generated) - 1]
    slack = _slack(dtype, rows)
    for i, tok in enumerate(generated):
        assert rows[i][tok] >= rows[i].max() - slack, (name, dtype, i, tok, int(rows[i].argmax()))


def _engine(folder, dtype, device, num_pages=256, **kw):
    from ferrisinfer_b200 import SchedulerConfig
    from ferrisinfer_b200.engine.engine import Engine

    sched = kw.pop("scheduler", None) or SchedulerConfig(
        max_batch_size=8, max_prefill_chunk_tokens=160, max_prefill_batch_tokens=384, max_sequence_length=1024,
        max_generated_tokens=64, min_prefix_share_tokens=32)
    return Engine(folder, dtype=dtype, device=device, page_size=PAGE, num_pages=num_pages, scheduler=sched, **kw)


def _pages_back(engine):
    cache = engine.runner.cache
    cache.check_invariants()
    assert not cache.requests
    cache.drop_idle()
    assert all(g.pool.num_used == 0 for g in cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["D", "0.5B"])
def test_greedy_generation_follows_the_plain_implementation(name, dtype, device, folders, oracle, monkeypatch):
    from ferrisinfer_b200 import SamplingParams
    from ferrisinfer_b200.kernels import ops

    vocab = CONFIGS[name]["vocab_size"]
    prompts = [helpers.random_ids(vocab, n, 3 * n) for n in (5, 140, 333, 61, 17)]
    engine = _engine(folders[name], dtype, device)
    calls = {"gemm_argmax": 0, "sample": 0}
    for fn in calls:
        real = getattr(ops, fn)

        def counted(*a, _fn=fn, _real=real, **k):
            calls[_fn] += 1
            return _real(*a, **k)

        monkeypatch.setattr(ops, fn, counted)
    outs = engine.generate(prompts, SamplingParams.greedy(max_new_tokens=12))
    assert ops.kernel_status() == 0
    # greedy rows are picked by the output head itself: in bfloat16 without logits, in 32-bit through the sampling kernel
    if dtype == "bfloat16":
        assert calls["gemm_argmax"] > 0 and calls["sample"] == 0
    else:
        assert calls["gemm_argmax"] == 0 and calls["sample"] > 0
    for prompt, out in zip(prompts, outs):
        assert len(out.generated_token_ids()) == 12
        _follows_plain(oracle, name, dtype, prompt, out.generated_token_ids())
    if dtype == "bfloat16":
        assert engine.runner.graph_replays > 0 and engine.steps_run_ahead > 0
    _pages_back(engine)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", SHARING)
def test_requests_that_begin_alike_share_pages(name, dtype, device, folders, oracle):
    """Six requests share a beginning of 200 tokens: the later ones hold the first one's pages, compute only what
    differs, and choose the tokens that the plain implementation chooses for their whole sequences."""
    from ferrisinfer_b200 import SamplingParams

    vocab = CONFIGS[name]["vocab_size"]
    stem = helpers.random_ids(vocab, 200, 77)
    prompts = [stem + helpers.random_ids(vocab, 5 + 9 * i, 200 + i) for i in range(6)]
    params = SamplingParams.greedy(max_new_tokens=8)
    engine = _engine(folders[name], dtype, device)
    first = engine.submit(prompts[0], params)
    while not engine.scheduler.running or engine.scheduler.running[0].num_computed < len(prompts[0]):
        engine.step()
    rest = [engine.submit(p, params) for p in prompts[1:]]
    seen_twice = False
    while engine.has_unfinished():
        engine.step()
        cache = engine.runner.cache
        cache.check_invariants()
        tables = [set(rc.tables[0]) for rc in cache.requests.values()]
        seen_twice |= any(a & b for i, a in enumerate(tables) for b in tables[i + 1:])
    outs = [engine.output_of(i) for i in [first] + rest]
    assert seen_twice, "a page id stood in two block tables"
    assert all(o.reused_prompt_tokens == 192 for o in outs[1:]) and outs[0].reused_prompt_tokens == 0
    assert engine.runner.cache.stats["shared_pages"] >= 5 * 12
    for prompt, out in zip(prompts, outs):
        _follows_plain(oracle, name, dtype, prompt, out.generated_token_ids())
    _pages_back(engine)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", SHARING)
def test_logits_over_shared_pages_are_the_plain_logits(name, dtype, device, folders, oracle):
    """Below the scheduler: requests are admitted with their prompts on a runner that shares pages, step in
    portions beside each other's single tokens, and the logits at EVERY computed position are compared with the
    plain implementation's.  One request ends and a later one still finds its pages."""
    from ferrisinfer_b200.engine.runner import ModelRunner, StepEntry
    from ferrisinfer_b200.weights import load_model

    torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    vocab = CONFIGS[name]["vocab_size"]
    stem = helpers.random_ids(vocab, 150, 5)
    requests = {"a": stem + helpers.random_ids(vocab, 40, 1), "b": stem + helpers.random_ids(vocab, 9, 2),
                "c": stem[:100] + helpers.random_ids(vocab, 70, 3), "d": stem + helpers.random_ids(vocab, 21, 4)}
    model, _ = load_model(folders[name], torch_dtype, device)
    runner = ModelRunner(model, torch_dtype, device, page_size=PAGE, num_pages=64, max_requests=4,
                         prefix_sharing=True, min_prefix_share_tokens=16, keep_finished=True)
    got, done = {}, {}

    def run(shares):
        """shares: request -> number of its next tokens in this step; logits at all of them."""
        entries = [StepEntry(r, requests[r][done[r]:done[r] + n], list(range(n))) for r, n in shares.items()]
        logits = runner.step(entries).detach().to("cpu", torch.float32).clone()
        row = 0
        for r, n in shares.items():
            for j in range(n):
                got[(r, done[r] + j)] = logits[row]
                row += 1
            done[r] += n

    runner.add_request("a", requests["a"])
    done["a"] = runner.num_tokens("a")
    assert done["a"] == 0
    run({"a": 160})  # ten full pages of the prompt are in the cache now
    runner.add_request("b", requests["b"])
    done["b"] = runner.num_tokens("b")
    assert done["b"] == 144, "nine full pages borrowed (never the whole of what they share, 150 tokens)"
    runner.add_request("c", requests["c"])
    done["c"] = runner.num_tokens("c")
    assert done["c"] == 96
    assert runner.cache.block_table("a", 0)[:6] == runner.cache.block_table("b", 0)[:6] == runner.cache.block_table("c", 0)[:6]
    run({"a": 1, "b": 7, "c": 50})
    run({"a": 1, "b": 1, "c": 23})
    run({"b": 1, "a": 28})
    runner.free_request("a")
    runner.free_request("b")
    runner.add_request("d", requests["d"])  # finds the pages that "a" and "b" left behind
    done["d"] = runner.num_tokens("d")
    assert done["d"] == 144 and runner.cache.stats["revived_pages"] > 0
    run({"d": 20, "c": 1})
    run({"d": 1})
    runner.free_request("c")
    runner.free_request("d")
    runner.cache.check_invariants()
    assert runner.cache.stats["shared_pages"] >= 9 + 6 + 9
    want = {}
    for r, ids in requests.items():
        rows = oracle(name, ids)
        want.update({(r, p): rows[p] for p in range(len(ids)) if (r, p) in got})
    assert len(want) == len(got) > 250
    from test_real_sizes_gpu import _tolerance

    bad = helpers.first_mismatch(got, want, **_tolerance(torch_dtype, want))
    assert bad is None, bad


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["D", "0.5B"])
def test_a_recorded_step_of_several_requests_is_replayed_with_another_division(name, dtype, device, folders, oracle):
    """Steps of 256 tokens from three requests whose longest share is 200: the shape is recorded the second time it
    comes and replayed afterwards with the tokens divided differently among the requests, the longest share in
    another place, other rows wanted and other positions.  What a recorded step takes from its metadata it has to
    take again at every replay."""
    from ferrisinfer_b200.engine.runner import ModelRunner, StepEntry
    from ferrisinfer_b200.weights import load_model

    torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    vocab = CONFIGS[name]["vocab_size"]
    model, _ = load_model(folders[name], torch_dtype, device)
    runner = ModelRunner(model, torch_dtype, device, page_size=PAGE, num_pages=160, max_requests=4)
    divisions = [((200, 30, 26), (3, 17, 40), ([199], [5], [25])),
                 ((200, 30, 26), (20, 2, 33), ([0], [29], [3])),
                 ((10, 200, 46), (35, 9, 1), ([9], [100], [45])),
                 ((46, 10, 200), (0, 50, 18), ([1], [0], [199]))]
    got, requests = {}, {}
    for k, (shares, before, wants) in enumerate(divisions):
        entries = []
        for j, (n, b, w) in enumerate(zip(shares, before, wants)):
            rid = f"s{k}r{j}"
            requests[rid] = helpers.random_ids(vocab, b + n, 31 * k + j)
            if b:
                runner.step([StepEntry(rid, requests[rid][:b], [])])
            entries.append(StepEntry(rid, requests[rid][b:], w))
        logits = runner.step(entries).detach().to("cpu", torch.float32).clone()
        for row, (e, b) in enumerate(zip(entries, before)):
            got[(e.request_id, b + e.want[0])] = logits[row]
        for e in entries:
            runner.free_request(e.request_id)
    assert runner.graph_replays == 2, "recorded at the second step, replayed by the third and fourth"
    want = {}
    for (rid, p) in got:
        want[(rid, p)] = oracle(name, requests[rid])[p]
    from test_real_sizes_gpu import _tolerance

    bad = helpers.first_mismatch(got, want, **_tolerance(torch_dtype, want))
    assert bad is None, bad


@pytest.mark.parametrize("name", ["D", "0.5B"])
def test_recorded_steps_outlive_the_growth_of_the_workspace(name, device, folders, oracle):
    """A decode step is recorded while the activation buffers are small; a long portion then makes them grow.  The
    recorded step still points at the old buffers: they must stay alive and untouched by anyone else.  Tensors
    allocated after the growth (which would receive the old buffers' memory had it been freed) keep their contents
    through further replays, and the replayed steps' logits are still the plain implementation's."""
    from ferrisinfer_b200.engine.runner import ModelRunner, StepEntry
    from ferrisinfer_b200.weights import load_model

    vocab = CONFIGS[name]["vocab_size"]
    model, _ = load_model(folders[name], torch.bfloat16, device)
    runner = ModelRunner(model, torch.bfloat16, device, page_size=PAGE, num_pages=64, max_requests=4)
    ids = {"a": helpers.random_ids(vocab, 60, 1), "b": helpers.random_ids(vocab, 50, 2)}
    long_ids = helpers.random_ids(vocab, 400, 3)
    got = {}
    for r in ids:
        runner.step([StepEntry(r, ids[r][:20], [])])
    pos = 20

    def decode():
        nonlocal pos
        logits = runner.step([StepEntry(r, [ids[r][pos]], [0]) for r in ids]).detach().to("cpu", torch.float32).clone()
        for row, r in enumerate(ids):
            got[(r, pos)] = logits[row]
        pos += 1

    for _ in range(4):
        decode()
    assert runner.graph_replays >= 2
    small = runner.workspace.bytes()
    runner.step([StepEntry("long", long_ids, [])])  # every activation buffer grows
    assert runner.workspace.replaced_buffers > 0 and runner.workspace.bytes() > small
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    sentinels = [torch.full((n,), 7.0, dtype=torch.float32, device=device) for n in (256, 1024, 4096, 16384, 65536) for _ in range(8)]
    for _ in range(6):
        decode()
    torch.cuda.synchronize()
    assert all(bool((s == 7.0).all()) for s in sentinels), "a replayed step wrote into memory that is not its own"
    want = {(r, p): oracle(name, ids[r])[p] for (r, p) in got}
    from test_real_sizes_gpu import _tolerance

    bad = helpers.first_mismatch(got, want, **_tolerance(torch.bfloat16, want))
    assert bad is None, bad


def test_decode_graphs_are_few_and_bounded(device, folders):
    """A pool of 1 to 8 decoding requests is served by one graph per bucket of batch size, all writing one logits
    buffer, and no more than MAX_GRAPHS recorded steps are ever kept."""
    from ferrisinfer_b200.engine.runner import ModelRunner, StepEntry
    from ferrisinfer_b200.weights import load_model

    model, _ = load_model(folders["D"], torch.bfloat16, device)
    runner = ModelRunner(model, torch.bfloat16, device, page_size=PAGE, num_pages=64, max_requests=8)
    vocab = CONFIGS["D"]["vocab_size"]
    for r in range(8):
        runner.step([StepEntry(r, helpers.random_ids(vocab, 5 + r, r), [])])
    solo = {}
    for n in (1, 2, 3, 4, 5, 6, 7, 8, 5, 3, 7):
        logits = runner.step([StepEntry(r, [r + 1], [0]) for r in range(n)])
        assert logits.shape == (n, vocab)
        solo[n] = logits.clone()
    assert len(runner._graphs) == 4, "batch sizes 1, 2, 4 and 8"
    buffers = {e.logits.data_ptr() for e in runner._graphs.values()}
    assert len(buffers) == 1
    runner.drop_graphs()
    runner.MAX_GRAPHS = 2
    rng = random.Random(1)
    for _ in range(12):
        n = rng.choice((1, 2, 4, 8))
        assert runner.step([StepEntry(r, [3], [0]) for r in range(n)]).shape == (n, vocab)
        assert len(runner._graphs) <= 2
    assert runner.graphs_dropped >= 2
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", DTYPES)
def test_preemption_and_random_arrivals_over_the_tensor_core_kernels(dtype, device, folders, oracle):
    """Ten requests arrive at random steps into a pool that is too small for them, with a step running ahead: some
    are preempted and recomputed, one is cancelled; whatever each of them generated is what the plain implementation
    chooses for its sequence."""
    from ferrisinfer_b200 import FinishReason, SamplingParams, SchedulerConfig

    name = "D"
    rng = random.Random(9)
    vocab = CONFIGS[name]["vocab_size"]
    n = 10
    prompts = [helpers.random_ids(vocab, rng.randint(3, 150), 40 + i) for i in range(n)]
    budgets = [rng.randint(2, 30) for _ in range(n)]
    sched = SchedulerConfig(max_batch_size=6, max_prefill_chunk_tokens=64, max_prefill_batch_tokens=160,
                            max_sequence_length=256, max_generated_tokens=32, min_prefix_share_tokens=32)
    engine = _engine(folders[name], dtype, device, num_pages=26, scheduler=sched)  # 416 tokens for requests of up to 180
    arrive = sorted(rng.randint(0, 12) for _ in range(n))
    ids, step = {}, 0
    while len(ids) < n or engine.has_unfinished():
        for i in range(n):
            if i not in ids and arrive[i] <= step:
                ids[i] = engine.submit(prompts[i], SamplingParams.greedy(max_new_tokens=budgets[i]))
        if step == arrive[2] + 3:
            engine.abort(ids[2])
        engine.step()
        engine.runner.cache.check_invariants()
        step += 1
        assert step < 3000
    assert engine.scheduler.stats["preemptions"] >= 1 and engine.steps_run_ahead > 0
    for i in range(n):
        out = engine.output_of(ids[i])
        got = out.generated_token_ids()
        if out.finish_reason is not FinishReason.CANCELLED:
            assert len(got) == budgets[i]
        if got:
            _follows_plain(oracle, name, dtype, prompts[i], got)
    _pages_back(engine)
