"""The engine against the plain implementation, cut and batched in every way, in 32-bit and in bfloat16."""

import pytest
import torch

import helpers
from helpers import TINY, TOL

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
SCORE_STD = 1.8
PAGE = {"A": 4, "B": 8, "C": 16, "D": 16}
LENGTHS = {"A": (5, 9, 17, 70), "B": (3, 11, 23, 40, 97), "C": (2, 33, 64), "D": (1, 16, 17, 95, 130)}


def _runner(folder, dtype, device, page_size, num_pages, max_requests=8):
    from ferrisinfer_b200.engine.runner import ModelRunner
    from ferrisinfer_b200.weights import load_model

    model, _ = load_model(folder, dtype, device)
    return ModelRunner(model, dtype, device, page_size=page_size, num_pages=num_pages, max_requests=max_requests)


def _requests(name, extra=()):
    vocab = TINY[name]["vocab_size"]
    lengths = tuple(LENGTHS[name]) + tuple(extra)
    return {f"r{i}": helpers.random_ids(vocab, n, 100 * i + n) for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    # queries and keys scaled up, so that the attention weights are far from uniform and the logits show a key
    # that is rotated wrongly, missing, or read from the wrong page
    return {name: helpers.make_folder(root, cfg, seed=11 + i, score_std=SCORE_STD) for i, (name, cfg) in enumerate(TINY.items())}


@pytest.fixture(scope="module")
def oracles(folders):
    out = {}
    for name, folder in folders.items():
        config, weights = helpers.read_folder(folder)
        out[name] = (config, weights)
    return out


def _check(name, dtype, device, folders, oracles, steps, requests, num_pages):
    runner = _runner(folders[name], dtype, device, PAGE[name], num_pages)
    got = helpers.replay(runner, steps)
    runner.cache.check_invariants()
    assert not runner.cache.requests, "every request of the trace has ended"
    assert all(g.pool.num_used == 0 for g in runner.cache.groups), "every page has come back"
    config, weights = oracles[name]
    want = helpers.oracle_logits(config, weights, requests)
    bad = helpers.first_mismatch(got, want, **TOL[dtype])
    assert bad is None, bad


def _pages_for(steps, page):
    return helpers.tokens_held(steps, round_to=page) // page


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_each_request_alone_and_whole(name, dtype, device, folders, oracles):
    requests = _requests(name)
    steps = helpers.trace_whole(requests)
    _check(name, dtype, device, folders, oracles, steps, requests, _pages_for(steps, PAGE[name]))


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_last_32_tokens_one_by_one(name, dtype, device, folders, oracles):
    requests = _requests(name, extra=(120,))
    steps = helpers.trace_tail_decoded(requests, tail=32)
    _check(name, dtype, device, folders, oracles, steps, requests, _pages_for(steps, PAGE[name]))


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_of_changing_size(name, dtype, device, folders, oracles):
    requests = _requests(name, extra=(131,))
    steps = helpers.trace_portions(requests)
    assert min(len(e["tokens"]) for s in steps for e in s["entries"]) <= 2
    _check(name, dtype, device, folders, oracles, steps, requests, _pages_for(steps, PAGE[name]))


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_requests_with_pages_used_again(name, dtype, device, folders, oracles):
    vocab = TINY[name]["vocab_size"]
    lengths = (45, 23, 61, 18, 37, 52, 29, 40)
    requests = {f"m{i}": helpers.random_ids(vocab, n, 7 * i + n) for i, n in enumerate(lengths)}
    steps = helpers.trace_mixed(requests, seed=5)
    assert max(len(s["entries"]) for s in steps) == 4
    assert any(len({len(e["tokens"]) == 1 for e in s["entries"]}) == 2 for s in steps), "portions beside decoded tokens"
    pages = _pages_for(steps, PAGE[name])
    assert pages * PAGE[name] < sum(lengths), "so few pages that they are used again"
    _check(name, dtype, device, folders, oracles, steps, requests, pages)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_long_decoding(dtype, device, folders, oracles):
    """A short prompt and then some three hundred tokens one by one, far past the window of B."""
    name = "B"
    requests = {"long": helpers.random_ids(TINY[name]["vocab_size"], 330, 3)}
    steps = helpers.trace_tail_decoded(requests, tail=322)
    _check(name, dtype, device, folders, oracles, steps, requests, _pages_for(steps, PAGE[name]))


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_decoding_a_batch_at_a_context_of_hundreds_of_keys(dtype, device, folders, oracles, monkeypatch):
    """Three requests of D (head size 64) with prompts of several hundred tokens, then decoded side by side: in
    bfloat16 the prompts' q/k/v products rotate and write the cache in their epilogue, the keys of each request
    are split into ranges over several CTAs, merged inside the output product, and the steps are replayed from
    a graph.  One of them ends early and a fourth takes its place."""
    from ferrisinfer_b200.kernels import ops

    fused_products = []
    real = ops.qkv_rope_gemm
    monkeypatch.setattr(ops, "qkv_rope_gemm", lambda *a, **k: (fused_products.append(1), real(*a, **k))[1])
    name = "D"
    vocab = TINY[name]["vocab_size"]
    requests = {"a": helpers.random_ids(vocab, 700, 1), "b": helpers.random_ids(vocab, 450, 2),
                "c": helpers.random_ids(vocab, 300, 3), "d": helpers.random_ids(vocab, 520, 4)}
    tail = {"a": 24, "b": 24, "c": 10, "d": 14}
    steps, n = [], 0
    for rid in ("a", "b", "c"):
        ids = requests[rid]
        head = len(ids) - tail[rid]
        for lo in range(0, head, 256):
            part = ids[lo:min(lo + 256, head)]
            steps.append({"step": n, "entries": [{"id": rid, "tokens": part, "want": [len(part) - 1]}], "end": []})
            n += 1
    done = {rid: len(requests[rid]) - tail[rid] for rid in ("a", "b", "c")}
    live = ["a", "b", "c"]
    while live:
        entries, ended = [], []
        for rid in live:
            p = done[rid]
            entries.append({"id": rid, "tokens": [requests[rid][p]], "want": [0]})
            done[rid] = p + 1
            if p + 1 == len(requests[rid]):
                ended.append(rid)
        steps.append({"step": n, "entries": entries, "end": ended})
        n += 1
        live = [r for r in live if r not in ended]
        if "c" in ended:  # the fourth request: its prompt whole beside the others' single tokens, then decoded with them
            ids = requests["d"]
            head = len(ids) - tail["d"]
            entries = [{"id": r, "tokens": [requests[r][done[r]]], "want": [0]} for r in live]
            for r in live:
                done[r] += 1
            entries.append({"id": "d", "tokens": ids[:head], "want": [head - 1]})
            steps.append({"step": n, "entries": entries, "end": []})
            n += 1
            done["d"] = head
            live.append("d")
    runner = _runner(folders[name], dtype, device, PAGE[name], _pages_for(steps, PAGE[name]))
    got = helpers.replay(runner, steps)
    runner.cache.check_invariants()
    config, weights = oracles[name]
    want = helpers.oracle_logits(config, weights, requests)
    want = {k: v for k, v in want.items() if k in got}
    assert len(got) > 70
    bad = helpers.first_mismatch(got, want, **TOL[dtype])
    assert bad is None, bad
    if dtype is torch.bfloat16:
        assert runner.graph_replays > 10
        assert len(fused_products) >= 3 * TINY[name]["num_hidden_layers"]
    else:
        assert not fused_products


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_a_recorded_long_step_runs_again_at_other_positions(dtype, device, folders, oracles):
    """Four requests of D whose second portions have the same shape (256 tokens, one request, block tables of
    the same width) but begin at different positions: the second is recorded as a graph, the third and fourth
    replay it.  Whatever a recorded step computes from the positions (rotation angles, cache slots) it has to
    compute again in every replay."""
    name = "D"
    vocab = TINY[name]["vocab_size"]
    firsts = {"a": 130, "b": 140, "c": 133, "d": 143}
    requests = {rid: helpers.random_ids(vocab, n + 256, 40 + i) for i, (rid, n) in enumerate(firsts.items())}
    steps = []
    for rid, n in firsts.items():
        ids = requests[rid]
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[:n], "want": [n - 1]}], "end": []})
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[n:], "want": [0, 100, 255]}], "end": [rid]})
    runner = _runner(folders[name], dtype, device, PAGE[name], _pages_for(steps, PAGE[name]))
    got = helpers.replay(runner, steps)
    assert runner.graph_replays >= 2
    config, weights = oracles[name]
    want = {k: v for k, v in helpers.oracle_logits(config, weights, requests).items() if k in got}
    assert len(want) == 16
    bad = helpers.first_mismatch(got, want, **TOL[dtype])
    assert bad is None, bad


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(name, dtype, device, folders, oracles):
    """Positions 0, 1, 2: a sequence of one token, and the first tokens fed one by one."""
    vocab = TINY[name]["vocab_size"]
    requests = {"one": helpers.random_ids(vocab, 1, 1), "three": helpers.random_ids(vocab, 3, 2)}
    steps = helpers.trace_tail_decoded(requests, tail=32)
    _check(name, dtype, device, folders, oracles, steps, requests, 8)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_window_pages_come_back_while_the_request_runs(dtype, device, folders):
    """In B's window group a long request never holds more pages than the window spans."""
    name = "B"
    runner = _runner(folders[name], dtype, device, PAGE[name], num_pages=40)
    ids = helpers.random_ids(TINY[name]["vocab_size"], 200, 9)
    from ferrisinfer_b200.engine.runner import StepEntry

    window_group = [g for g in runner.cache.groups if g.window is not None][0]
    full_group = [g for g in runner.cache.groups if g.window is None][0]
    most = 0
    for p in range(0, 200, 5):
        runner.step([StepEntry("w", ids[p:p + 5], [])])
        most = max(most, window_group.pool.num_used)
        runner.cache.check_invariants()
    span = -(-(TINY[name]["sliding_window"] + 5) // PAGE[name]) + 1
    assert most <= span, (most, span)
    assert full_group.pool.num_used == 200 // PAGE[name]
    runner.free_request("w")
    assert window_group.pool.num_used == 0 and full_group.pool.num_used == 0


def test_out_of_pages_is_an_error_and_changes_nothing(device, folders):
    from ferrisinfer_b200.engine.runner import StepEntry
    from ferrisinfer_b200.errors import OutOfPages

    runner = _runner(folders["A"], torch.float32, device, PAGE["A"], num_pages=4)
    ids = helpers.random_ids(256, 40, 1)
    runner.step([StepEntry("a", ids[:10], [])])
    used = runner.cache.groups[0].pool.num_used
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("a", ids[10:12], []), StepEntry("b", ids[:9], [])])
    assert runner.cache.groups[0].pool.num_used == used
    assert runner.num_tokens("a") == 10
    runner.cache.check_invariants()
