"""The engine at the LAYER sizes of the three published sizes of the architecture, against the plain implementation.

Two layers each, a vocabulary of a few thousand (so that the float64 oracle stays cheap), pages of 16, query and
key projections scaled so that the attention scores spread over about a unit.  What only these widths bring together
runs here and is compared: the weight-stationary products of single tokens with the RMSNorm formed on their way,
key ranges of a decode step merged through a thread-block cluster, graphs of decode steps filled up to a bucket, the
q/k/v product of long portions with rotation and cache write in its epilogue over 14 + 2 + 2 heads, the gate/up
product on CTA pairs, both head sizes of the tensor-core attention kernels.  Every way of cutting: whole, the last
32 tokens one by one, portions of changing size down to two tokens, and up to four live requests mixed with so few
pages that they are used again; in 32-bit and in bfloat16.

The oracle is tests/plain_qwen2.py in float64, run on the GPU with torch's own operators (the CPU needs minutes
at the widest of these sizes).
"""

import pytest
import torch

import helpers
from helpers import TOL

pytestmark = pytest.mark.gpu

PAGE = 16


def _config(hidden, heads, kv_heads, head_dim, intermediate, vocab, tied):
    return {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": vocab, "hidden_size": hidden,
            "intermediate_size": intermediate, "num_hidden_layers": 2, "num_attention_heads": heads,
            "num_key_value_heads": kv_heads, "head_dim": head_dim, "max_position_embeddings": 4096,
            "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "hidden_act": "silu", "tie_word_embeddings": tied,
            "use_sliding_window": False, "sliding_window": None, "max_window_layers": 2}


# layer sizes of Qwen2.5-0.5B, -1.5B and -7B; vocabularies that are no power of two
SIZES = {
    "0.5B": _config(896, 14, 2, 64, 4864, 2501, True),
    "1.5B": _config(1536, 12, 2, 128, 8960, 3001, True),
    "7B": _config(3584, 28, 4, 128, 18944, 2003, False),
}
LENGTHS = {"a": 760, "b": 300, "c": 131, "d": 45}
MIXED_LENGTHS = (420, 150, 61, 300, 37, 200)


def _tolerance(dtype, want: dict) -> dict:
    """The tolerance of the tiny configurations is absolute 1.5e-2 on logits of about 0.2 (bfloat16) and 2e-5 (32-bit);
    here the logits are several times larger (a hidden size of thousands times weights of N(0, 0.02)), and what an
    8-bit mantissa or a 32-bit sum leaves behind grows with them: the absolute part is scaled by the spread of the
    oracle's logits over 0.2."""
    spread = torch.stack(list(want.values())[:64]).std().item()
    t = dict(TOL[dtype])
    t["atol"] = t["atol"] * max(1.0, spread / 0.2)
    return t


@pytest.fixture(scope="module")
def models(tmp_path_factory, device):
    """name -> (folder, requests, oracle logits), made at first use and kept for the module."""
    root = tmp_path_factory.mktemp("real-sizes")
    made = {}

    def get(name):
        if name not in made:
            cfg = SIZES[name]
            folder = helpers.make_folder(root, cfg, seed=70 + len(made), score_std=1.0)
            config, weights = helpers.read_folder(folder)
            vocab = cfg["vocab_size"]
            requests = {rid: helpers.random_ids(vocab, n, 17 * n) for rid, n in LENGTHS.items()}
            mixed = {f"m{i}": helpers.random_ids(vocab, n, 5 * n + i) for i, n in enumerate(MIXED_LENGTHS)}
            want = helpers.oracle_logits(config, weights, {**requests, **mixed}, torch.float64, device=device)
            made[name] = (folder, requests, mixed, want)
        return made[name]

    return get


def _runner(folder, dtype, device, num_pages, **kw):
    from ferrisinfer_b200.engine.runner import ModelRunner
    from ferrisinfer_b200.weights import load_model

    model, _ = load_model(folder, dtype, device)
    return ModelRunner(model, dtype, device, page_size=PAGE, num_pages=num_pages, max_requests=8, **kw)


class _Calls:
    """Counts the calls of some functions of ``ops`` while the engine runs."""

    def __init__(self, monkeypatch, names):
        from ferrisinfer_b200.kernels import ops

        self.count = {n: 0 for n in names}
        for n in names:
            real = getattr(ops, n)

            def counted(*a, _n=n, _real=real, **k):
                self.count[_n] += 1
                return _real(*a, **k)

            monkeypatch.setattr(ops, n, counted)


def _check(name, dtype, device, models, steps, which, monkeypatch=None, expect=()):
    folder, requests, mixed, want = models(name)
    asked = {**requests, **mixed}
    calls = _Calls(monkeypatch, expect) if monkeypatch is not None else None
    runner = _runner(folder, dtype, device, helpers.tokens_held(steps, round_to=PAGE) // PAGE)
    got = helpers.replay(runner, steps)
    from ferrisinfer_b200.kernels import ops

    assert ops.kernel_status() == 0
    runner.cache.check_invariants()
    assert not runner.cache.requests and all(g.pool.num_used == 0 for g in runner.cache.groups)
    wanted = {k: v for k, v in want.items() if k[0] in which}
    assert set(wanted) == set(got)
    bad = helpers.first_mismatch(got, wanted, **_tolerance(dtype, wanted))
    assert bad is None, bad
    return runner, calls


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(SIZES))
def test_each_request_alone_and_whole(name, dtype, device, models, monkeypatch):
    _, requests, _, _ = models(name)
    steps = helpers.trace_whole(requests)
    _, calls = _check(name, dtype, device, models, steps, requests, monkeypatch, ("qkv_rope_gemm", "prefill_attention"))
    if dtype is torch.bfloat16:
        assert calls.count["qkv_rope_gemm"] >= 6, "long prompts rotate and store in the q/k/v product's epilogue"
        assert calls.count["prefill_attention"] >= 8
    else:
        assert calls.count["qkv_rope_gemm"] == 0 and calls.count["prefill_attention"] == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(SIZES))
def test_last_32_tokens_one_by_one(name, dtype, device, models, monkeypatch):
    _, requests, _, _ = models(name)
    steps = helpers.trace_tail_decoded(requests, tail=32)
    runner, calls = _check(name, dtype, device, models, steps, requests, monkeypatch, ("gemm_skinny",))
    if dtype is torch.bfloat16:
        assert runner.graph_replays >= 100, "single tokens are replayed from graphs"
        assert len(runner._graphs) <= 6, "one graph per width of block table, not per request"
        assert calls.count["gemm_skinny"] >= 8, "the products of single tokens run the weight-stationary kernel"
    else:
        assert calls.count["gemm_skinny"] == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(SIZES))
def test_portions_of_changing_size(name, dtype, device, models):
    _, requests, _, _ = models(name)
    steps = helpers.trace_portions(requests, sizes=(7, 2, 130, 3, 257, 2, 16, 4, 9, 2, 31, 6, 129))
    assert min(len(e["tokens"]) for s in steps for e in s["entries"]) <= 2
    _check(name, dtype, device, models, steps, requests)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(SIZES))
def test_mixed_requests_with_pages_used_again(name, dtype, device, models):
    _, _, mixed, _ = models(name)
    steps = helpers.trace_mixed(mixed, seed=3, sizes=(150, 2, 37, 131, 3, 64))
    assert max(len(s["entries"]) for s in steps) == 4
    assert any(len({len(e["tokens"]) == 1 for e in s["entries"]}) == 2 for s in steps), "portions beside decoded tokens"
    pages = helpers.tokens_held(steps, round_to=PAGE) // PAGE
    assert pages * PAGE < sum(MIXED_LENGTHS), "so few pages that they are used again"
    _check(name, dtype, device, models, steps, mixed)


def test_full_depth_and_vocabulary_bfloat16_follows_32_bit(device):
    """All 24 layers and the whole vocabulary of the smallest published size, random weights drawn on the device:
    eight requests with prompts of 2,000 tokens (in portions of 512 beside each other), then sixteen steps of
    decoding side by side, the same given tokens in both precisions.  The bfloat16 engine's logits stay within
    tolerance of the 32-bit engine's, and its best token is one that 32 bits put within a hair of their best."""
    from ferrisinfer_b200.config import resolve_config
    from ferrisinfer_b200.engine.runner import ModelRunner, StepEntry
    from ferrisinfer_b200.parts.model import build_model
    from ferrisinfer_b200.weights.loader import bind_tensors
    from ferrisinfer_b200.weights.random_init import random_tensors

    cfg = dict(SIZES["0.5B"], vocab_size=151936, num_hidden_layers=24, max_position_embeddings=32768)
    arch, typed = resolve_config(cfg)
    prompts = [helpers.random_ids(cfg["vocab_size"], 2000, 900 + i) for i in range(8)]
    forced = [helpers.random_ids(cfg["vocab_size"], 16, 950 + i) for i in range(8)]
    logits = {}
    for dtype in (torch.float32, torch.bfloat16):
        model = build_model(arch.plan(typed))
        bind_tensors(model, random_tensors(typed, 3, "bfloat16", device=device), dtype, device)
        runner = ModelRunner(model, dtype, device, page_size=PAGE, num_pages=8 * 130, max_requests=8)
        rows = []
        for lo in range(0, 2000, 512):
            hi = min(lo + 512, 2000)
            out = runner.step([StepEntry(i, p[lo:hi], [hi - lo - 1] if hi == 2000 else []) for i, p in enumerate(prompts)])
            if out is not None:
                rows.append(out.clone())
        for s in range(16):
            rows.append(runner.step([StepEntry(i, [forced[i][s]], [0]) for i in range(8)]).clone())
        logits[dtype] = torch.cat(rows).float()
        if dtype is torch.bfloat16:
            assert runner.graph_replays >= 12
        del runner, model
        torch.cuda.empty_cache()
    want, got = logits[torch.float32], logits[torch.bfloat16]
    assert want.shape == (8 * 17, cfg["vocab_size"]) and torch.isfinite(got).all()
    spread = want.std().item()
    err = (got - want).abs()
    assert err.max().item() <= TOL[torch.bfloat16]["atol"] * max(1.0, spread / 0.2) + TOL[torch.bfloat16]["rtol"] * want.abs().max().item()
    best = want.max(dim=1).values
    chosen = want.gather(1, got.argmax(dim=1, keepdim=True)).squeeze(1)
    assert (best - chosen).max().item() <= 0.1 * spread
