"""Each part of a layer alone, built from explicit sizes, against the plain function of the same part."""

import math
from types import SimpleNamespace

import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
F32, BF16 = torch.float32, torch.bfloat16
TOL = {F32: dict(atol=2e-5, rtol=1e-4), BF16: dict(atol=2e-2, rtol=3e-2)}


def rnd(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


class OnePart:
    """The least a 'model' must be for the step function to run it: here it wraps a single part."""

    bound = True

    def __init__(self, part, vocab_size, run):
        self.part, self.vocab_size, self.run = part, vocab_size, run
        self.plan = SimpleNamespace(max_positions=4096)
        self.result = None

    def cache_needs(self):
        need = getattr(self.part, "cache_need", lambda: None)()
        return [need]

    def forward(self, ctx, caches, logits_index, logits_out):
        self.result = self.run(self.part, ctx, caches[0])
        return None


def bind(part, prefix, tensors, dtype, device):
    from ferrisinfer_b200.parts.base import role_dtype

    placed = {}
    for spec in part.tensor_specs(prefix):
        if spec.name in tensors:
            assert tuple(tensors[spec.name].shape) == tuple(spec.shape)
            placed[spec.name] = tensors[spec.name].to(device=device, dtype=role_dtype(spec.role, dtype, F32)).contiguous()
    part.bind(placed, prefix)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_rmsnorm_part(dtype, device):
    from ferrisinfer_b200.parts import build_part, PartSpec

    norm = build_part("norm", PartSpec("rmsnorm", {"hidden_size": 200, "eps": 1e-4}))
    assert [(s.name, s.shape, s.role) for s in norm.tensor_specs("n")] == [("n.weight", (200,), "norm")]
    w = 1 + rnd((200,), 1, 0.1)
    bind(norm, "n", {"n.weight": w}, dtype, device)
    h = rnd((11, 200), 2, 2.0).to(device)
    out = torch.empty(11, 200, dtype=dtype, device=device)
    norm.forward(h, out)
    assert torch.allclose(out.cpu().double(), plain.rms_norm(h.cpu().double(), w.double(), 1e-4), **TOL[dtype])


def test_rotary_part_forms_frequencies_as_a_running_product():
    from ferrisinfer_b200.parts import build_part, PartSpec

    pos = build_part("position", PartSpec("rotary", {"head_dim": 48, "rotary_dim": 24, "theta": 50000.0}))
    table, rotary = pos.rotary_table("cpu")
    assert rotary == 24 and torch.equal(table, plain.rotary_inverse_frequencies(48, 24, 50000.0))
    none = build_part("position", PartSpec("none", {}))
    assert none.rotary_table("cpu") == (None, 0)
    with pytest.raises(ValueError):
        build_part("position", PartSpec("rotary", {"head_dim": 48, "rotary_dim": 25, "theta": 1.0}))


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_swiglu_part_adds_into_the_residual(dtype, device):
    from ferrisinfer_b200.engine.workspace import Workspace
    from ferrisinfer_b200.parts import build_part, PartSpec

    H, I, T = 72, 200, 13
    ffn = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}))
    w = {"f.gate_proj.weight": rnd((I, H), 3, 0.1), "f.up_proj.weight": rnd((I, H), 4, 0.1),
         "f.down_proj.weight": rnd((H, I), 5, 0.1)}
    stored = {n: t.to(dtype) for n, t in w.items()}
    bind(ffn, "f", dict(stored), dtype, device)
    x = rnd((T, H), 6).to(dtype)
    h0 = rnd((T, H), 7)
    h = h0.clone().to(device)
    ctx = SimpleNamespace(workspace=Workspace(device))
    ffn.forward(x.to(device), h, ctx)
    want = h0.double() + plain.swiglu_feed_forward(x.double(), stored["f.gate_proj.weight"].double(),
                                                   stored["f.up_proj.weight"].double(),
                                                   stored["f.down_proj.weight"].double())
    assert torch.allclose(h.cpu().double(), want, **TOL[dtype])


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("window, bias", [(None, True), (9, False)])
def test_attention_part_in_portions_equals_plain_attention(window, bias, dtype, device):
    """The mixer alone, stepped through the step function in portions, with sizes that no model here has."""
    from ferrisinfer_b200.engine.runner import ModelRunner, StepEntry
    from ferrisinfer_b200.parts import PartSpec, build_part

    H, nh, nkv, d, n = 40, 6, 2, 16, 45
    spec = PartSpec("gqa_attention", {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": d,
                                      "position": PartSpec("rotary", {"head_dim": d, "rotary_dim": 8, "theta": 777.0}),
                                      "window": window, "scale": 0.31})
    mixer = build_part("mixer", spec)
    names = {"q": (nh * d, H), "k": (nkv * d, H), "v": (nkv * d, H)}
    w = {f"a.{k}_proj.weight": rnd(shape, 10 + i, 0.2).to(dtype) for i, (k, shape) in enumerate(names.items())}
    w["a.o_proj.weight"] = rnd((H, nh * d), 14, 0.2).to(dtype)
    if bias:
        w.update({f"a.{k}_proj.bias": rnd((shape[0],), 20 + i, 0.2) for i, (k, shape) in enumerate(names.items())})
    bind(mixer, "a", dict(w), dtype, device)
    x_all = rnd((n, H), 30).to(dtype)
    outs = []

    def run(part, ctx, cache):
        rows = slice(run.offset, run.offset + ctx.num_tokens)
        h = torch.zeros(ctx.num_tokens, H, dtype=F32, device=device)
        part.forward(x_all[rows].to(device), h, ctx, cache, True)
        outs.append(h.cpu())
        run.offset += ctx.num_tokens

    run.offset = 0
    runner = ModelRunner(OnePart(mixer, 100, run), dtype, device, page_size=4, num_pages=16, max_requests=2)
    for size in (7, 2, 13, 1, 1, 21):
        runner.step([StepEntry("r", [0] * size, [])])
    got = torch.cat(outs).double()

    wd = {k: v.double() for k, v in w.items()}
    q = plain.linear(x_all.double(), wd["a.q_proj.weight"], wd.get("a.q_proj.bias")).view(n, nh, d)
    k = plain.linear(x_all.double(), wd["a.k_proj.weight"], wd.get("a.k_proj.bias")).view(n, nkv, d)
    v = plain.linear(x_all.double(), wd["a.v_proj.weight"], wd.get("a.v_proj.bias")).view(n, nkv, d)
    pos = list(range(n))
    q, k = plain.rope(q, pos, d, 8, 777.0), plain.rope(k, pos, d, 8, 777.0)
    # plain.attention scales by 1/sqrt(d); the part was given its own scale
    a = plain.attention(q * (0.31 * math.sqrt(d)), k, v, pos, window).reshape(n, nh * d)
    want = plain.linear(a, wd["a.o_proj.weight"])
    assert torch.allclose(got, want, **TOL[dtype]), (got - want).abs().max()


def test_embedding_and_tied_head(device):
    from ferrisinfer_b200.parts import PartSpec, build_part

    emb = build_part("embedding", PartSpec("token_embedding", {"vocab_size": 50, "hidden_size": 24}))
    head = build_part("output", PartSpec("linear_head", {"vocab_size": 50, "hidden_size": 24, "tied_to": "e.weight"}))
    assert head.tensor_specs("lm_head") == []
    table = rnd((50, 24), 40).to(device)
    emb.bind({"e.weight": table}, "e")
    head.bind({"e.weight": table}, "lm_head")
    h = torch.empty(3, 24, device=device)
    emb.forward(torch.tensor([4, 0, 49], dtype=torch.int32, device=device), h)
    assert torch.equal(h, table[[4, 0, 49]])
    logits = torch.empty(3, 50, device=device)
    head.forward(h, logits)
    assert torch.allclose(logits.cpu().double(), h.cpu().double() @ table.cpu().double().t(), atol=1e-5)
