"""A position encoding that acts on the attention SCORES, defined HERE, registered, built, loaded and stepped without a
change to the package's files.

The toy encoding leaves q and k alone and adds ``slope[head] * (j - P)`` to the score of the key at position j for the
query at position P: a penalty linear in the distance, steeper for later heads.  The attention mixer learns of it
through ``PositionEncoding.score_slopes`` and hands the slopes to the attention kernels; the general kernel then
attends, whatever the head size and precision (the tensor-core kernels know no such term).  Positions enter the
model in no other way, so a wrong distance (a page's edge, a portion's start, a request's offset in a mixed step)
shows in the logits.  This is nobody's model: it only shows that what a position encoding may do is not fixed to
rotations.
"""

import math
from dataclasses import asdict, dataclass

import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class ToyDistanceConfig:
    vocab_size: int = 130
    hidden_size: int = 48
    intermediate_size: int = 88
    num_heads: int = 6
    num_kv_heads: int = 2
    head_dim: int = 16
    steepest: float = 0.5
    eps: float = 1e-5
    architecture: str = "ToyDistanceForCausalLM"

    @classmethod
    def from_dict(cls, d):
        names = set(cls.__dataclass_fields__) - {"architecture"}
        return cls(**{k: d[k] for k in names if k in d}, architecture=d["architectures"][0])

    def to_dict(self):
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        d["model_type"] = "toy_distance"
        return d


def slopes_of(num_heads: int, steepest: float) -> torch.Tensor:
    """slope[h] = steepest / 2^(num_heads - 1 - h): the last head forgets fastest."""
    return torch.tensor([steepest / 2.0 ** (num_heads - 1 - h) for h in range(num_heads)], dtype=torch.float64)


def register_toy():
    from ferrisinfer_b200.config import register_architecture
    from ferrisinfer_b200.parts import LayerPlan, ModelPlan, PartSpec, PositionEncoding, RunStep, register_part

    class LinearDistance(PositionEncoding):
        graph_safe = True  # nothing of it runs in a step: the slopes are a constant tensor

        def __init__(self, num_heads, steepest):
            self.num_heads, self.steepest = num_heads, steepest
            self._slopes = {}

        def tensor_specs(self, prefix):
            return []

        def bind(self, tensors, prefix):
            pass

        def rotary_table(self, device=None):
            return (None, 0)  # nothing to rotate, and nothing to apply to q and k

        def score_slopes(self, num_heads, device=None):
            assert num_heads == self.num_heads
            key = str(device)
            if key not in self._slopes:
                self._slopes[key] = slopes_of(num_heads, self.steepest).float().to(device)
            return self._slopes[key]

    register_part("position", "toy_linear_distance", LinearDistance, replace=True)

    def plan(cfg: ToyDistanceConfig) -> ModelPlan:
        norm = PartSpec("rmsnorm", {"hidden_size": cfg.hidden_size, "eps": cfg.eps})
        dense = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
        attention = PartSpec("gqa_attention", {
            "hidden_size": cfg.hidden_size, "num_heads": cfg.num_heads, "num_kv_heads": cfg.num_kv_heads,
            "head_dim": cfg.head_dim, "window": None,
            "position": PartSpec("toy_linear_distance", {"num_heads": cfg.num_heads, "steepest": cfg.steepest})})
        layers = (LayerPlan("model.layers.0", attention, dense, norm, norm),
                  LayerPlan("model.layers.1", attention, dense, norm, norm))
        return ModelPlan(
            architecture=cfg.architecture, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
            embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}),
            embedding_prefix="model.embed_tokens", layers=layers, run_order=(RunStep(0), RunStep(1)),
            final_norm=norm, final_norm_prefix="model.norm",
            output=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "tied_to": None}),
            output_prefix="lm_head", max_positions=1024)

    register_architecture("ToyDistanceForCausalLM", ToyDistanceConfig, plan, replace=True)


def attention_with_slopes(q, k, v, slopes):
    """q [n, nh, d], k and v [n, nkv, d] of one sequence at positions 0..n-1; s = q . k / sqrt(d) + slope (j - P)."""
    n, nh, d = q.shape
    group = nh // k.shape[1]
    pos = torch.arange(n, dtype=torch.float64)
    distance = pos[None, :] - pos[:, None]  # j - P
    visible = distance <= 0
    out = torch.empty_like(q)
    for hq in range(nh):
        s = (q[:, hq] @ k[:, hq // group].t()) / math.sqrt(d) + slopes[hq] * distance
        out[:, hq] = torch.softmax(s.masked_fill(~visible, float("-inf")), dim=-1) @ v[:, hq // group]
    return out


def toy_plain_forward(cfg: ToyDistanceConfig, w: dict, ids):
    """Whole sequence, no cache, float64."""
    w = {k: v.double() for k, v in w.items()}
    n = len(ids)
    nh, nkv, d = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    slopes = slopes_of(nh, cfg.steepest)
    h = plain.embedding(ids, w["model.embed_tokens.weight"])
    for layer in (0, 1):
        p = f"model.layers.{layer}"
        y = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], cfg.eps)
        q = plain.linear(y, w[f"{p}.self_attn.q_proj.weight"], w.get(f"{p}.self_attn.q_proj.bias")).view(n, nh, d)
        k = plain.linear(y, w[f"{p}.self_attn.k_proj.weight"], w.get(f"{p}.self_attn.k_proj.bias")).view(n, nkv, d)
        v = plain.linear(y, w[f"{p}.self_attn.v_proj.weight"], w.get(f"{p}.self_attn.v_proj.bias")).view(n, nkv, d)
        h = h + plain.linear(attention_with_slopes(q, k, v, slopes).reshape(n, nh * d), w[f"{p}.self_attn.o_proj.weight"])
        y = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], cfg.eps)
        h = h + plain.swiglu_feed_forward(y, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                                          w[f"{p}.mlp.down_proj.weight"])
    return plain.linear(plain.rms_norm(h, w["model.norm.weight"], cfg.eps), w["lm_head.weight"])


# head size 16 in 32-bit; head size 64 in bfloat16, a geometry that the tensor-core kernels would take if the scores
# had no slopes
@pytest.mark.parametrize("dtype, head_dim, hidden", [(torch.float32, 16, 48), (torch.bfloat16, 64, 128)],
                         ids=["f32-d16", "bf16-d64"])
def test_a_position_encoding_that_adds_to_the_scores_is_registered_built_and_stepped(dtype, head_dim, hidden, device,
                                                                                      tmp_path, monkeypatch):
    from ferrisinfer_b200.engine.runner import ModelRunner
    from ferrisinfer_b200.kernels import ops
    from ferrisinfer_b200.weights import load_model

    register_toy()
    cfg = ToyDistanceConfig(head_dim=head_dim, hidden_size=hidden)
    folder = helpers.make_folder(tmp_path, cfg.to_dict(), seed=11, store_dtype="float32" if dtype is torch.float32 else "bfloat16")
    config, weights = helpers.read_folder(folder)
    model, loaded = load_model(folder, dtype, device)
    assert loaded == cfg and model.graph_safe
    requests = {f"t{i}": helpers.random_ids(cfg.vocab_size, n, 5 * n) for i, n in enumerate((70, 9, 33, 52))}
    want = {}
    for rid, ids in requests.items():
        logits = toy_plain_forward(cfg, weights, ids).float()
        for p in range(len(ids)):
            want[(rid, p)] = logits[p]
    # the slopes matter: without them the last rows' logits differ by far more than the tolerance
    flat = toy_plain_forward(ToyDistanceConfig(head_dim=head_dim, hidden_size=hidden, steepest=0.0), weights,
                             requests["t0"]).float()
    assert (flat[-1] - want[("t0", 69)]).abs().max().item() > 20 * helpers.TOL[dtype]["atol"]
    calls = {"general": 0, "other": 0}
    real_simt, real_decode, real_prefill = ops.paged_attention_simt, ops.decode_attention, ops.prefill_attention

    def general(*a, **k):
        calls["general"] += 1
        assert k.get("score_slopes") is not None
        return real_simt(*a, **k)

    def other(*a, **k):
        calls["other"] += 1
        return real_decode(*a, **k)

    monkeypatch.setattr(ops, "paged_attention_simt", general)
    monkeypatch.setattr(ops, "decode_attention", other)
    monkeypatch.setattr(ops, "prefill_attention", lambda *a, **k: calls.__setitem__("other", calls["other"] + 1) or real_prefill(*a, **k))
    replays = 0
    for steps in (helpers.trace_whole(requests), helpers.trace_tail_decoded(requests, tail=12),
                  helpers.trace_portions(requests), helpers.trace_mixed(requests, seed=4, max_live=3)):
        runner = ModelRunner(model, dtype, device, page_size=16, num_pages=helpers.tokens_held(steps, 16) // 16, max_requests=3)
        got = helpers.replay(runner, steps)
        bad = helpers.first_mismatch(got, want, **helpers.TOL[dtype])
        assert bad is None, bad
        runner.cache.check_invariants()
        replays += runner.graph_replays
    assert ops.kernel_status() == 0
    assert calls["general"] > 0 and calls["other"] == 0, "scores with slopes are the general kernel's"
    assert replays > 0, "single tokens are replayed from graphs: nothing of the encoding runs in a step"
