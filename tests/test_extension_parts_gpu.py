"""A feed-forward with routing and another position encoding, defined HERE, registered, built, loaded and stepped
without a change to the package's files.

The toy feed-forward sends each token to the one of E small gated experts that its router scores highest and
scales the expert's output by the router's probability.  The toy position encoding adds a sinusoid of the
position to every q and k head (it is not a rotation, so the attention mixer calls its ``apply`` and writes the
cache without rotating).  The toy architecture puts the routed feed-forward in layer 0 and the dense one in
layer 1.  None of this is anyone's model: it only shows that the kinds of a layer are data.
"""

import math
from dataclasses import asdict, dataclass

import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
F32 = torch.float32


@dataclass(frozen=True)
class ToyRoutedConfig:
    vocab_size: int = 150
    hidden_size: int = 40
    intermediate_size: int = 72
    expert_size: int = 24
    num_experts: int = 3
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 16
    amplitude: float = 0.5
    eps: float = 1e-6
    architecture: str = "ToyRoutedForCausalLM"

    @classmethod
    def from_dict(cls, d):
        names = set(cls.__dataclass_fields__) - {"architecture"}
        return cls(**{k: d[k] for k in names if k in d}, architecture=d["architectures"][0])

    def to_dict(self):
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        d["model_type"] = "toy_routed"
        return d


def sinusoid(positions: torch.Tensor, head_dim: int, amplitude: float) -> torch.Tensor:
    """[len(positions), head_dim]: amplitude * sin(p / 50^(i / head_dim) + i)."""
    i = torch.arange(head_dim, dtype=torch.float64, device=positions.device)
    return amplitude * torch.sin(positions.double()[:, None] / (50.0 ** (i / head_dim)) + i)


def register_toy():
    from ferrisinfer_b200.config import register_architecture
    from ferrisinfer_b200.parts import (FeedForward, LayerPlan, ModelPlan, PartSpec, PositionEncoding, RunStep, TensorSpec,
                                        register_part)

    class Top1Experts(FeedForward):
        def __init__(self, hidden_size, expert_size, num_experts):
            self.H, self.I, self.E = hidden_size, expert_size, num_experts
            self.router = self.gate = self.up = self.down = None

        def tensor_specs(self, prefix):
            specs = [TensorSpec(f"{prefix}.router.weight", (self.E, self.H), "vector")]  # kept in 32-bit
            for e in range(self.E):
                specs += [TensorSpec(f"{prefix}.experts.{e}.gate.weight", (self.I, self.H), "matrix"),
                          TensorSpec(f"{prefix}.experts.{e}.up.weight", (self.I, self.H), "matrix"),
                          TensorSpec(f"{prefix}.experts.{e}.down.weight", (self.H, self.I), "matrix")]
            return specs

        def bind(self, tensors, prefix):
            self.router = tensors[f"{prefix}.router.weight"]
            self.gate = [tensors[f"{prefix}.experts.{e}.gate.weight"] for e in range(self.E)]
            self.up = [tensors[f"{prefix}.experts.{e}.up.weight"] for e in range(self.E)]
            self.down = [tensors[f"{prefix}.experts.{e}.down.weight"] for e in range(self.E)]

        def forward(self, x, h, ctx):
            xf = x.float()
            prob = torch.softmax(xf @ self.router.t(), dim=-1)  # router in 32-bit
            top = prob.argmax(dim=-1)
            for e in range(self.E):
                rows = (top == e).nonzero().flatten()
                if rows.numel():
                    xe = xf[rows]
                    act = torch.nn.functional.silu(xe @ self.gate[e].float().t()) * (xe @ self.up[e].float().t())
                    h[rows] += (act @ self.down[e].float().t()) * prob[rows, e:e + 1]

    class AddedSinusoid(PositionEncoding):
        def __init__(self, head_dim, amplitude):
            self.head_dim, self.amplitude = head_dim, amplitude

        def tensor_specs(self, prefix):
            return []

        def bind(self, tensors, prefix):
            pass

        def apply(self, qkv, positions, num_heads, num_kv_heads, head_dim):
            enc = sinusoid(positions, head_dim, self.amplitude).to(qkv.dtype)
            heads = qkv[:, :(num_heads + num_kv_heads) * head_dim].view(qkv.shape[0], num_heads + num_kv_heads, head_dim)
            heads += enc[:, None, :]

    register_part("feed_forward", "toy_top1_experts", Top1Experts, replace=True)
    register_part("position", "toy_added_sinusoid", AddedSinusoid, replace=True)

    def plan(cfg: ToyRoutedConfig) -> ModelPlan:
        norm = PartSpec("rmsnorm", {"hidden_size": cfg.hidden_size, "eps": cfg.eps})
        dense = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
        routed = PartSpec("toy_top1_experts", {"hidden_size": cfg.hidden_size, "expert_size": cfg.expert_size,
                                               "num_experts": cfg.num_experts})
        attention = PartSpec("gqa_attention", {
            "hidden_size": cfg.hidden_size, "num_heads": cfg.num_heads, "num_kv_heads": cfg.num_kv_heads,
            "head_dim": cfg.head_dim, "window": None,
            "position": PartSpec("toy_added_sinusoid", {"head_dim": cfg.head_dim, "amplitude": cfg.amplitude})})
        layers = (LayerPlan("model.layers.0", attention, routed, norm, norm),
                  LayerPlan("model.layers.1", attention, dense, norm, norm))
        return ModelPlan(
            architecture=cfg.architecture, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
            embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}),
            embedding_prefix="model.embed_tokens", layers=layers, run_order=(RunStep(0), RunStep(1)),
            final_norm=norm, final_norm_prefix="model.norm",
            output=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "tied_to": None}),
            output_prefix="lm_head", max_positions=512)

    register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig, plan, replace=True)


def toy_plain_forward(cfg: ToyRoutedConfig, w: dict, ids):
    """Whole sequence, no cache, float64."""
    w = {k: v.double() for k, v in w.items()}
    n = len(ids)
    pos = list(range(n))
    enc = sinusoid(torch.tensor(pos), cfg.head_dim, cfg.amplitude)
    nh, nkv, d = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    h = plain.embedding(ids, w["model.embed_tokens.weight"])
    for layer in (0, 1):
        p = f"model.layers.{layer}"
        y = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], cfg.eps)
        q = plain.linear(y, w[f"{p}.self_attn.q_proj.weight"], w.get(f"{p}.self_attn.q_proj.bias")).view(n, nh, d) + enc[:, None]
        k = plain.linear(y, w[f"{p}.self_attn.k_proj.weight"], w.get(f"{p}.self_attn.k_proj.bias")).view(n, nkv, d) + enc[:, None]
        v = plain.linear(y, w[f"{p}.self_attn.v_proj.weight"], w.get(f"{p}.self_attn.v_proj.bias")).view(n, nkv, d)
        h = h + plain.linear(plain.attention(q, k, v, pos).reshape(n, nh * d), w[f"{p}.self_attn.o_proj.weight"])
        y = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], cfg.eps)
        if layer == 0:
            prob = torch.softmax(y @ w[f"{p}.mlp.router.weight"].t(), dim=-1)
            out = torch.zeros_like(h)
            for t in range(n):
                e = int(prob[t].argmax())
                m = f"{p}.mlp.experts.{e}"
                out[t] = plain.swiglu_feed_forward(y[t:t + 1], w[f"{m}.gate.weight"], w[f"{m}.up.weight"],
                                                   w[f"{m}.down.weight"])[0] * prob[t, e]
            h = h + out
        else:
            h = h + plain.swiglu_feed_forward(y, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                                              w[f"{p}.mlp.down_proj.weight"])
    return plain.linear(plain.rms_norm(h, w["model.norm.weight"], cfg.eps), w["lm_head.weight"])


def test_a_routed_feed_forward_and_another_position_encoding_are_registered_built_and_stepped(device, tmp_path):
    from ferrisinfer_b200.engine.runner import ModelRunner
    from ferrisinfer_b200.weights import load_model

    register_toy()
    cfg = ToyRoutedConfig()
    folder = helpers.make_folder(tmp_path, cfg.to_dict(), seed=9, store_dtype="float32")
    config, weights = helpers.read_folder(folder)
    assert "model.layers.0.mlp.experts.2.down.weight" in weights and "model.layers.1.mlp.gate_proj.weight" in weights
    assert weights["model.layers.0.mlp.router.weight"].shape == (cfg.num_experts, cfg.hidden_size)

    model, loaded = load_model(folder, "float32", device)
    assert loaded == cfg and not model.graph_safe, "the toy parts do not claim to be recordable"
    requests = {f"t{i}": helpers.random_ids(cfg.vocab_size, n, 7 * n) for i, n in enumerate((35, 6, 21, 48))}
    want, used = {}, set()
    for rid, ids in requests.items():
        logits = toy_plain_forward(cfg, weights, ids).float()
        for p in range(len(ids)):
            want[(rid, p)] = logits[p]
    for steps in (helpers.trace_whole(requests), helpers.trace_tail_decoded(requests, tail=12),
                  helpers.trace_portions(requests), helpers.trace_mixed(requests, seed=2, max_live=3)):
        runner = ModelRunner(model, F32, device, page_size=8, num_pages=helpers.tokens_held(steps, 8) // 8, max_requests=3)
        got = helpers.replay(runner, steps)
        bad = helpers.first_mismatch(got, want, atol=2e-5, rtol=1e-4)
        assert bad is None, bad
        runner.cache.check_invariants()
        assert runner.graph_replays == 0
