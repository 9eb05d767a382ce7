"""Another mixer and another architecture, defined HERE, registered, built, loaded and stepped without a change
to the package's files.

The toy mixer keeps a state of its own per request (no keys, no pages): s <- decay * s + x_t for each token in
order, out_t = s * gain.  The toy architecture puts it in layer 0, grouped-query attention in layer 1, names
layer 0 a second time in the run order (shared weights, a state of its own), and lets a last run of layer 1
read the cache that the earlier run of layer 1 wrote.  It is never anyone's model: it only shows that layers
are data.
"""

from dataclasses import asdict, dataclass

import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
F32 = torch.float32


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int = 120
    hidden_size: int = 48
    intermediate_size: int = 80
    num_heads: int = 3
    num_kv_heads: int = 1
    head_dim: int = 16
    decay: float = 0.75
    eps: float = 1e-5
    theta: float = 100.0
    architecture: str = "ToyDecayForCausalLM"

    @classmethod
    def from_dict(cls, d):
        names = set(cls.__dataclass_fields__) - {"architecture"}
        return cls(**{k: d[k] for k in names if k in d}, architecture=d["architectures"][0])

    def to_dict(self):
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        d["model_type"] = "toy_decay"
        return d


def register_toy():
    from ferrisinfer_b200.config import register_architecture
    from ferrisinfer_b200.parts import (FixedState, LayerPlan, Mixer, ModelPlan, PartSpec, RunStep, TensorSpec,
                                        register_part)

    class DecayMixer(Mixer):
        def __init__(self, hidden_size, decay):
            self.hidden_size, self.decay = hidden_size, decay
            self.gain = None

        def tensor_specs(self, prefix):
            return [TensorSpec(f"{prefix}.gain", (self.hidden_size,), "norm")]

        def bind(self, tensors, prefix):
            self.gain = tensors[f"{prefix}.gain"]

        def cache_need(self):
            return FixedState((self.hidden_size,), torch.float32)

        def forward(self, x, h, ctx, cache, owns_cache):
            for s in ctx.seqs:  # each request's tokens in order, its state carried in its slot
                state = cache.state[s.state_slot]
                for t in range(s.q_start, s.q_start + s.q_len):
                    state.mul_(self.decay).add_(x[t].float())
                    h[t] += state * self.gain

    register_part("mixer", "toy_decay", DecayMixer, replace=True)

    def plan(cfg: ToyConfig) -> ModelPlan:
        norm = PartSpec("rmsnorm", {"hidden_size": cfg.hidden_size, "eps": cfg.eps})
        ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
        attention = PartSpec("gqa_attention", {
            "hidden_size": cfg.hidden_size, "num_heads": cfg.num_heads, "num_kv_heads": cfg.num_kv_heads,
            "head_dim": cfg.head_dim, "window": None,
            "position": PartSpec("rotary", {"head_dim": cfg.head_dim, "rotary_dim": cfg.head_dim, "theta": cfg.theta})})
        decay = PartSpec("toy_decay", {"hidden_size": cfg.hidden_size, "decay": cfg.decay})
        layers = (LayerPlan("model.layers.0", decay, ffn, norm, norm), LayerPlan("model.layers.1", attention, ffn, norm, norm))
        return ModelPlan(
            architecture=cfg.architecture, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
            embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}),
            embedding_prefix="model.embed_tokens", layers=layers,
            run_order=(RunStep(0), RunStep(1), RunStep(0), RunStep(1, cache_of=1)),
            final_norm=norm, final_norm_prefix="model.norm",
            output=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                            "tied_to": "model.embed_tokens.weight"}),
            output_prefix="lm_head", max_positions=512)

    register_architecture("ToyDecayForCausalLM", ToyConfig, plan, replace=True)


def toy_plain_forward(cfg: ToyConfig, w: dict, ids):
    """Whole sequence, no cache, float64."""
    w = {k: v.double() for k, v in w.items()}
    n = len(ids)
    pos = list(range(n))
    h = plain.embedding(ids, w["model.embed_tokens.weight"])

    def ffn(h, p):
        y = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], cfg.eps)
        return h + plain.swiglu_feed_forward(y, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                                             w[f"{p}.mlp.down_proj.weight"])

    def decay_layer(h):
        p = "model.layers.0"
        y = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], cfg.eps)
        state = torch.zeros(cfg.hidden_size, dtype=torch.float64)
        out = []
        for t in range(n):
            state = cfg.decay * state + y[t]
            out.append(state * w[f"{p}.self_attn.gain"])
        return ffn(h + torch.stack(out), p)

    def attention_layer(h, kv_from=None):
        p = "model.layers.1"
        y = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], cfg.eps)
        nh, nkv, d = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        q = plain.linear(y, w[f"{p}.self_attn.q_proj.weight"], w[f"{p}.self_attn.q_proj.bias"]).view(n, nh, d)
        q = plain.rope(q, pos, d, d, cfg.theta)
        if kv_from is None:
            k = plain.linear(y, w[f"{p}.self_attn.k_proj.weight"], w[f"{p}.self_attn.k_proj.bias"]).view(n, nkv, d)
            v = plain.linear(y, w[f"{p}.self_attn.v_proj.weight"], w[f"{p}.self_attn.v_proj.bias"]).view(n, nkv, d)
            kv_from = (plain.rope(k, pos, d, d, cfg.theta), v)
        a = plain.attention(q, kv_from[0], kv_from[1], pos).reshape(n, nh * d)
        return ffn(h + plain.linear(a, w[f"{p}.self_attn.o_proj.weight"]), p), kv_from

    h = decay_layer(h)
    h, kv = attention_layer(h)
    h = decay_layer(h)  # the same weights again, a fresh state
    h, _ = attention_layer(h, kv_from=kv)  # reads the keys and values of the earlier run
    return plain.linear(plain.rms_norm(h, w["model.norm.weight"], cfg.eps), w["model.embed_tokens.weight"])


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(device, tmp_path):
    from ferrisinfer_b200.config import registered_architectures
    from ferrisinfer_b200.engine.runner import ModelRunner
    from ferrisinfer_b200.parts import FixedState, PagedKV
    from ferrisinfer_b200.weights import load_model

    register_toy()
    assert "ToyDecayForCausalLM" in registered_architectures()
    cfg = ToyConfig()
    folder = helpers.make_folder(tmp_path, cfg.to_dict(), seed=5, store_dtype="float32")
    config, weights = helpers.read_folder(folder)
    assert config["architectures"] == ["ToyDecayForCausalLM"] and "model.layers.0.self_attn.gain" in weights

    model, loaded = load_model(folder, "float32", device)
    assert loaded == cfg
    needs = model.cache_needs()
    assert isinstance(needs[0], FixedState) and isinstance(needs[1], PagedKV) and isinstance(needs[2], FixedState)
    assert needs[3] is None  # reads the cache of run 1

    requests = {f"t{i}": helpers.random_ids(cfg.vocab_size, n, n) for i, n in enumerate((40, 9, 27, 33, 18))}
    want = {}
    for rid, ids in requests.items():
        logits = toy_plain_forward(cfg, weights, ids).float()
        for p in range(len(ids)):
            want[(rid, p)] = logits[p]
    for steps in (helpers.trace_whole(requests), helpers.trace_portions(requests),
                  helpers.trace_mixed(requests, seed=1, max_live=3)):
        runner = ModelRunner(model, F32, device, page_size=4, num_pages=helpers.tokens_held(steps, 4) // 4,
                             max_requests=3)
        assert len(runner.cache.groups) == 1 and runner.cache.groups[0].members == [1]
        assert runner.cache.layer_caches[0].state.shape == (3, cfg.hidden_size)
        assert runner.cache.layer_caches[2].state.data_ptr() != runner.cache.layer_caches[0].state.data_ptr()
        got = helpers.replay(runner, steps)
        bad = helpers.first_mismatch(got, want, atol=2e-5, rtol=1e-4)
        assert bad is None, bad
        runner.cache.check_invariants()
