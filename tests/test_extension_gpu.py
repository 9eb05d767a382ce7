"""Another mixer and another architecture, defined HERE, registered, built, loaded and stepped without a change
to the package's files.

The toy mixer keeps a state of its own per request (no keys, no pages): s <- decay * s + x_t for each token in
order, out_t = s * gain.  It reads which token belongs to which request, and which slot holds that request's state,
from the step's DEVICE arrays alone (no loop over requests on the host), so it may be recorded into a CUDA graph:
its decode steps are replayed from graphs like the built-in mixers', padding rows and all.  The toy architecture
puts it in layer 0, grouped-query attention in layer 1, names
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
        graph_safe = True  # device-resident metadata only, no host loop, no synchronisation

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
            # s_t = decay^(j+1) s_before + sum_{i <= j} decay^(j-i) x_i for the j-th token of a request in this step:
            # a masked [T, T] matrix of powers of the decay built from ctx.token_seq, times the step's rows
            T = ctx.num_tokens
            seq = ctx.token_seq.long()
            rows = torch.arange(T, device=x.device)
            offset = rows - ctx.seq_q_start.long()[seq]
            lag = rows[:, None] - rows[None, :]
            same = (seq[:, None] == seq[None, :]) & (lag >= 0)
            powers = torch.where(same, torch.pow(self.decay, lag.clamp(min=0).float()), 0.0)
            slots = ctx.seq_state_slot.long()
            before = cache.state[slots[seq]]
            carried = torch.pow(self.decay, (offset + 1).float())[:, None] * before
            state = powers @ x.float() + carried
            h += state * self.gain
            last = ctx.seq_q_start.long()[1:] - 1  # each request's last row of the step holds its new state
            cache.state.index_copy_(0, slots, state[last])

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


VARIANTS = {
    # 32-bit, head size 16, pages of 4: the general attention kernel
    "f32": (ToyConfig(), torch.float32, 4, dict(atol=2e-5, rtol=1e-4)),
    # bfloat16, head size 64, pages of 16: the tensor-core attention kernels, also for the run that reads another
    # run's cache (its decode kernel rotates q and must take the token's key and value from the cache)
    "bf16": (ToyConfig(vocab_size=150, hidden_size=128, intermediate_size=96, num_heads=4, num_kv_heads=2, head_dim=64,
                       decay=0.6, theta=10000.0), torch.bfloat16, 16, helpers.TOL[torch.bfloat16]),
}


@pytest.mark.parametrize("variant", list(VARIANTS))
def test_a_toy_mixer_with_state_is_registered_built_and_stepped(variant, device, tmp_path):
    from ferrisinfer_b200.config import registered_architectures
    from ferrisinfer_b200.engine.runner import ModelRunner
    from ferrisinfer_b200.kernels import ops
    from ferrisinfer_b200.parts import FixedState, PagedKV
    from ferrisinfer_b200.weights import load_model

    cfg, dtype, page, tol = VARIANTS[variant]
    register_toy()
    assert "ToyDecayForCausalLM" in registered_architectures()
    folder = helpers.make_folder(tmp_path, cfg.to_dict(), seed=5, store_dtype="float32" if dtype is F32 else "bfloat16",
                                 score_std=1.5)
    config, weights = helpers.read_folder(folder)
    assert config["architectures"] == ["ToyDecayForCausalLM"] and "model.layers.0.self_attn.gain" in weights

    model, loaded = load_model(folder, dtype, device)
    assert loaded == cfg
    assert model.graph_safe, "a mixer with state that works from device arrays does not switch graphs off"
    needs = model.cache_needs()
    assert isinstance(needs[0], FixedState) and isinstance(needs[1], PagedKV) and isinstance(needs[2], FixedState)
    assert needs[3] is None  # reads the cache of run 1

    requests = {f"t{i}": helpers.random_ids(cfg.vocab_size, n, n) for i, n in enumerate((40, 9, 27, 33, 18, 70))}
    want = {}
    for rid, ids in requests.items():
        logits = toy_plain_forward(cfg, weights, ids).float()
        for p in range(len(ids)):
            want[(rid, p)] = logits[p]
    replays = 0
    for steps in (helpers.trace_whole(requests), helpers.trace_portions(requests), helpers.trace_tail_decoded(requests, 24),
                  helpers.trace_mixed(requests, seed=1, max_live=3)):
        runner = ModelRunner(model, dtype, device, page_size=page, num_pages=helpers.tokens_held(steps, page) // page,
                             max_requests=3)
        assert len(runner.cache.groups) == 1 and runner.cache.groups[0].members == [1]
        # one row per request slot and the padding slot's
        assert runner.cache.layer_caches[0].state.shape == (3 + 1, cfg.hidden_size)
        assert runner.cache.layer_caches[2].state.data_ptr() != runner.cache.layer_caches[0].state.data_ptr()
        got = helpers.replay(runner, steps)
        assert ops.kernel_status() == 0
        bad = helpers.first_mismatch(got, want, **tol)
        assert bad is None, bad
        runner.cache.check_invariants()
        replays += runner.graph_replays
    assert replays > 50, "the single-token steps of the model with the toy mixer were replayed from graphs"
