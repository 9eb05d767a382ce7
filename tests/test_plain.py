"""The plain implementation against the reference's own hand-computed unit-test vectors, and against itself
in float64 (the reference cannot be built here, so these vectors are the anchor that exists)."""

import json
import os

import pytest
import torch

import helpers
import plain_qwen2 as plain

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_unit_vectors.json")))


def close(got, expected, tol):
    got, expected = torch.as_tensor(got, dtype=torch.float32), torch.tensor(expected, dtype=torch.float32)
    assert got.shape == expected.shape
    assert (got - expected).abs().max().item() <= tol, (got, expected)


def test_rms_norm_vector():
    g = GOLDEN["rms_norm"]
    close(plain.rms_norm(torch.tensor(g["input"]), torch.tensor(g["weight"]), g["eps"]), g["expected"], g["tolerance"])


def test_softmax_vector():
    g = GOLDEN["softmax"]
    close(plain.softmax_rows(torch.tensor(g["input"])), g["expected"], g["tolerance"])


def test_silu_vector():
    g = GOLDEN["silu"]
    close(plain.silu(torch.tensor(g["input"])), g["expected"], g["tolerance"])


def test_rope_vector():
    g = GOLDEN["rope"]
    x = torch.tensor(g["input"])
    n = x.shape[0]
    positions = [g["position_offset"] + i for i in range(n)]
    close(plain.rope(x, positions, x.shape[-1], g["rotary_dims"], g["theta"]), g["expected"], g["tolerance"])


@pytest.mark.parametrize("case", ["causal_attention", "gqa_attention"])
def test_attention_vectors(case):
    g = GOLDEN[case]
    q, k, v = (torch.tensor(g[n]) for n in ("query", "key", "value"))
    close(plain.attention(q, k, v, list(range(q.shape[0]))), g["expected"], g["tolerance"])


def _block_weights(g):
    t = lambda m: torch.tensor(m).t().contiguous()  # the reference stores [in, out]; the folder [out, in]
    p = "model.layers.0"
    return {
        f"{p}.input_layernorm.weight": torch.tensor(g["norm"]),
        f"{p}.post_attention_layernorm.weight": torch.tensor(g["norm"]),
        f"{p}.self_attn.q_proj.weight": t(g["wq"]), f"{p}.self_attn.k_proj.weight": t(g["wk"]),
        f"{p}.self_attn.v_proj.weight": t(g["wv"]), f"{p}.self_attn.o_proj.weight": t(g["wo"]),
        f"{p}.mlp.up_proj.weight": t(g["w1"]), f"{p}.mlp.down_proj.weight": t(g["w2"]),
        f"{p}.mlp.gate_proj.weight": t(g["w3"]),
    }


@pytest.mark.parametrize("case", ["block", "gqa_block"])
def test_block_vectors(case):
    g = GOLDEN[case]
    h = torch.tensor(g["input"])
    dv = {"heads": g["heads"], "kv_heads": g["kv_heads"], "head_dim": g["head_dim"], "rotary_dims": g["rotary_dims"],
          "theta": 10000.0, "eps": g["eps"]}
    out = plain.block(h, _block_weights(g), "model.layers.0", list(range(h.shape[0])), dv, None)
    close(out, g["expected"], g["tolerance"])


def test_model_logits_vector():
    g = GOLDEN["model_logits"]
    eye, zero, one = torch.eye(2), torch.zeros(2, 2), torch.ones(2)
    p = "model.layers.0"
    weights = {
        "model.embed_tokens.weight": eye, "lm_head.weight": eye, "model.norm.weight": one,
        f"{p}.input_layernorm.weight": one, f"{p}.post_attention_layernorm.weight": one,
        f"{p}.self_attn.q_proj.weight": eye, f"{p}.self_attn.k_proj.weight": eye, f"{p}.self_attn.v_proj.weight": eye,
        f"{p}.self_attn.o_proj.weight": eye, f"{p}.mlp.up_proj.weight": zero, f"{p}.mlp.gate_proj.weight": zero,
        f"{p}.mlp.down_proj.weight": zero,
    }
    config = {"num_attention_heads": 1, "hidden_size": 2, "num_hidden_layers": 1, "rms_norm_eps": 1e-5,
              "partial_rotary_factor": 0.0, "tie_word_embeddings": False}
    close(plain.forward(config, weights, g["ids"]), g["expected"], g["tolerance"])


def test_float32_and_float64_agree(tmp_path):
    folder = helpers.make_folder(tmp_path, helpers.TINY_B, seed=3)
    config, weights = helpers.read_folder(folder)
    ids = helpers.random_ids(config["vocab_size"], 50, 1)
    a = plain.forward(config, weights, ids, torch.float32)
    b = plain.forward(config, weights, ids, torch.float64).to(torch.float32)
    assert (a - b).abs().max().item() < 2e-6


def test_window_limits_what_a_query_sees():
    """One key far outside the window carries a huge value; it must not show in the windowed output."""
    n, d = 30, 8
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(n, 1, d, generator=g) for _ in range(3))
    v[3] = 1000.0
    full = plain.attention(q, k, v, list(range(n)))
    windowed = plain.attention(q, k, v, list(range(n)), window=5)
    assert full[-1].abs().max() > 1.0
    assert windowed[-1].abs().max() < 10.0
    assert torch.allclose(windowed[:5], full[:5])  # the first five queries see everything either way
    assert windowed[7].abs().max() > 10.0  # position 7 still sees key 3 (7 - 5 < 3)
    assert windowed[8].abs().max() < 10.0  # position 8 does not


def test_sampler_walk_matches_the_reference_order():
    row = [0.1, 2.0, 1.0, 2.0, -1.0]
    tok, p = plain.greedy(row)
    assert tok == 1 and 0 < p < 1
    rng = plain.XorShift64Star(42)
    first = rng.next_f32()
    assert 0.0 <= first < 1.0
    rng = plain.XorShift64Star(42)
    tok, p = plain.sample(row, temperature=0.7, top_k=3, top_p=0.9, rng=rng)
    assert tok in (1, 3, 2)
    assert plain.sample(row, 0.0, 0, 1.0, rng)[0] == 1  # temperature 0 is greedy
    assert plain.sample(row, 1.0, 1, 1.0, rng)[0] == 1  # top_k 1 is greedy
