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


# ------------------------------------------------------------------------------------------------------------
# The reference's unit vectors above use head size 2, theta 1, one kv head and a zero feed-forward, so they do not
# tell rotate-half pairs from interleaved ones, fix no frequency schedule, no gate / up role and no head-to-kv-head
# mapping.  The reference cannot be run here, and model code of installed packages is not a source for this
# project, so those four readings rest on the cited lines.  What the tests below add is a second evaluation of each
# of them, element by element with ``math`` alone from the cited formula, at sizes where a slip in the vectorised
# code (a wrong slice, a transposed pair, a head mapped to the wrong kv head) shows.
# ------------------------------------------------------------------------------------------------------------
def test_rotary_pairs_and_frequencies_element_by_element():
    """crates/ferrisinfer-kernel/src/cpu/attention.rs:1254-1291: step = theta^(-2/d); inv_freq_i a running product;
    pairs (i, i + R/2); dims >= R untouched."""
    import math

    import numpy as np

    d, R, theta, pos = 8, 4, 100.0, 3
    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, 2, d, generator=g, dtype=torch.float64)
    got = plain.rope(x, [pos], d, R, theta)[0]
    step = np.float32(theta) ** (np.float32(-2.0) / np.float32(d))
    inv = [np.float32(1.0)]
    for _ in range(R // 2 - 1):
        inv.append(np.float32(inv[-1] * step))
    for head in range(2):
        want = x[0, head].tolist()
        for i in range(R // 2):
            angle = float(np.float32(np.float32(pos) * inv[i]))
            lo, hi = x[0, head, i].item(), x[0, head, i + R // 2].item()
            want[i] = lo * math.cos(angle) - hi * math.sin(angle)
            want[i + R // 2] = hi * math.cos(angle) + lo * math.sin(angle)
        assert max(abs(a - b) for a, b in zip(got[head].tolist(), want)) < 1e-12
    assert torch.equal(got[:, R:], x[0, :, R:])


def test_heads_read_their_kv_head_element_by_element():
    """crates/ferrisinfer-kernel/src/cpu/attention.rs:744-757: head hq reads kv head hq / (nh / nkv), keys 0..=P."""
    import math

    n, nh, nkv, d = 5, 6, 2, 4
    g = torch.Generator().manual_seed(2)
    q = torch.randn(n, nh, d, generator=g, dtype=torch.float64)
    k = torch.randn(n, nkv, d, generator=g, dtype=torch.float64)
    v = torch.randn(n, nkv, d, generator=g, dtype=torch.float64)
    got = plain.attention(q, k, v, list(range(n)))
    for p in range(n):
        for hq in range(nh):
            hk = hq // (nh // nkv)
            s = [sum(q[p, hq, c].item() * k[j, hk, c].item() for c in range(d)) / math.sqrt(d) for j in range(p + 1)]
            m = max(s)
            w = [math.exp(a - m) for a in s]
            for c in range(d):
                want = sum(w[j] * v[j, hk, c].item() for j in range(p + 1)) / sum(w)
                assert abs(got[p, hq, c].item() - want) < 1e-12


def test_gate_and_up_roles_element_by_element():
    """crates/ferrisinfer-runtime/src/reference.rs:346-368 with crates/ferrisinfer-io/src/hf.rs:437-457: the SiLU is
    taken of the gate_proj product (w3), which multiplies the up_proj product (w1)."""
    import math

    H, I = 3, 4
    g = torch.Generator().manual_seed(3)
    y = torch.randn(1, H, generator=g, dtype=torch.float64)
    wg, wu = (torch.randn(I, H, generator=g, dtype=torch.float64) for _ in range(2))
    wd = torch.randn(H, I, generator=g, dtype=torch.float64)
    got = plain.swiglu_feed_forward(y, wg, wu, wd)[0]
    act = []
    for i in range(I):
        gate = sum(y[0, c].item() * wg[i, c].item() for c in range(H))
        up = sum(y[0, c].item() * wu[i, c].item() for c in range(H))
        act.append(up * (gate * (1.0 / (1.0 + math.exp(-gate)))))
    for o in range(H):
        assert abs(got[o].item() - sum(act[i] * wd[o, i].item() for i in range(I))) < 1e-12
