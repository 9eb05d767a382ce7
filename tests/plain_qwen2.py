"""A plain, slow implementation of the Qwen2 decoder: whole sequences, no cache, one function per part.

It is the oracle of the tests.  It shares no code with the package: it reads config.json as a
dict and the tensors by their names in the model folder, and computes with torch's own operators
(float32, or float64 for a tighter oracle), on the CPU unless it is told another device.

It rests on the reference's formulas, each cited below by the file's path within
Micro-ATP/FerrisInfer.  The reference is Rust and cannot be compiled on this image (no cargo or
rustc), so it is never run; the hand-computed vectors of its unit tests are reproduced in
tests/golden/ and checked by tests/test_plain.py.

The sliding window (config keys use_sliding_window / sliding_window / max_window_layers) is not in
the reference, which never reads those keys (crates/ferrisinfer-io/src/hf.rs:315-369); here a
query at position P in a layer with index >= max_window_layers attends keys P-W+1..P.
"""

from __future__ import annotations

import math

import numpy as np
import torch


# ------------------------------------------------------------------------------------ config
def derived(config: dict) -> dict:
    """Sizes and constants with the reference's defaults (crates/ferrisinfer-io/src/hf.rs:315-369)."""
    heads = config["num_attention_heads"]
    head_dim = config.get("head_dim") or config["hidden_size"] // heads
    factor = config.get("partial_rotary_factor")
    factor = 1.0 if factor is None else factor
    layers = config["num_hidden_layers"]
    use_window = bool(config.get("use_sliding_window")) and config.get("sliding_window") is not None
    first_windowed = config.get("max_window_layers")
    first_windowed = layers if first_windowed is None else first_windowed
    return {
        "layers": layers,
        "heads": heads,
        "kv_heads": config.get("num_key_value_heads") or heads,
        "head_dim": head_dim,
        "rotary_dims": int(round(head_dim * factor)),
        "theta": 10000.0 if config.get("rope_theta") is None else config["rope_theta"],
        "eps": config["rms_norm_eps"],
        "tied": bool(config.get("tie_word_embeddings") or False),
        "windows": [config["sliding_window"] if (use_window and l >= first_windowed) else None for l in range(layers)],
    }


# ------------------------------------------------------------------------------------- parts
def embedding(ids, table):
    """h[t, :] = E[id_t, :]; no scaling (crates/ferrisinfer-kernel/src/cpu/attention.rs:3-99)."""
    return table[torch.as_tensor(ids, dtype=torch.long, device=table.device)]


def rms_norm(x, weight, eps):
    """mean_square = sum(x^2) / H; inv = 1 / sqrt(mean_square + eps); y = x * inv * w
    (crates/ferrisinfer-kernel/src/cpu/reduction.rs:35-41)."""
    mean_square = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    inv = 1.0 / torch.sqrt(mean_square + eps)
    return x * inv * weight


def linear(x, weight, bias=None):
    """y = x W^T (+ b).  The folder stores W as [out, in]; the reference transposes at load and
    computes out[n] += x[k] * W[k, n], then adds the bias per row
    (crates/ferrisinfer-kernel/src/cpu/matmul.rs:437-446; crates/ferrisinfer-runtime/src/reference.rs:1132-1191)."""
    y = x @ weight.t()
    return y if bias is None else y + bias


def rotary_inverse_frequencies(head_dim, rotary_dims, theta):
    """step = theta^(-2 / head_dim) in f32; inv_freq_0 = 1; inv_freq_{i+1} = inv_freq_i * step (a running
    product in f32; the exponent uses head_dim) (crates/ferrisinfer-kernel/src/cpu/attention.rs:1254-1276)."""
    step = np.power(np.float32(theta), np.float32(-2.0) / np.float32(head_dim), dtype=np.float32)
    freqs, f = [], np.float32(1.0)
    for _ in range(rotary_dims // 2):
        freqs.append(f)
        f = np.float32(f * step)
    return torch.tensor(np.array(freqs, dtype=np.float32))


def rope(x, positions, head_dim, rotary_dims, theta):
    """x: [n, heads, d].  angle = f32(pos) * inv_freq_i (an f32 product); pairs (i, i + R/2):
    lo' = lo cos - hi sin; hi' = hi cos + lo sin; dims >= R untouched
    (crates/ferrisinfer-kernel/src/cpu/attention.rs:1242-1292)."""
    if rotary_dims == 0:
        return x
    half = rotary_dims // 2
    inv_freq = rotary_inverse_frequencies(head_dim, rotary_dims, theta).to(x.device)  # f32
    pos = torch.as_tensor(positions, dtype=torch.float32, device=x.device)
    angle = (pos[:, None] * inv_freq[None, :]).to(torch.float32)  # the product itself is f32
    angle = angle.to(x.dtype)
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    lo, hi = x[..., :half], x[..., half:rotary_dims]
    out = x.clone()
    out[..., :half] = lo * cos - hi * sin
    out[..., half:rotary_dims] = hi * cos + lo * sin
    return out


def attention(q, k, v, positions, window=None):
    """q: [n, nh, d]; k, v: [n, nkv, d], all of one sequence whose rows stand at ``positions``
    (ascending).  Head hq reads kv head hq // (nh / nkv); s = (q . k) / sqrt(d); the query at
    position P attends keys at positions <= P (and > P - window); softmax; out = sum w v
    (crates/ferrisinfer-kernel/src/cpu/attention.rs:729-781; the running-maximum softmax of
    :1125-1155 equals the ordinary one)."""
    n, nh, d = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(d)
    pos = torch.as_tensor(positions, dtype=torch.long, device=q.device)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= pos[None, :] > (pos[:, None] - window)
    out = torch.empty_like(q)
    for hq in range(nh):
        hk = hq // group
        s = (q[:, hq, :] @ k[:, hk, :].t()) * scale
        s = s.masked_fill(~visible, float("-inf"))
        w = torch.softmax(s, dim=-1)
        out[:, hq, :] = w @ v[:, hk, :]
    return out


def silu(g):
    """g * 1 / (1 + exp(-g)) (crates/ferrisinfer-kernel/src/cpu/elementwise.rs:189-190)."""
    return g * (1.0 / (1.0 + torch.exp(-g)))


def swiglu_feed_forward(y, w_gate, w_up, w_down):
    """u = y W_up^T; g = silu(y W_gate^T); out = (u * g) W_down^T
    (crates/ferrisinfer-runtime/src/reference.rs:346-368; w1 = up_proj, w3 = gate_proj:
    crates/ferrisinfer-io/src/hf.rs:437-457)."""
    return linear(linear(y, w_up) * silu(linear(y, w_gate)), w_down)


def block(h, w, prefix, positions, dv, window):
    """Pre-norm residual block (crates/ferrisinfer-runtime/src/reference.rs:163-370)."""
    n = h.shape[0]
    nh, nkv, d = dv["heads"], dv["kv_heads"], dv["head_dim"]
    y = rms_norm(h, w[f"{prefix}.input_layernorm.weight"], dv["eps"])
    q = linear(y, w[f"{prefix}.self_attn.q_proj.weight"], w.get(f"{prefix}.self_attn.q_proj.bias"))
    k = linear(y, w[f"{prefix}.self_attn.k_proj.weight"], w.get(f"{prefix}.self_attn.k_proj.bias"))
    v = linear(y, w[f"{prefix}.self_attn.v_proj.weight"], w.get(f"{prefix}.self_attn.v_proj.bias"))
    q = rope(q.reshape(n, nh, d), positions, d, dv["rotary_dims"], dv["theta"])
    k = rope(k.reshape(n, nkv, d), positions, d, dv["rotary_dims"], dv["theta"])
    a = attention(q, k, v.reshape(n, nkv, d), positions, window).reshape(n, nh * d)
    h = h + linear(a, w[f"{prefix}.self_attn.o_proj.weight"])
    y = rms_norm(h, w[f"{prefix}.post_attention_layernorm.weight"], dv["eps"])
    return h + swiglu_feed_forward(y, w[f"{prefix}.mlp.gate_proj.weight"], w[f"{prefix}.mlp.up_proj.weight"],
                                   w[f"{prefix}.mlp.down_proj.weight"])


def forward(config: dict, weights: dict, ids, dtype=torch.float32, device=None):
    """Logits [n, V] of every position of the token sequence ``ids``
    (crates/ferrisinfer-runtime/src/reference.rs:517-524 with :372-423 and :145-149).
    ``weights`` holds the folder's tensors by name; they are widened to ``dtype`` first.
    ``device``: where torch computes (the tensors' own by default); the large configurations of the GPU tests
    run these same lines in float64 on the GPU, because the CPU takes minutes for them."""
    dv = derived(config)
    w = {n: t.to(device=device, dtype=dtype) for n, t in weights.items()}
    positions = list(range(len(ids)))
    h = embedding(ids, w["model.embed_tokens.weight"])
    for l in range(dv["layers"]):
        h = block(h, w, f"model.layers.{l}", positions, dv, dv["windows"][l])
    y = rms_norm(h, w["model.norm.weight"], dv["eps"])
    head = w["model.embed_tokens.weight"] if dv["tied"] else w["lm_head.weight"]
    return linear(y, head)


# ---------------------------------------------------------------------------------- sampling
def softmax_rows(x):
    """exp(x - max) / sum (crates/ferrisinfer-kernel/src/cpu/reduction.rs:75-141)."""
    e = torch.exp(x - x.max(dim=-1, keepdim=True).values)
    return e / e.sum(dim=-1, keepdim=True)


def greedy(logits_row):
    """argmax and its probability 1 / sum(exp(l - max)) (crates/ferrisinfer-runtime/src/sampler.rs:77-119).
    On an exact tie this engine takes the lowest index, as the reference's fused variant does
    (crates/ferrisinfer-kernel/src/cpu/matmul.rs:550-560)."""
    row = np.asarray(logits_row, dtype=np.float32)
    best = int(np.argmax(row))  # first maximum
    denom = np.float32(0.0)
    for v in row:
        denom = np.float32(denom + np.exp(np.float32(v - row[best]), dtype=np.float32))
    return best, float(np.float32(1.0) / denom)


class XorShift64Star:
    """x ^= x >> 12; x ^= x << 25; x ^= x >> 27; value = x * 0x2545F4914F6CDD1D; the top 24 bits
    give a float in [0, 1); seed 0 stands for 0x9e3779b97f4a7c15
    (crates/ferrisinfer-runtime/src/sampler.rs:50-75)."""

    MASK = (1 << 64) - 1

    def __init__(self, seed: int):
        self.state = 0x9E3779B97F4A7C15 if seed == 0 else seed & self.MASK

    def next_f32(self) -> float:
        x = self.state
        x ^= x >> 12
        x ^= (x << 25) & self.MASK
        x ^= x >> 27
        self.state = x
        value = (x * 0x2545F4914F6CDD1D) & self.MASK
        return float(np.float32(value >> 40) / np.float32(1 << 24))


def sample(logits_row, temperature, top_k, top_p, rng: XorShift64Star):
    """The reference's stochastic sampler (crates/ferrisinfer-runtime/src/sampler.rs:121-241):
    greedy if temperature <= 0, top_k == 1 or top_p <= 0; else the top_k largest logits sorted
    descending (ties: lower index first), w = exp(l/T - max/T) with T = max(T, f32 epsilon), the
    shortest prefix whose mass reaches top_p * total, one uniform draw u * retained_total, and a
    walk that subtracts weights until the threshold is <= 0.  top_k == 0 stands for the whole
    vocabulary (the reference clamps top_k to [1, V])."""
    row = np.asarray(logits_row, dtype=np.float32)
    V = row.shape[0]
    if temperature <= 0.0 or top_k == 1 or top_p <= 0.0:
        return greedy(row)
    k = V if top_k <= 0 else min(top_k, V)
    order = np.lexsort((np.arange(V), -row.astype(np.float64)))[:k]  # descending logit, ascending index
    T = np.float32(max(temperature, np.finfo(np.float32).eps))
    top = np.float32(row[order[0]] / T)
    weights = np.exp((row[order] / T - top).astype(np.float32)).astype(np.float32)
    total = np.float32(0.0)
    for wv in weights:
        total = np.float32(total + wv)
    p = np.float32(min(max(top_p, 0.0), 1.0))
    cutoff = total if p >= 1.0 else np.float32(total * p)
    retained, kept = np.float32(0.0), 0
    for wv in weights:
        retained = np.float32(retained + wv)
        kept += 1
        if retained >= cutoff:
            break
    kept = max(kept, 1)
    weights, order = weights[:kept], order[:kept]
    retained_total = np.float32(0.0)
    for wv in weights:
        retained_total = np.float32(retained_total + wv)
    threshold = np.float32(np.float32(rng.next_f32()) * retained_total)
    chosen = 0
    for i, wv in enumerate(weights):
        threshold = np.float32(threshold - wv)
        if threshold <= 0.0:
            chosen = i
            break
    return int(order[chosen]), float(weights[chosen] / retained_total)


def generate_greedy(config, weights, prompt, steps, dtype=torch.float32):
    """Greedy continuation by whole-sequence recomputation."""
    ids = list(prompt)
    out = []
    for _ in range(steps):
        logits = forward(config, weights, ids, dtype)
        tok, _ = greedy(logits[-1].to(torch.float32).numpy())
        out.append(tok)
        ids.append(tok)
    return out
