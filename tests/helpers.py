"""Shared by the tests: tiny configurations, model folders, traces cut in different ways, comparison."""

from __future__ import annotations

import json
import os
import random

import numpy as np
import torch

# Tiny configurations of the architecture that differ in every size and option.
TINY_A = {  # tied head, 4 heads over 2 kv heads, head 16, no window
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "max_position_embeddings": 512,
    "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "hidden_act": "silu", "tie_word_embeddings": True,
    "use_sliding_window": False, "sliding_window": None, "max_window_layers": 2,
}
TINY_B = {  # untied head, 3 heads over 1 kv head, head 32, sizes that are no power of two, a window from layer 1 on
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 384, "hidden_size": 96, "intermediate_size": 224, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "max_position_embeddings": 1024,
    "rms_norm_eps": 1e-5, "rope_theta": 1000000.0, "hidden_act": "silu", "tie_word_embeddings": False,
    "use_sliding_window": True, "sliding_window": 21, "max_window_layers": 1,
}
TINY_C = {  # head_dim that is not hidden / heads, as many kv heads as heads, half of each head rotated
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 301, "hidden_size": 80, "intermediate_size": 176, "num_hidden_layers": 1,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48, "max_position_embeddings": 640,
    "rms_norm_eps": 3e-6, "rope_theta": 50000.0, "partial_rotary_factor": 0.5, "hidden_act": "silu",
    "tie_word_embeddings": False,
}
TINY_D = {  # head size 64 and pages of 16: the geometry that the tensor-core attention kernels take in bfloat16
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 200, "hidden_size": 128, "intermediate_size": 192, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64, "max_position_embeddings": 2048,
    "rms_norm_eps": 1e-6, "rope_theta": 30000.0, "hidden_act": "silu", "tie_word_embeddings": True,
    "use_sliding_window": True, "sliding_window": 48, "max_window_layers": 1,
}
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}


def random_config(rng: random.Random) -> dict:
    """A configuration of the architecture with sizes drawn at random: head sizes in steps of 16 from 16 to 128,
    any grouping of heads, widths that are multiples of 8 or only of 2, with and without a window, tied or not."""
    d = rng.choice([16, 32, 48, 64, 64, 80, 96, 128, 128])
    nkv = rng.choice([1, 2, 3, 4])
    nh = nkv * rng.choice([1, 2, 3, 4, 7])
    hidden = rng.choice([nh * d if nh * d <= 640 else 8 * rng.randint(6, 40), 8 * rng.randint(6, 40),
                         4 * rng.randint(11, 70) + 2 * rng.randint(0, 1)])
    layers = rng.randint(1, 4)
    window_on = rng.random() < 0.5
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": rng.randint(150, 700),
           "hidden_size": hidden, "intermediate_size": rng.choice([8 * rng.randint(10, 90), 2 * rng.randint(40, 300)]),
           "num_hidden_layers": layers, "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": d,
           "max_position_embeddings": 1024, "rms_norm_eps": rng.choice([1e-6, 1e-5, 3e-6]),
           "rope_theta": rng.choice([10000.0, 1e6, 50000.0]), "hidden_act": "silu",
           "tie_word_embeddings": rng.random() < 0.5, "use_sliding_window": window_on,
           "sliding_window": rng.randint(5, 90) if window_on else None, "max_window_layers": rng.randint(0, layers)}
    if rng.random() < 0.2:
        cfg["partial_rotary_factor"] = 0.5
    return cfg


def make_folder(tmp_path, config: dict, seed: int, store_dtype="bfloat16", optional=True, score_std: float = None) -> str:
    """A model folder of random weights.  Weights of N(0, 0.02) give attention scores of a few hundredths: every
    key gets nearly the same weight, and a wrong rotation, a wrong key or a wrong window's edge hardly moves the
    logits.  ``score_std`` multiplies the query and key projections (and their biases) so that the scores of
    random tokens have about this standard deviation (hidden x 0.02^2 without it): the attention weights are
    then far from uniform and the logits depend on which key is where."""
    from ferrisinfer_b200.weights import write_model_folder

    folder = os.path.join(str(tmp_path), f"model-{seed}-{store_dtype}" + (f"-scores{score_std:g}" if score_std else ""))
    write_model_folder(config, seed, folder, store_dtype=store_dtype, optional=optional)
    if score_std:
        from safetensors.torch import load_file, save_file

        factor = (score_std / (config["hidden_size"] * 0.02 ** 2)) ** 0.5
        path = os.path.join(folder, "model.safetensors")
        tensors = load_file(path)
        for name, t in tensors.items():
            if ".q_proj." in name or ".k_proj." in name:
                tensors[name] = (t.float() * factor).to(t.dtype)
        save_file(tensors, path)
    return folder


def read_folder(folder: str):
    """(config dict, tensors by name) read with the safetensors package, not with the engine's reader."""
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    return config, load_file(os.path.join(folder, "model.safetensors"))


def random_ids(vocab: int, n: int, seed: int) -> list:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


# ------------------------------------------------------------------------------------ traces
def trace_whole(requests: dict) -> list:
    """Each request alone and whole: one step each, logits at every place."""
    steps = []
    for i, (rid, ids) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]})
    return steps


def trace_tail_decoded(requests: dict, tail: int = 32) -> list:
    """Most of each request in one step, then its last ``tail`` tokens one by one."""
    steps, n = [], 0
    for rid, ids in requests.items():
        head = max(1, len(ids) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": ids[:head], "want": list(range(head))}], "end": []})
        n += 1
        for p in range(head, len(ids)):
            last = p == len(ids) - 1
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [ids[p]], "want": [0]}],
                          "end": [rid] if last else []})
            n += 1
        if head == len(ids):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: dict, sizes=(7, 2, 13, 3, 5, 2, 16, 4, 9, 2, 31, 6)) -> list:
    """Each request in portions of changing size, down to two tokens."""
    steps, n = [], 0
    for r, (rid, ids) in enumerate(requests.items()):
        p, k = 0, r  # start the size pattern at a different place for each request
        while p < len(ids):
            size = min(sizes[k % len(sizes)], len(ids) - p)
            k += 1
            steps.append({"step": n, "entries": [{"id": rid, "tokens": ids[p:p + size], "want": list(range(size))}],
                          "end": [rid] if p + size == len(ids) else []})
            p += size
            n += 1
    return steps


def trace_mixed(requests: dict, seed: int, max_live: int = 4, prompt_fraction: float = 0.6,
                sizes=(5, 2, 11, 3, 8, 2, 17)) -> list:
    """Up to ``max_live`` requests at a time: the first ``prompt_fraction`` of each comes in portions
    of changing size, the rest token by token; portions of some requests stand beside decoded tokens
    of others; a request sometimes sits a step out; when one ends, the next one starts, so pages
    come back and are used again."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = {}  # rid -> [ids, pos, prompt_len, pattern index]
    steps, n = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting.pop(0)
            live[rid] = [ids, 0, min(len(ids), max(2, int(len(ids) * prompt_fraction))), rng.randrange(len(sizes))]
        entries, ended = [], []
        order = list(live)
        rng.shuffle(order)
        for rid in order:
            ids, pos, prompt_len, k = live[rid]
            if len(order) > 1 and rng.random() < 0.2:
                continue  # left out of this step, goes on later
            if pos < prompt_len:
                size = min(sizes[k % len(sizes)], prompt_len - pos)
                live[rid][3] += 1
            else:
                size = 1
            entries.append({"id": rid, "tokens": ids[pos:pos + size], "want": list(range(size))})
            live[rid][1] = pos + size
            if pos + size == len(ids):
                ended.append(rid)
        if not entries:
            continue
        steps.append({"step": n, "entries": entries, "end": ended})
        n += 1
        for rid in ended:
            del live[rid]
    return steps


def tokens_held(steps: list, round_to: int = 64) -> int:
    """Most tokens that live requests hold at any time, each count rounded up to ``round_to``."""
    held, most = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(-(-v // round_to) * round_to for v in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return most


def replay(runner, steps: list) -> dict:
    """Drive ``runner.step`` with a trace; returns {(request id, position): logits row (CPU fp32)}."""
    from ferrisinfer_b200.engine.runner import StepEntry

    out, pos = {}, {}
    for s in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        logits = runner.step(entries)
        if logits is not None:
            logits = logits.detach().to("cpu", torch.float32).clone()
        row = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = logits[row]
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            runner.free_request(rid)
            pos.pop(rid, None)
    return out


def oracle_logits(config: dict, weights: dict, requests: dict, dtype=torch.float64, device=None) -> dict:
    """{(request id, position): logits row (CPU fp32)} from the plain implementation, whole sequences."""
    import plain_qwen2

    if device is not None:
        weights = {n: t.to(device) for n, t in weights.items()}
    out = {}
    for rid, ids in requests.items():
        logits = plain_qwen2.forward(config, weights, ids, dtype).to("cpu", torch.float32)
        for p in range(len(ids)):
            out[(rid, p)] = logits[p]
    return out


def first_mismatch(got: dict, want: dict, atol: float, rtol: float):
    """None, or a description of the first (request, position) whose logits differ beyond tolerance."""
    missing = [k for k in want if k not in got]
    if missing:
        return f"{len(missing)} positions have no logits, first {sorted(missing, key=str)[0]}"
    worst = None
    for key in sorted(want, key=lambda k: (str(k[0]), k[1])):
        g, w = got[key], want[key]
        err = (g - w).abs()
        bound = atol + rtol * w.abs()
        if not torch.isfinite(g).all() or (err > bound).any():
            i = int((err - bound).argmax())
            return (f"request {key[0]!r} position {key[1]}: logit {i} is {g[i].item():.6g}, expected {w[i].item():.6g} "
                    f"(|diff| {err[i].item():.3g}, max |diff| {err.max().item():.3g}, tolerance {bound[i].item():.3g})")
    return worst


# fp32: fp32 sums of a few hundred terms against a float64 oracle.  bf16: activations are rounded to 8 bits of
# mantissa (2^-9 relative) a few dozen times on the way; logits of these tiny models are O(0.1).
TOL = {torch.float32: dict(atol=2e-5, rtol=1e-4), torch.bfloat16: dict(atol=1.5e-2, rtol=3e-2)}
