#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, random-weight Qwen2.5-0.5B sizes, bfloat16.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value``: decoded tokens a second at batch 8 and context 4,096: regions of exactly K
decode steps each, timed on the device with CUDA events (step function + sampling kernel; token ids preset on
the host), the cache refilled between regions so that every region ends at the same context; the median region
is reported, the fastest and slowest beside it.  ``e2e``: the same through ``Engine.step()``: host token ids in
(pinned metadata, one copy per step) and sampled tokens out (one read per step).  ``prefill``: one 2,048-token
prompt.  ``roofline``: bytes a decode step must read (every weight once, the cache of the live requests) over
its time, against the measured copy bandwidth.  ``points``: decode at batch 1 and 64 with their fractions of that
roofline, and the workloads of the two larger published sizes (a mixed batch of 32 requests at the 1.5B sizes;
decode, prefill and eight requests that share a prefix at the 7B sizes).  ``kernels``: what the step's dominant
kernels reach alone, each timed over the weights or caches of all layers in turn (more than L2 holds).  Peaks come
from MEASURED_PEAKS.json when present, else the fallback figures of this pool.

The weights (1 GB) and the cache are far larger than the 126 MB L2, so every step reads them from
HBM; no explicit L2 flush is needed between timed steps.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# layer sizes of Qwen2.5-0.5B (the configuration the benchmark is quoted on)
QWEN25_05B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 151936, "hidden_size": 896, "intermediate_size": 4864, "num_hidden_layers": 24,
    "num_attention_heads": 14, "num_key_value_heads": 2, "max_position_embeddings": 32768,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "hidden_act": "silu", "tie_word_embeddings": True,
    "use_sliding_window": False, "sliding_window": None, "max_window_layers": 24,
}
QWEN25_15B = dict(QWEN25_05B, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28, num_attention_heads=12,
                  num_key_value_heads=2, max_window_layers=28)
QWEN25_7B = dict(QWEN25_05B, vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                 num_attention_heads=28, num_key_value_heads=4, tie_word_embeddings=False, max_window_layers=28)
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        out = dict(FALLBACK_PEAKS)
        for k in out:
            if isinstance(d.get(k), (int, float)) and d[k] > 0:
                out[k] = float(d[k])
        return out, "measured"
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the timed regions run."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200", "-i", "0"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}


def model_numbers(cfg: dict) -> dict:
    H, I, L, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or H // nh
    Q, KV = nh * d, nkv * d
    layer_matrix = H * (Q + 2 * KV) + Q * H + 3 * H * I
    layer_vectors = (Q + 2 * KV) + 2 * H
    head = V * H
    untied = 0 if cfg.get("tie_word_embeddings") else V * H
    return {"layer_matrix": layer_matrix, "layer_vectors": layer_vectors, "head": head, "untied_embedding": untied,
            "kv_bytes_per_token": L * 2 * KV * 2, "d": d, "nh": nh, "L": L, "H": H, "V": V}


def decode_bytes(cfg, batch, context) -> float:
    n = model_numbers(cfg)
    weights = (n["L"] * (n["layer_matrix"] * 2 + n["layer_vectors"] * 4) + n["head"] * 2 + n["H"] * 4)  # tied or not: the head is read once
    return float(weights + batch * context * n["kv_bytes_per_token"])


def prefill_flops(cfg, T) -> float:
    n = model_numbers(cfg)
    linear = 2.0 * T * n["L"] * n["layer_matrix"] + 2.0 * n["head"]
    attention = n["L"] * 2.0 * T * T * n["d"] * n["nh"]
    return linear + attention


def build_engine(cfg, batch, context, extra_tokens=0):
    from ferrisinfer_b200 import SchedulerConfig
    from ferrisinfer_b200.engine.engine import Engine

    page = 16
    per_request = -(-(context + 8) // page)
    sched = SchedulerConfig(max_batch_size=batch, max_prefill_chunk_tokens=2048,
                            max_prefill_batch_tokens=max(2048, batch), max_sequence_length=context + 8,
                            max_generated_tokens=context)
    return Engine(config=cfg, seed=0, dtype="bfloat16", page_size=page, init_device="cuda",
                  num_pages=batch * per_request + -(-extra_tokens // page) + 4, scheduler=sched)


def fill_cache(engine, batch, context):
    """Give ``batch`` requests ``context`` tokens of cache without running the model: pages are taken
    from the pool as a real prompt would take them and filled with small random keys and values."""
    import torch

    cache = engine.runner.cache
    for lc in cache.layer_caches:
        if lc is not None and lc.k is not None:
            lc.k.normal_(0.0, 0.5)
            lc.v.normal_(0.0, 0.5)
    ids = []
    for b in range(batch):
        rid = f"bench{b}"
        cache.admit(rid)
        cache.extend(rid, context)
        cache.commit(rid, context)
        ids.append(rid)
    return ids


def time_decode(engine, batch, context, steps, warmup, regions=1):
    """Regions of exactly ``steps`` decode steps (step function with greedy sampling in its output head), each timed with CUDA
    events after ``warmup`` untimed steps; the cache is refilled before every region, so that each one ends at
    ``context``.  Returns (ms per step of each region, kernel launches of one region)."""
    import torch

    from ferrisinfer_b200.engine.runner import StepEntry
    from ferrisinfer_b200.kernels import ops

    vocab = engine.model.vocab_size
    gen = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, vocab, (steps + warmup, batch), generator=gen).tolist()
    times, launches = [], 0
    for _ in range(max(1, regions)):
        ids = fill_cache(engine, batch, context - steps - warmup - 1)

        def one(i):
            # as Engine.step runs a step of greedy requests: the output head picks the tokens, no logits are stored
            engine.runner.step([StepEntry(rid, [tokens[i][b]], [0]) for b, rid in enumerate(ids)], greedy=True)

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        launches0 = ops.launch_count() + engine.runner.graph_kernels
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(warmup, warmup + steps):
            one(i)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / steps)
        launches = ops.launch_count() + engine.runner.graph_kernels - launches0
        for rid in ids:
            engine.runner.free_request(rid)
    return times, launches


def time_prefill(engine, tokens, warmup=2, iters=3):
    import torch

    from ferrisinfer_b200.engine.runner import StepEntry

    vocab = engine.model.vocab_size
    gen = torch.Generator().manual_seed(2)
    times = []
    for i in range(warmup + iters):
        prompt = torch.randint(0, vocab, (tokens,), generator=gen).tolist()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.runner.step([StepEntry("prefill", prompt, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        engine.runner.free_request("prefill")
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def time_e2e(engine, batch, context, steps, warmup):
    """The same decode through Engine.step(): token ids come from and return to the host every step."""
    import torch

    from ferrisinfer_b200 import SamplingParams
    from ferrisinfer_b200.engine.scheduler import Phase

    start_ctx = context - steps - warmup - 2
    ids = fill_cache(engine, batch, start_ctx - 1)
    sched = engine.scheduler
    # hand the pre-filled requests to the scheduler as running, decoding sequences
    for b, rid in enumerate(ids):
        seq = sched.submit(rid, [(b * 7 + j) % engine.model.vocab_size for j in range(start_ctx)],
                           SamplingParams.greedy(max_new_tokens=steps + warmup + 1))
        sched.waiting.remove(seq)
        seq.phase, seq.num_computed, seq.slot = Phase.PREFILL, start_ctx - 1, engine.runner.cache.get(rid).slot
        sched.running.append(seq)
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    n = 0
    for _ in range(steps):
        n += sum(1 for o in engine.step() if o.token is not None)
    e1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms = max(e0.elapsed_time(e1), wall * 1e3) / steps
    for rid in ids:
        sched.cancel(rid)
    return ms, n, engine.runner.last_h2d_bytes, 8 * batch  # an int32 token and an fp32 probability per request


def time_mixed(cfg, requests=32, chunk=512, new_tokens=32, seed=3):
    """The mixed workload of the 1.5B sizes: ``requests`` prompts of 128 to 2,048 tokens, in portions of ``chunk``
    beside the decoded tokens of the requests that are further on, through Engine.generate.  Returns tokens
    (prompt + generated) a second and the wall time in ms."""
    import random

    import torch

    from ferrisinfer_b200 import SamplingParams, SchedulerConfig
    from ferrisinfer_b200.engine.engine import Engine

    rng = random.Random(seed)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.randint(128, 2048))] for _ in range(requests)]
    total = sum(len(p) for p in prompts) + requests * new_tokens
    sched = SchedulerConfig(max_batch_size=requests, max_prefill_chunk_tokens=chunk, max_prefill_batch_tokens=2 * chunk,
                            max_sequence_length=2048 + new_tokens + 8, max_generated_tokens=new_tokens)
    pages = sum(-(-(len(p) + new_tokens + 8) // 16) for p in prompts) + 8
    engine = Engine(config=cfg, seed=0, dtype="bfloat16", page_size=16, init_device="cuda", num_pages=pages, scheduler=sched)
    params = SamplingParams.greedy(max_new_tokens=new_tokens)
    engine.generate(prompts[:4], params)  # warm-up: kernels loaded, buffers sized
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = engine.generate(prompts, params)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    assert all(len(o.generated_tokens) == new_tokens for o in outs)
    del engine
    torch.cuda.empty_cache()
    return total / wall, wall * 1e3


def time_shared_prefix(cfg, requests=8, prefix=1024, tail=64, new_tokens=16):
    """Eight requests whose prompts share their first 1,024 tokens, through Engine.generate with prefix sharing:
    tokens (prompt + generated) a second, and how many prompt tokens were taken from shared pages."""
    import random

    import torch

    from ferrisinfer_b200 import SamplingParams, SchedulerConfig
    from ferrisinfer_b200.engine.engine import Engine

    rng = random.Random(11)
    stem = [rng.randrange(cfg["vocab_size"]) for _ in range(prefix)]
    prompts = [stem + [rng.randrange(cfg["vocab_size"]) for _ in range(tail + i)] for i in range(requests)]
    sched = SchedulerConfig(max_batch_size=requests, max_prefill_chunk_tokens=1024, max_prefill_batch_tokens=2048,
                            max_sequence_length=prefix + tail + requests + new_tokens + 8, max_generated_tokens=new_tokens)
    engine = Engine(config=cfg, seed=0, dtype="bfloat16", page_size=16, init_device="cuda",
                    num_pages=requests * 80 + 8, scheduler=sched, prefix_sharing=True)
    params = SamplingParams.greedy(max_new_tokens=new_tokens)
    engine.generate([p[:200] for p in prompts[:2]], params)
    engine.runner.cache.drop_idle()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    first = engine.submit(prompts[0], params)
    while not engine.scheduler.running or engine.scheduler.running[0].num_computed < len(prompts[0]):
        engine.step()
    rest = [engine.submit(p, params) for p in prompts[1:]]
    while engine.has_unfinished():
        engine.step()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    outs = [engine.output_of(i) for i in [first] + rest]
    reused = sum(o.reused_prompt_tokens for o in outs)
    total = sum(len(p) for p in prompts) + requests * new_tokens
    del engine
    torch.cuda.empty_cache()
    return total / wall, reused


def larger_sizes(steps, warmup) -> dict:
    """The workloads of the 1.5B and 7B sizes: random weights drawn on the device, same harness as the headline."""
    import torch

    out = {}
    # the median of three runs: the workload is a few hundred steps of changing shapes, some recorded on the way
    runs = sorted(time_mixed(dict(QWEN25_15B))[0] for _ in range(3))
    out["q15b_mixed32_tok_s"] = round(runs[1], 1)
    cfg = dict(QWEN25_7B)
    steps = max(8, steps // 4)
    for b in (1, 8, 64):
        engine = build_engine(cfg, b, CONTEXT, extra_tokens=PREFILL_TOKENS if b == 8 else 0)
        times, _ = time_decode(engine, b, CONTEXT, steps, warmup)
        ms = statistics.median(times)
        out[f"q7b_decode_b{b}"] = round(b / ms * 1e3, 1)
        out[f"q7b_decode_b{b}_frac"] = round(decode_bytes(cfg, b, CONTEXT) / (ms * 1e-3) / 1e9 / load_peaks()[0]["hbm_gbs"], 4)
        if b == 8:
            pms = time_prefill(engine, PREFILL_TOKENS)
            out["q7b_prefill_2048_tok_s"] = round(PREFILL_TOKENS / pms * 1e3, 1)
            out["q7b_prefill_frac"] = round(prefill_flops(cfg, PREFILL_TOKENS) / (pms * 1e-3) / (load_peaks()[0]["bf16_tflops"] * 1e12), 4)
        del engine
        torch.cuda.empty_cache()
    tok_s, reused = time_shared_prefix(cfg)
    out["q7b_shared_prefix8_tok_s"] = round(tok_s, 1)
    out["q7b_shared_prefix8_reused_tokens"] = reused
    return out


def kernel_numbers(engine, cfg, peaks) -> dict:
    """What the dominant kernels of the step reach alone.  Each is recorded once per layer into a CUDA graph, over
    that layer's own weights or cache (all layers together are far more than L2 holds), and the graph is timed."""
    import math

    import torch

    from ferrisinfer_b200.kernels import ops
    from ferrisinfer_b200.parts.base import PagedMeta, StepContext

    dev = engine.device
    n = model_numbers(cfg)
    H, I, L, d, nh, nkv = n["H"], cfg["intermediate_size"], n["L"], n["d"], n["nh"], cfg["num_key_value_heads"]
    blocks = engine.model.blocks
    out = {}

    def timed(body, reps=3):
        body()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            body()
        g.replay()
        torch.cuda.synchronize()
        best = None
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            best = e0.elapsed_time(e1) if best is None else min(best, e0.elapsed_time(e1))
        return best * 1e-3 / L  # seconds per launch

    # decode, 8 tokens: gate/up and down (weight bytes a second)
    T = 8
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    act = torch.empty(T, I, dtype=torch.bfloat16, device=dev)
    h = torch.zeros(T, H, dtype=torch.float32, device=dev)
    sec = timed(lambda: [ops.gemm_swiglu(x, b.feed_forward.gate_up, act) for b in blocks])
    out["decode_gate_up_gbs"] = round(2 * I * H * 2 / sec / 1e9, 1)
    sec = timed(lambda: [ops.gemm(act, b.feed_forward.down, None, h, accumulate=True) for b in blocks])
    out["decode_down_gbs"] = round(I * H * 2 / sec / 1e9, 1)
    # the output head, 8 rows
    logits = torch.empty(T, n["V"], dtype=torch.float32, device=dev)
    w_head = engine.model.output.weight
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ops.gemm(x, w_head, None, logits)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(4):
        ops.gemm(x, w_head, None, logits)
    e1.record()
    torch.cuda.synchronize()
    out["lm_head_gbs"] = round(n["V"] * H * 2 / (e0.elapsed_time(e1) * 1e-3 / 4) / 1e9, 1)
    # decode attention, 64 requests at context 4,096, over every layer's cache
    B = 64
    caches = [c for c in engine.runner.cache.layer_caches if c is not None and c.k is not None]
    pages_per = CONTEXT // 16
    have = caches[0].k.shape[0]
    if have >= B * pages_per:
        tables = torch.arange(B * pages_per, dtype=torch.int32, device=dev).view(B, pages_per)
        ws = engine.runner.workspace
        ctx = StepContext(num_tokens=B, num_seqs=B, token_ids=torch.zeros(B, dtype=torch.int32, device=dev),
                          positions=torch.full((B,), CONTEXT - 1, dtype=torch.int32, device=dev),
                          token_seq=torch.arange(B, dtype=torch.int32, device=dev),
                          seq_q_start=torch.arange(B + 1, dtype=torch.int32, device=dev),
                          seq_start_pos=torch.full((B,), CONTEXT - 1, dtype=torch.int32, device=dev),
                          seq_state_slot=torch.zeros(B, dtype=torch.int32, device=dev), seqs=[], paged={}, max_q_len=1,
                          max_kv_len=CONTEXT, act_dtype=torch.bfloat16, workspace=ws, device=dev)
        slots = (tables[:, -1] * 16 + 15).contiguous()
        meta = PagedMeta(block_tables=tables, slot_mapping=slots, page_size=16)
        qkv = torch.randn(B, (nh + 2 * nkv) * d, device=dev).to(torch.bfloat16)
        o = torch.empty(B, nh * d, dtype=torch.bfloat16, device=dev)
        inv_freq, rot = blocks[0].mixer.position.rotary_table(dev)
        sec = timed(lambda: [ops.attention_step(qkv, o, c.k, c.v, meta, ctx, nh, nkv, d, inv_freq, rot, 0, 1.0 / math.sqrt(d))
                             for c in caches])
        out["decode_attention_b64_gbs"] = round(B * CONTEXT * 2 * nkv * d * 2 / sec / 1e9, 1)
    # prefill, 2,048 tokens: the gate/up product and the attention
    Tp = PREFILL_TOKENS
    xp = torch.randn(Tp, H, device=dev).to(torch.bfloat16)
    actp = torch.empty(Tp, I, dtype=torch.bfloat16, device=dev)
    sec = timed(lambda: [ops.gemm_swiglu(xp, b.feed_forward.gate_up, actp) for b in blocks])
    out["prefill_gate_up_tflops"] = round(2.0 * Tp * 2 * I * H / sec / 1e12, 1)
    if have >= Tp // 16:
        tables = torch.arange(Tp // 16, dtype=torch.int32, device=dev).view(1, -1)
        qkvp = torch.randn(Tp, (nh + 2 * nkv) * d, device=dev).to(torch.bfloat16)
        op = torch.empty(Tp, nh * d, dtype=torch.bfloat16, device=dev)
        q_start = torch.tensor([0, Tp], dtype=torch.int32, device=dev)
        start_pos = torch.zeros(1, dtype=torch.int32, device=dev)
        sec = timed(lambda: [ops.prefill_attention(qkvp, op, c.k, c.v, tables, q_start, start_pos, 1, Tp, nh, nkv, d, 0,
                                                   1.0 / math.sqrt(d)) for c in caches])
        out["prefill_attention_tflops"] = round(2.0 * Tp * Tp * d * nh / sec / 1e12, 1)  # causal: half of 4 T^2 d nh
    # the temperature sampler, 8 rows of the whole vocabulary
    from ferrisinfer_b200 import SamplingParams

    params = [SamplingParams(temperature=0.7, top_k=20, top_p=0.9, seed=42 + i) for i in range(T)]
    engine.sampler.sample(logits, params, list(range(T)))
    torch.cuda.synchronize()
    e0.record()
    for _ in range(4):
        engine.sampler.sample(logits, params, list(range(T)))
    e1.record()
    torch.cuda.synchronize()
    out["sampler_top_k_top_p_b8_us"] = round(e0.elapsed_time(e1) * 1e3 / 4, 1)
    return out


def reference_arm(args) -> int:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference is a Rust workspace (no Python package, no GPU kernel); this image has no "
                       "cargo or rustc, so it can be neither installed with pip nor built",
    }))
    return 0


def timeline(args) -> int:
    """One decode step at the bench's sizes, seen from inside: when each kernel's CTAs entered, passed their
    programmatic-launch wait and ended, and the marks of its phases."""
    os.environ["FERRIS_NVCC_FLAGS"] = (os.environ.get("FERRIS_NVCC_FLAGS", "") + " -DFERRIS_TIMELINE").strip()
    import torch

    from ferrisinfer_b200.engine.runner import StepEntry
    from ferrisinfer_b200.kernels.timeline import StepTimeline, summarize

    cfg = dict(QWEN25_05B)
    if args.layers:
        cfg["num_hidden_layers"] = cfg["max_window_layers"] = args.layers
    if args.timeline == "prefill":
        engine = build_engine(cfg, 1, CONTEXT, extra_tokens=PREFILL_TOKENS)
        tl = StepTimeline(engine.device)
        gen = torch.Generator().manual_seed(2)
        for i in range(3):
            prompt = torch.randint(0, engine.model.vocab_size, (PREFILL_TOKENS,), generator=gen).tolist()
            if i == 2:
                tl.reset()
            engine.runner.step([StepEntry("p", prompt, [PREFILL_TOKENS - 1])])
            torch.cuda.synchronize()
            engine.runner.free_request("p")
        launches = tl.read()
        print(f"prefill of {PREFILL_TOKENS} tokens, {cfg['num_hidden_layers']} layers (times in us)")
        first = next(i for i, l in enumerate(launches) if "attention" in l.kernel)
        for l in launches[first + 6:first + 14]:
            print(f"{l.kernel:26s} ctas {l.ctas:5d}  entry {l.entry_us:8.2f}  start {l.start_us:8.2f}  end {l.end_us:8.2f}")
        print(summarize(launches))
        return 0
    engine = build_engine(cfg, args.batch, CONTEXT)
    tl = StepTimeline(engine.device)
    ids = fill_cache(engine, args.batch, CONTEXT - 16)
    def one(i):
        engine.runner.step([StepEntry(rid, [(7 * i + b) % 1000], [0]) for b, rid in enumerate(ids)], greedy=True)

    for i in range(4):
        one(i)
    tl.reset()
    one(4)
    launches = tl.read()
    print(f"decode step, batch {args.batch}, context {CONTEXT}, {cfg['num_hidden_layers']} layers "
          "(times in us; 'start' = first CTA past its launch wait)")
    per_layer = 5
    first = next(i for i, l in enumerate(launches) if "attention" in l.kernel) - 1
    for l in launches[first + per_layer:first + 2 * per_layer] + launches[-3:]:
        marks = " ".join("  -  " if m is None else f"{m:5.2f}" for m in l.marks_us[:6])
        print(f"{l.kernel:26s} ctas {l.ctas:5d}  entry {l.entry_us:8.2f}  start {l.start_us:8.2f}  end {l.end_us:8.2f}"
              f"  marks {marks}")
    print(summarize(launches))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--skip-points", action="store_true", help="no decode at batch 1 and 64")
    ap.add_argument("--skip-extra", action="store_true", help="no workloads of the 1.5B and 7B sizes, no per-kernel numbers")
    ap.add_argument("--regions", type=int, default=5, help="timed regions of --steps decode steps each (the median is reported)")
    ap.add_argument("--timeline", nargs="?", const="decode", choices=["decode", "prefill"], default=None,
                    help="instead of the measurement: the timeline of one decode step (or of one prefill of 2,048 "
                         "tokens) from hooks inside the kernels (a build of the kernel library of its own; prints a "
                         "table, no JSON line)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.timeline:
        return timeline(args)
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported (nothing here spans GPUs)")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch

    cfg = dict(QWEN25_05B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
        cfg["max_window_layers"] = args.layers
    peaks, peak_source = load_peaks()
    clocks = ClockSampler()

    engine = build_engine(cfg, args.batch, CONTEXT, extra_tokens=PREFILL_TOKENS)
    clocks.start()
    region_ms, launches = time_decode(engine, args.batch, CONTEXT, args.steps, args.warmup, regions=args.regions)
    ms = statistics.median(region_ms)
    prefill_ms = time_prefill(engine, PREFILL_TOKENS)
    e2e_ms, e2e_tokens, h2d, d2h = time_e2e(engine, args.batch, CONTEXT, args.steps, args.warmup)
    points, kernels = {}, {}
    if not args.skip_extra:
        del engine
        torch.cuda.empty_cache()
        # the per-kernel numbers want the cache of 64 requests at the bench's context
        engine = build_engine(cfg, 64, CONTEXT)
        kernels = kernel_numbers(engine, cfg, peaks)
    if not args.skip_points:
        for b in (1, 64):
            del engine
            torch.cuda.empty_cache()
            engine = build_engine(cfg, b, CONTEXT)
            times, _ = time_decode(engine, b, CONTEXT, max(8, args.steps // 2), args.warmup, regions=min(3, args.regions))
            pms = statistics.median(times)
            points[f"decode_b{b}"] = round(b / pms * 1e3, 1)
            points[f"decode_b{b}_frac"] = round(decode_bytes(cfg, b, CONTEXT) / (pms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
    del engine
    torch.cuda.empty_cache()
    if not args.skip_extra:
        points.update(larger_sizes(args.steps, args.warmup))
    clock_record = clocks.stop()

    value = args.batch / ms * 1e3
    bytes_step = decode_bytes(cfg, args.batch, CONTEXT)
    achieved = bytes_step / (ms * 1e-3) / 1e9
    flops = prefill_flops(cfg, PREFILL_TOKENS)
    n = model_numbers(cfg)
    line = {
        "metric": "decode tok/s at batch 8, context 4096 (Qwen2.5-0.5B sizes, random weights)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "ms_per_step_min": round(min(region_ms), 4), "ms_per_step_max": round(max(region_ms), 4),
        "regions": len(region_ms), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded uniform token ids, random-init weights)", "impl": "ours",
        "config": {
            "model": "Qwen2.5-0.5B sizes", "layers": cfg["num_hidden_layers"], "layers_of_model": full_layers,
            "hidden": n["H"], "heads": n["nh"], "kv_heads": cfg["num_key_value_heads"], "head_dim": n["d"],
            "intermediate": cfg["intermediate_size"], "vocab": n["V"], "tied": True, "global_batch": args.batch,
            "seq_len": CONTEXT, "kv_page": 16, "parallelism": "single GPU",
            "l2": "weights and cache exceed L2; no flush", "peaks": peak_source,
        },
        "e2e": {"value": round(e2e_tokens / args.steps / e2e_ms * 1e3, 1), "unit": "tok/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 4),
                "how": "Engine.step(): step metadata from pinned host memory, sampled tokens back to the host every "
                       "step; the next step is queued while the GPU runs (it reads its token ids on the device)"},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "kernels": kernels,
        "clocks": clock_record,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
