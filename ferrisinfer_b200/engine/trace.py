"""Trace replay: feed given token ids through a model step by step and write the logits.

It samples nothing and has no forward pass, cache or loader of its own: it loads the folder with
``weights.load_model`` and drives ``ModelRunner.step``, the step function that generation uses.
The reference has no such tool; its nearest relatives are the mode-equivalence unit tests
(crates/ferrisinfer-runtime/src/reference.rs:1431-1675).

Input, one JSON object a line on standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits at the wanted places
(order of the entries, then of ``want``) as little-endian float32 [wanted, vocab].  After every step
a line ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

PAGE_SIZE = 16
MAX_LIVE_REQUESTS = 16


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                   help="bfloat16: the kernels and precisions that serving uses; float32: everything in true 32-bit")
    p.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens that live requests hold at any time (each rounded up to a multiple of 64)")
    p.add_argument("--page-size", type=int, default=PAGE_SIZE, help=argparse.SUPPRESS)
    return p


def main(argv=None, stdin=None, stdout=None) -> int:
    args = build_parser().parse_args(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    from ..kernels import ops
    from ..weights.loader import load_model, parse_dtype
    from .runner import ModelRunner, StepEntry

    ops.require_device()
    device = torch.device("cuda", torch.cuda.current_device())
    dtype = parse_dtype(args.dtype)
    model, _cfg = load_model(args.model, dtype, device)
    page = args.page_size
    num_pages = max(1, -(-args.max_tokens // page))
    runner = ModelRunner(model, dtype, device, page_size=page, num_pages=num_pages,
                         max_requests=MAX_LIVE_REQUESTS)
    os.makedirs(args.out, exist_ok=True)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", [])]
        logits = runner.step(entries)
        if logits is not None:
            arr = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
            tmp = os.path.join(args.out, f".{step}.f32.tmp")
            arr.tofile(tmp)
            os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        else:
            torch.cuda.synchronize(device)
        for rid in rec.get("end", []):
            if runner.has_request(rid):
                runner.free_request(rid)
        stdout.write(f"done {step}\n")
        stdout.flush()
    return 0
