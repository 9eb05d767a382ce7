"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits read back from <step>.f32 files."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
from helpers import TINY, TOL

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_trace(folder, dtype, steps, out_dir, max_tokens, vocab):
    proc = subprocess.Popen(
        [os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out_dir),
         "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    got, pos = {}, {}
    for s in steps:
        proc.stdin.write(json.dumps(s) + "\n")
        proc.stdin.flush()
        line = proc.stdout.readline().strip()
        assert line == f"done {s['step']}", line
        wanted = sum(len(e["want"]) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if wanted:
            rows = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(wanted, vocab).copy())
        else:
            assert not os.path.exists(path)
        row = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = rows[row]
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            pos.pop(rid, None)
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0
    return got


LENGTHS = {"A": (70, 33, 101, 48, 64, 90), "B": (70, 33, 101, 48, 64, 90),
           # head size 64: in bfloat16 the tensor-core kernels, and prompts long enough for the long-step ones
           "D": (260, 33, 150, 140, 64)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_replay_in_every_way_of_cutting(name, dtype, device, tmp_path):
    folder = helpers.make_folder(tmp_path, TINY[name], seed=41, score_std=1.8)
    config, weights = helpers.read_folder(folder)
    vocab = config["vocab_size"]
    lengths = LENGTHS[name]
    requests = {f"q{i}": helpers.random_ids(vocab, n, 3 * i + n) for i, n in enumerate(lengths)}
    want = helpers.oracle_logits(config, weights, requests)
    tol = TOL[torch.float32 if dtype == "float32" else torch.bfloat16]
    traces = {
        "whole": helpers.trace_whole(requests),
        "tail": helpers.trace_tail_decoded(requests, tail=32),
        "portions": helpers.trace_portions(requests),
        "mixed": helpers.trace_mixed(requests, seed=2),
    }
    # some steps ask for only some places, or none
    for s in traces["portions"][::3]:
        for e in s["entries"]:
            e["want"] = e["want"][-1:]
    for s in traces["mixed"][::4]:
        for e in s["entries"][:1]:
            e["want"] = []
    for kind, steps in traces.items():
        out_dir = tmp_path / f"{kind}-{dtype}"
        got = run_trace(folder, dtype, steps, out_dir, helpers.tokens_held(steps), vocab)
        expected = {k: v for k, v in want.items() if k in got}
        assert len(got) > 50
        bad = helpers.first_mismatch(got, expected, **tol)
        assert bad is None, f"{kind}: {bad}"
