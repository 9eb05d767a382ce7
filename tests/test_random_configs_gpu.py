"""Configurations drawn at random, replayed in every way of cutting against the plain implementation: what the
four hand-made tiny configurations do not reach (head sizes 80, 96, 128; seven heads to a group; widths that are
only multiples of 2 or 4; a window in some layers only; half-rotated heads; pages of 4 to 32)."""

import random

import pytest
import torch

import helpers
from helpers import TOL

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [3, 16, 25, 27, 30, 50, 53, 89])
def test_random_configuration_in_every_way_of_cutting(seed, device, tmp_path):
    from ferrisinfer_b200.engine.runner import ModelRunner
    from ferrisinfer_b200.weights import load_model

    rng = random.Random(seed)
    cfg = helpers.random_config(rng)
    page = rng.choice([4, 8, 16, 16, 32])
    lengths = [rng.randint(1, 40), rng.randint(20, 140), rng.randint(2, 70), rng.randint(60, 300), rng.randint(1, 20)]
    requests = {f"r{i}": helpers.random_ids(cfg["vocab_size"], n, seed * 10 + i) for i, n in enumerate(lengths)}
    folder = helpers.make_folder(tmp_path, cfg, seed=seed, optional=rng.random() < 0.7, score_std=rng.choice((None, 0.5, 1.0)))
    config, weights = helpers.read_folder(folder)
    want = helpers.oracle_logits(config, weights, requests)
    traces = {"whole": helpers.trace_whole(requests), "tail": helpers.trace_tail_decoded(requests),
              "portions": helpers.trace_portions(requests), "mixed": helpers.trace_mixed(requests, seed)}
    for dtype in (torch.float32, torch.bfloat16):
        model, _ = load_model(folder, dtype, device)
        for kind, steps in traces.items():
            pages = helpers.tokens_held(steps, round_to=page) // page
            runner = ModelRunner(model, dtype, device, page_size=page, num_pages=pages, max_requests=8)
            got = helpers.replay(runner, steps)
            runner.cache.check_invariants()
            assert all(g.pool.num_used == 0 for g in runner.cache.groups)
            bad = helpers.first_mismatch(got, want, **TOL[dtype])
            assert bad is None, f"{cfg} page {page} {dtype} {kind}: {bad}"
