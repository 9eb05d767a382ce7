"""Turns the logits a step returns into one token per request, on the GPU.

Each request's xorshift64* state lives in its state slot (a [slots] int64 tensor that the cache
manager zeroes at admission); ``seed_slot`` writes a request's seed there.  Sampling reads the
per-row options from small device tensors and launches one kernel for the whole batch.
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from ..kernels import ops
from ..parts.base import FixedState
from .params import SamplingParams

RNG_STATE = "sampler_rng"
RNG_NEED = FixedState((), torch.int64)


def _as_signed64(x: int) -> int:
    x &= (1 << 64) - 1
    return x - (1 << 64) if x >= 1 << 63 else x


class Sampler:
    def __init__(self, rng_states: torch.Tensor):
        self.rng_states = rng_states  # int64 [slots]
        self.device = rng_states.device
        self._staging = []  # ring of (pinned [4, n] fp32, event of the last copy out of it)
        self._next = 0

    def seed_slot(self, slot: int, seed: int) -> None:
        """seed 0 keeps the slot's zero, which the kernel reads as the reference's default constant."""
        self.rng_states[slot] = _as_signed64(seed)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], slots: Sequence[int]):
        """(tokens int32 [n], probabilities fp32 [n]) on the device for fp32 ``logits`` [n, V]."""
        n = logits.shape[0]
        tokens = torch.empty(n, dtype=torch.int32, device=self.device)
        probs = torch.empty(n, dtype=torch.float32, device=self.device)
        if all(p.is_greedy for p in params):
            ops.sample(logits, tokens, probs)
            return tokens, probs
        # the rows' options go up in one asynchronous copy from pinned memory
        if not self._staging:
            self._staging = [[None, None] for _ in range(4)]
        slot = self._staging[self._next]
        self._next = (self._next + 1) % len(self._staging)
        if slot[1] is not None:
            slot[1].synchronize()
        if slot[0] is None or slot[0].shape[1] < n:
            slot[0] = torch.empty(4, max(n, 64), dtype=torch.float32).pin_memory()
            slot[1] = torch.cuda.Event()
        host = slot[0].numpy()[:, :n]
        ints = host.view(np.int32)
        for i, (p, s) in enumerate(zip(params, slots)):
            host[0, i] = p.temperature if not p.is_greedy else 0.0
            ints[1, i] = p.top_k
            host[2, i] = min(max(p.top_p, 0.0), 1.0)
            ints[3, i] = s
        dev = torch.empty(4, n, dtype=torch.float32, device=self.device)
        dev.copy_(slot[0][:, :n], non_blocking=True)
        slot[1].record(torch.cuda.current_stream(self.device))
        ops.sample(logits, tokens, probs, temperature=dev[0], top_k=dev[1].view(torch.int32), top_p=dev[2],
                   slots=dev[3].view(torch.int32), rng_states=self.rng_states)
        return tokens, probs
