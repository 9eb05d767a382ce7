"""Sampling options of a request.

Names and meanings follow the reference's ``SamplerConfig``
(crates/ferrisinfer-runtime/src/sampler.rs:3-41): ``temperature`` (<= 0: greedy), ``top_k``
(1: greedy; the reference clamps it to [1, vocabulary]; here 0 also stands for the whole
vocabulary), ``top_p`` (<= 0: greedy; clamped to [0, 1]), ``repetition_penalty`` (stored and, as
in the reference, never applied), ``seed`` (0: the constant 0x9e3779b97f4a7c15).  The presets are
the reference's: ``greedy()`` and ``chat_default()`` = temperature 0.7, top_k 20, top_p 0.9, seed 42.
``max_new_tokens`` (default 128) and ``stop_token_id`` are the fields of the reference's
``GenerationRequest`` (crates/ferrisinfer-runtime/src/session.rs:48-65).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 1
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    seed: int = 0
    max_new_tokens: int = 128
    stop_token_id: Optional[int] = None
    # further ids that end the request (the reference's command line stops on the end-of-turn marker or on
    # eos_token_id: crates/ferrisinfer-cli/src/main.rs:904-919)
    stop_token_ids: tuple = ()

    @classmethod
    def greedy(cls, **kw) -> "SamplingParams":
        return cls(temperature=0.0, top_k=1, top_p=1.0, seed=0, **kw)

    @classmethod
    def chat_default(cls, **kw) -> "SamplingParams":
        return cls(temperature=0.7, top_k=20, top_p=0.9, seed=42, **kw)

    def stops(self, token: int) -> bool:
        """Whether ``token`` ends the request."""
        return (self.stop_token_id is not None and token == self.stop_token_id) or token in self.stop_token_ids

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1 or self.top_p <= 0.0

    def __post_init__(self):
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be >= 0")
        if self.seed < 0 or self.seed >= 1 << 64:
            raise ValueError("seed must fit in 64 bits")
        object.__setattr__(self, "stop_token_ids", tuple(int(t) for t in self.stop_token_ids))
