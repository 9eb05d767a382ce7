"""The Python entry point: load or create a model, queue requests, step, generate.

The reference's entry points are ``InferenceEngine`` (a factory of sessions and schedulers:
crates/ferrisinfer-runtime/src/engine.rs:17-69), ``Session::generate_reference_from_tokens(ids,
max_new_tokens, stop_token_id)`` for one request (crates/ferrisinfer-runtime/src/session.rs:264-332)
and ``ReferenceScheduler::submit`` / ``execute_next_tick`` for many
(crates/ferrisinfer-runtime/src/scheduler.rs:208-251, 393-415).  ``Engine`` keeps those three ways:
``generate`` (prompts in, outputs out), ``submit`` + ``step`` (continuous batching), with the same
request fields (prompt token ids, max_new_tokens = 128, stop_token_id) and the same output fields
(prompt_token_ids, generated tokens with their probabilities, finish_reason).  Text in and out is the
tokenizer's business and not part of the engine: requests are token ids.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Sequence as Seq

import torch

from ..config.registry import resolve_config
from ..kernels import ops
from ..parts.model import build_model
from ..sampling import RNG_NEED, RNG_STATE, Sampler, SamplingParams
from ..weights.loader import bind_tensors, load_model, parse_dtype
from ..weights.random_init import random_tensors
from .runner import ModelRunner, StepEntry
from .scheduler import FinishReason, Scheduler, SchedulerConfig, Sequence


@dataclass
class TokenSample:
    """crates/ferrisinfer-runtime/src/sampler.rs:44-48."""

    token_id: int
    probability: float


@dataclass
class GenerationOutput:
    """crates/ferrisinfer-runtime/src/session.rs:75-90, without the text."""

    request_id: Any
    prompt_token_ids: list
    generated_tokens: list  # list[TokenSample]
    finish_reason: FinishReason
    preemptions: int = 0
    reused_prompt_tokens: int = 0

    def generated_token_ids(self) -> list:
        return [t.token_id for t in self.generated_tokens]


@dataclass
class StepOutput:
    request_id: Any
    token: Optional[TokenSample]
    finished: bool
    finish_reason: Optional[FinishReason]


class Engine:
    def __init__(self, model=None, *, config=None, seed: int = 0, dtype="bfloat16", device=None,
                 page_size: int = 16, num_pages: Optional[int] = None, gpu_memory_fraction: float = 0.5,
                 scheduler: Optional[SchedulerConfig] = None, init_device="cpu", prefix_sharing: bool = True):
        """``model``: a model folder (config.json + safetensors).  Or ``config`` (a folder, dict or
        typed configuration) with ``seed``: random weights, no folder needed.
        ``num_pages``: pages per page group; by default what ``gpu_memory_fraction`` of the free device
        memory holds.  ``init_device``: where random weights are drawn ("cpu": the values a model folder
        written with the same seed holds; a CUDA device: other values, much faster for large models).
        ``prefix_sharing``: requests whose prompts begin with the same full pages as a live request's share
        those pages instead of recomputing them (where every layer keeps all keys)."""
        ops.require_device()
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.dtype = parse_dtype(dtype)
        if model is not None:
            self.model, self.config = load_model(model, self.dtype, self.device)
        elif config is not None:
            arch, self.config = resolve_config(config)
            self.model = build_model(arch.plan(self.config))
            bind_tensors(self.model, random_tensors(self.config, seed, "bfloat16", device=init_device), self.dtype, self.device)
        else:
            raise ValueError("give a model folder, or a configuration and a seed")
        self.scheduler_config = scheduler or SchedulerConfig()
        sc = self.scheduler_config
        needs = self.model.cache_needs()
        if num_pages is None:
            num_pages = self._pages_that_fit(needs, page_size, gpu_memory_fraction, sc)
        self.runner = ModelRunner(self.model, self.dtype, self.device, page_size=page_size, num_pages=num_pages,
                                  max_requests=sc.max_batch_size, max_model_len=sc.max_sequence_length,
                                  extra_states={RNG_STATE: RNG_NEED}, prefix_sharing=prefix_sharing,
                                  min_prefix_share_tokens=sc.min_prefix_share_tokens)
        self.sampler = Sampler(self.runner.cache.state_tensors[RNG_STATE])
        self.scheduler = Scheduler(sc, self.runner.cache, on_admit=self._on_admit, on_preempt=self._on_preempt)
        self._next_id = 0

    # ------------------------------------------------------------------ set-up
    def _pages_that_fit(self, needs, page_size, fraction, sc) -> int:
        from ..parts.base import PagedKV

        item = 2 if self.dtype == torch.bfloat16 else 4
        per_page = sum(2 * n.num_kv_heads * n.head_dim * page_size * item for n in needs if isinstance(n, PagedKV))
        if per_page == 0:
            return 1
        free, _total = torch.cuda.mem_get_info(self.device)
        pages = int(free * fraction) // per_page
        most = sc.max_batch_size * (-(-sc.max_sequence_length // page_size))
        return max(1, min(pages, most))

    def _on_admit(self, seq: Sequence) -> None:
        state = seq.saved_rng_state if seq.saved_rng_state is not None else seq.params.seed
        self.sampler.seed_slot(seq.slot, state)

    def _on_preempt(self, seq: Sequence) -> None:
        seq.saved_rng_state = int(self.sampler.rng_states[seq.slot].item()) & ((1 << 64) - 1)

    # ---------------------------------------------------------------- requests
    def submit(self, prompt_token_ids: Seq[int], params: Optional[SamplingParams] = None, request_id=None):
        """Queue one request; returns its id (crates/ferrisinfer-runtime/src/scheduler.rs:208-251)."""
        if request_id is None:
            request_id = self._next_id
            self._next_id += 1
        vocab = self.model.vocab_size
        if any((not isinstance(t, int)) or t < 0 or t >= vocab for t in prompt_token_ids):
            raise ValueError(f"prompt token ids must be integers in [0, {vocab})")
        self.scheduler.submit(request_id, prompt_token_ids, params or SamplingParams())
        return request_id

    def abort(self, request_id) -> bool:
        return self.scheduler.cancel(request_id) is not None

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    # -------------------------------------------------------------------- step
    def step(self) -> list:
        """One scheduler step: run it, sample, record.  Returns a StepOutput for every request that
        got a new token or finished."""
        plan = self.scheduler.schedule()
        if not plan.entries:
            return []
        entries, sampling = [], []
        for e in plan.entries:
            seq = e.seq
            tokens = seq.token_slice(e.start, e.count)
            wants = e.samples and len(seq.generated) < seq.max_new_tokens \
                and seq.num_tokens < self.scheduler_config.max_sequence_length
            entries.append(StepEntry(seq.request_id, tokens, [e.count - 1] if wants else []))
            if wants:
                sampling.append(seq)
        logits = self.runner.step(entries)
        sampled = {}
        if sampling:
            tokens, probs = self.sampler.sample(logits, [s.params for s in sampling], [s.slot for s in sampling])
            host = torch.stack([tokens.to(torch.float64), probs.to(torch.float64)]).cpu()
            for i, s in enumerate(sampling):
                sampled[s.request_id] = (int(host[0, i].item()), float(host[1, i].item()))
        self.scheduler.update(plan, sampled)
        out = []
        for e in plan.entries:
            seq = e.seq
            got = sampled.get(seq.request_id)
            finished = seq.finish_reason is not None
            if got is not None or finished:
                out.append(StepOutput(seq.request_id, TokenSample(*got) if got else None, finished, seq.finish_reason))
        return out

    # ---------------------------------------------------------------- generate
    def generate(self, prompts, params=None) -> list:
        """Run ``prompts`` (a list of token-id lists, or one list) to the end; one GenerationOutput each,
        in the order given.  ``params``: one SamplingParams for all, or one per prompt."""
        single = bool(prompts) and isinstance(prompts[0], int)
        if single:
            prompts = [prompts]
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams for all prompts, or one per prompt")
        ids = [self.submit(list(p), sp) for p, sp in zip(prompts, params)]
        while self.scheduler.has_unfinished():
            if not self.step() and not self.scheduler.running and self.scheduler.waiting:
                raise RuntimeError("the scheduler cannot make progress")
        outs = [self.output_of(i) for i in ids]
        return outs[0] if single else outs

    def output_of(self, request_id) -> GenerationOutput:
        seq = self.scheduler.finished.pop(request_id)
        return GenerationOutput(
            request_id, list(seq.prompt),
            [TokenSample(t, p) for t, p in zip(seq.generated, seq.probabilities)],
            seq.finish_reason, seq.preemptions, seq.reused_prompt_tokens)


def generate(model, prompts, params: Optional[SamplingParams] = None, **engine_options) -> list:
    """One call from a model folder and prompts (lists of token ids) to outputs."""
    return Engine(model, **engine_options).generate(prompts, params)
