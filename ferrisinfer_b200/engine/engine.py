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
from .scheduler import FinishReason, Phase, ScheduledEntry, Scheduler, SchedulerConfig, Sequence, StepPlan


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
class _InFlight:
    """A step that has been queued on the GPU: its plan, the requests it samples for, the sampled tokens
    on the device and the pinned host buffers (tokens, probabilities, event) they are copied to."""

    plan: StepPlan
    sampling: list
    tokens: Optional[torch.Tensor] = None
    host: Optional[list] = None


@dataclass
class StepOutput:
    request_id: Any
    token: Optional[TokenSample]
    finished: bool
    finish_reason: Optional[FinishReason]


class Engine:
    def __init__(self, model=None, *, config=None, seed: int = 0, dtype="bfloat16", device=None,
                 page_size: int = 16, num_pages: Optional[int] = None, gpu_memory_fraction: float = 0.5,
                 scheduler: Optional[SchedulerConfig] = None, init_device="cpu", prefix_sharing: bool = True,
                 run_ahead: bool = True, keep_finished_prefixes: bool = True):
        """``model``: a model folder (config.json + safetensors).  Or ``config`` (a folder, dict or
        typed configuration) with ``seed``: random weights, no folder needed.
        ``num_pages``: pages per page group; by default what ``gpu_memory_fraction`` of the free device
        memory holds.  ``init_device``: where random weights are drawn ("cpu": the values a model folder
        written with the same seed holds; a CUDA device: other values, much faster for large models).
        ``prefix_sharing``: requests whose prompts begin with the same full pages as a live request's share
        those pages instead of recomputing them (where every layer keeps all keys).  ``keep_finished_prefixes``:
        such pages stay in the cache after the last request that held them has ended (or was preempted), for
        later requests with the same beginning, until a request needs their room.
        ``run_ahead``: queue the next decode step while the GPU still runs the current one (see ``step``)."""
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
                                  min_prefix_share_tokens=sc.min_prefix_share_tokens,
                                  keep_finished=keep_finished_prefixes)
        self.sampler = Sampler(self.runner.cache.state_tensors[RNG_STATE])
        self.scheduler = Scheduler(sc, self.runner.cache, on_admit=self._on_admit, on_preempt=self._on_preempt)
        self._next_id = 0
        self.run_ahead = bool(run_ahead)
        self.steps_run_ahead = 0
        self._in_flight: Optional[_InFlight] = None
        self._results = [[None, None, None] for _ in range(3)]  # pinned (tokens, probabilities, event), in turn
        self._results_next = 0

    # ------------------------------------------------------------------ set-up
    def _pages_that_fit(self, needs, page_size, fraction, sc) -> int:
        """Pages per group that ``fraction`` of the free device memory holds, after what the per-request state of
        fixed size (mixers' and the sampler's, one row per request slot and one more) takes from it."""
        from ..parts.base import FixedState, PagedKV

        item = 2 if self.dtype == torch.bfloat16 else 4
        per_page = sum(2 * n.num_kv_heads * n.head_dim * page_size * item for n in needs if isinstance(n, PagedKV))
        if per_page == 0:
            return 1
        states = [n for n in needs if isinstance(n, FixedState)] + [RNG_NEED]
        state_bytes = 0
        for n in states:
            count = 1
            for s in n.shape:
                count *= int(s)
            state_bytes += (sc.max_batch_size + 1) * count * torch.empty((), dtype=n.dtype).element_size()
        free, _total = torch.cuda.mem_get_info(self.device)
        pages = max(0, int(free * fraction) - state_bytes) // per_page
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

    add_request = submit

    def abort(self, request_id) -> bool:
        return self.scheduler.cancel(request_id) is not None

    def step_raw(self, entries) -> Optional[torch.Tensor]:
        """The step function itself, below the scheduler: ``entries`` is a list of ``StepEntry`` (request id, its next
        tokens, the places among them whose logits are wanted); returns fp32 logits [wanted, vocab] or None.  This is
        what trace replay drives; requests stepped this way are the caller's to end (``runner.free_request``)."""
        return self.runner.step(entries)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    # -------------------------------------------------------------------- step
    def step(self) -> list:
        """One scheduler step: run it, sample, record.  Returns a StepOutput for every request that
        got a new token or finished.

        While the GPU runs a step of decoding requests, the host prepares and queues the step after it
        (``run_ahead``): that step needs the requests' lengths, which are known, and their new tokens,
        which it reads on the device from where the sampler of the running step puts them.  The host
        then waits for the running step's tokens and records them.  A request that ends on a stop token
        (or is cancelled) has one step too many in flight; its share of that step is dropped."""
        if self._in_flight is None:
            self._in_flight = self._launch(self.scheduler.schedule())
            if self._in_flight is None:
                return []
        current = self._in_flight
        self._in_flight = self._launch_ahead(current) if self.run_ahead else None
        out, void = self._complete(current)
        if void and self._in_flight is None and self.scheduler.has_unfinished():
            return self.step()  # every request of that step had ended before it: run a fresh one
        return out

    def _launch(self, plan, device_tokens=None) -> Optional["_InFlight"]:
        if not plan.entries:
            return None
        entries, sampling = [], []
        ahead = device_tokens is not None
        for e in plan.entries:
            seq = e.seq
            tokens = [0] if ahead else seq.token_slice(e.start, e.count)
            wants = ahead or (e.samples and len(seq.generated) < seq.max_new_tokens
                              and seq.num_tokens < self.scheduler_config.max_sequence_length)
            entries.append(StepEntry(seq.request_id, tokens, [e.count - 1] if wants else []))
            if wants:
                sampling.append(seq)
        # rows that all take their most likely token are sampled by the step itself (its output head stores no logits)
        greedy = bool(sampling) and all(s.params.is_greedy for s in sampling)
        logits = self.runner.step(entries, device_tokens=device_tokens, greedy=greedy)
        flight = _InFlight(plan, sampling)
        if sampling:
            n = len(sampling)
            if greedy:
                flight.tokens, probs = logits
            else:
                flight.tokens, probs = self.sampler.sample(logits, [s.params for s in sampling], [s.slot for s in sampling])
            buf = self._results[self._results_next]
            self._results_next = (self._results_next + 1) % len(self._results)
            if buf[0] is None or buf[0].numel() < n:
                size = max(n, self.scheduler_config.max_batch_size)
                buf[0] = torch.empty(size, dtype=torch.int32).pin_memory()
                buf[1] = torch.empty(size, dtype=torch.float32).pin_memory()
                buf[2] = torch.cuda.Event()
            buf[0][:n].copy_(flight.tokens, non_blocking=True)
            buf[1][:n].copy_(probs, non_blocking=True)
            buf[2].record(torch.cuda.current_stream(self.device))
            flight.host = buf
        return flight

    def _launch_ahead(self, current: "_InFlight") -> Optional["_InFlight"]:
        """Queue the step after ``current`` if it is sure to be the same requests decoding one token more."""
        sched, cfg = self.scheduler, self.scheduler_config
        plan = current.plan
        if sched.waiting or plan.preempted or len(plan.entries) != len(sched.running) \
                or len(current.sampling) != len(plan.entries):
            return None
        cache = self.runner.cache
        short = {g.gid: 0 for g in cache.groups}
        for e in plan.entries:
            seq = e.seq
            if not e.samples or seq.phase is Phase.FINISHED or seq.phase is Phase.WAITING:
                return None
            # after the running step the request has one token more; it must be sure to go on after that
            if len(seq.generated) + 2 > seq.max_new_tokens or seq.num_tokens + 2 > cfg.max_sequence_length:
                return None
            for gid, n in cache.pages_needed(seq.request_id, e.start + e.count + 1).items():
                short[gid] += n
        free = cache.free_pages()
        if any(short[g] > free[g] for g in short):
            return None  # pages are short: the scheduler decides who waits, with the tokens in hand
        nxt = StepPlan([ScheduledEntry(e.seq, e.start + e.count, 1, True) for e in plan.entries])
        self.steps_run_ahead += 1
        return self._launch(nxt, device_tokens=current.tokens)

    def _complete(self, flight: "_InFlight") -> list:
        """Wait for the step's tokens, hand them to the scheduler, report."""
        sampled = {}
        if flight.sampling:
            tok, prob, event = flight.host
            event.synchronize()
            n = len(flight.sampling)
            toks, probs = tok[:n].tolist(), prob[:n].tolist()
            for i, s in enumerate(flight.sampling):
                sampled[s.request_id] = (toks[i], probs[i])
        live = [e for e in flight.plan.entries if e.seq.phase is not Phase.FINISHED and e.seq.phase is not Phase.WAITING]
        self.scheduler.update(flight.plan, sampled)
        out = []
        for e in live:
            seq = e.seq
            got = sampled.get(seq.request_id)
            finished = seq.finish_reason is not None
            if got is not None or finished:
                out.append(StepOutput(seq.request_id, TokenSample(*got) if got else None, finished, seq.finish_reason))
        return out, not live

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
