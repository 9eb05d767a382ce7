"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes, finishes, frees.

The reference's scheduler (crates/ferrisinfer-runtime/src/scheduler.rs:109-648) plans a tick that is
either all prefill or all decode, gives prefill priority with a fairness counter
(:253-328), cuts a prompt into chunks of ``max_prefill_chunk_tokens`` under a per-tick budget
``max_prefill_batch_tokens`` with at most ``max_batch_size`` sequences (:271-312), and releases a
sequence's resources when it finishes (:452-456, 521-525).  Its sequences own private caches, so
pages never run out across requests.

Here a step is mixed, which removes the prefill-or-decode choice: every step carries one token for
each decoding request, and what is left of the token budget is filled with portions of prompts in
arrival order.  The option names and defaults are the reference's; the finish reasons are the
reference's (crates/ferrisinfer-runtime/src/sequence.rs:35-41) with the same order of checks
(crates/ferrisinfer-runtime/src/scheduler.rs:433-443, 493-507).

**When pages run out** (all requests share one pool):
1. a request that can never fit (its prompt plus its token budget exceeds ``max_sequence_length`` or
   the pool) is refused at ``submit``;
2. nothing new is admitted while the pool cannot hold the first portion;
3. a portion of a prompt is shortened to what the free pages hold, down to nothing;
4. if a decoding request cannot get the page its next token needs, or no running request can go on
   at all, the request admitted LAST is preempted: its pages and slot go back, its tokens (prompt and generated) are kept, and it returns
   to the front of the waiting queue, to be recomputed as one prompt when pages are free again.
   Its sampler state is carried over, so what it generates does not change.

The scheduler is host-side bookkeeping only; it sees the cache manager through ``pages_needed``,
``free_pages``, ``admit``, ``release`` and never touches a tensor.
"""

from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Optional

from ..errors import SchedulerError
from ..sampling.params import SamplingParams


class FinishReason(enum.Enum):
    STOP_TOKEN = "StopToken"
    MAX_NEW_TOKENS = "MaxNewTokens"
    SESSION_LIMIT = "SessionLimit"
    SEQUENCE_LENGTH = "SequenceLength"
    CANCELLED = "Cancelled"


class Phase(enum.Enum):
    WAITING = "Waiting"
    PREFILL = "Prefill"
    DECODE = "Decode"
    FINISHED = "Finished"


@dataclass
class SchedulerConfig:
    """Names and defaults of the reference's SchedulerConfig
    (crates/ferrisinfer-runtime/src/scheduler.rs:16-35) and SessionConfig
    (crates/ferrisinfer-runtime/src/session.rs:29-46)."""

    max_batch_size: int = 16  # most requests in one step
    max_prefill_chunk_tokens: int = 256  # largest portion of one prompt in one step
    max_prefill_batch_tokens: int = 1024  # token budget of one step (decoded tokens count too)
    max_sequence_length: int = 4096  # prompt + generated tokens of one request
    max_generated_tokens: int = 512  # cap on any request's max_new_tokens
    min_prefix_share_tokens: int = 64  # shorter common prefixes are not shared


@dataclass
class Sequence:
    request_id: Any
    prompt: list
    params: SamplingParams
    requested_max_new_tokens: int
    max_new_tokens: int
    arrival: int
    generated: list = field(default_factory=list)
    probabilities: list = field(default_factory=list)
    num_computed: int = 0  # tokens whose keys and values are in the cache
    phase: Phase = Phase.WAITING
    finish_reason: Optional[FinishReason] = None
    slot: Optional[int] = None
    saved_rng_state: Optional[int] = None
    preemptions: int = 0
    reused_prompt_tokens: int = 0  # tokens taken from other requests' pages instead of being computed

    @property
    def tokens(self) -> list:
        return self.prompt + self.generated

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.generated)

    def token_slice(self, start: int, count: int) -> list:
        """tokens[start : start + count] without building the whole list."""
        n = len(self.prompt)
        if start >= n:
            return self.generated[start - n:start - n + count]
        if start + count <= n:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.generated[:start + count - n]

    @property
    def pending(self) -> int:
        """Tokens that are known but not in the cache yet."""
        return self.num_tokens - self.num_computed


@dataclass
class ScheduledEntry:
    seq: Sequence
    start: int  # position of the first token of this step's share
    count: int
    samples: bool  # the share ends at the request's last known token: a new token is sampled


@dataclass
class StepPlan:
    entries: list = field(default_factory=list)
    preempted: list = field(default_factory=list)
    admitted: list = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache, on_admit=None, on_preempt=None):
        """``on_admit(seq)`` runs after a request got its slot; ``on_preempt(seq)`` before a preempted
        request's slot is given back (the engine saves and restores the sampler state there)."""
        self.on_admit, self.on_preempt = on_admit, on_preempt
        if config.max_batch_size <= 0 or config.max_prefill_chunk_tokens <= 0 or config.max_prefill_batch_tokens <= 0:
            raise SchedulerError("scheduler limits must be positive")
        self.config = config
        self.cache = cache
        self.waiting: deque = deque()
        self.running: list = []  # in order of admission
        self.finished: dict = {}
        self._arrivals = 0
        self.stats = {"steps": 0, "preemptions": 0, "tokens": 0, "sampled": 0}

    # ------------------------------------------------------------------- submit
    def submit(self, request_id, prompt, params: SamplingParams) -> Sequence:
        """Queue a request (crates/ferrisinfer-runtime/src/scheduler.rs:208-251: an empty prompt and a
        prompt longer than the sequence limit are refused; the token budget is capped by the session's)."""
        prompt = list(prompt)
        cfg = self.config
        if not prompt:
            raise SchedulerError("a request needs at least one prompt token")
        if len(prompt) > cfg.max_sequence_length:
            raise SchedulerError(f"the prompt has {len(prompt)} tokens; max_sequence_length is {cfg.max_sequence_length}")
        if any(s.request_id == request_id for s in list(self.waiting) + self.running):
            raise SchedulerError(f"request {request_id!r} is already queued")
        budget = min(params.max_new_tokens, cfg.max_generated_tokens)
        most = min(len(prompt) + budget, cfg.max_sequence_length)
        ps = self.cache.page_size
        for g in self.cache.groups:
            window = g.window
            span = most if window is None else min(most, window + 2 * ps)
            if -(-span // ps) > g.pool.num_pages:
                raise SchedulerError(
                    f"request {request_id!r} can reach {most} tokens, which the cache ({g.pool.num_pages} pages "
                    f"of {ps} in group {g.gid}) can never hold")
        seq = Sequence(request_id, prompt, params, params.max_new_tokens, budget, self._arrivals)
        self._arrivals += 1
        self.waiting.append(seq)
        return seq

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ----------------------------------------------------------------- schedule
    def schedule(self) -> StepPlan:
        """Plan one step.  If no running request can go on (every one is part-way through its prompt
        and the pool is exhausted), requests are preempted from the back until one can."""
        plan = StepPlan()
        while True:
            self._plan(plan)
            if plan.entries or not self.running:
                return plan
            if len(self.running) == 1:
                raise SchedulerError(
                    f"request {self.running[0].request_id!r} cannot go on although it has the cache to itself")
            self._preempt(self.running[-1], plan)

    def _plan(self, plan: StepPlan) -> None:
        cfg, cache = self.config, self.cache
        budget = cfg.max_prefill_batch_tokens
        reserve = {g.gid: 0 for g in cache.groups}

        def fits(seq, new_total):
            need = cache.pages_needed(seq.request_id, new_total)
            free = cache.free_pages()
            return all(need[g] + reserve[g] <= free[g] for g in need), need

        def take(need):
            for g, n in need.items():
                reserve[g] += n

        # 1. one token for each decoding request, preempting from the back if pages are short
        decoding = [s for s in self.running if s.phase is Phase.DECODE]
        i = 0
        while i < len(decoding):
            seq = decoding[i]
            if budget <= 0 or len(plan.entries) >= cfg.max_batch_size:
                break
            ok, need = fits(seq, seq.num_computed + 1)
            if ok:
                take(need)
                plan.entries.append(ScheduledEntry(seq, seq.num_computed, 1, True))
                budget -= 1
                i += 1
                continue
            victim = self.running[-1]
            self._preempt(victim, plan)
            # the victim's pages are free now; what was reserved for it (if it was planned already) is void
            kept = [e for e in plan.entries if e.seq is not victim]
            if len(kept) != len(plan.entries):
                plan.entries = kept
                budget += 1
                reserve = {g.gid: 0 for g in cache.groups}
                for e in plan.entries:
                    take(cache.pages_needed(e.seq.request_id, e.start + e.count))
            decoding = [s for s in decoding if s is not victim]
            i = min(i, len(decoding))

        # 2. portions of prompts: requests that are part-way first, then new ones in arrival order
        for seq in [s for s in self.running if s.phase is Phase.PREFILL]:
            if budget <= 0 or len(plan.entries) >= cfg.max_batch_size:
                break
            budget -= self._plan_portion(seq, budget, plan, fits, take)
        while self.waiting and budget > 0 and len(plan.entries) < cfg.max_batch_size \
                and len(self.running) < cfg.max_batch_size and cache.num_free_slots > 0:
            seq = self.waiting[0]
            if seq in plan.preempted:
                break  # preempted in this very step: it waits for the next one
            rc = cache.admit(seq.request_id, seq.tokens)
            seq.num_computed = rc.num_tokens  # > 0 if leading pages are shared with a live request
            first = min(seq.pending, cfg.max_prefill_chunk_tokens, budget)
            ok, _ = fits(seq, seq.num_computed + first)
            if not ok and self.running:
                # not even the first portion fits while others run: wait (a lone request takes what fits)
                cache.release(seq.request_id)
                seq.num_computed = 0
                break
            self.waiting.popleft()
            seq.slot = rc.slot
            seq.phase = Phase.PREFILL
            seq.reused_prompt_tokens += rc.num_tokens
            self.running.append(seq)
            plan.admitted.append(seq)
            if self.on_admit:
                self.on_admit(seq)
            used = self._plan_portion(seq, budget, plan, fits, take)
            budget -= used
            if used == 0:
                break

    def _plan_portion(self, seq, budget, plan, fits, take) -> int:
        cfg = self.config
        count = min(seq.pending, cfg.max_prefill_chunk_tokens, budget)
        while count > 0:
            ok, need = fits(seq, seq.num_computed + count)
            if ok:
                take(need)
                plan.entries.append(ScheduledEntry(seq, seq.num_computed, count, count == seq.pending))
                return count
            # shorten to the end of the last page that still fits
            ps = self.cache.page_size
            shorter = ((seq.num_computed + count - 1) // ps) * ps - seq.num_computed
            count = shorter if shorter < count else count - 1
        return 0

    def _preempt(self, seq: Sequence, plan: StepPlan) -> None:
        self.running.remove(seq)
        if self.on_preempt:
            self.on_preempt(seq)
        self.cache.release(seq.request_id)
        seq.phase = Phase.WAITING
        seq.num_computed = 0
        seq.slot = None
        seq.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(seq)
        plan.preempted.append(seq)

    # ------------------------------------------------------------------- update
    def update(self, plan: StepPlan, sampled: dict) -> list:
        """The step ran.  ``sampled``: request id -> (token, probability) for the entries that sample.
        Returns the sequences that finished, whose pages and slots are released here."""
        cfg = self.config
        done = []
        self.stats["steps"] += 1
        self.stats["tokens"] += plan.num_tokens
        for e in plan.entries:
            seq = e.seq
            if seq.phase is Phase.FINISHED or seq.phase is Phase.WAITING:
                continue  # finished or cancelled while this step was running: its share is void
            seq.num_computed = e.start + e.count
            if not e.samples:
                continue
            reason = None
            if len(seq.generated) >= seq.max_new_tokens:
                # nothing may be generated (max_new_tokens == 0, or recomputed after the budget was met)
                reason = self._budget_reason(seq)
            elif seq.num_tokens >= cfg.max_sequence_length:
                reason = FinishReason.SEQUENCE_LENGTH
            else:
                token, prob = sampled[seq.request_id]
                seq.generated.append(int(token))
                seq.probabilities.append(float(prob))
                seq.phase = Phase.DECODE
                self.stats["sampled"] += 1
                if seq.params.stops(int(token)):
                    reason = FinishReason.STOP_TOKEN
                elif len(seq.generated) >= seq.max_new_tokens:
                    reason = self._budget_reason(seq)
                elif seq.num_tokens >= cfg.max_sequence_length:
                    reason = FinishReason.SEQUENCE_LENGTH
            if reason is not None:
                self._finish(seq, reason)
                done.append(seq)
        return done

    @staticmethod
    def _budget_reason(seq: Sequence) -> FinishReason:
        """MaxNewTokens, or SessionLimit if the session's cap was the smaller one
        (crates/ferrisinfer-runtime/src/sequence.rs:173-179)."""
        return FinishReason.SESSION_LIMIT if seq.max_new_tokens < seq.requested_max_new_tokens \
            else FinishReason.MAX_NEW_TOKENS

    def _finish(self, seq: Sequence, reason: FinishReason) -> None:
        seq.phase = Phase.FINISHED
        seq.finish_reason = reason
        if seq in self.running:
            self.running.remove(seq)
            self.cache.release(seq.request_id)
        elif seq in self.waiting:
            self.waiting.remove(seq)
        seq.slot = None
        self.finished[seq.request_id] = seq

    def cancel(self, request_id) -> Optional[Sequence]:
        """Take a request out wherever it is; what it holds is given back."""
        for seq in list(self.running) + list(self.waiting):
            if seq.request_id == request_id:
                self._finish(seq, FinishReason.CANCELLED)
                return seq
        return None
