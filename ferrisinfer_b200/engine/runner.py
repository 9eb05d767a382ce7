"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

The reference runs one request at a time: ``Session::prefill_tokens`` for a chunk of two or more
tokens appended at the committed position, the decode path for one token
(crates/ferrisinfer-runtime/src/session.rs:220-262), and a scheduler tick is all prefill or all
decode, executed sequence by sequence (crates/ferrisinfer-runtime/src/scheduler.rs:393-415).  Here
ONE step carries any mix: portions of prompts beside single decoded tokens, cut anywhere.  The
step packs all tokens into one array with per-token positions and cache slots and per-request block
tables, writes the step's keys and values into the cache, runs every layer once over all tokens,
and forms logits only at the rows asked for.  Afterwards the requests' token counts advance
(the reference's ``advance(n)``: crates/ferrisinfer-runtime/src/session.rs:371,407).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import NO_PAGE, CacheManager
from ..errors import CacheError, FerrisError, OutOfPages
from ..kernels import ops
from ..parts.base import FixedState, PagedMeta, SeqInfo, StepContext
from ..parts.model import DecoderModel
from .workspace import Workspace


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them (0-based
    indices into ``tokens``) whose logits are wanted."""

    request_id: Any
    tokens: Sequence[int]
    want: Sequence[int] = ()


class ModelRunner:
    """Owns the model, the cache manager and the workspace; ``step`` is the only way tokens run."""

    def __init__(self, model: DecoderModel, dtype: torch.dtype, device, page_size: int, num_pages: int,
                 max_requests: int, max_model_len: Optional[int] = None, extra_states: Optional[dict] = None):
        if not model.bound:
            raise FerrisError("the model has no weights bound")
        self.model = model
        self.dtype = dtype
        self.device = torch.device(device)
        self.vocab_size = model.vocab_size
        self.max_model_len = int(max_model_len or model.plan.max_positions)
        self.cache = CacheManager(model.cache_needs(), page_size, num_pages, max_requests, dtype=dtype,
                                  device=self.device, extra_states=extra_states)
        self.workspace = Workspace(self.device)
        self.steps_run = 0
        self.last_h2d_bytes = 0
        self._pinned = None

    # ------------------------------------------------------------------ requests
    def add_request(self, request_id) -> int:
        return self.cache.admit(request_id).slot

    def has_request(self, request_id) -> bool:
        return self.cache.has(request_id)

    def free_request(self, request_id) -> int:
        return self.cache.release(request_id)

    def num_tokens(self, request_id) -> int:
        return self.cache.get(request_id).num_tokens

    # ---------------------------------------------------------------------- step
    def step(self, entries: Sequence[StepEntry], out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run the tokens of ``entries`` as one batch from the cache that earlier steps left.
        Returns fp32 logits [wanted, vocab] in the order of the entries and of their ``want``
        (None if nothing is wanted).  Requests that are not admitted yet are admitted."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return None
        ctx, logits_index = self._prepare(entries)
        n_want = 0 if logits_index is None else logits_index.numel()
        logits = None
        if n_want:
            logits = out if out is not None else self.workspace.get("logits", (n_want, self.vocab_size), torch.float32)
        self.model.forward(ctx, self.cache.layer_caches, logits_index, logits)
        for e, s in zip(entries, ctx.seqs):
            self.cache.commit(e.request_id, s.start_pos + s.q_len)
        self.steps_run += 1
        return logits

    def _upload(self, pieces) -> torch.Tensor:
        """One copy of the step's int32 metadata, host (pinned) to device."""
        total = sum(p.size for p in pieces)
        if self.device.type != "cuda":
            return torch.from_numpy(np.concatenate(pieces)).to(self.device)
        if self._pinned is None or self._pinned.numel() < total:
            self._pinned = torch.empty(max(total, 4096) * 2, dtype=torch.int32).pin_memory()
        host = self._pinned.numpy()
        off = 0
        for p in pieces:
            host[off:off + p.size] = p.reshape(-1)
            off += p.size
        dev = torch.empty(total, dtype=torch.int32, device=self.device)
        dev.copy_(self._pinned[:total], non_blocking=True)
        # the pinned buffer is rewritten by the next step: the copy must have left it by then
        torch.cuda.current_stream(self.device).synchronize()
        self.last_h2d_bytes = total * 4
        return dev

    # ----------------------------------------------------------- step preparation
    def _prepare(self, entries):
        cache = self.cache
        seen = set()
        T = 0
        for e in entries:
            if e.request_id in seen:
                raise FerrisError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            n = len(e.tokens)
            for w in e.want:
                if not (0 <= w < n):
                    raise FerrisError(f"request {e.request_id!r}: wanted place {w} is not among its {n} tokens")
            T += n
        for e in entries:
            if not cache.has(e.request_id):
                cache.admit(e.request_id)
        # all pages of the step or none
        short = {g.gid: 0 for g in cache.groups}
        for e in entries:
            rc = cache.get(e.request_id)
            total = rc.num_tokens + len(e.tokens)
            if total > self.max_model_len:
                raise FerrisError(f"request {e.request_id!r} would reach {total} tokens; the limit is {self.max_model_len}")
            for gid, n in cache.pages_needed(e.request_id, total).items():
                short[gid] += n
        for g in cache.groups:
            if short[g.gid] > g.pool.num_free:
                raise OutOfPages(f"the step needs {short[g.gid]} new pages in group {g.gid}; "
                                 f"{g.pool.num_free} of {g.pool.num_pages} are free")
        for e in entries:
            cache.extend(e.request_id, cache.get(e.request_id).num_tokens + len(e.tokens))

        S = len(entries)
        ps = cache.page_size
        token_ids = np.empty(T, dtype=np.int32)
        positions = np.empty(T, dtype=np.int32)
        token_seq = np.empty(T, dtype=np.int32)
        q_start = np.zeros(S + 1, dtype=np.int32)
        start_pos = np.empty(S, dtype=np.int32)
        state_slot = np.empty(S, dtype=np.int32)
        want_rows = []
        seqs = []
        max_q = max_kv = 0
        row = 0
        for i, e in enumerate(entries):
            rc = cache.get(e.request_id)
            n = len(e.tokens)
            toks = np.asarray(e.tokens, dtype=np.int64)
            if toks.min() < 0 or toks.max() >= self.vocab_size:
                raise FerrisError(f"request {e.request_id!r}: a token id lies outside [0, {self.vocab_size})")
            token_ids[row:row + n] = toks
            positions[row:row + n] = np.arange(rc.num_tokens, rc.num_tokens + n, dtype=np.int32)
            token_seq[row:row + n] = i
            q_start[i + 1] = row + n
            start_pos[i] = rc.num_tokens
            state_slot[i] = rc.slot
            want_rows += [row + w for w in e.want]
            seqs.append(SeqInfo(e.request_id, row, n, rc.num_tokens, rc.slot))
            max_q = max(max_q, n)
            max_kv = max(max_kv, rc.num_tokens + n)
            row += n
        max_blocks = max(1, -(-max_kv // ps))
        group_arrays = []
        for g in cache.groups:
            slot_mapping = np.empty(T, dtype=np.int32)
            tables = np.full((S, max_blocks), NO_PAGE, dtype=np.int32)
            for i, (e, s) in enumerate(zip(entries, seqs)):
                table = cache.block_table(e.request_id, g.gid)
                tables[i, :len(table)] = table
                pos = positions[s.q_start:s.q_start + s.q_len]
                pages = tables[i, pos // ps]
                if (pages < 0).any():
                    raise CacheError(f"request {e.request_id!r}: a token of the step has no page in group {g.gid}")
                slot_mapping[s.q_start:s.q_start + s.q_len] = pages * ps + pos % ps
            group_arrays.append((slot_mapping, tables))
        want = np.asarray(want_rows, dtype=np.int32)

        pieces = [token_ids, positions, token_seq, q_start, start_pos, state_slot, want]
        for slot_mapping, tables in group_arrays:
            pieces += [slot_mapping, tables.reshape(-1)]
        dev = self._upload(pieces)
        views = []
        off = 0
        for p in pieces:
            views.append(dev[off:off + p.size])
            off += p.size
        paged = {}
        for k, g in enumerate(cache.groups):
            paged[g.gid] = PagedMeta(block_tables=views[7 + 2 * k + 1].view(S, max_blocks),
                                     slot_mapping=views[7 + 2 * k], page_size=ps)
        ctx = StepContext(
            num_tokens=T, num_seqs=S, token_ids=views[0], positions=views[1], token_seq=views[2],
            seq_q_start=views[3], seq_start_pos=views[4], seq_state_slot=views[5], seqs=seqs, paged=paged,
            max_q_len=max_q, max_kv_len=max_kv, act_dtype=self.dtype, workspace=self.workspace, device=self.device,
        )
        return ctx, (views[6] if want.size else None)
