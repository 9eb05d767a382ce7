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

import gc
from collections import OrderedDict
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


@dataclass
class _HostStep:
    """A step laid out on the host: the int32 pieces that go to the device, and what the host keeps.
    ``T``, ``S`` and ``n_want`` count the rows on the device, padding rows included; ``real`` is the number
    of requests (and of wanted rows) that the caller brought."""

    pieces: list
    T: int
    S: int
    max_q: int
    max_kv: int
    max_blocks: int
    seqs: list
    n_want: int
    real: int = 0


@dataclass
class _GraphEntry:
    meta: torch.Tensor  # static device buffer of the step's metadata
    ctx: StepContext
    logits_index: torch.Tensor
    logits: torch.Tensor
    greedy: Any = None  # (tokens, probabilities) of a step that samples greedily on its way
    graph: Any = None
    kernels: int = 0  # kernel launches that one replay stands for


class ModelRunner:
    """Owns the model, the cache manager and the workspace; ``step`` is the only way tokens run.

    Steps in which every request brings exactly one token and wants its logits (decoding) are replayed
    from CUDA graphs: the ~150 kernel launches of a step become one.  Such a step is filled up with padding
    rows to the next of a few batch sizes (``DECODE_BUCKETS``), so that a pool of 1..N decoding requests needs
    a handful of graphs, one per (batch size, width of the block tables); a padding row is a token at position
    0 of a request that does not exist, whose key, value and state go to the cache manager's padding page and
    padding slot, and whose logits nobody reads.  All decode graphs write one shared logits buffer.  Any other
    shape of step is recorded when it comes a second time (portions of a fixed size recur); the rest launch
    their kernels one by one.  At most ``MAX_GRAPHS`` recorded steps are kept, the least recently replayed
    goes first.  The metadata of a recorded step lives in a static device buffer that is rewritten before
    each replay."""

    N_FIXED = 7  # token_ids, positions, token_seq, q_start, start_pos, state_slot, want
    MAX_GRAPHS = 48  # recorded shapes of step, decode steps included
    MAX_GRAPH_LOGITS_BYTES = 64 << 20  # a recorded step that is no decode step owns its logits buffer
    DECODE_BUCKETS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512)

    def __init__(self, model: DecoderModel, dtype: torch.dtype, device, page_size: int, num_pages: int,
                 max_requests: int, max_model_len: Optional[int] = None, extra_states: Optional[dict] = None,
                 cuda_graphs: bool = True, prefix_sharing: bool = False, min_prefix_share_tokens: int = 0,
                 keep_finished: bool = False):
        if not model.bound:
            raise FerrisError("the model has no weights bound")
        self.model = model
        self.dtype = dtype
        self.device = torch.device(device)
        self.vocab_size = model.vocab_size
        self.max_model_len = int(max_model_len or model.plan.max_positions)
        self.cache = CacheManager(model.cache_needs(), page_size, num_pages, max_requests, dtype=dtype,
                                  device=self.device, extra_states=extra_states, prefix_sharing=prefix_sharing,
                                  min_prefix_share_tokens=min_prefix_share_tokens, keep_finished=keep_finished)
        self.workspace = Workspace(self.device)
        self.steps_run = 0
        self.last_h2d_bytes = 0
        self._staging = []  # ring of (pinned buffer, event of the last copy out of it)
        self._staging_next = 0
        self.cuda_graphs = bool(cuda_graphs) and self.device.type == "cuda" and getattr(model, "graph_safe", False)
        self.max_requests = int(max_requests)
        self._graphs: OrderedDict = OrderedDict()  # shape of step -> recorded step, least recently replayed first
        self._shapes_seen: dict = {}
        self._decode_logits: Optional[torch.Tensor] = None  # [largest bucket, vocab], shared by the decode graphs
        self.graph_replays = 0
        self.graph_kernels = 0  # kernel launches made through graph replays
        self.graphs_dropped = 0

    # ------------------------------------------------------------------ requests
    def add_request(self, request_id, prompt: Optional[Sequence[int]] = None) -> int:
        """Admit a request; returns its state slot.  With ``prompt`` (its known tokens) and prefix sharing on,
        leading full pages that the cache already holds are borrowed: ``num_tokens(request_id)`` then says how
        many tokens the request need not bring."""
        return self.cache.admit(request_id, None if prompt is None else list(prompt)).slot

    def has_request(self, request_id) -> bool:
        return self.cache.has(request_id)

    def free_request(self, request_id) -> int:
        return self.cache.release(request_id)

    def num_tokens(self, request_id) -> int:
        return self.cache.get(request_id).num_tokens

    # ---------------------------------------------------------------------- step
    def step(self, entries: Sequence[StepEntry], out: Optional[torch.Tensor] = None,
             device_tokens: Optional[torch.Tensor] = None, greedy: bool = False):
        """Run the tokens of ``entries`` as one batch from the cache that earlier steps left.
        Returns fp32 logits [wanted, vocab] in the order of the entries and of their ``want``
        (None if nothing is wanted).  Requests that are not admitted yet are admitted.
        The returned tensor is the runner's own buffer: it is overwritten by the next step.
        ``device_tokens`` (int32 on the device, one per entry): every entry brings one token whose id the
        host does not know yet (it was sampled by a step that is still running); the ids in ``entries`` are
        placeholders and the step reads the real ones from this tensor.
        ``greedy``: instead of the logits the step returns (tokens int32 [wanted], probabilities fp32 [wanted]) on
        the device, each wanted row's most likely token (the lowest index among equals) and its probability; the
        output head then stores no logits where its kernel can avoid it.  The two tensors are the runner's own too."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return None
        if device_tokens is not None and (any(len(e.tokens) != 1 for e in entries) or device_tokens.numel() != len(entries)
                                          or device_tokens.dtype != torch.int32):
            raise FerrisError("tokens on the device: one int32 for each entry of one token is needed")
        decode = all(len(e.tokens) == 1 and len(e.want) == 1 and e.want[0] == 0 for e in entries)
        graphs = self.cuda_graphs and out is None
        host = self._layout(entries, pad_to=self._bucket(len(entries)) if (decode and graphs) else 0)
        greedy = bool(greedy) and host.n_want > 0 and out is None
        if graphs and self._graph_worthwhile(host, decode, greedy):
            logits = self._step_graph(host, device_tokens, decode, greedy)
        else:
            dev = self._upload(host.pieces)
            if device_tokens is not None:
                dev[:host.real].copy_(device_tokens)
            ctx, logits_index = self._context(host, dev)
            logits = None
            if greedy:
                logits = (torch.empty(host.n_want, dtype=torch.int32, device=self.device),
                          torch.empty(host.n_want, dtype=torch.float32, device=self.device))
                self.model.forward(ctx, self.cache.layer_caches, logits_index, None, greedy_out=logits)
            else:
                if host.n_want:
                    logits = out if out is not None else self.workspace.get("logits", (host.n_want, self.vocab_size),
                                                                            torch.float32)
                self.model.forward(ctx, self.cache.layer_caches, logits_index, logits)
        for e, s in zip(entries, host.seqs):
            self.cache.commit(e.request_id, s.start_pos + s.q_len)
        self.steps_run += 1
        return logits

    def _bucket(self, requests: int) -> int:
        """The batch size a decode step of ``requests`` single tokens is filled up to."""
        for b in self.DECODE_BUCKETS:
            if b >= requests:
                return b
        return requests

    @staticmethod
    def _shape_key(host: _HostStep, greedy: bool = False) -> tuple:
        """What fixes every launch of a step: the counts of tokens, requests, wanted rows and single tokens beside
        portions, the longest share and the width of the block tables.  Everything else (which tokens, positions,
        pages, how the tokens divide among the requests, which rows are wanted) is data in the step's metadata
        buffer."""
        return (host.T, host.S, host.max_q, host.max_blocks, host.n_want, int(host.pieces[-1].size), bool(greedy))

    def _graph_worthwhile(self, host: _HostStep, decode: bool, greedy: bool = False) -> bool:
        """Decode steps are recorded at first sight; any other shape of step when it comes a second time (portions of
        a fixed size recur, most mixed steps do not), unless its logits would make the graph's own buffer large."""
        if decode:
            return True
        key = self._shape_key(host, greedy)
        if key in self._graphs:
            return True
        seen = self._shapes_seen.get(key, 0)
        if len(self._shapes_seen) > 4096:
            self._shapes_seen.clear()
        self._shapes_seen[key] = seen + 1
        return seen >= 1 and (greedy or host.n_want * self.vocab_size * 4 <= self.MAX_GRAPH_LOGITS_BYTES)

    def drop_graphs(self) -> None:
        """Forget every recorded step (their buffers go with them)."""
        if self._graphs:
            torch.cuda.synchronize(self.device)
            self.graphs_dropped += len(self._graphs)
            self._graphs.clear()
        self.workspace.unpin()

    def _step_graph(self, host: _HostStep, device_tokens: Optional[torch.Tensor] = None,
                    decode: bool = False, greedy: bool = False):
        key = self._shape_key(host, greedy)
        entry = self._graphs.get(key)
        if entry is None:
            while len(self._graphs) >= self.MAX_GRAPHS:
                # the least recently replayed goes; nothing of it may still be running when its memory is freed
                torch.cuda.synchronize(self.device)
                self._graphs.popitem(last=False)
                self.graphs_dropped += 1
            total = sum(p.size for p in host.pieces)
            meta = torch.zeros(total, dtype=torch.int32, device=self.device)
            self._upload(host.pieces, meta)
            if device_tokens is not None:
                meta[:host.real].copy_(device_tokens)
            ctx, logits_index = self._context(host, meta)
            # launch geometry that depends on the keys' length is fixed for the width of the block table
            ctx.max_kv_len = host.max_blocks * self.cache.page_size
            logits = None
            picked = None
            if greedy:
                picked = (torch.empty(host.n_want, dtype=torch.int32, device=self.device),
                          torch.empty(host.n_want, dtype=torch.float32, device=self.device))
            elif host.n_want and decode:
                if self._decode_logits is None:
                    rows = max(self._bucket(self.max_requests), host.n_want)
                    self._decode_logits = torch.empty(rows, self.vocab_size, dtype=torch.float32, device=self.device)
                if host.n_want <= self._decode_logits.shape[0]:
                    logits = self._decode_logits[:host.n_want]
            if host.n_want and logits is None and not greedy:
                logits = torch.empty(host.n_want, self.vocab_size, dtype=torch.float32, device=self.device)
            entry = _GraphEntry(meta, ctx, logits_index, logits, picked)
            # the first step of this shape runs eagerly (it also sizes every workspace buffer) ...
            self.model.forward(ctx, self.cache.layer_caches, logits_index, logits, greedy_out=picked)
            # ... and is then recorded for the steps to come; from here on the workspace keeps what it replaces
            self.workspace.pin()
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            # No garbage collection while the stream records: a collection that frees pinned buffers or events of
            # an engine that is no longer used would issue calls that are not permitted during capture.
            collecting = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph):
                    self.model.forward(ctx, self.cache.layer_caches, logits_index, logits, greedy_out=picked)
            finally:
                if collecting:
                    gc.enable()
            entry.kernels = ops.launch_count() - before
            entry.graph = graph
            self._graphs[key] = entry
            # the capture itself ran nothing, but the eager run before it did: the result is in ``logits``
            return self._result(entry, host, decode)
        self._graphs.move_to_end(key)
        self._upload(host.pieces, entry.meta)
        if device_tokens is not None:
            entry.meta[:host.real].copy_(device_tokens)  # the token ids are the first piece of the metadata
        entry.ctx.seqs = host.seqs
        entry.graph.replay()
        self.graph_replays += 1
        self.graph_kernels += entry.kernels
        return self._result(entry, host, decode)

    @staticmethod
    def _result(entry: _GraphEntry, host: _HostStep, decode: bool):
        """What a recorded step hands back: its logits, or its tokens and probabilities; without the padding rows."""
        if entry.greedy is not None:
            return (entry.greedy[0][:host.real], entry.greedy[1][:host.real]) if decode else entry.greedy
        return entry.logits[:host.real] if decode else entry.logits

    # ------------------------------------------------------------------- upload
    def _upload(self, pieces, dest: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One copy of the step's int32 metadata from pinned host memory to the device."""
        total = sum(p.size for p in pieces)
        if self.device.type != "cuda":
            flat = torch.from_numpy(np.concatenate([p.reshape(-1) for p in pieces]))
            if dest is None:
                return flat.to(self.device)
            dest[:total].copy_(flat)
            return dest
        if not self._staging:
            self._staging = [[None, None] for _ in range(4)]
        slot = self._staging[self._staging_next]
        self._staging_next = (self._staging_next + 1) % len(self._staging)
        if slot[1] is not None:
            slot[1].synchronize()  # the copy that last read this buffer has finished (long ago, as a rule)
        if slot[0] is None or slot[0].numel() < total:
            slot[0] = torch.empty(max(total * 2, 16384), dtype=torch.int32).pin_memory()
            slot[1] = torch.cuda.Event()
        host = slot[0].numpy()
        off = 0
        for p in pieces:
            host[off:off + p.size] = p.reshape(-1)
            off += p.size
        if dest is None:
            dest = torch.empty(total, dtype=torch.int32, device=self.device)
        dest[:total].copy_(slot[0][:total], non_blocking=True)
        slot[1].record(torch.cuda.current_stream(self.device))
        self.last_h2d_bytes = total * 4
        return dest

    # ----------------------------------------------------------- step preparation
    def _layout(self, entries, pad_to: int = 0) -> _HostStep:
        """Check the step, take its pages (all of the step or none; a refused step leaves no trace in the
        cache) and lay its metadata out.  ``pad_to``: a step of single tokens is filled up to this many rows."""
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
        S = len(entries)
        if T == S:  # one token each
            token_ids = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=S)
        else:
            token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if token_ids.min() < 0 or token_ids.max() >= self.vocab_size:
            raise FerrisError(f"a token id of the step lies outside [0, {self.vocab_size})")
        token_ids = token_ids.astype(np.int32)
        admitted_here = []
        try:
            for e in entries:
                if not cache.has(e.request_id):
                    cache.admit(e.request_id)
                    admitted_here.append(e.request_id)
            # all pages of the step or none
            short = {g.gid: 0 for g in cache.groups}
            for e in entries:
                rc = cache.get(e.request_id)
                total = rc.num_tokens + len(e.tokens)
                if total > self.max_model_len:
                    raise FerrisError(
                        f"request {e.request_id!r} would reach {total} tokens; the limit is {self.max_model_len}")
                for gid, n in cache.pages_needed(e.request_id, total).items():
                    short[gid] += n
            free = cache.free_pages()
            for g in cache.groups:
                if short[g.gid] > free[g.gid]:
                    raise OutOfPages(f"the step needs {short[g.gid]} new pages in group {g.gid}; "
                                     f"{free[g.gid]} of {g.pool.num_pages} are free")
        except FerrisError:
            for rid in admitted_here:
                cache.release(rid)
            raise
        for e in entries:
            cache.extend(e.request_id, cache.get(e.request_id).num_tokens + len(e.tokens))

        ps = cache.page_size
        rcs = [cache.get(e.request_id) for e in entries]
        q_lens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=S)
        start_pos = np.fromiter((rc.num_tokens for rc in rcs), dtype=np.int32, count=S)
        state_slot = np.fromiter((rc.slot for rc in rcs), dtype=np.int32, count=S)
        pad = max(0, pad_to - S) if T == S else 0
        if pad:
            # padding rows: one token (id 0) at position 0 of a request that holds the padding page and slot
            token_ids = np.concatenate([token_ids, np.zeros(pad, dtype=np.int32)])
            q_lens = np.concatenate([q_lens, np.ones(pad, dtype=np.int32)])
            start_pos = np.concatenate([start_pos, np.zeros(pad, dtype=np.int32)])
            state_slot = np.concatenate([state_slot, np.full(pad, cache.padding_slot, dtype=np.int32)])
        real, S, T = S, S + pad, T + pad
        q_start = np.zeros(S + 1, dtype=np.int32)
        np.cumsum(q_lens, out=q_start[1:])
        if T == S:
            token_seq = np.arange(S, dtype=np.int32)
            positions = start_pos.copy()
        else:
            token_seq = np.repeat(np.arange(S, dtype=np.int32), q_lens)
            positions = (np.arange(T, dtype=np.int32) - q_start[token_seq] + start_pos[token_seq]).astype(np.int32)
        want_rows = []
        seqs = []
        for i, (e, rc) in enumerate(zip(entries, rcs)):
            row = int(q_start[i])
            if len(e.want) == 1:
                want_rows.append(row + e.want[0])
            elif e.want:
                want_rows += [row + w for w in e.want]
            seqs.append(SeqInfo(e.request_id, row, int(q_lens[i]), rc.num_tokens, rc.slot))
        want_rows += list(range(real, S))  # the padding rows' logits are formed too: the step's shape is its bucket's
        max_q = int(q_lens.max())
        max_kv = int((start_pos + q_lens).max())
        # block tables are as wide as the next power of two of what the longest request needs, so that the
        # shapes a decode graph is recorded with recur
        need_blocks = max(1, -(-max_kv // ps))
        max_blocks = 8
        while max_blocks < need_blocks:
            max_blocks *= 2
        max_blocks = min(max_blocks, max(need_blocks, -(-self.max_model_len // ps)))
        group_arrays = []
        for g in cache.groups:
            tables = np.full((S, max_blocks), NO_PAGE, dtype=np.int32)
            for i, e in enumerate(entries):
                arr = cache.block_table_array(e.request_id, g.gid)
                tables[i, :arr.size] = arr
            if pad:
                tables[real:, 0] = cache.padding_page(g.gid)
            pages = tables[token_seq, positions // ps]
            if (pages < 0).any():
                raise CacheError(f"a token of the step has no page in group {g.gid}")
            slot_mapping = (pages * ps + positions % ps).astype(np.int32)
            group_arrays.append((slot_mapping, tables))
        want = np.asarray(want_rows, dtype=np.int32)
        pieces = [token_ids, positions, token_seq, q_start, start_pos, state_slot, want]
        for slot_mapping, tables in group_arrays:
            pieces += [slot_mapping, tables.reshape(-1)]
        singles = [s.q_start for s in seqs if s.q_len == 1] if max_q > 1 else []
        pieces.append(np.asarray(singles, dtype=np.int32))
        return _HostStep(pieces, T, S, max_q, max_kv, max_blocks, seqs, int(want.size), real)

    def _context(self, host: _HostStep, dev: torch.Tensor):
        views = []
        off = 0
        for p in host.pieces:
            views.append(dev[off:off + p.size])
            off += p.size
        paged = {}
        for k, g in enumerate(self.cache.groups):
            paged[g.gid] = PagedMeta(block_tables=views[self.N_FIXED + 2 * k + 1].view(host.S, host.max_blocks),
                                     slot_mapping=views[self.N_FIXED + 2 * k], page_size=self.cache.page_size)
        ctx = StepContext(
            num_tokens=host.T, num_seqs=host.S, token_ids=views[0], positions=views[1], token_seq=views[2],
            seq_q_start=views[3], seq_start_pos=views[4], seq_state_slot=views[5], seqs=host.seqs, paged=paged,
            max_q_len=host.max_q, max_kv_len=host.max_kv, act_dtype=self.dtype, workspace=self.workspace,
            device=self.device, single_rows=views[-1] if host.pieces[-1].size else None,
        )
        return ctx, (views[6] if host.n_want else None)
