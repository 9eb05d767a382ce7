"""Interfaces of the parts a layer is put together from, and what a step hands them.

A part is built from explicit sizes and constants (never from a model's
configuration object), lists the tensors it reads (``tensor_specs``), receives
them (``bind``) and computes on the tokens of one step (``forward``).  No part
knows which model, or which layer of it, it is in.

Activations: the residual stream ``h`` is fp32 ``[T, H]`` in both precisions;
norms read it and write the compute dtype (bf16 or fp32); mixers and
feed-forwards read the normed rows and ADD their result into ``h``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from .plan import TensorSpec


# ----------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class PagedKV:
    """The mixer keeps a key and a value of ``num_kv_heads x head_dim`` per token, in pages.
    ``window``: None = every past token is read; n = only the last n (the current one included),
    so pages that lie wholly behind the window are given back while the request runs."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """The mixer keeps a tensor of ``shape`` per request, whatever the request's length.
    It is zeroed when a request is admitted."""

    shape: tuple
    dtype: torch.dtype = torch.float32


# ----------------------------------------------------------------------------- step context
@dataclass
class PagedMeta:
    """Device metadata of one page group for one step."""

    block_tables: torch.Tensor  # int32 [S, max_blocks]; -1 = no page
    slot_mapping: torch.Tensor  # int32 [T]; page * page_size + slot of each token of the step
    page_size: int


@dataclass
class SeqInfo:
    """Host-side description of one request's share of a step."""

    request_id: Any
    q_start: int  # first row of the step's token arrays
    q_len: int
    start_pos: int  # tokens of the request that were in the cache before this step
    state_slot: int


@dataclass
class StepContext:
    """Everything a part may need about the step: device arrays and their host twins."""

    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor  # int32 [T]
    positions: torch.Tensor  # int32 [T] absolute position of each token
    token_seq: torch.Tensor  # int32 [T] index of the token's request within the step
    seq_q_start: torch.Tensor  # int32 [S + 1]
    seq_start_pos: torch.Tensor  # int32 [S]
    seq_state_slot: torch.Tensor  # int32 [S]
    seqs: list  # list[SeqInfo]
    paged: dict  # group id -> PagedMeta
    max_q_len: int
    max_kv_len: int
    act_dtype: torch.dtype
    workspace: Any  # engine.workspace.Workspace
    device: torch.device = None
    # in a step that mixes portions of prompts with single tokens: the rows (int32, device) of the
    # requests that bring exactly one token, so that kernels made for either kind can share the step
    single_rows: Optional[torch.Tensor] = None
    # what parts compute once per pass of the model and share across layers, under keys of their own; the
    # model empties it when a pass begins
    shared: dict = field(default_factory=dict)

    @property
    def all_decode(self) -> bool:
        return self.max_q_len == 1


@dataclass
class LayerCache:
    """What one run of a layer's mixer owns in the cache.

    ``group``: id of the page group (PagedKV) whose block tables address ``k`` and ``v``
    ([pages, kv heads, page size, head dim]); ``state``: [slots, *shape] for FixedState.
    """

    need: Any
    group: Optional[int] = None
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None


# ----------------------------------------------------------------------------- part interfaces
class Part:
    """Base of every part."""

    def tensor_specs(self, prefix: str) -> list:
        """The tensors this part reads, named under ``prefix``."""
        return []

    def bind(self, tensors: dict, prefix: str) -> None:
        """Receive the loaded tensors (on the device, in the dtype their role gives).
        Optional tensors that the folder lacks are absent from ``tensors``."""


class Norm(Part):
    def forward(self, h: torch.Tensor, out: torch.Tensor, row_index: Optional[torch.Tensor] = None) -> None:
        """out[i] = norm(h[row_index[i]] or h[i]); h fp32, out in the compute dtype."""
        raise NotImplementedError

    def lazy(self, h: torch.Tensor, out: torch.Tensor):
        """An object that stands for norm(h): ``materialize()`` computes it into ``out`` (once).  A norm
        whose arithmetic a matrix-product kernel can do on its way returns a richer object that such a
        kernel recognises; the default is to compute at once."""
        self.forward(h, out)
        return out


class PositionEncoding(Part):
    """How positions enter a mixer.  ``rotary_table`` lets the attention mixer fuse the
    rotation with its cache write; a kind without one is applied through ``apply``; a kind that acts on
    the attention scores instead of (or beside) q and k says so with ``score_slopes``."""

    # as for Mixer: True if ``apply`` may be recorded into a CUDA graph (kinds with a rotary table never run it)
    graph_safe = False

    def rotary_table(self, device=None) -> Optional[tuple]:
        """``(inv_freq, R)`` if the encoding is a rotate-half rotation of the first R dims of
        each head by ``pos * inv_freq[i]`` (inv_freq fp32 [R/2] on ``device``; ``(None, 0)`` =
        nothing to rotate), which the attention mixer fuses with its cache write.
        ``None`` = not of that form: the mixer calls ``apply`` instead."""
        return None

    def apply(self, qkv: torch.Tensor, positions: torch.Tensor, num_heads: int, num_kv_heads: int,
              head_dim: int) -> None:
        """Encode positions into the q and k heads of ``qkv`` in place."""
        raise NotImplementedError

    def score_slopes(self, num_heads: int, device=None) -> Optional[torch.Tensor]:
        """fp32 [num_heads] on ``device`` if the encoding adds ``slopes[head] * (j - P)`` to the score of the key at
        position j for the query at position P (a penalty linear in the distance; j <= P); None (the default) if it
        adds nothing to the scores.  Such scores are attended by the general kernel in every precision."""
        return None


class Mixer(Part):
    """What mixes the tokens of a request: attention over cached keys and values, a recurrence over a state
    of fixed size, or anything else that declares its need with ``cache_need``.

    A step hands the mixer all its tokens as one batch; which row belongs to which request is told twice, on
    the host (``ctx.seqs``, a list of ``SeqInfo``) and on the device.  A mixer that wants its steps recorded
    into CUDA graphs (``graph_safe``) works from the device arrays alone, because a replayed step runs no
    Python: ``ctx.token_seq`` [T] (index of each row's request within the step), ``ctx.positions`` [T],
    ``ctx.seq_q_start`` [S + 1] (first row of each request; rows of a request are consecutive and in order),
    ``ctx.seq_start_pos`` [S] (tokens the request held before the step), ``ctx.seq_state_slot`` [S] (the row
    of ``cache.state`` that is the request's, for a ``FixedState`` need) and, for a ``PagedKV`` need,
    ``ctx.paged[cache.group]`` (block tables [S, max_blocks] and the cache slot of every row).  The shapes
    T and S are those of the recorded step; the contents change from replay to replay.  A decode step may
    carry padding rows after the real ones: single tokens at position 0 of requests that do not exist, whose
    state slot and page are the cache manager's padding slot and padding page, so whatever a mixer writes
    for them lands where nobody reads.  A mixer with state must carry the state across steps through its
    slot and process a request's rows in order; it may not assume that a step holds the whole request."""

    # True if forward takes its input ``x`` either as a tensor or as the object that ``Norm.lazy`` returns
    # (which it hands to ``ops.gemm`` unchanged, or turns into a tensor with ``materialize()``).
    accepts_lazy_norm = False
    # True if forward only launches work on the current stream from device-resident metadata (no host
    # loops over requests, no synchronisation, no read of ``ctx.seqs``), so that a step can be recorded into
    # a CUDA graph.  One part that says False switches graphs off for the whole model.
    graph_safe = False

    def cache_need(self):
        """PagedKV, FixedState or None."""
        return None

    def forward(self, x: torch.Tensor, h: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache],
                owns_cache: bool) -> None:
        """h += mix(x).  ``owns_cache`` False: read ``cache`` but do not write it."""
        raise NotImplementedError


class FeedForward(Part):
    accepts_lazy_norm = False  # as for Mixer
    graph_safe = False  # as for Mixer

    def forward(self, x: torch.Tensor, h: torch.Tensor, ctx: StepContext) -> None:
        """h += feed_forward(x)."""
        raise NotImplementedError


class Block(Part):
    graph_safe = False

    def cache_need(self):
        return None

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache], owns_cache: bool) -> None:
        raise NotImplementedError


def role_dtype(role: str, compute_dtype: torch.dtype, stored: torch.dtype) -> torch.dtype:
    """Device dtype of a tensor of ``role`` stored as ``stored`` when the engine computes in
    ``compute_dtype``: matrices and embeddings in the compute dtype; vectors in fp32 (an exact
    widening of bf16; a vector stored in 32-bit stays so); integer tables int32."""
    if role in ("matrix", "embedding"):
        return compute_dtype
    if role in ("bias", "norm", "vector"):
        return torch.float32
    if role == "int_table":
        return torch.int32
    raise ValueError(f"unknown tensor role '{role}'")


__all__ = [
    "PagedKV", "FixedState", "PagedMeta", "SeqInfo", "StepContext", "LayerCache", "Part", "Norm",
    "PositionEncoding", "Mixer", "FeedForward", "Block", "TensorSpec", "role_dtype",
]
