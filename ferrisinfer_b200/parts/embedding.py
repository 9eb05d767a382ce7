"""Token embedding and the output head as parts.

Embedding: h[t, :] = E[id_t, :], no scaling (crates/ferrisinfer-kernel/src/cpu/attention.rs:3-99).
Output head: logits[v] = sum_k y[k] W[v, k], no bias, only for the rows asked
(crates/ferrisinfer-runtime/src/reference.rs:145-149); tied = the embedding table is W
(crates/ferrisinfer-runtime/src/reference.rs:976-982).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part, TensorSpec
from .plan import register_part


class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight = None

    def tensor_specs(self, prefix):
        return [TensorSpec(f"{prefix}.weight", (self.vocab_size, self.hidden_size), "embedding")]

    def bind(self, tensors, prefix):
        self.weight = tensors[f"{prefix}.weight"]

    def forward(self, token_ids, h):
        ops.embed_gather(self.weight, token_ids, h)


class OutputHead(Part):
    """``tied_to``: tensor name of the embedding table to use as the output matrix, or None
    when the folder has a matrix of its own under ``prefix``."""

    def __init__(self, vocab_size: int, hidden_size: int, tied_to=None):
        self.vocab_size, self.hidden_size, self.tied_to = int(vocab_size), int(hidden_size), tied_to
        self.weight = None

    def tensor_specs(self, prefix):
        if self.tied_to:
            return []
        return [TensorSpec(f"{prefix}.weight", (self.vocab_size, self.hidden_size), "matrix")]

    def bind(self, tensors, prefix):
        self.weight = tensors[self.tied_to if self.tied_to else f"{prefix}.weight"]

    def forward(self, y, logits):
        """logits fp32 [n, V] = y [n, H] W^T."""
        ops.gemm(y, self.weight, None, logits)

    def forward_greedy(self, y, tokens, probs, workspace):
        """tokens int32 [n] = the index of each row's greatest logit (the lowest among equals), probs fp32 [n] its
        softmax probability; the logits themselves are stored nowhere where a kernel can avoid it (the reference's
        fused product + argmax: crates/ferrisinfer-kernel/src/cpu/matmul.rs:190-274)."""
        ops.greedy_head(y, self.weight, tokens, probs, workspace)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("output", "linear_head", OutputHead)
