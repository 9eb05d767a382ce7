"""The gated SiLU feed-forward (SwiGLU) as a part.

  u = y W_up^T;  g = y W_gate^T;  m = u * (g * sigmoid(g));  h += m W_down^T
(crates/ferrisinfer-runtime/src/reference.rs:346-368; the reference's w1 is up_proj and w3 is
gate_proj: crates/ferrisinfer-io/src/hf.rs:437-457).  No bias.  Gate and up are held as one
[2I, H] matrix (gate rows first) so that one matrix product feeds the activation.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, TensorSpec
from .plan import register_part


class SwiGLU(FeedForward):
    accepts_lazy_norm = True  # x goes to ops.gemm_swiglu and nowhere else
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.gate_up = None
        self.down = None

    def tensor_specs(self, prefix):
        H, I = self.hidden_size, self.intermediate_size
        return [
            TensorSpec(f"{prefix}.gate_proj.weight", (I, H), "matrix"),
            TensorSpec(f"{prefix}.up_proj.weight", (I, H), "matrix"),
            TensorSpec(f"{prefix}.down_proj.weight", (H, I), "matrix"),
        ]

    def bind(self, tensors, prefix):
        self.gate_up = torch.cat(
            [tensors.pop(f"{prefix}.gate_proj.weight"), tensors.pop(f"{prefix}.up_proj.weight")], dim=0
        ).contiguous()
        self.down = tensors[f"{prefix}.down_proj.weight"]

    def forward(self, x, h, ctx):
        T, I = x.shape[0], self.intermediate_size
        act = ctx.workspace.get("ffn_act", (T, I), x.dtype)
        ops.gemm_swiglu(x, self.gate_up, act, ctx.workspace)
        ops.gemm(act, self.down, None, h, accumulate=True)


register_part("feed_forward", "swiglu", SwiGLU)
