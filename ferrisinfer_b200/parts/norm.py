"""RMSNorm as a part: sizes and eps are parameters; statistics are fp32.

  ms = sum(x^2) / H;  r = 1 / sqrt(ms + eps);  y_j = (x_j * r) * w_j
(crates/ferrisinfer-kernel/src/cpu/reduction.rs:35-41).
"""

from __future__ import annotations

from ..kernels import ops
from .base import Norm, TensorSpec
from .plan import register_part


class RMSNorm(Norm):
    def __init__(self, hidden_size: int, eps: float):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.weight = None

    def tensor_specs(self, prefix):
        return [TensorSpec(f"{prefix}.weight", (self.hidden_size,), "norm")]

    def bind(self, tensors, prefix):
        self.weight = tensors[f"{prefix}.weight"]

    def forward(self, h, out, row_index=None):
        ops.rmsnorm(h, self.weight, self.eps, out, row_index)

    def lazy(self, h, out):
        return ops.LazyRMSNorm(h, self.weight, self.eps, out)


register_part("norm", "rmsnorm", RMSNorm)
