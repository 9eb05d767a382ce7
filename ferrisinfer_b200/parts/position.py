"""Position encodings as parts.

``RotaryEncoding``: rotate-half rotary positions over the first ``rotary_dim``
dims of each head.  Frequencies as the reference forms them, a running product
in f32 (crates/ferrisinfer-kernel/src/cpu/attention.rs:1254-1276):
``step = theta ** (-2 / head_dim)``, ``inv_freq[0] = 1``,
``inv_freq[i + 1] = inv_freq[i] * step`` (the exponent uses head_dim, not
rotary_dim).  The angle ``float(pos) * inv_freq[i]`` and its sine and cosine
are fp32, formed in the kernel that also writes the cache.

``NoPosition``: nothing is encoded (the keys go to the cache as they are).
"""

from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .base import PositionEncoding
from .plan import register_part


def rotary_inverse_frequencies(head_dim: int, rotary_dim: int, theta: float) -> np.ndarray:
    step = np.float32(np.power(np.float32(theta), np.float32(-2.0) / np.float32(head_dim), dtype=np.float32))
    out = np.empty(rotary_dim // 2, dtype=np.float32)
    f = np.float32(1.0)
    for i in range(rotary_dim // 2):
        out[i] = f
        f = np.float32(f * step)
    return out


class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, head_dim: int, rotary_dim: int, theta: float):
        if rotary_dim % 2 or not (0 <= rotary_dim <= head_dim):
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        self.head_dim, self.rotary_dim, self.theta = int(head_dim), int(rotary_dim), float(theta)
        self._host = rotary_inverse_frequencies(self.head_dim, self.rotary_dim, self.theta)
        self._device = {}

    def rotary_table(self, device=None):
        if self.rotary_dim == 0:
            return None, 0
        device = torch.device(device if device is not None else "cuda")
        key = str(device)
        if key not in self._device:
            self._device[key] = torch.from_numpy(self._host.copy()).to(device)
        return self._device[key], self.rotary_dim

    def angles(self, ctx):
        """(cos, sin) of position x frequency for the tokens of the step, fp32 [T, rotary_dim / 2, 2]: computed by
        the first layer of a pass that asks, shared with the other layers of the same frequencies."""
        key = ("rotary_angles", self.head_dim, self.rotary_dim, self.theta)
        angles = ctx.shared.get(key)
        if angles is None:
            inv_freq, _ = self.rotary_table(ctx.positions.device)
            angles = ctx.workspace.get(f"rotary_angles_{len(ctx.shared)}", (ctx.positions.numel(), inv_freq.numel(), 2),
                                       torch.float32)
            ops.rotary_angles(ctx.positions, inv_freq, angles)
            ctx.shared[key] = angles
        return angles


class NoPosition(PositionEncoding):
    graph_safe = True

    def rotary_table(self, device=None):
        return None, 0


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoPosition)
