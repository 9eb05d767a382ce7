"""Named activation buffers that live across steps.

The reference keeps its scratch tensors in per-session workspaces sized for one token or one
chunk (crates/ferrisinfer-runtime/src/reference.rs:16-106).  Here a part asks for a buffer by name
and shape; the storage behind a name grows to the largest size ever asked and is reused, so a
steady state allocates nothing and buffer addresses stay fixed (which CUDA-graph replay needs).
"""

from __future__ import annotations

import torch


class Workspace:
    def __init__(self, device):
        self.device = torch.device(device)
        self._buffers: dict = {}
        self.frozen = False

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        count = 1
        for s in shape:
            count *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < count:
            if self.frozen:
                raise RuntimeError(f"workspace buffer '{name}' would have to grow while its addresses are frozen")
            buf = torch.empty(max(count, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:count].view(*shape)

    def reserve(self, name: str, shape, dtype: torch.dtype) -> None:
        self.get(name, shape, dtype)

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())
