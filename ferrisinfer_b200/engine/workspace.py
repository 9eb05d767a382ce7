"""Named activation buffers that live across steps.

The reference keeps its scratch tensors in per-session workspaces sized for one token or one
chunk (crates/ferrisinfer-runtime/src/reference.rs:16-106).  Here a part asks for a buffer by name
and shape; the storage behind a name grows to the largest size ever asked and is reused, so a
steady state allocates nothing.

A recorded CUDA graph replays the addresses it was recorded with.  Once a step has been recorded
(``pin()``), a buffer that has to grow is REPLACED, never freed: the old storage stays alive, at its
address, for the graphs that name it, and steps that run after the growth (recorded or not) use the
new one.  ``unpin()`` lets the replaced buffers go when no recorded step is left.
"""

from __future__ import annotations

import torch


class Workspace:
    def __init__(self, device):
        self.device = torch.device(device)
        self._buffers: dict = {}
        self._replaced: list = []  # outgrown buffers that recorded steps may still point at
        self._pinned = False

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        count = 1
        for s in shape:
            count *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < count:
            if buf is not None and self._pinned:
                self._replaced.append(buf)
            buf = torch.empty(max(count, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:count].view(*shape)

    def reserve(self, name: str, shape, dtype: torch.dtype) -> None:
        self.get(name, shape, dtype)

    def pin(self) -> None:
        """From now on the address of every buffer handed out stays valid."""
        self._pinned = True

    def unpin(self) -> None:
        """No recorded step names a buffer any more: outgrown ones may go."""
        self._pinned = False
        self._replaced.clear()

    @property
    def replaced_buffers(self) -> int:
        return len(self._replaced)

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values()) + sum(
            b.numel() * b.element_size() for b in self._replaced)
