"""Reading and writing the safetensors container.

Format (crates/ferrisinfer-io/src/safetensors.rs:242-293): 8 bytes little-endian
header length, a JSON header ``{name: {dtype, shape, data_offsets}}`` (the
``__metadata__`` entry is skipped), then the raw little-endian data.  A model
folder holds either one ``model.safetensors`` or a
``model.safetensors.index.json`` whose ``weight_map`` names the shard of each
tensor (crates/ferrisinfer-io/src/safetensors.rs:97-164).

The checks follow the reference's (truncated header, header that is not UTF-8
JSON, missing dtype / shape / offsets, end < start, byte length that does not
equal dtype size x shape, data beyond the end of the file:
crates/ferrisinfer-io/src/safetensors.rs:254-389).  Unlike the reference,
nothing is converted to f32 or transposed here: a tensor comes back in the
dtype and layout it is stored in.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass

import torch

from ..errors import WeightFileError

_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple
    file: str
    begin: int  # absolute byte offset in the file
    end: int


def _read_header(path: str) -> dict[str, TensorEntry]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise WeightFileError(f"{path}: truncated (no header length)")
        (n,) = struct.unpack("<Q", head)
        if 8 + n > size:
            raise WeightFileError(f"{path}: header length {n} runs beyond the end of the file")
        raw = f.read(n)
    try:
        header = json.loads(raw.decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise WeightFileError(f"{path}: header is not UTF-8 JSON ({e})") from None
    if not isinstance(header, dict):
        raise WeightFileError(f"{path}: header must be a JSON object")
    base = 8 + n
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        if not isinstance(meta, dict) or not {"dtype", "shape", "data_offsets"} <= set(meta):
            raise WeightFileError(f"{path}: tensor '{name}' lacks dtype, shape or data_offsets")
        if meta["dtype"] not in _DTYPES:
            raise WeightFileError(
                f"{path}: tensor '{name}' has dtype {meta['dtype']}, supported: {', '.join(_DTYPES)}"
            )
        dtype, item = _DTYPES[meta["dtype"]]
        shape = tuple(int(s) for s in meta["shape"])
        begin, end = (int(v) for v in meta["data_offsets"])
        if end < begin:
            raise WeightFileError(f"{path}: tensor '{name}' has data_offsets end < start")
        count = 1
        for s in shape:
            count *= s
        if end - begin != count * item:
            raise WeightFileError(
                f"{path}: tensor '{name}' holds {end - begin} bytes, "
                f"but {meta['dtype']} x {list(shape)} needs {count * item}"
            )
        if base + end > size:
            raise WeightFileError(f"{path}: tensor '{name}' runs beyond the end of the file")
        out[name] = TensorEntry(name, dtype, shape, path, base + begin, base + end)
    return out


class SafetensorsFolder:
    """All tensors of a model folder, by name, read lazily through mmap."""

    def __init__(self, folder: str):
        self.folder = folder
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        self.entries: dict[str, TensorEntry] = {}
        if os.path.exists(index):
            with open(index, "r", encoding="utf-8") as f:
                try:
                    weight_map = json.load(f)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError) as e:
                    raise WeightFileError(f"{index}: no usable weight_map ({e})") from None
            shards: dict[str, dict[str, TensorEntry]] = {}
            for name, shard in weight_map.items():
                path = os.path.join(folder, shard)
                if shard not in shards:
                    if not os.path.exists(path):
                        raise WeightFileError(f"{index} names shard '{shard}', which is absent")
                    shards[shard] = _read_header(path)
                if name not in shards[shard]:
                    raise WeightFileError(f"{index}: tensor '{name}' is not in shard '{shard}'")
                self.entries[name] = shards[shard][name]
        elif os.path.exists(single):
            self.entries = _read_header(single)
        else:
            raise WeightFileError(
                f"{folder}: neither model.safetensors nor model.safetensors.index.json found"
            )
        self._maps: dict[str, mmap.mmap] = {}

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple:
        return self.entries[name].shape

    def dtype(self, name: str) -> torch.dtype:
        return self.entries[name].dtype

    def _map_of(self, path: str) -> mmap.mmap:
        mm = self._maps.get(path)
        if mm is None:
            with open(path, "rb") as f:
                mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps[path] = mm
        return mm

    def raw(self, name: str):
        """The tensor's bytes as a read-only uint8 numpy array over the file's mapping: nothing is copied, pages
        come in as they are touched."""
        import numpy as np

        e = self.entries[name]
        return np.frombuffer(self._map_of(e.file), dtype=np.uint8, count=e.end - e.begin, offset=e.begin)

    def read(self, name: str) -> torch.Tensor:
        """The tensor as stored (a CPU tensor that owns its memory: one copy out of the mapping)."""
        e = self.entries[name]
        count = 1
        for s in e.shape:
            count *= s
        if count == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        flat = torch.from_numpy(self.raw(name).copy()).view(e.dtype)
        return flat.reshape(e.shape)

    def close(self) -> None:
        for mm in self._maps.values():
            try:
                mm.close()
            except BufferError:
                pass
        self._maps.clear()


def write_safetensors(path: str, tensors: dict[str, torch.Tensor]) -> None:
    """Write ``tensors`` (CPU, contiguous or not) as one safetensors file."""
    header = {}
    offset = 0
    order = sorted(tensors)
    blobs = []
    for name in order:
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightFileError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        header[name] = {
            "dtype": _NAMES[t.dtype],
            "shape": list(t.shape),
            "data_offsets": [offset, offset + len(raw)],
        }
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
