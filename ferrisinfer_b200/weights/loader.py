"""From a model folder to a bound model: tensors by name, checked against what the parts ask for.

The reference walks a list of tensor plans (external name, expected shape, required flag) and
fails at the first missing tensor or wrong shape (crates/ferrisinfer-io/src/hf.rs:274-299); its
``inspect`` command reports all of them without loading (crates/ferrisinfer-io/src/hf.rs:66-118).
Here the list comes from the model's parts (``tensor_specs``), and ONE ``WeightLoadError`` lists
every missing tensor, every unexpected tensor and every wrong shape.

Dtypes on the device: matrices and embeddings in the engine's compute dtype (bfloat16 stays
bfloat16; float32 mode widens exactly); vectors (biases, norm weights) in fp32, which is an exact
widening of bf16 and leaves a tensor stored in 32-bit as it is; integer tables int32.
Nothing is transposed: the kernels take the folder's [out, in] layout.
"""

from __future__ import annotations

import os
from typing import Any, Optional

import torch

from ..config.registry import resolve_config
from ..errors import WeightLoadError
from ..parts.base import role_dtype
from ..parts.model import DecoderModel, build_model
from .safetensors_io import SafetensorsFolder

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          "f32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype must be bfloat16 or float32, found {dtype}")
        return dtype
    try:
        return DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"compute dtype must be bfloat16 or float32, found {dtype!r}") from None


def check_tensors(specs, found: dict, ignorable=(), where: str = "") -> None:
    """``found``: name -> shape of what the folder (or dict) holds.  Raises one WeightLoadError."""
    wanted = {s.name: s for s in specs}
    missing = [s.name for s in specs if s.required and s.name not in found]
    unexpected = [n for n in found if n not in wanted and n not in ignorable]
    wrong = [
        (n, wanted[n].shape, tuple(found[n])) for n in found if n in wanted and tuple(found[n]) != tuple(wanted[n].shape)
    ]
    if missing or unexpected or wrong:
        raise WeightLoadError(sorted(missing), sorted(unexpected), sorted(wrong), where)


def inspect_folder(folder: str) -> dict:
    """What the reference's ``inspect-hf`` reports (crates/ferrisinfer-cli/src/main.rs:503-589):
    architecture, sizes, and whether the folder's tensors fit, without loading any."""
    arch, cfg = resolve_config(folder)
    model = build_model(arch.plan(cfg))
    st = SafetensorsFolder(folder)
    specs = model.tensor_specs()
    found = {n: st.shape(n) for n in st.names()}
    report = {
        "architecture": arch.name,
        "config": cfg.to_dict(),
        "tensors_in_folder": len(found),
        "tensors_wanted": len([s for s in specs if s.required]),
        "stored_dtypes": sorted({str(st.dtype(n)).replace("torch.", "") for n in st.names()}),
        "parameters": sum(int(torch.Size(found[n]).numel()) for n in found),
        "problems": None,
    }
    try:
        check_tensors(specs, found, model.plan.extra.get("ignorable_tensors", ()), folder)
    except WeightLoadError as e:
        report["problems"] = {"missing": e.missing, "unexpected": e.unexpected,
                              "wrong_shape": [(n, list(a), list(b)) for n, a, b in e.wrong_shape]}
    st.close()
    return report


def bind_tensors(model: DecoderModel, tensors: dict, compute_dtype: torch.dtype, device) -> None:
    """Check ``tensors`` (name -> CPU or device tensor) against the model, move them to
    ``device`` in the dtype their role gives, and hand them to the parts."""
    specs = model.tensor_specs()
    check_tensors(specs, {n: tuple(t.shape) for n, t in tensors.items()},
                  model.plan.extra.get("ignorable_tensors", ()), "the given tensors")
    placed = {}
    for s in specs:
        if s.name in tensors:
            t = tensors[s.name]
            placed[s.name] = t.to(device=device, dtype=role_dtype(s.role, compute_dtype, t.dtype)).contiguous()
    model.bind(placed)


def load_model(folder: str, dtype="bfloat16", device="cuda") -> tuple:
    """(model, config) of ``folder`` (config.json + safetensors), bound to ``device``."""
    compute_dtype = parse_dtype(dtype)
    arch, cfg = resolve_config(folder)
    model = build_model(arch.plan(cfg))
    st = SafetensorsFolder(folder)
    try:
        specs = model.tensor_specs()
        check_tensors(specs, {n: st.shape(n) for n in st.names()},
                      model.plan.extra.get("ignorable_tensors", ()), folder)
        placed = {}
        for s in specs:
            if s.name in st.entries:
                t = st.read(s.name)
                placed[s.name] = t.to(device=device, dtype=role_dtype(s.role, compute_dtype, t.dtype)).contiguous()
        model.bind(placed)
    finally:
        st.close()
    return model, cfg
