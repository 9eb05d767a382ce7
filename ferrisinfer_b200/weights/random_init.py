"""Random weights from a configuration and a seed, as tensors or as a model folder.

The reference has no such mode (its tests write weight maps by hand:
crates/ferrisinfer-runtime/src/reference.rs:1715-1837).  Each tensor is drawn from a
generator seeded by (seed, tensor name), so a tensor does not depend on which others exist:
matrices, embeddings and biases N(0, 0.02); norm weights 1 + N(0, 0.02); integer tables zero.
``write_model_folder`` writes config.json and model.safetensors, which the loader then reads
like any other folder.
"""

from __future__ import annotations

import hashlib
import json
import os

import torch

from ..config.registry import resolve_config
from ..parts.model import build_model
from .loader import parse_dtype
from .safetensors_io import write_safetensors

INIT_STD = 0.02


def _generator(seed: int, name: str, device="cpu") -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensor(spec, seed: int, store_dtype: torch.dtype, device="cpu"):
    if spec.role == "int_table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    g = _generator(seed, spec.name, device)
    t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device) * INIT_STD
    if spec.role == "norm":
        t = t + 1.0
    return t.to(store_dtype)


def random_tensors(config, seed: int, store_dtype="bfloat16", optional: bool = True, device="cpu") -> dict:
    """name -> tensor for every tensor the architecture's parts ask for (optional ones, such as the
    q/k/v biases, included unless ``optional`` is False).  Drawn on ``device``: the CPU stream is the
    one that model folders are written from; a CUDA device draws other values, faster."""
    arch, cfg = resolve_config(config)
    store = parse_dtype(store_dtype)
    model = build_model(arch.plan(cfg))
    out = {}
    for spec in model.tensor_specs():
        if spec.required or optional:
            out[spec.name] = random_tensor(spec, seed, store, device)
    return out


def write_model_folder(config, seed: int, folder: str, store_dtype="bfloat16", optional: bool = True) -> str:
    """Write ``folder``/config.json and ``folder``/model.safetensors; returns ``folder``."""
    arch, cfg = resolve_config(config)
    os.makedirs(folder, exist_ok=True)
    d = cfg.to_dict()
    d["torch_dtype"] = "bfloat16" if parse_dtype(store_dtype) == torch.bfloat16 else "float32"
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(d, f, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"), random_tensors(cfg, seed, store_dtype, optional))
    return folder
