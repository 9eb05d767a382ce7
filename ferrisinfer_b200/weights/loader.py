"""From a model folder to a bound model: tensors by name, checked against what the parts ask for.

The reference walks a list of tensor plans (external name, expected shape, required flag) and
fails at the first missing tensor or wrong shape (crates/ferrisinfer-io/src/hf.rs:274-299); its
``inspect`` command reports all of them without loading (crates/ferrisinfer-io/src/hf.rs:66-118).
Here the list comes from the model's parts (``tensor_specs``), and ONE ``WeightLoadError`` lists
every missing tensor, every unexpected tensor and every wrong shape.

A folder is read straight from the files' mappings into a ring of pinned staging buffers by a few threads
(the reference loads its tensor plans on ``available_parallelism`` threads with a file handle each:
crates/ferrisinfer-io/src/hf.rs:224-272), and each filled buffer goes to the device with an asynchronous
copy on a stream of its own while the threads page in what comes next; the change of dtype, where there is
one, happens on the device.

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


def check_tensors(specs, found: dict, ignorable=(), where: str = "", strict: bool = True) -> list:
    """``found``: name -> shape of what the folder (or dict) holds.  Raises ONE WeightLoadError that lists every
    missing tensor, every unexpected tensor and every wrong shape.  ``strict`` False: tensors that the model
    does not ask for are no error; their names are returned (the reference never looks at them:
    crates/ferrisinfer-io/src/hf.rs:274-299 reads by plan)."""
    wanted = {s.name: s for s in specs}
    missing = [s.name for s in specs if s.required and s.name not in found]
    unexpected = [n for n in found if n not in wanted and n not in ignorable]
    wrong = [
        (n, wanted[n].shape, tuple(found[n])) for n in found if n in wanted and tuple(found[n]) != tuple(wanted[n].shape)
    ]
    if missing or wrong or (unexpected and strict):
        raise WeightLoadError(sorted(missing), sorted(unexpected), sorted(wrong), where)
    return sorted(unexpected)


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


STAGING_BYTES = 64 << 20  # one pinned staging buffer
STAGING_BUFFERS = 4
READER_THREADS = 4


def _to_device_pipelined(st: SafetensorsFolder, names: list, device: torch.device) -> dict:
    """name -> device tensor in the STORED dtype.  Reader threads copy pieces of at most STAGING_BYTES from the
    files' mappings into pinned buffers; this thread sends each filled buffer on with an asynchronous copy on a
    side stream and hands the buffer back once that copy has finished."""
    import queue
    from concurrent.futures import ThreadPoolExecutor

    import numpy as np

    out, jobs = {}, []
    for name in names:
        e = st.entries[name]
        t = torch.empty(e.shape, dtype=e.dtype, device=device)
        out[name] = t
        nbytes = e.end - e.begin
        flat = t.view(-1).view(torch.uint8) if nbytes else None
        for lo in range(0, nbytes, STAGING_BYTES):
            jobs.append((name, flat, lo, min(lo + STAGING_BYTES, nbytes)))
    if not jobs:
        return out
    most = max(hi - lo for _, _, lo, hi in jobs)
    free: queue.Queue = queue.Queue()
    for _ in range(STAGING_BUFFERS):
        free.put((torch.empty(most, dtype=torch.uint8).pin_memory(), torch.cuda.Event()))
    stream = torch.cuda.Stream(device)

    def fill(job):
        name, _flat, lo, hi = job
        buf, event = free.get()
        event.synchronize()  # the copy that last read this buffer is done
        np.copyto(buf.numpy()[:hi - lo], st.raw(name)[lo:hi])  # pages come in here, outside the interpreter lock
        return buf, event

    with ThreadPoolExecutor(max_workers=READER_THREADS) as pool:
        # no more jobs in flight than there are buffers, or the readers would wait on each other
        pending, nxt = [], 0
        while nxt < len(jobs) or pending:
            while nxt < len(jobs) and len(pending) < STAGING_BUFFERS:
                pending.append((jobs[nxt], pool.submit(fill, jobs[nxt])))
                nxt += 1
            (name, flat, lo, hi), fut = pending.pop(0)
            buf, event = fut.result()
            with torch.cuda.stream(stream):
                flat[lo:hi].copy_(buf[:hi - lo], non_blocking=True)
                event.record(stream)
            free.put((buf, event))
    stream.synchronize()
    return out


def load_model(folder: str, dtype="bfloat16", device="cuda", strict: bool = True) -> tuple:
    """(model, config) of ``folder`` (config.json + safetensors), bound to ``device``.
    ``strict`` False: tensors of the folder that no part asks for are left alone instead of being an error;
    their names are in ``model.unexpected_tensors``."""
    compute_dtype = parse_dtype(dtype)
    device = torch.device(device)
    arch, cfg = resolve_config(folder)
    model = build_model(arch.plan(cfg))
    st = SafetensorsFolder(folder)
    try:
        specs = model.tensor_specs()
        model.unexpected_tensors = check_tensors(specs, {n: st.shape(n) for n in st.names()},
                                                 model.plan.extra.get("ignorable_tensors", ()), folder, strict)
        wanted = [s for s in specs if s.name in st.entries]
        if device.type == "cuda":
            stored = _to_device_pipelined(st, [s.name for s in wanted], device)
        else:
            stored = {s.name: st.read(s.name).to(device) for s in wanted}
        placed = {}
        for s in wanted:
            t = stored.pop(s.name)
            placed[s.name] = t.to(dtype=role_dtype(s.role, compute_dtype, t.dtype)).contiguous()
        model.bind(placed)
    finally:
        st.close()
    return model, cfg
