"""Timeline of a step as it runs on the GPU, from hooks inside the kernels.

The hooks exist only in a library built with ``FERRIS_NVCC_FLAGS=-DFERRIS_TIMELINE`` (set in the
environment before the first kernel call; the build gets a name of its own).  Every instrumented
kernel then records, per launch, the earliest entry of one of its CTAs, the earliest moment a CTA
passed its programmatic-launch wait (from there on it may read what the kernel before it wrote) and
the latest end of a CTA, in nanoseconds of the GPU's global timer; one chosen thread of the grid
also leaves marks at the kernel's phases.  The hooks cost a microsecond or two per launch, so the
numbers are for comparing phases and kernels with one another, not for reporting throughput.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import torch

from ..errors import KernelError
from . import ops

WORDS = 16  # per slot: kernel id, CTAs, entry, start, end, CTAs done, ten marks
UNITS = ("elementwise", "gemm_tcgen05", "gemm_skinny", "attention_mma", "sampling")
KERNELS = {
    1: "embedding", 2: "rmsnorm", 3: "rotary + cache write", 4: "decode attention", 5: "greedy sampling",
    6: "rmsnorm (warp per row)", 7: "prefill attention (mma.sync)", 8: "prefill attention (tcgen05)",
    9: "rotary angles", 26: "long q/k/v gemm + rotary + cache write",
    22: "long gemm -> bf16", 23: "long gemm -> fp32", 24: "long gemm += fp32", 25: "long gemm swiglu",
    30: "pair gemm -> bf16", 31: "pair gemm -> fp32", 32: "pair gemm += fp32", 33: "pair gemm swiglu",
    10: "gemm -> bf16", 11: "gemm -> fp32", 12: "gemm += fp32", 13: "gemm swiglu",
    14: "norm + gemm -> bf16", 15: "norm + gemm -> fp32", 16: "norm + gemm += fp32", 17: "norm + gemm swiglu",
    40: "skinny gemm -> bf16", 41: "skinny gemm -> fp32", 42: "skinny gemm += fp32", 43: "skinny gemm swiglu",
    44: "skinny norm + gemm -> bf16", 45: "skinny norm + gemm -> fp32", 46: "skinny norm + gemm += fp32",
    47: "skinny norm + gemm swiglu",
    21: "gemm + argmax", 27: "argmax merge",
    18: "merge + gemm -> bf16", 19: "merge + gemm -> fp32", 20: "merge + gemm += fp32",
}


@dataclass
class Launch:
    kernel: str
    ctas: int
    entry_us: float  # all times in microseconds after the first launch's start
    start_us: float
    end_us: float
    marks_us: list = field(default_factory=list)  # after the marking thread's own wait; None where not set


class StepTimeline:
    def __init__(self, device, capacity: int = 4096):
        lib = ops._lib()
        if not hasattr(lib, "ferris_timeline_install_" + UNITS[0]):
            raise KernelError("the kernel library has no timeline hooks: set FERRIS_NVCC_FLAGS=-DFERRIS_TIMELINE "
                              "before the first kernel call")
        self.capacity = capacity
        self.buf = torch.zeros(2 + WORDS * capacity, dtype=torch.int64, device=device)
        for unit in UNITS:
            code = getattr(lib, "ferris_timeline_install_" + unit)(ctypes.c_void_p(self.buf.data_ptr()))
            if code != 0:
                raise KernelError(f"timeline: installing the buffer in {unit} failed (CUDA error {code})")
        self.reset()

    def reset(self) -> None:
        torch.cuda.synchronize(self.buf.device)
        self.buf.zero_()
        self.buf[1] = self.capacity
        slots = self.buf[2:].view(self.capacity, WORDS)
        slots[:, 2] = -1  # entry and start are minima: begin with all ones
        slots[:, 3] = -1
        torch.cuda.synchronize(self.buf.device)

    def read(self) -> list:
        torch.cuda.synchronize(self.buf.device)
        n = int(self.buf[0].item())
        rows = self.buf[2:2 + WORDS * n].view(n, WORDS).cpu().tolist()
        if not rows:
            return []
        t0 = rows[0][3]
        out = []
        for kid, ctas, entry, start, end, _done, *marks in rows:
            own = marks[9]
            out.append(Launch(KERNELS.get(kid, f"kernel {kid}"), ctas, (entry - t0) / 1e3, (start - t0) / 1e3,
                              (end - t0) / 1e3, [(m - own) / 1e3 if (m and own) else None for m in marks[:9]]))
        return out


def summarize(launches: list) -> str:
    """A table by kernel: launches, time between start and end, time from the end of the launch before to the
    start, time between entry and start (what the kernel could do before its wait), per launch."""
    by = {}
    prev_end = None
    for l in launches:
        d = by.setdefault(l.kernel, [0, 0.0, 0.0, 0.0])
        d[0] += 1
        d[1] += l.end_us - l.start_us
        d[2] += (l.start_us - prev_end) if prev_end is not None else 0.0
        d[3] += l.start_us - l.entry_us
        prev_end = l.end_us
    lines = [f"{'kernel':26s} {'launches':>8s} {'run us':>8s} {'gap us':>8s} {'early us':>8s}   (per launch)"]
    for name, (n, run, gap, early) in by.items():
        lines.append(f"{name:26s} {n:8d} {run / n:8.2f} {gap / n:8.2f} {early / n:8.2f}")
    lines.append(f"span {launches[-1].end_us - launches[0].start_us:.1f} us over {len(launches)} launches")
    return "\n".join(lines)
