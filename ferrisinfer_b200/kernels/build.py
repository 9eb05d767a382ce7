"""Compiles the CUDA sources under ``csrc/`` into one shared library for sm_100a and loads it.

The library is built with ``nvcc`` at the first call that needs it (seconds per
file; the sources include no PyTorch header) and kept beside the package in
``ferrisinfer_b200/_native/``; when that folder cannot be written, in a
per-user folder under the system's temporary directory.  The file name carries
a hash of the sources and flags, so an edited source never meets a stale binary.
While it compiles, a line goes to stderr for each file and every few seconds.

There is no fallback: if the library cannot be built or loaded, the caller gets
a ``KernelError`` that says why.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

from ..errors import KernelError

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(_PKG, "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
# more flags from the environment, e.g. FERRIS_NVCC_FLAGS=-DFERRIS_TIMELINE for the build with timeline hooks
NVCC_FLAGS += os.environ.get("FERRIS_NVCC_FLAGS", "").split()

_lock = threading.Lock()
_lib = None


def _sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _find_nvcc() -> str:
    for cand in (
        os.environ.get("FERRIS_NVCC"),
        os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
        shutil.which("nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelError("nvcc not found (looked at $FERRIS_NVCC, $CUDA_HOME/bin, PATH, /usr/local/cuda/bin)")


def _digest() -> str:
    h = hashlib.sha256()
    for name in _sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dirs() -> list[str]:
    dirs = [os.path.join(_PKG, "_native")]
    dirs.append(os.path.join(tempfile.gettempdir(), f"ferrisinfer_b200-{os.getuid()}", "_native"))
    return dirs


def _writable_dir() -> str:
    errors = []
    for d in _build_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe-{os.getpid()}")
            with open(probe, "w") as f:
                f.write("")
            os.unlink(probe)
            return d
        except OSError as e:
            errors.append(f"{d}: {e}")
    raise KernelError("no writable folder for the compiled kernels: " + "; ".join(errors))


def library_path(build: bool = True, verbose: bool = True) -> str:
    """Path of the compiled library, building it first if it is absent."""
    name = f"libferris_kernels-{_digest()}.so"
    for d in _build_dirs():
        p = os.path.join(d, name)
        if os.path.isfile(p):
            return p
    if not build:
        raise KernelError(f"the kernel library {name} has not been built")
    return _compile(os.path.join(_writable_dir(), name), verbose)


def _say(msg: str) -> None:
    print(f"[ferrisinfer_b200] {msg}", file=sys.stderr, flush=True)


def _compile(target: str, verbose: bool) -> str:
    nvcc = _find_nvcc()
    out_dir = os.path.dirname(target)
    work = tempfile.mkdtemp(prefix="build-", dir=out_dir)
    srcs = _sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA sources for sm_100a with {nvcc} (first use; takes a minute or two)")
    t0 = time.time()
    procs = []
    jobs = max(1, min(len(srcs), (os.cpu_count() or 2)))
    pending = list(srcs)
    objects = []
    failed = None
    last_note = time.time()
    try:
        while pending or procs:
            while pending and len(procs) < jobs:
                src = pending.pop(0)
                obj = os.path.join(work, src[:-3] + ".o")
                objects.append(obj)
                cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
                if verbose:
                    _say(f"  nvcc {src}")
                log = open(obj + ".log", "w+")
                procs.append((src, subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT), log))
            still = []
            for src, p, log in procs:
                if p.poll() is None:
                    still.append((src, p, log))
                    continue
                log.seek(0)
                out = log.read()
                log.close()
                if p.returncode != 0:
                    failed = f"nvcc failed on {src}:\n{out}"
                    pending.clear()
            procs = still
            if failed:
                for _, p, _log in procs:
                    p.kill()
                raise KernelError(failed)
            if procs:
                time.sleep(0.2)
                if verbose and time.time() - last_note > 10:
                    _say(f"  still compiling ({', '.join(s for s, _, _l in procs)}; {time.time() - t0:.0f} s)")
                    last_note = time.time()
        tmp_so = os.path.join(work, "lib.so")
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp_so, *objects]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise KernelError(f"linking the kernel library failed:\n{r.stdout}")
        os.replace(tmp_so, target)
        for old in os.listdir(out_dir):  # binaries of earlier source versions
            if old.startswith("libferris_kernels-") and old.endswith(".so") and old != os.path.basename(target):
                try:
                    os.unlink(os.path.join(out_dir, old))
                except OSError:
                    pass
    finally:
        shutil.rmtree(work, ignore_errors=True)
    if verbose:
        _say(f"built {os.path.basename(target)} in {time.time() - t0:.0f} s")
    return target


def load_library(verbose: bool = True) -> ctypes.CDLL:
    """The compiled kernels as a ctypes library (built on first use)."""
    global _lib
    with _lock:
        if _lib is None:
            path = library_path(build=True, verbose=verbose)
            try:
                _lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load {path}: {e}") from None
            _lib.ferris_last_error.restype = ctypes.c_char_p
        return _lib
