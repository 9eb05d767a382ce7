"""Python face of the CUDA kernels: one function per kernel, taking torch CUDA tensors.

Every function checks dtypes, contiguity and sizes, then launches on the current
CUDA stream through the C ABI of the compiled library.  Nothing here computes on
the CPU or falls back to a library: a tensor that is not on a CUDA device, or a
library that cannot be built or loaded, raises ``KernelError``.

The library keeps small tables (tensor maps it has made, shared-memory allowances, the text of the
last error) without locks: one thread at a time may call into it, which is how the engine drives it.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..errors import KernelError
from . import build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_c_int = ctypes.c_int
_c_float = ctypes.c_float
_c_void_p = ctypes.c_void_p


_VP, _I, _F, _LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
# Argument types of the launchers on the model's path: with these declared, plain Python ints and floats go straight
# to C (a pointer would otherwise be cut to 32 bits, and wrapping every argument in a ctypes object costs microseconds).
_SIGNATURES = {
    "ferris_gemm_tcgen05": [_VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _I, _I, _VP, _VP, _VP],
    "ferris_norm_gemm_tcgen05": [_VP, _VP, _F, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _I, _VP],
    "ferris_merge_gemm_tcgen05": [_VP, _I, _I, _I, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _VP],
    "ferris_qkv_rope_gemm_tcgen05": [_VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _VP],
    "ferris_rotary_angles": [_VP, _VP, _VP, _I, _I, _VP],
    "ferris_rmsnorm": [_VP, _VP, _VP, _VP, _I, _I, _I, _F, _VP],
    "ferris_rope_cache_write": [_VP, _I, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _VP],
    "ferris_prefill_attention": [_VP, _I, _VP, _I, _VP, _VP, _LL, _VP, _I, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _F, _I, _VP],
    "ferris_decode_attention_rope": [_VP, _I, _VP, _I, _VP, _VP, _LL, _VP, _I, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I,
                                     _F, _I, _VP, _I, _VP],
    "ferris_gemm_argmax_tcgen05": [_VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _VP, _VP],
    "ferris_gemm_skinny": [_VP, _I, _VP, _VP, _F, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _I, _VP],
    "ferris_gemm_skinny_takes": [_I, _I, _I, _I, _I],
    "ferris_embed_gather": [_VP, _I, _VP, _VP, _I, _I, _I, _VP, _VP],
}
_declared = False


def _lib():
    global _declared
    lib = build.load_library()
    if not _declared:
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = ctypes.c_int
        _declared = True
    return lib


def _dt(t: torch.Tensor, what: str) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]) -> _c_void_p:
    return _c_void_p(0 if t is None else t.data_ptr())


def _stream() -> _c_void_p:
    """The raw handle of torch's current stream on the current device."""
    return _c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _need(t: torch.Tensor, what: str, dtype=None, contiguous: bool = True) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{what} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, found {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


def _rows(t: torch.Tensor, what: str) -> tuple[int, int, int]:
    """(rows, cols, row stride) of a 2-D tensor whose rows are contiguous."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{what} must be a CUDA tensor (there is no CPU path)")
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{what} must be 2-D with contiguous rows, found shape {tuple(t.shape)} strides {t.stride()}")
    return t.shape[0], t.shape[1], t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


_launches = 0


def launch_count() -> int:
    """How many kernels this process has launched through this module."""
    return _launches


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    _launches += kernels
    if code != 0:
        msg = _lib().ferris_last_error().decode("utf-8", "replace")
        kind = "refused its arguments" if code < 0 else f"failed (CUDA error {code})"
        raise KernelError(f"{what} {kind}: {msg}")


def require_device() -> None:
    """Raise unless a CUDA device of compute capability 10.x is current and the library loads."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is available; this engine has no CPU path")
    arch = _lib().ferris_device_arch()
    if arch < 0:
        raise KernelError("cannot query the CUDA device: " + _lib().ferris_last_error().decode())
    if arch // 10 != 10:
        raise KernelError(f"the kernels are built for sm_100a; the current device is sm_{arch}")


# ------------------------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None):
    """out[t, :] = table[ids[t], :] as fp32.  ids int32 [T]; out fp32 [T, H]."""
    _need(table, "embedding table")
    _need(ids, "token ids", torch.int32)
    _need(out, "embedding output", torch.float32)
    T, H = out.shape
    if table.dim() != 2 or table.shape[1] != H or ids.numel() != T:
        raise KernelError(f"embed_gather: table {tuple(table.shape)}, ids {tuple(ids.shape)}, out {tuple(out.shape)}")
    _check(
        _lib().ferris_embed_gather(_ptr(table), _dt(table, "embedding table"), _ptr(ids), _ptr(out), _c_int(T),
                                   _c_int(H), _c_int(table.shape[0]), _ptr(status), _stream()),
        "embed_gather",
    )


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            row_index: Optional[torch.Tensor] = None):
    """out[i] = rmsnorm(x[row_index[i]] or x[i]) * weight.  x fp32 [T, H]; weight fp32 [H]."""
    _need(x, "rmsnorm input", torch.float32)
    _need(weight, "rmsnorm weight", torch.float32)
    _need(out, "rmsnorm output")
    rows, H = out.shape
    if x.shape[1] != H or weight.numel() != H:
        raise KernelError(f"rmsnorm: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if row_index is not None:
        _need(row_index, "rmsnorm row index", torch.int32)
        if row_index.numel() != rows:
            raise KernelError("rmsnorm: one row index per output row is needed")
    elif x.shape[0] != rows:
        raise KernelError("rmsnorm: input and output row counts differ")
    _check(
        _lib().ferris_rmsnorm(x.data_ptr(), weight.data_ptr(), None if row_index is None else row_index.data_ptr(),
                              out.data_ptr(), _dt(out, "rmsnorm output"), rows, H, eps, _stream()),
        "rmsnorm",
    )


def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
              accumulate: bool = False):
    """out[t, n] (+)= sum_k x[t, k] w[n, k] + bias[n] with fp32 FMAs on the CUDA cores."""
    M, K, ldx = _rows(x, "gemm input")
    N, K2, ldw = _rows(w, "gemm weight")
    M2, N2, ldo = _rows(out, "gemm output")
    if K != K2 or M != M2 or N != N2 or x.dtype != w.dtype:
        raise KernelError(f"gemm: x {tuple(x.shape)} {x.dtype}, w {tuple(w.shape)} {w.dtype}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32)
        if bias.numel() != N:
            raise KernelError("gemm: bias length differs from the output width")
    _check(
        _lib().ferris_gemm_simt(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _dt(x, "gemm input"), _dt(out, "gemm output"),
                                _c_int(M), _c_int(N), _c_int(K), _c_int(ldx), _c_int(ldw), _c_int(ldo),
                                _c_int(1 if accumulate else 0), _stream()),
        "gemm",
    )


# Scratch of the tensor-core GEMM's K split: fp32 partials and per-tile counters.  Buffers only ever grow, and
# outgrown ones are kept alive, because a captured CUDA graph may still point at them.
_gemm_buffers: dict = {}
_gemm_retired: list = []
_GEMM_COUNTERS = 8192


def _gemm_scratch(device, floats: int, counters: int):
    key = str(device)
    entry = _gemm_buffers.get(key)
    if entry is None or entry[0].numel() < floats or entry[1].numel() < counters:
        if entry is not None:
            _gemm_retired.append(entry)
        size = max(floats, 1 << 20, 0 if entry is None else entry[0].numel())
        entry = (torch.empty(size, dtype=torch.float32, device=device),
                 torch.zeros(max(counters, _GEMM_COUNTERS), dtype=torch.int32, device=device))
        _gemm_buffers[key] = entry
    return entry


def tensor_core_gemm_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    """bf16 operands with contiguous rows, K and the row strides multiples of 8, 16-byte aligned bases."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2:
        return False
    K = x.shape[1]
    ldx = x.stride(0) if x.shape[0] > 1 else max(x.stride(0), K)
    ldw = w.stride(0) if w.shape[0] > 1 else max(w.stride(0), K)
    return (K % 8 == 0 and ldx % 8 == 0 and ldw % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and (K <= 1 or (x.stride(1) == 1 and w.stride(1) == 1)))


_uses_clusters = None


def gemm_tcgen05(x, w, bias, out, mode: int, n_out: Optional[int] = None, up_row_offset: int = 0):
    """out = x w^T on the tcgen05 tensor cores.  mode 0: bf16 store (+bias); 1: fp32 store (+bias);
    2: fp32 out += ; 3: bf16 silu(x w[:N]^T) * (x w[up_row_offset:up_row_offset+N]^T)."""
    global _uses_clusters
    T, K, ldx = _rows(x, "gemm input")
    rows_w, K2, ldw = _rows(w, "gemm weight")
    T2, N, ldo = _rows(out, "gemm output")
    if n_out is not None and n_out != N:
        raise KernelError("gemm: output width differs from what was asked")
    want_dtype = torch.bfloat16 if mode in (0, 3) else torch.float32
    if K != K2 or T != T2 or out.dtype != want_dtype:
        raise KernelError(f"gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}, mode {mode}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32)
        if bias.numel() != N:
            raise KernelError("gemm: bias length differs from the output width")
    lib = _lib()
    if _uses_clusters is None:
        _uses_clusters = bool(lib.ferris_gemm_uses_clusters())
    scratch = cnt = None
    if not _uses_clusters:
        # K splits that add up through global memory need scratch and counters
        bt, splits, floats, counters = _c_int(), _c_int(), ctypes.c_longlong(), _c_int()
        lib.ferris_gemm_tcgen05_plan(_c_int(T), _c_int(N), _c_int(K), _c_int(2 if mode == 3 else 1), ctypes.byref(bt),
                                     ctypes.byref(splits), ctypes.byref(floats), ctypes.byref(counters))
        if splits.value > 1:
            scratch, cnt = _gemm_scratch(x.device, floats.value, counters.value)
    _check(
        lib.ferris_gemm_tcgen05(x.data_ptr(), w.data_ptr(), None if bias is None else bias.data_ptr(), out.data_ptr(),
                                mode, T, N, K, ldx, ldw, ldo, rows_w, up_row_offset,
                                None if scratch is None else scratch.data_ptr(), None if cnt is None else cnt.data_ptr(),
                                _stream()),
        "tensor-core gemm",
    )


def gemm_plan(tokens: int, outputs: int, k: int, accumulators: int = 1) -> tuple[int, int]:
    """How the short-step tcgen05 kernel would cut a product: (token tile, K splits)."""
    bt, splits, floats, counters = _c_int(), _c_int(), ctypes.c_longlong(), _c_int()
    _lib().ferris_gemm_tcgen05_plan(_c_int(tokens), _c_int(outputs), _c_int(k), _c_int(accumulators), ctypes.byref(bt),
                                    ctypes.byref(splits), ctypes.byref(floats), ctypes.byref(counters))
    return bt.value, splits.value


def gemm_argmax(x, w, out_token, out_prob, scratch):
    """out_token[t] = the lowest index among the greatest of (x w^T)[t, :], out_prob[t] = its softmax probability
    (may be None): the output head of rows that all take their greatest logit, on the tcgen05 tensor cores, without
    storing the logits.  At most 128 rows; ``scratch``: fp32, ``gemm_argmax_scratch_floats`` long."""
    T, K, ldx = _rows(x, "gemm input")
    N, K2, ldw = _rows(w, "gemm weight")
    if K != K2 or T > 128 or not tensor_core_gemm_takes(x, w):
        raise KernelError(f"product + argmax: x {tuple(x.shape)}, w {tuple(w.shape)} are not taken")
    _need(out_token, "tokens", torch.int32)
    if out_prob is not None:
        _need(out_prob, "probabilities", torch.float32)
    _need(scratch, "scratch", torch.float32)
    if out_token.numel() != T or (out_prob is not None and out_prob.numel() != T) \
            or scratch.numel() < gemm_argmax_scratch_floats(T, N):
        raise KernelError("product + argmax: one token (and probability) per row and enough scratch are needed")
    _check(
        _lib().ferris_gemm_argmax_tcgen05(x.data_ptr(), w.data_ptr(), out_token.data_ptr(),
                                          None if out_prob is None else out_prob.data_ptr(), T, N, K, ldx, ldw, N,
                                          scratch.data_ptr(), _stream()),
        "product + argmax",
    )


def gemm_argmax_scratch_floats(rows: int, outputs: int) -> int:
    return 4 * rows * ((outputs + 127) // 128)


GREEDY_HEAD_MAX_ROWS = 96


def greedy_head(y, w, out_token, out_prob, workspace):
    """The output head and greedy sampling of the rows ``y`` [n, H] in one: out_token int32 [n], out_prob fp32 [n].
    bf16 rows, at most 96: the product that stores no logits; anything else: logits into the workspace, then the
    sampling kernel's greedy rows.  The same tokens and probabilities either way (up to the rounding of the sums).
    (The product's epilogue reduces over the 128 outputs of a tile, which lie across the lanes of its warps, with
    three warp reductions a token.  With three of its CTAs to an SM that hides behind the weights' way in: measured
    inside the decode step of the 0.5B sizes against stored logits and the sampling kernel, ms a step at 17 / 24 / 48 /
    64 / 96 / 128 rows: 1.212 / 1.260 / 1.633 / 1.733 / 2.382 / 2.492 against 1.227 / 1.276 / 1.638 / 1.743 / 2.420 /
    2.487.)"""
    n, V = y.shape[0], w.shape[0]
    if n <= GREEDY_HEAD_MAX_ROWS and tensor_core_gemm_takes(y, w):
        scratch = workspace.get("argmax_tiles", (gemm_argmax_scratch_floats(n, V),), torch.float32)
        gemm_argmax(y, w, out_token, out_prob, scratch)
        return
    logits = workspace.get("logits", (n, V), torch.float32)
    gemm(y, w, None, logits)
    sample(logits, out_token, out_prob)


GEMM_PAIRS_NONE, GEMM_PAIRS_ALL, GEMM_PAIRS_SWIGLU = 0, 1, 2


def set_gemm_pairs(which=GEMM_PAIRS_SWIGLU) -> None:
    """Which products of long steps (more than 128 tokens) run on pairs of CTAs that share one 256-row MMA
    (cta_group::2): none, all, or the gate / up product only (the default, also of the library: see the
    measurements beside ferris_gemm_pair_enabled in csrc/gemm_tcgen05.cu).  True / False mean all / none."""
    _lib().ferris_set_gemm_pair(_c_int(int(which)))


def set_gemm_long_min(tokens: int = 0) -> None:
    """From how many tokens on a product runs the token-major kernel (never below 128); 0: the library's default."""
    _lib().ferris_set_gemm_long_min(_c_int(int(tokens)))


class LazyRMSNorm:
    """The RMSNorm of the residual rows ``h`` that has not been computed yet.  A matrix product that can form
    it on its way (``gemm`` / ``gemm_swiglu`` for short bf16 steps) takes it as its input and no norm kernel
    runs; everyone else calls ``materialize()`` and gets the normed rows, computed once."""

    def __init__(self, h: torch.Tensor, weight: torch.Tensor, eps: float, out_buffer: torch.Tensor):
        self.h, self.weight, self.eps, self._out, self._done = h, weight, float(eps), out_buffer, False

    @property
    def shape(self):
        return self._out.shape

    @property
    def dtype(self):
        return self._out.dtype

    def materialize(self) -> torch.Tensor:
        if not self._done:
            rmsnorm(self.h, self.weight, self.eps, self._out)
            self._done = True
        return self._out


def _norm_gemm_takes(x: "LazyRMSNorm", w: torch.Tensor, accs: int) -> bool:
    """Whether the short-step kernel can form the norm itself: bf16, at most 16 tokens, and a K split that
    leaves all of a CTA's slices resident at once."""
    T, K = x.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or T > 16 or K % 8 or x._done:
        return False
    if not (x.h.is_cuda and x.h.dtype == torch.float32 and x.h.is_contiguous() and x.h.data_ptr() % 16 == 0
            and x.weight.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0):
        return False
    return bool(_lib().ferris_gemm_tcgen05_builds_tokens(_c_int(T), _c_int(w.shape[0] // accs), _c_int(K), _c_int(accs)))


def norm_gemm_tcgen05(x: "LazyRMSNorm", w, bias, out, mode: int, up_row_offset: int = 0):
    """out = rmsnorm(h) w^T in one kernel (modes as gemm_tcgen05)."""
    T, K = x.shape
    rows_w, K2, ldw = _rows(w, "gemm weight")
    T2, N, ldo = _rows(out, "gemm output")
    want_dtype = torch.bfloat16 if mode in (0, 3) else torch.float32
    if K != K2 or T != T2 or out.dtype != want_dtype:
        raise KernelError(f"norm + gemm: h {tuple(x.h.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32)
    _check(
        _lib().ferris_norm_gemm_tcgen05(x.h.data_ptr(), x.weight.data_ptr(), x.eps, w.data_ptr(),
                                        None if bias is None else bias.data_ptr(), out.data_ptr(), mode, T, N, K, ldw,
                                        ldo, rows_w, up_row_offset, _stream()),
        "norm + gemm",
    )


class LazySplitMerge:
    """The attention rows of a single-token step whose key ranges (splits) have not been merged yet: the
    partial results lie in ``scratch``.  A matrix product that can merge them on its way (``gemm`` for short
    bf16 steps) takes this as its input and no merge kernel runs; everyone else calls ``materialize()``."""

    def __init__(self, scratch: torch.Tensor, out_buffer: torch.Tensor, num_heads: int, head_dim: int, splits: int):
        self.scratch, self._out, self._done = scratch, out_buffer, False
        self.num_heads, self.head_dim, self.splits = int(num_heads), int(head_dim), int(splits)

    @property
    def shape(self):
        return self._out.shape

    @property
    def dtype(self):
        return self._out.dtype

    def materialize(self) -> torch.Tensor:
        if not self._done:
            T, _, ldo = _rows(self._out, "attention output")
            _check(_lib().ferris_decode_merge(_ptr(self.scratch), _ptr(self._out), _c_int(ldo), _c_int(T),
                                              _c_int(self.num_heads), _c_int(self.head_dim), _c_int(self.splits), _stream()),
                   "decode merge")
            self._done = True
        return self._out


def _merge_gemm_takes(x: "LazySplitMerge", w: torch.Tensor) -> bool:
    """Whether the short-step kernel can merge the key ranges itself (the limits of the fused norm)."""
    T, K = x.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or T > 16 or x._done or w.shape[1] != K:
        return False
    if not (w.data_ptr() % 16 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0 and x.scratch.data_ptr() % 16 == 0):
        return False
    return bool(_lib().ferris_gemm_tcgen05_builds_tokens(_c_int(T), _c_int(w.shape[0]), _c_int(K), _c_int(1)))


def merge_gemm_tcgen05(x: "LazySplitMerge", w, bias, out, mode: int):
    """out (+)= merge(partial attention results) w^T in one kernel (modes 0-2 as gemm_tcgen05)."""
    T, K = x.shape
    rows_w, K2, ldw = _rows(w, "gemm weight")
    T2, N, ldo = _rows(out, "gemm output")
    want_dtype = torch.bfloat16 if mode == 0 else torch.float32
    if K != K2 or T != T2 or out.dtype != want_dtype or mode not in (0, 1, 2):
        raise KernelError(f"merge + gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32)
    _check(
        _lib().ferris_merge_gemm_tcgen05(_ptr(x.scratch), _c_int(x.num_heads), _c_int(x.head_dim), _c_int(x.splits),
                                         _ptr(w), _ptr(bias), _ptr(out), _c_int(mode), _c_int(T), _c_int(N), _c_int(ldw),
                                         _c_int(ldo), _c_int(rows_w), _stream()),
        "merge + gemm",
    )


def set_gemm_skinny(on: bool = True) -> None:
    """Steps of at most 16 tokens on the weight-stationary kernel of csrc/gemm_skinny.cu (True, the default, also
    of the library unless FERRIS_GEMM_SKINNY=0), or on the tcgen05 kernel with its K split over a cluster (False)."""
    _lib().ferris_set_gemm_skinny(_c_int(1 if on else 0))
    _skinny_shapes.clear()


_skinny_shapes: dict = {}


def gemm_skinny_enabled() -> bool:
    return bool(_lib().ferris_gemm_skinny_enabled())


def _skinny_takes(x, w, out, accs: int) -> bool:
    """Whether the skinny kernel takes this product: bf16, at most 16 tokens, K a multiple of 8, aligned rows, and a
    number of outputs that its plan covers (``x``: a tensor or a LazyRMSNorm that has not been computed)."""
    T, K = x.shape
    if T > 16 or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.dim() != 2 or w.shape[1] != K or K % 8:
        return False
    if w.stride(1) != 1 or w.stride(0) % 8 or w.data_ptr() % 16:
        return False
    if isinstance(x, LazyRMSNorm):
        if x._done or not (x.h.is_cuda and x.h.dtype == torch.float32 and x.h.is_contiguous() and x.h.data_ptr() % 16 == 0
                           and x.weight.data_ptr() % 16 == 0):
            return False
    elif not (x.dim() == 2 and x.is_cuda and x.stride(1) == 1 and (x.stride(0) % 8 == 0 or T == 1) and x.data_ptr() % 16 == 0):
        return False
    N = out.shape[1]
    formed = isinstance(x, LazyRMSNorm)  # rows that the kernel forms stand whole in shared memory; others may stream
    key = (T > 8, N, K, accs, formed)
    takes = _skinny_shapes.get(key)
    if takes is None:
        takes = bool(_lib().ferris_gemm_skinny_takes(T, N, K, accs, 0 if formed else 1))
        _skinny_shapes[key] = takes
    return takes


def gemm_skinny(x, w, bias, out, mode: int, up_row_offset: int = 0):
    """out (+)= x w^T (+ bias) for at most 16 tokens; ``x`` a bf16 tensor or a LazyRMSNorm (formed in the kernel).
    Modes as gemm_tcgen05."""
    T, K = x.shape
    rows_w, K2, ldw = _rows(w, "gemm weight")
    T2, N, ldo = _rows(out, "gemm output")
    want_dtype = torch.bfloat16 if mode in (0, 3) else torch.float32
    if K != K2 or T != T2 or out.dtype != want_dtype:
        raise KernelError(f"skinny gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}, mode {mode}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32)
        if bias.numel() != N:
            raise KernelError("gemm: bias length differs from the output width")
    lazy = isinstance(x, LazyRMSNorm)
    ldx = K if lazy else (x.stride(0) if T > 1 else max(x.stride(0), K))
    _check(
        _lib().ferris_gemm_skinny(None if lazy else x.data_ptr(), ldx, x.h.data_ptr() if lazy else None,
                                  x.weight.data_ptr() if lazy else None, x.eps if lazy else 0.0, w.data_ptr(),
                                  None if bias is None else bias.data_ptr(), out.data_ptr(), mode, T, N, K, ldw, ldo,
                                  rows_w, up_row_offset, _stream()),
        "skinny gemm",
    )


def _mode_of(out, accumulate: bool) -> int:
    return 2 if accumulate else (0 if out.dtype == torch.bfloat16 else 1)


def gemm(x, w, bias, out, accumulate: bool = False):
    """The matrix product of the model, out (+)= x w^T + bias: for bf16 operands the skinny kernel (at most 16
    tokens) or the tcgen05 kernels, the CUDA-core kernel for everything else (all of the 32-bit path).  ``x`` may
    be a LazyRMSNorm or a LazySplitMerge."""
    if isinstance(x, LazySplitMerge):
        if w.shape[0] == out.shape[1] and _merge_gemm_takes(x, w):
            merge_gemm_tcgen05(x, w, bias, out, 2 if accumulate else (0 if out.dtype == torch.bfloat16 else 1))
            return
        x = x.materialize()
    if w.shape[0] == out.shape[1] and x.shape[0] <= 16 and gemm_skinny_enabled() and _skinny_takes(x, w, out, 1):
        gemm_skinny(x, w, bias, out, _mode_of(out, accumulate))
        return
    if isinstance(x, LazyRMSNorm):
        if w.shape[0] == out.shape[1] and _norm_gemm_takes(x, w, 1):
            norm_gemm_tcgen05(x, w, bias, out, 2 if accumulate else (0 if out.dtype == torch.bfloat16 else 1))
            return
        x = x.materialize()
    if tensor_core_gemm_takes(x, w) and w.shape[0] == out.shape[1]:
        if accumulate:
            gemm_tcgen05(x, w, bias, out, 2)
        else:
            gemm_tcgen05(x, w, bias, out, 0 if out.dtype == torch.bfloat16 else 1)
        return
    gemm_simt(x, w, bias, out, accumulate)


def gemm_swiglu(x, gate_up_weight, out, workspace=None):
    """out [T, I] = silu(x Wg^T) * (x Wu^T) with gate_up_weight = [Wg; Wu] ([2I, K]).  bf16: one tensor-core
    kernel with two accumulators (the [T, 2I] intermediate never exists); otherwise a product and the SwiGLU kernel."""
    T, I = out.shape
    if gate_up_weight.shape[0] != 2 * I:
        raise KernelError(f"gemm_swiglu: weight {tuple(gate_up_weight.shape)} for {I} outputs")
    if T <= 16 and out.dtype == torch.bfloat16 and gemm_skinny_enabled() and _skinny_takes(x, gate_up_weight, out, 2):
        gemm_skinny(x, gate_up_weight, None, out, 3, up_row_offset=I)
        return
    if isinstance(x, LazyRMSNorm):
        if out.dtype == torch.bfloat16 and _norm_gemm_takes(x, gate_up_weight, 2):
            norm_gemm_tcgen05(x, gate_up_weight, None, out, 3, up_row_offset=I)
            return
        x = x.materialize()
    if tensor_core_gemm_takes(x, gate_up_weight) and out.dtype == torch.bfloat16:
        gemm_tcgen05(x, gate_up_weight, None, out, 3, up_row_offset=I)
        return
    if workspace is not None:
        gate_up = workspace.get("ffn_gate_up", (T, 2 * I), x.dtype)
    else:
        gate_up = torch.empty(T, 2 * I, dtype=x.dtype, device=x.device)
    gemm_simt(x, gate_up_weight, None, gate_up)
    swiglu(gate_up, out)


def swiglu(gate_up: torch.Tensor, out: torch.Tensor):
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _need(gate_up, "swiglu input")
    _need(out, "swiglu output", gate_up.dtype)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I):
        raise KernelError(f"swiglu: input {tuple(gate_up.shape)}, output {tuple(out.shape)}")
    _check(_lib().ferris_swiglu(_ptr(gate_up), _ptr(out), _dt(out, "swiglu"), _c_int(T), _c_int(I), _stream()), "swiglu")


def rotary_angles(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor):
    """out [T, len(inv_freq), 2] fp32 = (cos, sin)(float(position) * inv_freq), as the rotary kernels form them."""
    _need(positions, "positions", torch.int32)
    _need(inv_freq, "rotary frequencies", torch.float32)
    _need(out, "rotary angles", torch.float32)
    T, half = positions.numel(), inv_freq.numel()
    if out.numel() != 2 * T * half:
        raise KernelError(f"rotary_angles: output {tuple(out.shape)} for {T} positions x {half} frequencies")
    _check(_lib().ferris_rotary_angles(_ptr(positions), _ptr(inv_freq), _ptr(out), T, half, _stream()), "rotary angles")


QKV_ROPE_MIN_TOKENS = 128


def qkv_rope_gemm_takes(x, w, qkv, num_heads, num_kv_heads, head_dim, rotary_dim, k_cache) -> bool:
    """Whether ``qkv_rope_gemm`` takes this step: bf16 on the tensor cores, at least 128 tokens, heads of 64 or
    128 rotated whole."""
    return (isinstance(x, torch.Tensor) and qkv.shape[0] >= QKV_ROPE_MIN_TOKENS and head_dim in (64, 128)
            and rotary_dim == head_dim and qkv.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
            and w.shape[0] == (num_heads + 2 * num_kv_heads) * head_dim == qkv.shape[1]
            and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0 and tensor_core_gemm_takes(x, w))


def qkv_rope_gemm(x, w, bias, qkv, angles, slot_mapping, k_cache, v_cache, num_heads, num_kv_heads, head_dim):
    """The q/k/v product of a long step with rotation and cache write in its epilogue: ``qkv[:, :nh d]`` gets the
    rotated queries (its key and value columns are left as they were), the paged cache the rotated keys and
    the values at ``slot_mapping`` (None: nothing is stored, for a layer that reads another layer's cache).
    ``angles``: from ``rotary_angles`` for the step's positions."""
    T, K, ldx = _rows(x, "q/k/v input")
    rows_w, K2, ldw = _rows(w, "q/k/v weight")
    T2, N, ldo = _rows(qkv, "q/k/v output")
    _need(angles, "rotary angles", torch.float32)
    _need(k_cache, "key cache", torch.bfloat16)
    _need(v_cache, "value cache", torch.bfloat16)
    page_size = k_cache.shape[2]
    if (K != K2 or T != T2 or qkv.dtype != torch.bfloat16 or N != (num_heads + 2 * num_kv_heads) * head_dim
            or angles.numel() != T * head_dim or k_cache.dim() != 4
            or k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape):
        raise KernelError(f"qkv_rope_gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, qkv {tuple(qkv.shape)}, "
                          f"cache {tuple(k_cache.shape)}, angles {tuple(angles.shape)}")
    if bias is not None:
        _need(bias, "q/k/v bias", torch.float32)
        if bias.numel() != N:
            raise KernelError("qkv_rope_gemm: bias length differs from the output width")
    if slot_mapping is not None:
        _need(slot_mapping, "slot mapping", torch.int32)
        if slot_mapping.numel() != T:
            raise KernelError("qkv_rope_gemm: one cache slot per token is needed")
    _check(
        _lib().ferris_qkv_rope_gemm_tcgen05(x.data_ptr(), w.data_ptr(), None if bias is None else bias.data_ptr(),
                                            qkv.data_ptr(), T, K, ldx, ldw, ldo, rows_w, angles.data_ptr(),
                                            None if slot_mapping is None else slot_mapping.data_ptr(),
                                            k_cache.data_ptr(), v_cache.data_ptr(), num_heads, num_kv_heads, head_dim,
                                            page_size, _stream()),
        "q/k/v product with rotation",
    )


def rope_cache_write(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                     slot_mapping: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                     v_cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                     rotary_dim: int, page_size: int, write_kv: bool = True):
    """Rotate q and k of ``qkv`` [T, (nh + 2 nkv) d] by position; store k and v into the paged cache."""
    _need(qkv, "qkv")
    _need(positions, "positions", torch.int32)
    T = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim or positions.numel() != T:
        raise KernelError(f"rope_cache_write: qkv {tuple(qkv.shape)} for {num_heads}+2x{num_kv_heads} heads of {head_dim}")
    if rotary_dim > 0:
        _need(inv_freq, "rotary frequencies", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("rope_cache_write: one frequency per rotated pair is needed")
    if write_kv:
        _need(slot_mapping, "slot mapping", torch.int32)
        _need(k_cache, "key cache", qkv.dtype)
        _need(v_cache, "value cache", qkv.dtype)
        if slot_mapping.numel() != T or k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) \
                or v_cache.shape != k_cache.shape:
            raise KernelError(f"rope_cache_write: cache {tuple(k_cache.shape)} does not fit "
                              f"[pages, {num_kv_heads}, {page_size}, {head_dim}]")
    _check(
        _lib().ferris_rope_cache_write(_ptr(qkv), _dt(qkv, "qkv"), _ptr(positions), _ptr(inv_freq),
                                       _ptr(slot_mapping if write_kv else None), _ptr(k_cache if write_kv else None),
                                       _ptr(v_cache if write_kv else None), _c_int(T), _c_int(num_heads),
                                       _c_int(num_kv_heads), _c_int(head_dim), _c_int(rotary_dim), _c_int(page_size),
                                       _c_int(1 if write_kv else 0), _stream()),
        "rope_cache_write",
    )


def paged_attention_simt(qkv: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         block_tables: torch.Tensor, token_seq: torch.Tensor, positions: torch.Tensor,
                         num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float,
                         score_slopes: Optional[torch.Tensor] = None):
    """General attention over the paged cache; q is read from the first nh*d columns of ``qkv``.
    ``score_slopes`` (fp32 [num_heads]): the score of a query at position P and the key at position j gets
    slopes[head] * (j - P) added."""
    T, _, ldq = _rows(qkv, "attention queries")
    T2, width, ldo = _rows(out, "attention output")
    _need(k_cache, "key cache", qkv.dtype)
    _need(v_cache, "value cache", qkv.dtype)
    _need(block_tables, "block tables", torch.int32)
    _need(token_seq, "token-to-request map", torch.int32)
    _need(positions, "positions", torch.int32)
    if T != T2 or width != num_heads * head_dim or out.dtype != qkv.dtype or qkv.shape[1] < num_heads * head_dim:
        raise KernelError(f"attention: q {tuple(qkv.shape)}, out {tuple(out.shape)}")
    if k_cache.dim() != 4 or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim or block_tables.dim() != 2:
        raise KernelError(f"attention: cache {tuple(k_cache.shape)}, tables {tuple(block_tables.shape)}")
    if score_slopes is not None:
        _need(score_slopes, "score slopes", torch.float32)
        if score_slopes.numel() != num_heads:
            raise KernelError("attention: one score slope per query head is needed")
    _check(
        _lib().ferris_paged_attention_simt(_ptr(qkv), _c_int(ldq), _ptr(out), _c_int(ldo), _ptr(k_cache), _ptr(v_cache),
                                           _dt(qkv, "attention"), _ptr(block_tables), _c_int(block_tables.shape[1]),
                                           _ptr(token_seq), _ptr(positions), _c_int(T), _c_int(num_heads),
                                           _c_int(num_kv_heads), _c_int(head_dim), _c_int(k_cache.shape[2]),
                                           _c_int(window or 0), _c_float(scale), _ptr(score_slopes), _stream()),
        "paged attention",
    )


def kernel_status() -> int:
    """Reads and clears the device status word (synchronises).  0: no kernel gave up a bounded wait;
    otherwise (code << 16) | place."""
    return int(_lib().ferris_kernel_status())


def check_kernel_status() -> None:
    v = kernel_status()
    if v:
        raise KernelError(f"a kernel gave up a bounded wait (code {v >> 16}, place {v & 0xffff}); its results are wrong")


_sm_count = None


def sm_count() -> int:
    global _sm_count
    if _sm_count is None:
        _sm_count = max(1, _lib().ferris_sm_count())
    return _sm_count


def tensor_core_attention_takes(dtype, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the TMA + tensor-core attention kernels take this geometry (the general kernel takes the rest)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 16 == 0
            and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16)


def decode_splits(tokens: int, num_kv_heads: int, max_kv_len: int) -> int:
    """Into how many key ranges a single-token step is split, so that the GPU's SMs have work:
    one CTA per SM at most (each streams its keys through four per-warp pipelines and holds most of the
    SM's shared memory, so a CTA more than there are SMs would wait for a second round), and at least
    eight 16-key tiles per CTA."""
    base = max(1, tokens * num_kv_heads)
    want = max(1, sm_count() // base)
    most = max(1, (max_kv_len // 16) // 8)
    return max(1, min(want, most))


def decode_attention(qkv, out, k_cache, v_cache, block_tables, token_seq, positions, num_heads, num_kv_heads,
                     head_dim, window, scale, splits, scratch, rows: Optional[torch.Tensor] = None):
    """Split-KV attention for single tokens (bf16, head size 64 or 128): every row of the step, or the rows
    that ``rows`` (int32) names when the step also carries portions of prompts."""
    T, _, ldq = _rows(qkv, "attention queries")
    _, _, ldo = _rows(out, "attention output")
    n = T if rows is None else rows.numel()
    need = n * num_heads * splits * (head_dim + 2) if splits > 1 else 0
    if need and (scratch is None or scratch.numel() < need or scratch.dtype != torch.float32):
        raise KernelError(f"decode attention with {splits} splits needs {need} floats of scratch")
    common = (_ptr(qkv), _c_int(ldq), _ptr(out), _c_int(ldo), _ptr(k_cache), _ptr(v_cache),
              ctypes.c_longlong(k_cache.shape[0]), _ptr(block_tables), _c_int(block_tables.shape[1]), _ptr(token_seq),
              _ptr(positions))
    tail = (_c_int(num_heads), _c_int(num_kv_heads), _c_int(head_dim), _c_int(k_cache.shape[2]), _c_int(window or 0),
            _c_float(scale), _c_int(splits), _ptr(scratch if need else None), _stream())
    kernels = 2 if splits > 1 else 1  # the attention kernel and the merge of its key ranges
    if rows is None:
        _check(_lib().ferris_decode_attention(*common, _c_int(T), *tail), "decode attention", kernels)
    else:
        _need(rows, "rows of the single tokens", torch.int32)
        _check(_lib().ferris_decode_attention_listed(*common, _ptr(rows), _c_int(rows.numel()), *tail), "decode attention",
               kernels)


def prefill_attention(qkv, out, k_cache, v_cache, block_tables, seq_q_start, seq_start_pos, num_seqs, max_q_len,
                      num_heads, num_kv_heads, head_dim, window, scale, skip_single: bool = False):
    """Tensor-core attention for portions of prompts (bf16, head size 64 or 128).  ``skip_single``: requests
    that bring one token are left out (the decode kernel takes them)."""
    _, _, ldq = _rows(qkv, "attention queries")
    _, _, ldo = _rows(out, "attention output")
    _check(
        _lib().ferris_prefill_attention(_ptr(qkv), _c_int(ldq), _ptr(out), _c_int(ldo), _ptr(k_cache), _ptr(v_cache),
                                        ctypes.c_longlong(k_cache.shape[0]), _ptr(block_tables),
                                        _c_int(block_tables.shape[1]), _ptr(seq_q_start), _ptr(seq_start_pos),
                                        _c_int(num_seqs), _c_int(max_q_len), _c_int(num_heads), _c_int(num_kv_heads),
                                        _c_int(head_dim), _c_int(k_cache.shape[2]), _c_int(window or 0), _c_float(scale),
                                        _c_int(1 if skip_single else 0), _stream()),
        "prefill attention",
    )


def set_prefill_tcgen05(on=True) -> None:
    """Portions of prompts on the tcgen05 attention kernel (True / 1, the default), on the mma.sync kernel it
    replaced (False / 0), or on the tcgen05 kernel with one softmax group at every head size (2)."""
    _lib().ferris_set_prefill_tcgen05(_c_int(int(on)))


def attention_step(qkv, out, k_cache, v_cache, meta, ctx, num_heads, num_kv_heads, head_dim, inv_freq, rotary_dim,
                   window, scale, write_kv: bool = True, lazy_merge: bool = False, rotated: bool = False,
                   score_slopes: Optional[torch.Tensor] = None):
    """Everything between the q/k/v product and the output product of an attention layer: rotate q and k by
    position, put k and v into the paged cache (``meta``: the step's block tables and slots for the cache's
    page group), attend.  A step of single tokens with whole-head rotation on the tensor-core path is ONE
    kernel (the split-KV kernel rotates and writes on its way); everything else is the rotary / cache-write
    kernel followed by ``paged_attention``.  Returns ``out``; with ``lazy_merge`` it may return a
    LazySplitMerge instead (``out`` not yet written), which ``gemm`` takes as its input.  ``rotated``: the
    q/k/v product has rotated and stored already (``qkv_rope_gemm``), only attention is left.
    ``score_slopes`` (fp32 [num_heads], of a position encoding that acts on the scores): slopes[head] * (j - P) is
    added to the score of the key at position j for the query at position P; the general kernel then attends."""
    T = qkv.shape[0]
    page_size = k_cache.shape[2]
    if rotated:
        paged_attention(qkv, out, k_cache, v_cache, meta.block_tables, ctx, num_heads, num_kv_heads, head_dim, window, scale,
                        score_slopes=score_slopes)
        return out
    if (ctx.max_q_len == 1 and rotary_dim == head_dim and inv_freq is not None and score_slopes is None
            and tensor_core_attention_takes(qkv.dtype, num_heads, num_kv_heads, head_dim, page_size)):
        _need(k_cache, "key cache", qkv.dtype)
        _need(v_cache, "value cache", qkv.dtype)
        _need(meta.block_tables, "block tables", torch.int32)
        _need(meta.slot_mapping, "slot mapping", torch.int32)
        _need(inv_freq, "rotary frequencies", torch.float32)
        if (k_cache.dim() != 4 or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim
                or v_cache.shape != k_cache.shape or qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim
                or out.shape != (T, num_heads * head_dim) or out.dtype != qkv.dtype
                or inv_freq.numel() != head_dim // 2 or meta.slot_mapping.numel() != T):
            raise KernelError(f"attention step: qkv {tuple(qkv.shape)}, cache {tuple(k_cache.shape)}, out {tuple(out.shape)}")
        kv_span = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        # Who merges the key ranges: with the skinny products the attention kernel itself (the ranges of a token and
        # kv head are a thread-block cluster that adds them through its shared memory); otherwise the output product
        # on its way (lazy_merge) or a merge kernel
        in_cluster = gemm_skinny_enabled()
        if in_cluster:
            splits = int(_lib().ferris_decode_cluster_splits(T, num_kv_heads, head_dim, kv_span))
            in_cluster = splits >= 1
        if not in_cluster:
            splits = decode_splits(T, num_kv_heads, kv_span)
        need = T * num_heads * splits * (head_dim + 2) if (splits > 1 and not in_cluster) else 0
        scratch = ctx.workspace.get("attn_split_scratch", (need,), torch.float32) if need else None
        leave = bool(lazy_merge and need)
        mode = 3 if in_cluster else (0 if leave else 1)
        _, _, ldq = _rows(qkv, "attention queries")
        _, _, ldo = _rows(out, "attention output")
        _check(
            _lib().ferris_decode_attention_rope(
                _ptr(qkv), _c_int(ldq), _ptr(out), _c_int(ldo), _ptr(k_cache), _ptr(v_cache),
                ctypes.c_longlong(k_cache.shape[0]), _ptr(meta.block_tables), _c_int(meta.block_tables.shape[1]),
                _ptr(ctx.token_seq), _ptr(ctx.positions), _ptr(inv_freq), _ptr(meta.slot_mapping if write_kv else None),
                _c_int(T), _c_int(num_heads), _c_int(num_kv_heads), _c_int(head_dim), _c_int(page_size),
                _c_int(window or 0), _c_float(scale), _c_int(splits), _ptr(scratch), _c_int(mode), _stream()),
            "decode attention with rotation", 2 if (splits > 1 and mode == 1) else 1,
        )
        return LazySplitMerge(scratch, out, num_heads, head_dim, splits) if leave else out
    rope_cache_write(qkv, ctx.positions, inv_freq, meta.slot_mapping, k_cache, v_cache, num_heads, num_kv_heads,
                     head_dim, rotary_dim, page_size, write_kv=write_kv)
    paged_attention(qkv, out, k_cache, v_cache, meta.block_tables, ctx, num_heads, num_kv_heads, head_dim, window, scale,
                    score_slopes=score_slopes)
    return out


def paged_attention(qkv, out, k_cache, v_cache, block_tables, ctx, num_heads, num_kv_heads, head_dim, window, scale,
                    score_slopes: Optional[torch.Tensor] = None):
    """Attention of the step's tokens over the paged cache (their own keys are in it already).
    ``ctx`` is the step context.  bf16 with head size 64 / 128 runs on the tensor cores: the split-KV
    kernel when every request brings one token, the prefill kernel otherwise; every other geometry, the
    32-bit path, and scores with slopes added (``score_slopes``) run the general kernel."""
    _need(k_cache, "key cache", qkv.dtype)
    _need(v_cache, "value cache", qkv.dtype)
    _need(block_tables, "block tables", torch.int32)
    if k_cache.dim() != 4 or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim \
            or v_cache.shape != k_cache.shape or block_tables.dim() != 2:
        raise KernelError(f"attention: cache {tuple(k_cache.shape)}, tables {tuple(block_tables.shape)}")
    if out.dtype != qkv.dtype or out.shape[1] != num_heads * head_dim or out.shape[0] != qkv.shape[0]:
        raise KernelError(f"attention: q {tuple(qkv.shape)}, out {tuple(out.shape)}")
    if score_slopes is not None or not tensor_core_attention_takes(qkv.dtype, num_heads, num_kv_heads, head_dim, k_cache.shape[2]):
        paged_attention_simt(qkv, out, k_cache, v_cache, block_tables, ctx.token_seq, ctx.positions, num_heads,
                             num_kv_heads, head_dim, window, scale, score_slopes=score_slopes)
        return
    T = qkv.shape[0]
    singles = getattr(ctx, "single_rows", None)
    if ctx.max_q_len == 1 or singles is not None:
        # single tokens: all rows of the step, or the listed ones beside portions of prompts
        n = T if ctx.max_q_len == 1 else singles.numel()
        kv_span = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        splits = decode_splits(n, num_kv_heads, kv_span)
        scratch = None
        if splits > 1:
            scratch = ctx.workspace.get("attn_split_scratch", (n * num_heads * splits * (head_dim + 2),), torch.float32)
        decode_attention(qkv, out, k_cache, v_cache, block_tables, ctx.token_seq, ctx.positions, num_heads,
                         num_kv_heads, head_dim, window, scale, splits, scratch,
                         rows=None if ctx.max_q_len == 1 else singles)
    if ctx.max_q_len > 1:
        prefill_attention(qkv, out, k_cache, v_cache, block_tables, ctx.seq_q_start, ctx.seq_start_pos, ctx.num_seqs,
                          ctx.max_q_len, num_heads, num_kv_heads, head_dim, window, scale,
                          skip_single=singles is not None)


def sample(logits: torch.Tensor, out_token: torch.Tensor, out_prob: Optional[torch.Tensor] = None,
           temperature: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None,
           top_p: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
           rng_states: Optional[torch.Tensor] = None):
    """One token per row of fp32 ``logits`` [n, V].  Without ``temperature``: argmax (lowest index on
    ties).  With it: per-row temperature, top_k (<= 0: whole vocabulary), top_p, and one draw from
    ``rng_states[slots[row]]`` (int64 xorshift64* states, advanced in place)."""
    n, V, ld = _rows(logits, "logits")
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    _need(out_token, "sampled tokens", torch.int32)
    if out_token.numel() != n:
        raise KernelError("sample: one output token per row is needed")
    if out_prob is not None:
        _need(out_prob, "sample probabilities", torch.float32)
    if temperature is not None:
        _need(temperature, "temperatures", torch.float32)
        _need(top_k, "top_k", torch.int32)
        _need(top_p, "top_p", torch.float32)
        _need(slots, "generator slots", torch.int32)
        _need(rng_states, "generator states", torch.int64)
        if not (temperature.numel() == top_k.numel() == top_p.numel() == slots.numel() == n):
            raise KernelError("sample: one temperature, top_k, top_p and slot per row is needed")
    _check(
        _lib().ferris_sample(_ptr(logits), _c_int(ld), _c_int(n), _c_int(V), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                             _ptr(slots), _ptr(rng_states), _ptr(out_token), _ptr(out_prob), _stream()),
        "sample",
    )
