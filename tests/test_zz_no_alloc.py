"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some embedders of the kernel library cannot hand it a scratch buffer because they cannot allocate device memory
where they call it (inside another framework's callback, or after all device memory was given out).  For them the
library has ``ferris_decode_attention_static_scratch``, which keeps the per-split partial results in an array built
into the library.  This test calls that symbol directly with raw device pointers, twice in a row with different
inputs (so what the first call left in the shared array is stale for the second), and compares each result bit for
bit with the regular entry point, which gets its scratch from the caller, and within rounding with the attention
formula itself.  It also checks that a request too large for the
built-in array is refused with a message instead of running.

The file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_FLOATS = 2 * 1024 * 1024


def _case(device, seed, nh, nkv, d, page, kv_lens):
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-kv // page) for kv in kv_lens]
    total = sum(blocks) + 2
    order = torch.randperm(total, generator=g)
    tables = torch.full((len(kv_lens), max(blocks)), -1, dtype=torch.int32)
    used = 0
    for s, nb in enumerate(blocks):
        tables[s, :nb] = order[used:used + nb].to(torch.int32)
        used += nb
    k = torch.randn(total, nkv, page, d, generator=g).to(torch.bfloat16).to(device)
    v = torch.randn(total, nkv, page, d, generator=g).to(torch.bfloat16).to(device)
    T = len(kv_lens)
    qkv = torch.randn(T, (nh + 2 * nkv) * d, generator=g).to(torch.bfloat16).to(device)
    token_seq = torch.arange(T, dtype=torch.int32, device=device)
    positions = torch.tensor([kv - 1 for kv in kv_lens], dtype=torch.int32, device=device)
    return qkv, k, v, tables.to(device), token_seq, positions


def _plain_attention(qkv, k, v, tables, positions, nh, nkv, d, window, scale):
    """One query per request at its last position, over the paged keys and values, in float64 on the CPU."""
    qkv, k, v, tables = qkv.cpu().double(), k.cpu().double(), v.cpu().double(), tables.cpu()
    page = k.shape[2]
    out = torch.empty(qkv.shape[0], nh * d, dtype=torch.float64)
    for t in range(qkv.shape[0]):
        P = int(positions[t])
        lo = max(0, P - window + 1) if window else 0
        keys = torch.arange(lo, P + 1)
        pages, offs = tables[t, keys // page].long(), keys % page
        for h in range(nh):
            hk = h // (nh // nkv)
            kk, vv = k[pages, hk, offs], v[pages, hk, offs]
            w = torch.softmax((kk @ qkv[t, h * d:(h + 1) * d]) * scale, dim=0)
            out[t, h * d:(h + 1) * d] = w @ vv
    return out.float()


def _call_static(lib, qkv, out, k, v, tables, token_seq, positions, nh, nkv, d, window, scale, splits):
    fn = lib.ferris_decode_attention_static_scratch
    fn.restype = ctypes.c_int
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    return fn(p(qkv), ctypes.c_int(qkv.stride(0)), p(out), ctypes.c_int(out.stride(0)), p(k), p(v),
              ctypes.c_longlong(k.shape[0]), p(tables), ctypes.c_int(tables.shape[1]), p(token_seq), p(positions),
              ctypes.c_int(qkv.shape[0]), ctypes.c_int(nh), ctypes.c_int(nkv), ctypes.c_int(d), ctypes.c_int(k.shape[2]),
              ctypes.c_int(window), ctypes.c_float(scale), ctypes.c_int(splits),
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_entry_point_matches_the_regular_one(device):
    from ferrisinfer_b200.kernels import build, ops

    lib = build.load_library()
    nh, nkv, d, page = 14, 2, 64, 16
    scale = 1.0 / math.sqrt(d)
    for call, (seed, kv_lens, splits, window) in enumerate([(1, [700, 33, 1500, 16], 6, 0), (2, [90, 1200, 257], 5, 300)]):
        qkv, k, v, tables, token_seq, positions = _case(device, seed, nh, nkv, d, page, kv_lens)
        T = qkv.shape[0]
        want = torch.empty(T, nh * d, dtype=torch.bfloat16, device=device)
        scratch = torch.empty(T * nh * splits * (d + 2), dtype=torch.float32, device=device)
        ops.decode_attention(qkv, want, k, v, tables, token_seq, positions, nh, nkv, d, window, scale, splits, scratch)
        got = torch.full_like(want, float("nan"))
        rc = _call_static(lib, qkv, got, k, v, tables, token_seq, positions, nh, nkv, d, window, scale, splits)
        assert rc == 0, lib.ferris_last_error().decode()
        torch.cuda.synchronize()
        assert ops.kernel_status() == 0
        assert torch.isfinite(got.float()).all()
        # the same kernel with the same key ranges: where the partial results lie changes no bit of the result
        assert torch.equal(got, want), f"call {call}"
        # and the result is the attention itself: softmax(q . k / sqrt(d)) v over the keys each query may see
        plain_out = _plain_attention(qkv, k, v, tables, positions, nh, nkv, d, window, scale)
        assert torch.allclose(got.float().cpu(), plain_out, atol=2e-2, rtol=2e-2), f"call {call}"


def test_static_scratch_entry_point_refuses_what_does_not_fit(device):
    from ferrisinfer_b200.kernels import build

    lib = build.load_library()
    nh, nkv, d, page = 32, 2, 128, 16
    qkv, k, v, tables, token_seq, positions = _case(device, 3, nh, nkv, d, page, [64] * 64)
    splits = 9
    assert 64 * nh * splits * (d + 2) > STATIC_SCRATCH_FLOATS
    out = torch.zeros(64, nh * d, dtype=torch.bfloat16, device=device)
    rc = _call_static(lib, qkv, out, k, v, tables, token_seq, positions, nh, nkv, d, 0, 0.1, splits)
    assert rc < 0
    message = lib.ferris_last_error().decode()
    assert "exceed the built-in scratch" in message and str(STATIC_SCRATCH_FLOATS) in message
    torch.cuda.synchronize()
    assert out.abs().sum().item() == 0, "nothing ran"
