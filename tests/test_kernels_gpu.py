"""Each kernel alone against a plain fp32 PyTorch reference of the same op, at sizes other than the engine's.

Where random data would hide a fault, the inputs are made so that it shows: one far key that must dominate,
keys just inside and just outside a window, pages in shuffled order, ragged shapes.
"""

import math

import numpy as np
import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16


def tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == F32 else dict(atol=2e-2, rtol=2e-2)


def rnd(shape, dtype, device, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(device)


# ------------------------------------------------------------------------------------ embedding
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_embed_gather(dtype, device):
    from ferrisinfer_b200.kernels import ops

    table = rnd((1000, 200), dtype, device, 1)
    ids = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32, device=device)
    out = torch.empty(5, 200, dtype=F32, device=device)
    ops.embed_gather(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())
    status = torch.zeros(1, dtype=torch.int32, device=device)
    bad = torch.tensor([3, 1000, 7], dtype=torch.int32, device=device)
    out = torch.empty(3, 200, dtype=F32, device=device)
    ops.embed_gather(table, bad, out, status)
    assert status.item() == 2 and out[1].abs().sum().item() == 0 and torch.equal(out[2], table[7].float())


# ------------------------------------------------------------------------------------- rmsnorm
@pytest.mark.parametrize("out_dtype", [F32, BF16])
@pytest.mark.parametrize("hidden, eps", [(1000, 1e-5), (3584, 1e-6), (48, 3e-3), (1538, 1e-6), (4100, 1e-5)])
@pytest.mark.parametrize("n", [37, 131])  # few rows: a block per row; many: a warp per row
def test_rmsnorm(n, hidden, eps, out_dtype, device):
    from ferrisinfer_b200.kernels import ops

    x = rnd((n, hidden), F32, device, 2, scale=3.0)
    w = 1 + rnd((hidden,), F32, device, 3, scale=0.1)
    want = plain.rms_norm(x.cpu().double(), w.cpu().double(), eps)
    out = torch.empty(n, hidden, dtype=out_dtype, device=device)
    ops.rmsnorm(x, w, eps, out)
    assert torch.allclose(out.cpu().double(), want, **tol(out_dtype))
    picks = [n - 1, 0, 0, 11] * (1 if n < 64 else 17)
    rows = torch.tensor(picks, dtype=torch.int32, device=device)
    out = torch.empty(len(picks), hidden, dtype=out_dtype, device=device)
    ops.rmsnorm(x, w, eps, out, rows)
    assert torch.allclose(out.cpu().double(), want[rows.cpu().long()], **tol(out_dtype))


# ---------------------------------------------------------------------------------------- gemm
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("M, N, K", [(1, 7, 33), (5, 130, 72), (67, 300, 1000), (64, 64, 16), (130, 65, 17)])
def test_gemm_simt(M, N, K, dtype, device):
    from ferrisinfer_b200.kernels import ops

    x, w = rnd((M, K), dtype, device, 4), rnd((N, K), dtype, device, 5, scale=0.1)
    bias = rnd((N,), F32, device, 6)
    want = x.cpu().double() @ w.cpu().double().t()
    out = torch.empty(M, N, dtype=dtype, device=device)
    ops.gemm_simt(x, w, None, out)
    assert torch.allclose(out.cpu().double(), want, **tol(dtype))
    out32 = torch.empty(M, N, dtype=F32, device=device)
    ops.gemm_simt(x, w, bias, out32)
    assert torch.allclose(out32.cpu().double(), want + bias.cpu().double(), atol=1e-4, rtol=1e-5)
    acc = rnd((M, N), F32, device, 7)
    before = acc.clone()
    ops.gemm_simt(x, w, None, acc, accumulate=True)
    assert torch.allclose(acc.cpu().double(), before.cpu().double() + want, atol=1e-4, rtol=1e-5)
    # rows of a wider buffer (a column slice) as input
    wide = rnd((M, K + 24), dtype, device, 8)
    out = torch.empty(M, N, dtype=dtype, device=device)
    ops.gemm_simt(wide[:, 8:8 + K], w, None, out)
    assert torch.allclose(out.cpu().double(), wide[:, 8:8 + K].cpu().double() @ w.cpu().double().t(), **tol(dtype))


def test_gemm_rows_do_not_depend_on_the_batch(device):
    from ferrisinfer_b200.kernels import ops

    x, w = rnd((70, 200), F32, device, 9), rnd((150, 200), F32, device, 10)
    full = torch.empty(70, 150, dtype=F32, device=device)
    ops.gemm_simt(x, w, None, full)
    one = torch.empty(1, 150, dtype=F32, device=device)
    ops.gemm_simt(x[41:42], w, None, one)
    assert torch.equal(one[0], full[41])


# ------------------------------------------------------------------------- tensor-core gemm
TC_SHAPES = [(1, 1152, 896), (8, 1152, 896), (64, 896, 4864), (5, 130, 72), (16, 128, 64), (17, 300, 1000),
             (300, 256, 128), (2048, 384, 256), (33, 1000, 80), (257, 129, 200),
             (8, 3584, 18944), (8, 4608, 3584),  # K splits whose clusters do not pack evenly into GPCs
             (32, 1536, 8960), (100, 1536, 1536),  # few tiles and a long K: clusters of more than 8 CTAs
             # long steps whose tiles are 224, 192 and 160 weight rows wide (one round of CTAs instead of two)
             (4096, 896, 256), (2048, 1536, 192), (1024, 3584, 128), (2048, 1200, 72)]


def test_few_tiles_with_a_long_k_are_split_beyond_the_portable_cluster_size(device):
    """The down projection of a step of 17 to 127 tokens: 7 tiles of 128 rows would leave most SMs idle with 8 K
    splits; where the GPU holds enough clusters of 16 CTAs at once the plan uses them (TC_SHAPES runs such shapes
    through every epilogue, twice for equality)."""
    from ferrisinfer_b200.kernels import ops

    ops.require_device()
    for T, N, K in [(64, 896, 4864), (32, 1536, 8960), (100, 1536, 1536)]:
        bt, splits = ops.gemm_plan(T, N, K)
        tiles = (N + 127) // 128
        assert bt == (T + 15) // 16 * 16 and 1 <= splits <= 16
        assert tiles * splits <= ops.sm_count()
        assert splits <= (K + 63) // 64 // 2, "at least two K slices a CTA"
    if ops.sm_count() >= 128:
        assert ops.gemm_plan(64, 896, 4864)[1] > 8
    # two accumulators (gate and up) keep to the portable size
    assert ops.gemm_plan(64, 256, 4864, 2)[1] <= 8


def _gemm_reference(x, w, bias=None):
    y = x.cpu().double() @ w.cpu().double().t()
    return y if bias is None else y + bias.cpu().double()


def _close(got, want, K, out_dtype):
    # fp32 accumulation of K bf16 products, then one rounding to the output type
    scale = want.abs().max().item() + 1e-6
    atol = scale * (2e-2 if out_dtype == BF16 else 2e-5 * math.sqrt(K) + 1e-5)
    err = (got.cpu().double() - want).abs().max().item()
    assert err <= atol, (err, atol)


@pytest.mark.parametrize("T, N, K", TC_SHAPES)
def test_gemm_tcgen05_store_and_accumulate(T, N, K, device):
    from ferrisinfer_b200.kernels import ops

    x, w = rnd((T, K), BF16, device, 21), rnd((N, K), BF16, device, 22, scale=0.1)
    bias = rnd((N,), F32, device, 23)
    assert ops.tensor_core_gemm_takes(x, w)
    want = _gemm_reference(x, w)
    out = torch.full((T, N), float("nan"), dtype=BF16, device=device)
    ops.gemm_tcgen05(x, w, bias, out, 0)
    _close(out, want + bias.cpu().double(), K, BF16)
    out32 = torch.full((T, N), float("nan"), dtype=F32, device=device)
    ops.gemm_tcgen05(x, w, None, out32, 1)
    _close(out32, want, K, F32)
    again = torch.empty_like(out32)
    ops.gemm_tcgen05(x, w, None, again, 1)
    assert torch.equal(again, out32), "the K split adds its partials in a fixed order"
    acc = rnd((T, N), F32, device, 24)
    before = acc.clone()
    ops.gemm_tcgen05(x, w, bias, acc, 2)
    _close(acc - before, want + bias.cpu().double(), K, F32)
    assert ops.kernel_status() == 0


@pytest.mark.parametrize("T, N, K", [(300, 896, 4864), (700, 896, 4864), (200, 1536, 8960), (513, 1152, 896), (260, 130, 1000),
                                     (1000, 384, 2048)])
def test_gemm_of_a_few_hundred_tokens_on_either_kernel(T, N, K, device):
    """Steps between 128 and about a thousand tokens run the token-major kernel or, where its few tiles would leave
    most SMs idle, the weight-major one with several token tiles and a K split over a cluster: both, and the
    library's own choice, against the plain product, in every mode."""
    from ferrisinfer_b200.kernels import ops

    x, w = rnd((T, K), BF16, device, 51), rnd((N, K), BF16, device, 52, scale=0.1)
    bias = rnd((N,), F32, device, 53)
    want = _gemm_reference(x, w)
    I = N // 2
    want_act = want[:, I:2 * I] * plain.silu(want[:, :I])
    base = rnd((T, N), F32, device, 54)
    try:
        for long_min in (128, 1 << 30, 0):
            ops.set_gemm_long_min(long_min)
            out = torch.full((T, N), float("nan"), dtype=BF16, device=device)
            ops.gemm_tcgen05(x, w, bias, out, 0)
            _close(out, want + bias.cpu().double(), K, BF16)
            out32 = torch.full((T, N), float("nan"), dtype=F32, device=device)
            ops.gemm_tcgen05(x, w, None, out32, 1)
            _close(out32, want, K, F32)
            again = torch.empty_like(out32)
            ops.gemm_tcgen05(x, w, None, again, 1)
            assert torch.equal(again, out32)
            acc = base.clone()
            ops.gemm_tcgen05(x, w, bias, acc, 2)
            _close(acc - base, want + bias.cpu().double(), K, F32)
            act = torch.full((T, I), float("nan"), dtype=BF16, device=device)
            ops.gemm_tcgen05(x, w, None, act, 3, up_row_offset=I)
            _close(act, want_act, K, BF16)
            assert ops.kernel_status() == 0
    finally:
        ops.set_gemm_long_min(0)


@pytest.mark.parametrize("T, I, K", [(1, 4864, 896), (8, 300, 96), (64, 4864, 896), (130, 128, 64), (700, 224, 96)])
def test_gemm_tcgen05_swiglu(T, I, K, device):
    from ferrisinfer_b200.kernels import ops

    x, w = rnd((T, K), BF16, device, 25), rnd((2 * I, K), BF16, device, 26, scale=0.2)
    out = torch.full((T, I), float("nan"), dtype=BF16, device=device)
    ops.gemm_swiglu(x, w, out)
    y = _gemm_reference(x, w)
    want = y[:, I:] * plain.silu(y[:, :I])
    _close(out, want, K, BF16)
    assert ops.kernel_status() == 0


@pytest.mark.parametrize("T, N, K, mode", [(300, 256, 128, 0), (2048, 384, 256, 2), (257, 129, 200, 1), (700, 448, 96, 3),
                                           (2048, 9728, 896, 3), (130, 256, 64, 3), (1000, 896, 4864, 2)])
def test_gemm_on_cta_pairs(T, N, K, mode, device):
    """Long steps on pairs of CTAs (one MMA of 256 rows over two SMs, each holding half of the weight rows): the same
    numbers as the kernel on single CTAs, and as the plain product."""
    from ferrisinfer_b200.kernels import ops

    x, w = rnd((T, K), BF16, device, 41), rnd((N, K), BF16, device, 42, scale=0.1)
    bias = rnd((N,), F32, device, 43) if mode in (0, 1) else None
    n_out = N // 2 if mode == 3 else N
    dtype = BF16 if mode in (0, 3) else F32
    base = rnd((T, n_out), F32, device, 44) if mode == 2 else None

    def run():
        out = base.clone() if mode == 2 else torch.full((T, n_out), float("nan"), dtype=dtype, device=device)
        ops.gemm_tcgen05(x, w, bias, out, mode, up_row_offset=n_out if mode == 3 else 0)
        torch.cuda.synchronize()
        assert ops.kernel_status() == 0
        return out

    ops.set_gemm_pairs(ops.GEMM_PAIRS_NONE)
    try:
        single = run()
        ops.set_gemm_pairs(ops.GEMM_PAIRS_ALL)
        paired = run()
    finally:
        ops.set_gemm_pairs()  # back to the default
    assert torch.equal(paired, single), (paired.float() - single.float()).abs().max()
    ref = _gemm_reference(x, w, bias)
    if mode == 3:
        ref = ref[:, n_out:] * plain.silu(ref[:, :n_out])
    if mode == 2:
        ref = ref + base.cpu().double()
    _close(paired, ref, K, dtype)


@pytest.fixture
def skinny_off():
    """The products of short steps on the tcgen05 kernel with its K split over a cluster, as before the skinny kernel."""
    from ferrisinfer_b200.kernels import ops

    ops.set_gemm_skinny(False)
    yield
    ops.set_gemm_skinny(True)


@pytest.mark.parametrize("skinny", [True, False], ids=["skinny", "tcgen05"])
@pytest.mark.parametrize("T", [1, 8, 16])
@pytest.mark.parametrize("N, K", [(1152, 896), (130, 72), (896, 512), (300, 1000)])
def test_gemm_with_rmsnorm_formed_on_its_way(T, N, K, skinny, device, request):
    """ops.gemm given the not-yet-computed norm of the residual rows: one kernel, same numbers as norm then product."""
    from ferrisinfer_b200.kernels import ops

    if not skinny:
        request.getfixturevalue("skinny_off")
    h = rnd((T, K), F32, device, 31, scale=2.0)
    nw = 1 + rnd((K,), F32, device, 32, scale=0.1)
    w = rnd((N, K), BF16, device, 33, scale=0.1)
    bias = rnd((N,), F32, device, 34)
    eps = 1e-5
    y = torch.empty(T, K, dtype=BF16, device=device)
    ops.rmsnorm(h, nw, eps, y)
    want = torch.empty(T, N, dtype=BF16, device=device)
    ops.gemm(y, w, bias, want)
    lazy = ops.LazyRMSNorm(h, nw, eps, torch.full((T, K), float("nan"), dtype=BF16, device=device))
    launches = ops.launch_count()
    got = torch.full((T, N), float("nan"), dtype=BF16, device=device)
    ops.gemm(lazy, w, bias, got)
    assert ops.launch_count() - launches == 1 and not lazy._done, "no norm kernel ran"
    scale = want.float().abs().max().item()
    assert (got.float() - want.float()).abs().max().item() <= 2e-2 * scale
    ref = plain.rms_norm(h.cpu().double(), nw.cpu().double(), eps).to(BF16).double() @ w.cpu().double().t() + bias.cpu().double()
    assert (got.cpu().double() - ref).abs().max().item() <= 2e-2 * scale
    # accumulation into the residual, and the gated feed-forward's first product
    acc = rnd((T, N), F32, device, 35)
    before = acc.clone()
    ops.gemm(ops.LazyRMSNorm(h, nw, eps, y.clone()), w, None, acc, accumulate=True)
    assert ((acc - before).cpu().double() - (ref - bias.cpu().double())).abs().max().item() <= 2e-2 * scale
    if N % 2 == 0:
        I = N // 2
        out = torch.full((T, I), float("nan"), dtype=BF16, device=device)
        ops.gemm_swiglu(ops.LazyRMSNorm(h, nw, eps, y.clone()), w, out)
        g = ref - bias.cpu().double()
        want_act = g[:, I:] * plain.silu(g[:, :I])
        assert (out.cpu().double() - want_act).abs().max().item() <= 3e-2 * (want_act.abs().max().item() + 1e-3)
    assert ops.kernel_status() == 0


def test_lazy_norm_is_computed_where_no_kernel_can_form_it(device):
    from ferrisinfer_b200.kernels import ops

    h = rnd((100, 256), F32, device, 36)  # 100 tokens: beyond the fused kernel
    nw = 1 + rnd((256,), F32, device, 37, scale=0.1)
    w = rnd((64, 256), BF16, device, 38, scale=0.1)
    lazy = ops.LazyRMSNorm(h, nw, 1e-6, torch.empty(100, 256, dtype=BF16, device=device))
    out = torch.empty(100, 64, dtype=BF16, device=device)
    ops.gemm(lazy, w, None, out)
    assert lazy._done
    want = plain.rms_norm(h.cpu().double(), nw.cpu().double(), 1e-6).to(BF16).double() @ w.cpu().double().t()
    assert (out.cpu().double() - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    h32 = rnd((4, 64), F32, device, 39)  # the 32-bit path always computes the norm
    lazy32 = ops.LazyRMSNorm(h32, torch.ones(64, device=device), 1e-6, torch.empty(4, 64, device=device))
    out32 = torch.empty(4, 8, device=device)
    ops.gemm(lazy32, rnd((8, 64), F32, device, 40), None, out32)
    assert lazy32._done


def test_gemm_dispatch_takes_strided_rows_and_refuses_nothing_silently(device):
    from ferrisinfer_b200.kernels import ops

    wide = rnd((40, 256 + 64), BF16, device, 27)
    w = rnd((200, 256), BF16, device, 28, scale=0.1)
    x = wide[:, 32:32 + 256]  # rows 320 apart, start 64 bytes into the row: takes the tensor-core path
    assert ops.tensor_core_gemm_takes(x, w)
    out = torch.empty(40, 200, dtype=BF16, device=device)
    ops.gemm(x, w, None, out)
    _close(out, _gemm_reference(x, w), 256, BF16)
    odd = rnd((40, 100), BF16, device, 29)[:, :99]  # K = 99: the CUDA-core kernel runs instead
    w2 = rnd((50, 99), BF16, device, 30)
    assert not ops.tensor_core_gemm_takes(odd, w2)
    out = torch.empty(40, 50, dtype=BF16, device=device)
    ops.gemm(odd, w2, None, out)
    _close(out, _gemm_reference(odd, w2), 99, BF16)


# -------------------------------------------------------------------------------------- swiglu
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_swiglu(dtype, device):
    from ferrisinfer_b200.kernels import ops

    gu = rnd((9, 600), dtype, device, 11, scale=2.0)
    out = torch.empty(9, 300, dtype=dtype, device=device)
    ops.swiglu(gu, out)
    g, u = gu[:, :300].cpu().double(), gu[:, 300:].cpu().double()
    assert torch.allclose(out.cpu().double(), u * plain.silu(g), **tol(dtype))


# ------------------------------------------------------------------------- rope + cache write
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("nh, nkv, d, rotary, page", [(6, 3, 48, 24, 8), (4, 1, 16, 16, 4), (2, 2, 128, 128, 16),
                                                      (3, 1, 32, 0, 8)])
def test_rope_cache_write(nh, nkv, d, rotary, page, dtype, device):
    from ferrisinfer_b200.kernels import ops

    T, pages = 21, 9
    qkv = rnd((T, (nh + 2 * nkv) * d), dtype, device, 12)
    src = qkv.clone()
    positions = torch.tensor([0, 1, 2, 7, 8, 9, 500, 501, 31999, 32000, 3, 3, 3, 40, 41, 42, 43, 44, 45, 46, 47],
                             dtype=torch.int32, device=device)
    slots = torch.randperm(pages * page, generator=torch.Generator().manual_seed(1))[:T].to(torch.int32).to(device)
    slots[5] = -1  # nothing is written for this token
    k_cache = torch.zeros(pages, nkv, page, d, dtype=dtype, device=device)
    v_cache = torch.zeros_like(k_cache)
    inv_freq = torch.tensor(plain.rotary_inverse_frequencies(d, rotary, 1e6).numpy(), device=device) if rotary else None
    ops.rope_cache_write(qkv, positions, inv_freq, slots, k_cache, v_cache, nh, nkv, d, rotary, page)
    s3 = src.cpu().float().view(T, nh + 2 * nkv, d)
    pos = positions.cpu().tolist()
    q_want = plain.rope(s3[:, :nh].double(), pos, d, rotary, 1e6)
    k_want = plain.rope(s3[:, nh:nh + nkv].double(), pos, d, rotary, 1e6)
    got = qkv.cpu().double().view(T, nh + 2 * nkv, d)
    # the angle is the same fp32 product in the kernel and in the plain implementation, also at position 32000
    t = dict(atol=2e-5, rtol=1e-5) if dtype == F32 else dict(atol=3e-2, rtol=2e-2)
    assert torch.allclose(got[:, :nh], q_want, **t)
    assert torch.equal(got[:, nh:], s3[:, nh:].double())  # k and v stay as they were in the buffer
    small = [i for i, p in enumerate(pos) if p < 1000]
    assert torch.allclose(got[small, :nh], q_want[small], **tol(dtype))
    for i in range(T):
        slot = slots[i].item()
        if slot < 0:
            continue
        pg, off = slot // page, slot % page
        assert torch.allclose(k_cache[pg, :, off].cpu().double(), k_want[i], **t)
        assert torch.equal(v_cache[pg, :, off].cpu().double(), s3[i, nh + nkv:].double())
    written = {s.item() for s in slots if s.item() >= 0}
    for slot in range(pages * page):
        if slot not in written:
            assert k_cache[slot // page, :, slot % page].abs().sum().item() == 0
    again = src.clone()
    ops.rope_cache_write(again, positions, inv_freq, None, None, None, nh, nkv, d, rotary, page, write_kv=False)
    assert torch.equal(again.view(T, -1, d)[:, :nh], qkv.view(T, -1, d)[:, :nh])


@pytest.mark.gpu
@pytest.mark.parametrize("T,nh,nkv,d,K,page", [(128, 2, 1, 64, 64, 16), (300, 14, 2, 64, 896, 64), (257, 3, 1, 128, 136, 32),
                                               (6400, 5, 2, 64, 72, 64), (1000, 1, 1, 128, 264, 16),
                                               # tiles of 192 weight rows (three heads of 64) and of 256 (two heads of 128)
                                               (2048, 20, 2, 64, 72, 64), (2048, 12, 2, 128, 136, 32)])
def test_qkv_product_with_rotation_and_cache_write_in_its_epilogue(T, nh, nkv, d, K, page, device):
    """Queries rotated into the output rows, keys rotated and values straight into the paged cache, against the
    product in fp64 rotated by the plain implementation; tokens with slot -1 and all other slots stay untouched."""
    from ferrisinfer_b200.kernels import ops

    N = (nh + 2 * nkv) * d
    x = rnd((T, K), BF16, device, 31)
    w = rnd((N, K), BF16, device, 32) * (K ** -0.5)
    bias = rnd((N,), F32, device, 33)
    g = torch.Generator().manual_seed(5)
    positions = torch.randint(0, 5000, (T,), generator=g, dtype=torch.int32)
    positions[:3] = torch.tensor([0, 1, 32000])
    pages = (T + page - 1) // page + 3
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32)
    slots[7] = -1
    slots[T - 1] = -1
    positions, slots = positions.to(device), slots.to(device)
    k_cache = torch.full((pages, nkv, page, d), 7.0, dtype=BF16, device=device)
    v_cache = torch.full_like(k_cache, 7.0)
    qkv = torch.full((T, N), 7.0, dtype=BF16, device=device)
    inv_freq = torch.tensor(plain.rotary_inverse_frequencies(d, d, 1e6).numpy(), device=device)
    angles = torch.empty(T, d // 2, 2, dtype=F32, device=device)
    ops.rotary_angles(positions, inv_freq, angles)
    a = (positions.cpu().float()[:, None] * inv_freq.cpu()[None, :])  # the same fp32 product
    assert torch.allclose(angles[..., 0].cpu().double(), torch.cos(a.double()), atol=1e-6)
    assert torch.allclose(angles[..., 1].cpu().double(), torch.sin(a.double()), atol=1e-6)
    assert ops.qkv_rope_gemm_takes(x, w, qkv, nh, nkv, d, d, k_cache)
    ops.qkv_rope_gemm(x, w, bias, qkv, angles, slots, k_cache, v_cache, nh, nkv, d)

    y = (x.cpu().double() @ w.cpu().double().t() + bias.cpu().double()).view(T, nh + 2 * nkv, d)
    pos = positions.cpu().tolist()
    q_want = plain.rope(y[:, :nh], pos, d, d, 1e6)
    k_want = plain.rope(y[:, nh:nh + nkv], pos, d, d, 1e6)
    v_want = y[:, nh + nkv:]
    t = dict(atol=3e-2, rtol=2e-2)
    small = [i for i, p in enumerate(pos) if p < 32000]  # the angle at 32000 differs in the last fp32 bits
    got = qkv.cpu().double().view(T, nh + 2 * nkv, d)
    assert torch.allclose(got[small, :nh], q_want[small], **tol(BF16))
    assert torch.allclose(got[:, :nh], q_want, **t)
    assert (got[:, nh:] == 7.0).all()  # the key and value columns of the buffer are not written
    sl = slots.cpu()
    live = sl >= 0
    kc, vc = k_cache.cpu().double(), v_cache.cpu().double()
    k_got = kc[sl[live] // page, :, sl[live] % page]
    v_got = vc[sl[live] // page, :, sl[live] % page]
    assert torch.allclose(k_got, k_want[live], **t)
    assert torch.allclose(v_got, v_want[live], **tol(BF16))
    untouched = torch.ones(pages * page, dtype=torch.bool)
    untouched[sl[live].long()] = False
    flat_k = kc.permute(0, 2, 1, 3).reshape(pages * page, nkv, d)
    flat_v = vc.permute(0, 2, 1, 3).reshape(pages * page, nkv, d)
    assert (flat_k[untouched] == 7.0).all() and (flat_v[untouched] == 7.0).all()

    # a layer that reads another layer's cache: queries only
    k2, v2 = torch.full_like(k_cache, 7.0), torch.full_like(v_cache, 7.0)
    q2 = torch.full_like(qkv, 7.0)
    ops.qkv_rope_gemm(x, w, bias, q2, angles, None, k2, v2, nh, nkv, d)
    assert torch.equal(q2, qkv) and (k2 == 7.0).all() and (v2 == 7.0).all()
    # and the same numbers as the product followed by the rotary kernel, up to one more rounding to bf16
    ref = torch.empty_like(qkv)
    ops.gemm(x, w, bias, ref)
    ops.rope_cache_write(ref, positions, inv_freq, slots, k2, v2, nh, nkv, d, d, page)
    assert torch.allclose(ref.view(T, -1, d)[:, :nh].float(), qkv.view(T, -1, d)[:, :nh].float(), atol=3e-2, rtol=2e-2)
    assert torch.allclose(k2.float(), k_cache.float(), atol=3e-2, rtol=2e-2)



# ----------------------------------------------------------------------------------- attention
class AttentionCase:
    """A batch of requests over a shuffled page pool; keys and values are set by position."""

    def __init__(self, device, dtype, nh, nkv, d, page, seqs, seed=0, window=0):
        # seqs: list of (kv_len, q_len): the last q_len positions of each request are the step's queries
        self.nh, self.nkv, self.d, self.page, self.window = nh, nkv, d, page, window
        g = torch.Generator().manual_seed(seed)
        blocks = [-(-kv // page) for kv, _ in seqs]
        total = sum(blocks) + 3
        order = torch.randperm(total, generator=g).tolist()
        self.max_blocks = max(blocks)
        tables = torch.full((len(seqs), self.max_blocks), -1, dtype=torch.int32)
        self.k = [torch.randn(kv, nkv, d, generator=g) for kv, _ in seqs]
        self.v = [torch.randn(kv, nkv, d, generator=g) for kv, _ in seqs]
        self.q = [torch.randn(ql, nh, d, generator=g) for _, ql in seqs]
        self.seqs = seqs
        used = 0
        for s, nb in enumerate(blocks):
            tables[s, :nb] = torch.tensor(order[used:used + nb], dtype=torch.int32)
            used += nb
        self.tables, self.total, self.dtype, self.device = tables, total, dtype, device

    def device_inputs(self):
        nh, nkv, d, page = self.nh, self.nkv, self.d, self.page
        k_cache = torch.full((self.total, nkv, page, d), 7.0)  # stale contents of pages that nobody owns
        v_cache = torch.full((self.total, nkv, page, d), -7.0)
        for s, (kv, _) in enumerate(self.seqs):
            for p in range(kv):
                pg = self.tables[s, p // page].item()
                k_cache[pg, :, p % page] = self.k[s][p]
                v_cache[pg, :, p % page] = self.v[s][p]
        T = sum(ql for _, ql in self.seqs)
        qkv = torch.zeros(T, (nh + 2 * nkv) * d)
        token_seq, positions = [], []
        row = 0
        for s, (kv, ql) in enumerate(self.seqs):
            qkv[row:row + ql, :nh * d] = self.q[s].reshape(ql, nh * d)
            token_seq += [s] * ql
            positions += list(range(kv - ql, kv))
            row += ql
        to = lambda t, dt: t.to(dt).to(self.device)
        from types import SimpleNamespace

        from ferrisinfer_b200.engine.workspace import Workspace

        starts = [0]
        for _, ql in self.seqs:
            starts.append(starts[-1] + ql)
        ctx = SimpleNamespace(token_seq=to(torch.tensor(token_seq), torch.int32),
                              seq_q_start=to(torch.tensor(starts), torch.int32),
                              seq_start_pos=to(torch.tensor([kv - ql for kv, ql in self.seqs]), torch.int32),
                              workspace=Workspace(self.device),
                              single_rows=(to(torch.tensor([starts[i] for i, (_, ql) in enumerate(self.seqs) if ql == 1]),
                                              torch.int32)
                                           if any(ql == 1 for _, ql in self.seqs) and any(ql > 1 for _, ql in self.seqs)
                                           else None),
                              positions=to(torch.tensor(positions), torch.int32),
                              seqs=[SimpleNamespace(q_start=sum(q for _, q in self.seqs[:i]), q_len=ql, start_pos=kv - ql)
                                    for i, (kv, ql) in enumerate(self.seqs)],
                              num_tokens=T, num_seqs=len(self.seqs), max_q_len=max(ql for _, ql in self.seqs),
                              max_kv_len=max(kv for kv, _ in self.seqs))
        return (to(qkv, self.dtype), to(k_cache, self.dtype), to(v_cache, self.dtype),
                self.tables.to(self.device), ctx, T)

    def reference(self):
        """Plain attention per request in float64, from the values as the storage type rounds them."""
        outs = []
        r = lambda t: t.to(self.dtype).double()
        for s, (kv, ql) in enumerate(self.seqs):
            q_all = torch.zeros(kv, self.nh, self.d, dtype=torch.float64)
            q_all[kv - ql:] = r(self.q[s])
            o = plain.attention(q_all, r(self.k[s]), r(self.v[s]), list(range(kv)), self.window or None)
            outs.append(o[kv - ql:].reshape(ql, self.nh * self.d))
        return torch.cat(outs)


def attention_impls():
    from ferrisinfer_b200.kernels import ops

    def simt(qkv, out, k, v, tables, ctx, nh, nkv, d, window, scale):
        ops.paged_attention_simt(qkv, out, k, v, tables, ctx.token_seq, ctx.positions, nh, nkv, d, window, scale)

    return {"simt": simt, "dispatch": ops.paged_attention}


def run_attention(case, impl):
    qkv, k, v, tables, ctx, T = case.device_inputs()
    out = torch.full((T, case.nh * case.d), float("nan"), dtype=case.dtype, device=case.device)
    attention_impls()[impl](qkv, out, k, v, tables, ctx, case.nh, case.nkv, case.d, case.window,
                            1.0 / math.sqrt(case.d))
    torch.cuda.synchronize()
    from ferrisinfer_b200.kernels import ops

    assert ops.kernel_status() == 0, "a bounded wait ran out"
    return out.cpu().double()


ATT_TOL = {F32: dict(atol=2e-5, rtol=1e-4), BF16: dict(atol=2e-2, rtol=2e-2)}


@pytest.mark.parametrize("impl", ["simt", "dispatch"])
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("nh, nkv, d, page", [(4, 2, 16, 4), (3, 1, 32, 8), (5, 5, 48, 16), (14, 2, 64, 16),
                                              (12, 2, 128, 16), (7, 1, 64, 16), (2, 1, 256, 32), (6, 2, 80, 16),
                                              (12, 1, 64, 16), (16, 1, 128, 16)])  # groups of more than 8 heads
def test_attention_mixed_batch(nh, nkv, d, page, dtype, impl, device):
    """Whole prompts, portions and single decoded tokens in one batch, lengths at and around page edges."""
    seqs = [(1, 1), (page, page), (page + 1, 1), (3 * page, 1), (3 * page - 1, 2), (77, 77), (130, 17), (200, 1), (5, 3)]
    case = AttentionCase(device, dtype, nh, nkv, d, page, seqs, seed=nh * d)
    got, want = run_attention(case, impl), case.reference()
    assert torch.isfinite(got).all()
    assert torch.allclose(got, want, **ATT_TOL[dtype]), (got - want).abs().max()


@pytest.mark.parametrize("impl", ["simt", "dispatch"])
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("q_len", [1, 5, 64])
def test_attention_finds_one_far_key_among_hundreds(q_len, dtype, impl, device):
    """Key 37 of 900 is aligned with every query and scaled up: the output must be its value."""
    nh, nkv, d, page, kv = 8, 2, 64, 16, 900
    case = AttentionCase(device, dtype, nh, nkv, d, page, [(kv, q_len), (300, 1)], seed=3)
    direction = torch.randn(d, generator=torch.Generator().manual_seed(9))
    direction = direction / direction.norm()
    case.q[0][:] = direction * 6.0 + 0.05 * case.q[0]
    case.k[0][37] = direction * 30.0
    case.v[0][37] = torch.arange(d).float().repeat(nkv, 1) / d + 3.0
    got, want = run_attention(case, impl), case.reference()
    row = got[q_len - 1].view(nh, d)
    assert (row - case.v[0][37][0].to(dtype).double()).abs().max() < 0.05
    assert torch.allclose(got, want, **ATT_TOL[dtype])


@pytest.mark.parametrize("impl", ["simt", "dispatch"])
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("decode_only", [False, True])
@pytest.mark.parametrize("window, page, d", [(21, 8, 32), (16, 16, 32), (33, 16, 64), (5, 4, 16), (16, 16, 64),
                                             (47, 32, 128), (100, 16, 64)])
def test_attention_window_edges(window, page, d, decode_only, dtype, impl, device):
    """The key at P - W + 1 is the last one inside the window; the key at P - W is outside.  Both carry loud
    values, so a window that is off by one shows."""
    nh, nkv = 4, 2
    seqs = [(100, 1), (100, 30), (window, 1), (window + 1, 2), (64, 64), (300, 1)]
    if decode_only:
        seqs = [(kv, 1) for kv, _ in seqs]
    case = AttentionCase(device, dtype, nh, nkv, d, page, seqs, seed=window, window=window)
    P = 99
    case.v[0][P - window + 1] += 50.0  # inside: must show
    if P - window >= 0:
        case.v[0][P - window] -= 5000.0  # outside: must not
    got, want = run_attention(case, impl), case.reference()
    assert got[0].max() > 0.5 and got[0].min() > -100.0
    assert torch.allclose(got, want, atol=ATT_TOL[dtype]["atol"] * 10, rtol=ATT_TOL[dtype]["rtol"])


@pytest.mark.parametrize("impl", ["simt", "dispatch"])
def test_attention_long_context_decode_batch(impl, device):
    """Decoding at a context of several thousand keys for a batch of requests of unequal length."""
    nh, nkv, d, page = 14, 2, 64, 16
    seqs = [(4096, 1), (4095, 1), (2049, 1), (17, 1), (4081, 1), (3000, 1), (1, 1), (2048, 1)]
    case = AttentionCase(device, BF16, nh, nkv, d, page, seqs, seed=11)
    got, want = run_attention(case, impl), case.reference()
    assert torch.allclose(got, want, **ATT_TOL[BF16]), (got - want).abs().max()


@pytest.mark.parametrize("nh, nkv, d, window", [(14, 2, 64, 0), (12, 2, 128, 0), (4, 4, 64, 40), (7, 1, 64, 0),
                                                (24, 2, 64, 0), (16, 1, 128, 0)])  # groups of 12 and 16: 16-row products
def test_attention_step_of_single_tokens_rotates_and_writes_on_its_way(nh, nkv, d, window, device):
    """The one-kernel path of a decode step against the two-kernel path: same output, same cache."""
    from ferrisinfer_b200.kernels import ops
    from ferrisinfer_b200.parts.base import PagedMeta

    page = 16
    seqs = [(4096, 1), (1, 1), (16, 1), (17, 1), (33, 1), (700, 1), (48, 1), (49, 1)]
    case = AttentionCase(device, BF16, nh, nkv, d, page, seqs, seed=d + nh, window=window)
    qkv, k, v, tables, ctx, T = case.device_inputs()
    g = torch.Generator().manual_seed(5)
    qkv[:, nh * d:] = torch.randn(T, 2 * nkv * d, generator=g).to(BF16).to(device)  # the tokens' own k and v
    slots = torch.tensor([tables[i, (kv - 1) // page].item() * page + (kv - 1) % page for i, (kv, _) in enumerate(seqs)],
                         dtype=torch.int32, device=device)
    inv_freq = torch.tensor(plain.rotary_inverse_frequencies(d, d, 1e6).numpy(), device=device)
    meta = PagedMeta(block_tables=tables, slot_mapping=slots, page_size=page)
    scale = 1.0 / math.sqrt(d)
    # two kernels
    qkv2, k2, v2 = qkv.clone(), k.clone(), v.clone()
    want = torch.empty(T, nh * d, dtype=BF16, device=device)
    ops.rope_cache_write(qkv2, ctx.positions, inv_freq, slots, k2, v2, nh, nkv, d, d, page)
    ops.paged_attention(qkv2, want, k2, v2, tables, ctx, nh, nkv, d, window, scale)
    # one kernel
    qkv1, k1, v1 = qkv.clone(), k.clone(), v.clone()
    got = torch.full_like(want, float("nan"))
    ops.attention_step(qkv1, got, k1, v1, meta, ctx, nh, nkv, d, inv_freq, d, window, scale)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert torch.equal(k1, k2) and torch.equal(v1, v2), "the cache holds the same rotated keys and values"
    assert torch.equal(qkv1, qkv), "the fused path leaves the step's qkv rows alone"
    assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2), (got.float() - want.float()).abs().max()
    # a layer that reads another layer's cache: q is rotated, nothing is written, and the token's key and value are
    # the ones the cache holds, not the ones in this layer's own qkv rows (which are made different here)
    k3, v3 = k2.clone(), v2.clone()
    other = qkv.clone()
    other[:, nh * d:] = torch.randn(T, 2 * nkv * d, generator=g).to(BF16).to(device)
    again = torch.full_like(want, float("nan"))
    ops.attention_step(other, again, k3, v3, meta, ctx, nh, nkv, d, inv_freq, d, window, scale, write_kv=False)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert torch.equal(k3, k2) and torch.equal(v3, v2)
    assert torch.allclose(again.float(), want.float(), atol=2e-2, rtol=2e-2), (again.float() - want.float()).abs().max()


@pytest.mark.parametrize("nh, nkv, d, window", [(14, 2, 64, 0), (12, 2, 128, 0), (8, 8, 64, 100), (3, 1, 128, 0)])
def test_prefill_attention_on_tcgen05_and_on_mma_sync(nh, nkv, d, window, device):
    """The prefill kernels (scores and products in tensor memory by tcgen05.mma, with two groups of softmax warps on
    alternate blocks of keys where they fit and with one; mma.sync fragments in registers) against the plain
    attention and against each other: whole prompts past several blocks of 128 keys, a portion at the end of a long
    context, rows that end inside a block of 128, prompts of one and of two blocks (the second group has no block
    or one), a single token beside them."""
    from ferrisinfer_b200.kernels import ops

    seqs = [(700, 700), (1500, 130), (129, 129), (4, 4), (300, 1), (128, 128), (256, 256)]
    case = AttentionCase(device, BF16, nh, nkv, d, 16, seqs, seed=nh + d, window=window)
    want = case.reference()
    got = {}
    try:
        for mode in (1, 0, 2):
            ops.set_prefill_tcgen05(mode)
            got[mode] = run_attention(case, "dispatch")
    finally:
        ops.set_prefill_tcgen05(True)
    for mode in (1, 0, 2):
        assert torch.allclose(got[mode], want, **ATT_TOL[BF16]), (mode, (got[mode] - want).abs().max())
    assert (got[1] - got[0]).abs().max() <= 2 * ATT_TOL[BF16]["atol"]
    assert (got[1] - got[2]).abs().max() <= 2 * ATT_TOL[BF16]["atol"]


@pytest.mark.parametrize("impl", ["simt", "dispatch"])
def test_attention_single_tokens_beside_portions_at_long_context(impl, device):
    """Single tokens whose keys are split into ranges, at rows of the step that come after portions of prompts
    (their partial results must not lie where another row's do)."""
    nh, nkv, d, page = 14, 2, 64, 16
    seqs = [(600, 3), (4096, 1), (3000, 1), (40, 40), (2048, 1), (1000, 1), (9, 2), (4000, 1)]
    case = AttentionCase(device, BF16, nh, nkv, d, page, seqs, seed=23)
    got, want = run_attention(case, impl), case.reference()
    assert torch.allclose(got, want, **ATT_TOL[BF16]), (got - want).abs().max()


@pytest.mark.parametrize("nh, nkv, d, T", [(14, 2, 64, 8), (12, 2, 128, 3), (7, 1, 64, 16), (14, 2, 64, 1)])
def test_output_product_merges_the_key_ranges_on_its_way(nh, nkv, d, T, device, skinny_off):
    """A decode step that leaves the partial results of its key ranges to the product that follows, against the
    same step with the merge kernel (the path of the tcgen05 short-step products)."""
    from ferrisinfer_b200.kernels import ops
    from ferrisinfer_b200.parts.base import PagedMeta

    page, H = 16, 896
    lengths = [4096, 2500, 4000, 3333, 4090, 2049, 3000, 3500, 2100, 2200, 2300, 2400, 2600, 2700, 2800, 2900][:T]
    seqs = [(kv, 1) for kv in lengths]
    case = AttentionCase(device, BF16, nh, nkv, d, page, seqs, seed=T + d)
    qkv, k, v, tables, ctx, _ = case.device_inputs()
    g = torch.Generator().manual_seed(6)
    qkv[:, nh * d:] = torch.randn(T, 2 * nkv * d, generator=g).to(BF16).to(device)
    slots = torch.tensor([tables[i, (kv - 1) // page].item() * page + (kv - 1) % page for i, (kv, _) in enumerate(seqs)],
                         dtype=torch.int32, device=device)
    inv_freq = torch.tensor(plain.rotary_inverse_frequencies(d, d, 1e6).numpy(), device=device)
    meta = PagedMeta(block_tables=tables, slot_mapping=slots, page_size=page)
    scale = 1.0 / math.sqrt(d)
    w_o = rnd((H, nh * d), BF16, device, 7, scale=0.05)
    h0 = rnd((T, H), F32, device, 8)

    eager = torch.empty(T, nh * d, dtype=BF16, device=device)
    k1, v1 = k.clone(), v.clone()
    assert ops.attention_step(qkv.clone(), eager, k1, v1, meta, ctx, nh, nkv, d, inv_freq, d, 0, scale) is eager
    want = h0.clone()
    ops.gemm(eager, w_o, None, want, accumulate=True)

    buf = torch.full_like(eager, float("nan"))
    k2, v2 = k.clone(), v.clone()
    lazy = ops.attention_step(qkv.clone(), buf, k2, v2, meta, ctx, nh, nkv, d, inv_freq, d, 0, scale, lazy_merge=True)
    assert isinstance(lazy, ops.LazySplitMerge), "these lengths are split into key ranges"
    assert ops._merge_gemm_takes(lazy, w_o)
    got = h0.clone()
    ops.gemm(lazy, w_o, None, got, accumulate=True)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert torch.isnan(buf.float()).all(), "no merge kernel ran"
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    assert torch.allclose(got, want, **tol(BF16)), (got - want).abs().max()
    # a consumer that cannot merge gets the merged rows from the merge kernel
    assert torch.equal(lazy.materialize(), eager)


# ------------------------------------------------------------------------------------ sampling
def test_argmax_takes_the_lowest_index_among_equal_maxima(device):
    from ferrisinfer_b200.kernels import ops

    logits = rnd((6, 5000), F32, device, 20)
    logits[0, 4000] = logits[0, 17] = 9.0
    logits[1, 4999] = 9.0
    logits[2, 0] = 9.0
    logits[3] = -3.0  # all equal
    logits[4, 123] = float("inf")
    tok = torch.empty(6, dtype=torch.int32, device=device)
    prob = torch.empty(6, dtype=F32, device=device)
    ops.sample(logits, tok, prob)
    want = [plain.greedy(logits[i].cpu().numpy()) for i in range(6)]
    assert tok.cpu().tolist()[:4] == [17, 4999, 0, 0] and tok[4].item() == 123
    assert tok[5].item() == want[5][0]
    for i in (0, 1, 2, 3, 5):
        assert abs(prob[i].item() - want[i][1]) < 1e-6 * max(1.0, 1 / want[i][1]) + 1e-6


@pytest.mark.parametrize("T, N, K", [(1, 2501, 64), (8, 151936, 896), (64, 3001, 1536), (100, 777, 128), (128, 4096, 264),
                                     (5, 100, 72)])
def test_output_head_picks_the_greatest_logit_without_storing_the_logits(T, N, K, device):
    """The product + argmax kernel against the plain greedy sampler over logits in float64, and against the stored
    logits followed by the sampling kernel (the same token).  Rows are made so
    that the best logit lies at the vocabulary's first and last index, in the last, partly filled tile, and twice
    (the lower index wins)."""
    from ferrisinfer_b200.engine.workspace import Workspace
    from ferrisinfer_b200.kernels import ops

    x = rnd((T, K), BF16, device, 61)
    w = rnd((N, K), BF16, device, 62, scale=0.05)
    # a weight row that is a multiple of a token's own row gives that token a logit that stands out
    plant = {0: [N - 1], 1 % T: [0]} if T > 1 else {0: [N - 1]}
    if T > 2:
        plant[2] = [N // 2 + 1, 7]  # twice the same logit: index 7 wins
    if T > 3:
        plant[3] = [N - 3, N - 2]
    for t, rows in plant.items():
        for r in rows:
            w[r] = (x[t].float() * 0.5).to(BF16)
    tok = torch.full((T,), -1, dtype=torch.int32, device=device)
    prob = torch.full((T,), float("nan"), dtype=F32, device=device)
    scratch = torch.empty(ops.gemm_argmax_scratch_floats(T, N), dtype=F32, device=device)
    launches = ops.launch_count()
    ops.gemm_argmax(x, w, tok, prob, scratch)
    assert ops.launch_count() - launches == 1  # one call: the product and the merge of its tiles
    logits = torch.empty(T, N, dtype=F32, device=device)
    ops.gemm(x, w, None, logits)
    tok2 = torch.empty(T, dtype=torch.int32, device=device)
    prob2 = torch.empty(T, dtype=F32, device=device)
    ops.sample(logits, tok2, prob2)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert torch.equal(tok, tok2)
    # the stored logits of few tiles are summed over a K split, the fused product's are not: they differ by a rounding
    # of the logit (~1e-6 absolute), and so do the probabilities
    assert torch.allclose(prob, prob2, rtol=5e-5, atol=1e-7)
    for t, rows in plant.items():
        if t in (0, 1 % T) or T > 2:
            assert tok[t].item() == min(rows), (t, tok[t].item(), rows)
    exact = x.double() @ w.double().T
    best = exact.max(dim=1).values
    chosen = exact.gather(1, tok.long().unsqueeze(1)).squeeze(1)
    assert ((best - chosen) <= 1e-3 * best.abs().clamp(min=1.0)).all()
    want_prob = torch.softmax(exact, dim=1).gather(1, tok.long().unsqueeze(1)).squeeze(1)
    assert torch.allclose(prob.double(), want_prob, rtol=2e-3, atol=1e-6)
    # through the part's entry: the same for bf16 rows; 32-bit rows go through stored logits and the sampling kernel
    ws = Workspace(device)
    for rows in (x, x.float()):
        weight = w if rows.dtype == BF16 else w.float()
        tok3 = torch.full((T,), -1, dtype=torch.int32, device=device)
        prob3 = torch.empty(T, dtype=F32, device=device)
        ops.greedy_head(rows, weight, tok3, prob3, ws)
        if rows.dtype == BF16:
            assert torch.equal(tok3, tok) and torch.allclose(prob3, prob, rtol=5e-5, atol=1e-7)
            if T <= ops.GREEDY_HEAD_MAX_ROWS:
                assert torch.equal(prob3, prob), "few rows go through the product that stores no logits"
        else:
            got = exact.gather(1, tok3.long().unsqueeze(1)).squeeze(1)
            assert ((best - got) <= 1e-5 * best.abs().clamp(min=1.0)).all()


def exact_interval(row, T, k, p, token):
    """In float64: the mass before ``token`` and through it in the reference's order (descending logit, ascending
    index), after the top-k and top-p cuts, both as fractions of the retained mass; None if the token was cut."""
    V = row.shape[0]
    order = np.lexsort((np.arange(V), -row.astype(np.float64)))
    k = V if k <= 0 else min(k, V)
    order = order[:k]
    Tc = max(np.float32(T), np.finfo(np.float32).eps)
    w = np.exp((row[order] / Tc - row[order[0]] / Tc).astype(np.float64))
    cum = np.cumsum(w)
    kept = k
    if p < 1.0:
        kept = int(np.searchsorted(cum, cum[-1] * np.float64(np.float32(p)), side="left")) + 1
        kept = min(max(kept, 1), k)
    where = np.nonzero(order[:kept + 1] == token)[0]  # one more than kept: the cut itself may fall within rounding
    if where.size == 0:
        return None
    i = int(where[0])
    total = cum[kept - 1]
    return (cum[i] - w[i]) / total, cum[i] / total


@pytest.mark.parametrize("V", [257, 5000, 151936])
def test_sampling_matches_the_plain_sampler(V, device):
    """Rows with different temperatures, top_k and top_p; each row draws from its own generator state.
    The chosen token must be the one whose span of the retained mass (float64, the reference's order) holds the
    draw u.  For small vocabularies it must also be the token that the reference's sequential f32 walk picks
    (over 150,000 tokens that walk's own f32 sums are coarser than a token's span, so it is no oracle there)."""
    from ferrisinfer_b200.kernels import ops

    rows = 24 if V > 100000 else 48
    g = torch.Generator().manual_seed(V)
    logits = (torch.randn(rows, V, generator=g) * 2.0)
    logits[3, 10:20] = logits[3, 5]  # ties
    logits[4] = torch.round(logits[4])  # many ties
    options = [(0.7, 0, 1.0), (1.0, 20, 0.9), (0.3, 0, 0.5), (1.5, 50, 1.0), (0.7, 5, 0.1), (2.0, 0, 0.95),
               (0.0, 0, 1.0), (0.7, 1, 1.0), (1e-9, 0, 1.0), (1.0, 100000000, 0.999)]
    temperature = torch.tensor([options[i % len(options)][0] for i in range(rows)])
    top_k = torch.tensor([options[i % len(options)][1] for i in range(rows)], dtype=torch.int32)
    top_p = torch.tensor([options[i % len(options)][2] for i in range(rows)])
    slots = torch.randperm(64, generator=g)[:rows].to(torch.int32)
    states = torch.randint(1, 2**62, (64,), generator=g)
    states[slots[2]] = 0  # stands for the default seed
    dev_states = states.clone().to(device)
    tok = torch.empty(rows, dtype=torch.int32, device=device)
    prob = torch.empty(rows, dtype=F32, device=device)
    for draw in range(3):
        ops.sample(logits.to(device), tok, prob, temperature.to(device), top_k.to(device), top_p.to(device),
                   slots.to(device), dev_states)
        differ = 0
        for r in range(rows):
            T, k, p = temperature[r].item(), top_k[r].item(), top_p[r].item()
            row = logits[r].numpy()
            rng = plain.XorShift64Star(int(states[slots[r]].item()))
            greedy = T <= 0 or k == 1 or p <= 0
            if greedy:
                assert tok[r].item() == plain.greedy(row)[0]
                assert dev_states[slots[r]].item() == states[slots[r]].item(), "greedy rows draw nothing"
                continue
            if V <= 5000:
                want_tok, want_prob = plain.sample(row, T, k, p, plain.XorShift64Star(rng.state))
                if tok[r].item() != want_tok:
                    differ += 1
                else:
                    assert abs(prob[r].item() - want_prob) < 1e-3 * want_prob + 1e-6
            u = rng.next_f32()
            states[slots[r]] = rng.state - (1 << 64) if rng.state >= 1 << 63 else rng.state
            assert dev_states[slots[r]].item() == states[slots[r]].item(), "the generator advances once per draw"
            span = exact_interval(row, T, k, p, tok[r].item())
            assert span is not None, (r, "the chosen token lies outside the top-k / top-p set")
            lo, hi = span
            assert lo - 1e-5 <= u <= hi + 1e-5, (r, T, k, p, u, lo, hi)
            assert abs(prob[r].item() - (hi - lo)) < 1e-3 * (hi - lo) + 1e-6
        assert differ <= 1, differ


@pytest.mark.parametrize("V", [3, 7, 33, 1000])
def test_sampling_at_the_edges(V, device):
    """Vocabularies smaller than the row's eight CTAs have parts, rows with -inf entries (a masked vocabulary), one
    finite logit only, logits spread over hundreds of units (everything but the top falls below the histogram's range)
    and rows of one value: the chosen token's span of the retained mass holds the draw, in float64."""
    from ferrisinfer_b200.kernels import ops

    g = torch.Generator().manual_seed(V)
    base = torch.randn(6, V, generator=g) * 2.0
    base[1, ::2] = float("-inf")                      # every second token masked
    base[2] = float("-inf")
    base[2, V // 2] = 0.3                             # one token left
    base[3] = torch.linspace(-300.0, 40.0, V)         # a spread far beyond the histogram's range at T = 0.5
    base[4] = 1.25                                    # all equal
    base[5, : max(1, V // 3)] = float("-inf")
    options = [(0.8, 0, 1.0), (1.0, 0, 0.9), (0.7, 5, 1.0), (0.5, 0, 0.95), (1.0, 2, 1.0), (1.3, 0, 0.5)]
    rows = base.shape[0]
    temperature = torch.tensor([o[0] for o in options])
    top_k = torch.tensor([o[1] for o in options], dtype=torch.int32)
    top_p = torch.tensor([o[2] for o in options])
    slots = torch.arange(rows, dtype=torch.int32)
    states = torch.randint(1, 2**62, (rows,), generator=g)
    dev_states = states.clone().to(device)
    tok = torch.empty(rows, dtype=torch.int32, device=device)
    prob = torch.empty(rows, dtype=F32, device=device)
    for draw in range(4):
        ops.sample(base.to(device), tok, prob, temperature.to(device), top_k.to(device), top_p.to(device),
                   slots.to(device), dev_states)
        torch.cuda.synchronize()
        assert ops.kernel_status() == 0
        for r in range(rows):
            T, k, p = options[r]
            row = base[r].numpy()
            rng = plain.XorShift64Star(int(states[r].item()))
            u = rng.next_f32()
            states[r] = rng.state - (1 << 64) if rng.state >= 1 << 63 else rng.state
            assert dev_states[r].item() == states[r].item()
            chosen = tok[r].item()
            assert 0 <= chosen < V and row[chosen] > float("-inf"), (r, chosen)
            span = exact_interval(row, T, k, p, chosen)
            assert span is not None, (r, chosen)
            lo, hi = span
            assert lo - 1e-5 <= u <= hi + 1e-5, (r, u, lo, hi)
            assert abs(prob[r].item() - (hi - lo)) < 1e-3 * (hi - lo) + 1e-6


def test_sampling_distribution(device):
    """Ten thousand draws at temperature 1 from a row of five tokens follow softmax."""
    from ferrisinfer_b200.kernels import ops

    row = torch.tensor([[1.0, 2.0, 0.0, -1.0, 1.5]])
    n = 10000
    logits = row.repeat(n, 1).to(device)
    states = torch.arange(1, n + 1, dtype=torch.int64, device=device) * 2654435761
    tok = torch.empty(n, dtype=torch.int32, device=device)
    ops.sample(logits, tok, None, torch.ones(n, device=device), torch.zeros(n, dtype=torch.int32, device=device),
               torch.ones(n, device=device), torch.arange(n, dtype=torch.int32, device=device), states)
    freq = torch.bincount(tok.cpu().long(), minlength=5).double() / n
    want = torch.softmax(row[0].double(), 0)
    assert (freq - want).abs().max() < 0.02, (freq, want)


# ------------------------------------------------------------------------------- skinny gemm
SKINNY_SHAPES = [(1152, 896), (896, 4864), (130, 72), (300, 1000), (9728, 896),
                 (4608, 3584), (896, 6016),  # slabs that do not fit into shared memory: the stages are a ring
                 (9472, 64), (7, 8), (17920, 1536),  # 64 rows per CTA; one K block of 8; more CTAs than SMs
                 (1536, 8960), (3584, 18944)]  # long rows: the step's rows travel with the weights through the ring


@pytest.mark.parametrize("T", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N, K", SKINNY_SHAPES)
def test_gemm_skinny(T, N, K, device):
    """The weight-stationary product of short steps alone: every mode against the product in float64, twice the
    same bits, and a row's result whatever else is in the step."""
    from ferrisinfer_b200.kernels import ops

    wide = rnd((T, K + 16), BF16, device, 51)
    x = wide[:, 8:8 + K]  # rows of a wider buffer
    w = rnd((N, K), BF16, device, 52, scale=0.1)
    bias = rnd((N,), F32, device, 53)
    want = _gemm_reference(x, w)
    out = torch.full((T, N), float("nan"), dtype=BF16, device=device)
    if not ops._skinny_takes(x, w, out, 1):
        # more than 8 tokens beside slabs of 64 rows leave no room for a ring of weights
        assert T > 8 and N > 9000
        pytest.skip("left to the tcgen05 kernel")
    ops.gemm_skinny(x, w, bias, out, 0)
    _close(out, want + bias.cpu().double(), K, BF16)
    out32 = torch.full((T, N), float("nan"), dtype=F32, device=device)
    ops.gemm_skinny(x, w, None, out32, 1)
    _close(out32, want, K, F32)
    again = torch.empty_like(out32)
    ops.gemm_skinny(x, w, None, again, 1)
    assert torch.equal(again, out32)
    one = torch.empty(1, N, dtype=F32, device=device)
    ops.gemm_skinny(x[T - 1:T], w, None, one, 1)
    if T <= 8:
        assert torch.equal(one[0], out32[T - 1]), "a row's sum does not depend on the rows beside it"
    else:
        # more than 8 tokens may be cut into other groups of K blocks: the same sum in another order
        assert torch.allclose(one[0], out32[T - 1], rtol=1e-5, atol=1e-5 * math.sqrt(K) * want.abs().max().item())
    acc = rnd((T, N), F32, device, 54)
    before = acc.clone()
    ops.gemm_skinny(x, w, bias, acc, 2)
    _close(acc - before, want + bias.cpu().double(), K, F32)
    if N % 2 == 0:
        I = N // 2
        act = torch.full((T, I), float("nan"), dtype=BF16, device=device)
        if ops._skinny_takes(x, w, act, 2):
            ops.gemm_skinny(x, w, None, act, 3, up_row_offset=I)
            want_act = want[:, I:] * plain.silu(want[:, :I])
            assert (act.cpu().double() - want_act).abs().max().item() <= 3e-2 * (want_act.abs().max().item() + 1e-3)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0


def test_gemm_skinny_leaves_tall_products_and_long_steps_to_the_other_kernels(device):
    from ferrisinfer_b200.errors import KernelError
    from ferrisinfer_b200.kernels import ops

    w = rnd((151936, 64), BF16, device, 55)
    x = rnd((4, 64), BF16, device, 56)
    assert not ops._skinny_takes(x, w, torch.empty(4, 151936, device=device), 1)  # the output head
    w2 = rnd((256, 64), BF16, device, 57)
    assert not ops._skinny_takes(rnd((17, 64), BF16, device, 58), w2, torch.empty(17, 256, device=device), 1)
    assert not ops._skinny_takes(rnd((4, 60), BF16, device, 59), rnd((256, 60), BF16, device, 60),
                                 torch.empty(4, 256, device=device), 1)
    with pytest.raises(KernelError):
        ops.gemm_skinny(rnd((17, 64), BF16, device, 58), w2, None, torch.empty(17, 256, dtype=BF16, device=device), 0)


@pytest.mark.parametrize("nh, nkv, d, T, window", [(14, 2, 64, 8, 0), (12, 2, 128, 3, 0), (7, 1, 64, 16, 0), (14, 2, 64, 1, 0),
                                                   (4, 4, 64, 5, 1000), (24, 2, 64, 6, 0), (16, 1, 128, 9, 0),
                                                   (14, 2, 64, -2, 0), (12, 2, 128, -1, 0)])  # T < 0: -T long requests
def test_decode_attention_merges_its_key_ranges_in_a_cluster(nh, nkv, d, T, window, device, request):
    """With the skinny products the decode kernel merges the partial results of its key ranges itself: the ranges of
    a (token, kv head) are the CTAs of a thread-block cluster, which adds them through its shared memory in the
    order of the ranges.  One launch, no scratch; the same bits launch after launch; and the merge kernel's result
    within rounding (the two paths cut the keys into ranges of different lengths)."""
    from ferrisinfer_b200.kernels import ops
    from ferrisinfer_b200.parts.base import PagedMeta

    page = 16
    span = 4096
    if T < 0:
        # one or two requests of some 20,000 keys: block tables of 16,384 keys and more are cut into up to 16 ranges,
        # a cluster larger than the portable 8
        T, span = -T, 20000
        lengths = [20000, 17001][:T]
    else:
        lengths = [4096, 2500, 4000, 3333, 4090, 2049, 3000, 3500, 2100, 2200, 2300, 2400, 2600, 2700, 2800, 2900][:T]
    seqs = [(kv, 1) for kv in lengths]
    case = AttentionCase(device, BF16, nh, nkv, d, page, seqs, seed=T + d, window=window)
    qkv, k, v, tables, ctx, _ = case.device_inputs()
    g = torch.Generator().manual_seed(6)
    qkv[:, nh * d:] = torch.randn(T, 2 * nkv * d, generator=g).to(BF16).to(device)
    slots = torch.tensor([tables[i, (kv - 1) // page].item() * page + (kv - 1) % page for i, (kv, _) in enumerate(seqs)],
                         dtype=torch.int32, device=device)
    inv_freq = torch.tensor(plain.rotary_inverse_frequencies(d, d, 1e6).numpy(), device=device)
    meta = PagedMeta(block_tables=tables, slot_mapping=slots, page_size=page)
    scale = 1.0 / math.sqrt(d)
    ranges = ops._lib().ferris_decode_cluster_splits(T, nkv, d, min(window, span) if window else ctx.max_kv_len)
    assert ranges > (8 if span > 16384 else 1)
    got = []
    for _ in range(3):
        out = torch.full((T, nh * d), float("nan"), dtype=BF16, device=device)
        k1, v1 = k.clone(), v.clone()
        launches = ops.launch_count()
        assert ops.attention_step(qkv.clone(), out, k1, v1, meta, ctx, nh, nkv, d, inv_freq, d, window, scale,
                                  lazy_merge=True) is out
        assert ops.launch_count() - launches == 1
        got.append(out)
    # keys and values as the two planes of one tensor (as the cache manager allocates them): a tile of keys and the
    # tile of values of the same tokens come with one copy; the result is the same to the bit
    planes = torch.stack([k, v]).contiguous()
    paired = torch.full((T, nh * d), float("nan"), dtype=BF16, device=device)
    ops.attention_step(qkv.clone(), paired, planes[0], planes[1], meta, ctx, nh, nkv, d, inv_freq, d, window, scale)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert torch.equal(got[0], got[1]) and torch.equal(got[0], got[2]) and torch.equal(paired, got[0])
    assert torch.equal(planes[0], k1) and torch.equal(planes[1], v1)
    request.getfixturevalue("skinny_off")
    want = torch.full((T, nh * d), float("nan"), dtype=BF16, device=device)
    k2, v2 = k.clone(), v.clone()
    ops.attention_step(qkv.clone(), want, k2, v2, meta, ctx, nh, nkv, d, inv_freq, d, window, scale)
    assert torch.allclose(got[0].float(), want.float(), atol=2e-2, rtol=2e-2), (got[0].float() - want.float()).abs().max()
    assert torch.equal(k1, k2) and torch.equal(v1, v2)


# ------------------------------------------------------------------------- switches of the library
def test_products_with_the_older_k_split_and_without_programmatic_launch():
    """FERRIS_GEMM_CLUSTER=0 (partials of a K split in global scratch, added by the CTA that finishes last) and
    FERRIS_PDL=0 (plain stream order) are read once per process: the product tests run again in a process of
    their own with both set."""
    import os
    import subprocess
    import sys

    env = dict(os.environ, FERRIS_GEMM_CLUSTER="0", FERRIS_PDL="0")
    here = os.path.dirname(os.path.abspath(__file__))
    done = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_kernels_gpu.py"), "-q", "-x", "-m", "gpu",
                           "-k", "gemm_tcgen05_store or gemm_tcgen05_swiglu or rows_do_not_depend", "-p", "no:cacheprovider"],
                          env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    assert " passed" in done.stdout
