"""Each kernel alone against a plain fp32/fp64 torch reference, at sizes other than the
engine's tiny models: widths that are no power of two, every head size class, tails in
every dimension, pages handed out in scrambled order and poisoned with NaN."""

from __future__ import annotations

import math
from pathlib import Path

import pytest
import torch

import plain_gpt2 as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _ops():
    from ayaka_b200.kernels import ops
    return ops


def _randn(*shape, seed=0, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [1, 100, 1600])
def test_embed_rows(dtype, width):
    ops = _ops()
    table, pos = _randn(37, width, seed=1, dtype=dtype), _randn(19, width, seed=2, dtype=dtype)
    index = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32, device=DEV)
    add = torch.tensor([18, 0, 3, 4, 4], dtype=torch.int32, device=DEV)
    out = torch.full((7, width + 3), float("nan"), device=DEV)[:, :width]
    bad = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embed_rows(table, index, out, add_table=pos, add_index=add, bad_index=bad)
    expected = table.float()[index.long()] + pos.float()[add.long()]
    torch.testing.assert_close(out[:5], expected, rtol=0, atol=0)
    assert torch.isnan(out[5:]).all() and int(bad.item()) == 0
    ops.embed_rows(table, index, out, bad_index=bad)
    torch.testing.assert_close(out[:5], table.float()[index.long()], rtol=0, atol=0)
    index[2] = 37
    ops.embed_rows(table, index, out, bad_index=bad)
    assert int(bad.item()) == 1


@pytest.mark.parametrize("width", [1, 96, 1600, 5000])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_layer_norm(width, out_dtype):
    ops = _ops()
    x = _randn(9, width, seed=3, scale=3.0) + 5.0
    gamma, beta = _randn(width, seed=4) + 1.0, _randn(width, seed=5)
    out = torch.zeros(9, width, dtype=out_dtype, device=DEV)
    ops.layer_norm(x, gamma, beta, 1e-6, out)
    expected = plain.layer_norm(x.double(), gamma.double(), beta.double(), 1e-6)
    tol = dict(rtol=1e-5, atol=1e-5) if out_dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(out.double(), expected, **tol)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    picked = torch.zeros(3, width, dtype=out_dtype, device=DEV)
    ops.layer_norm(x, gamma, beta, 1e-6, picked, rows=rows)
    torch.testing.assert_close(picked, out[rows.long()], rtol=0, atol=0)


# ---------------------------------------------------------------------------------------------
def _linear_reference(a, w, bias, activation, residual):
    y = a.double() @ w.double().t()
    if bias is not None:
        y = y + bias.double()
    if activation == "gelu_tanh":
        y = plain.gelu(y, "gelu_new")
    elif activation == "gelu_erf":
        y = plain.gelu(y, "gelu")
    if residual is not None:
        y = y + residual.double()
    return y


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (33, 77, 50), (130, 64, 257)])
@pytest.mark.parametrize("activation", ["none", "gelu_tanh", "gelu_erf"])
def test_linear_float32_is_true_fp32(m, n, k, activation):
    ops = _ops()
    a = _randn(m, k, seed=6)
    w = _randn(n, k, seed=7, scale=1 / math.sqrt(k))
    bias = _randn(n, seed=8)
    out = torch.zeros(m, n, device=DEV)
    ops.linear(a, w, bias, out, activation=activation)
    torch.testing.assert_close(out.double(), _linear_reference(a, w, bias, activation, None),
                               rtol=1e-5, atol=1e-5)
    if activation == "none":
        base = _randn(m, n, seed=9)
        acc = base.clone()
        ops.linear(a, w, bias, acc, residual=True)
        torch.testing.assert_close(acc.double(), _linear_reference(a, w, bias, "none", base),
                                   rtol=1e-5, atol=1e-5)


def test_linear_float32_sees_what_tf32_would_lose():
    """A product whose exact value needs more than TF32's 10 mantissa bits."""
    ops = _ops()
    a = torch.tensor([[1.0 + 2 ** -14, 1.0]], device=DEV)
    w = torch.tensor([[1.0, -1.0]], device=DEV)
    out = torch.zeros(1, 1, device=DEV)
    ops.linear(a, w, None, out)
    assert out.item() == 2 ** -14


GEMM_SHAPES = [(128, 128, 64), (1, 64, 64), (5, 24, 8), (200, 300, 136), (130, 1000, 1600),
               (300, 200, 6400), (3, 50257, 160), (2048, 640, 512)]


@pytest.mark.parametrize("kernel", ["simt", "tcgen05"])
@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
def test_linear_bfloat16(kernel, m, n, k):
    ops = _ops()
    a = _randn(m, k, seed=10, dtype=torch.bfloat16)
    w = _randn(n, k, seed=11, dtype=torch.bfloat16, scale=1 / math.sqrt(k))
    bias = _randn(n, seed=12)
    exact = _linear_reference(a, w, bias, "none", None)
    out32 = torch.full((m, n), float("nan"), device=DEV)
    ops.linear(a, w, bias, out32, kernel=kernel)
    torch.testing.assert_close(out32.double(), exact, rtol=1e-4, atol=1e-4)
    out16 = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    ops.linear(a, w, bias, out16, activation="gelu_tanh", kernel=kernel)
    torch.testing.assert_close(out16.double(), _linear_reference(a, w, bias, "gelu_tanh", None),
                               rtol=1e-2, atol=1e-2)
    base = _randn(m, n, seed=13)
    acc = base.clone()
    ops.linear(a, w, None, acc, residual=True, kernel=kernel)
    torch.testing.assert_close(acc.double(), _linear_reference(a, w, None, "none", base),
                               rtol=1e-4, atol=1e-4)
    if kernel == "tcgen05":
        from ayaka_b200.kernels import gemm_tc
        gemm_tc.check_status(a.device)


@pytest.mark.parametrize("tile_n", [64, 128, 192, 256, 1128, 1192, 1256, 2192, 2256, 3002,
                                    3004])
def test_linear_tcgen05_tiles_and_strides(tile_n):
    """Every tile width, operands that are column ranges of wider buffers, rows limited."""
    ops = _ops()
    from ayaka_b200.kernels import gemm_tc
    m, n, k = 70, 333, 200
    a_wide = _randn(96, 3 * k, seed=14, dtype=torch.bfloat16)
    a = a_wide[:, k:2 * k]
    w = _randn(n, k, seed=15, dtype=torch.bfloat16, scale=1 / math.sqrt(k))
    out = torch.full((96, n + 5), float("nan"), device=DEV)[:, :n]
    gemm_tc.linear_bf16(a, w, None, out, m, 0, False, tile_n=tile_n)
    gemm_tc.check_status(a.device)
    torch.testing.assert_close(out[:m].double(), a[:m].double() @ w.double().t(),
                               rtol=1e-4, atol=1e-4)
    assert torch.isnan(out[m:]).all()
    half = torch.full((96, n + 3), float("nan"), device=DEV, dtype=torch.bfloat16)[:, :n]
    gemm_tc.linear_bf16(a, w, None, half, m, 0, False, tile_n=tile_n)
    gemm_tc.check_status(a.device)
    torch.testing.assert_close(half[:m].double(), a[:m].double() @ w.double().t(),
                               rtol=1e-2, atol=1e-2)
    assert torch.isnan(half[m:]).all()


@pytest.mark.parametrize("tile_n", [1192, 1256, 2192, 2256])
@pytest.mark.parametrize("m,n,k", [(600, 700, 520), (2048, 1600, 1600), (257, 4800, 64),
                                   (300, 712, 136)])
def test_linear_tcgen05_many_tiles(tile_n, m, n, k):
    """The persistent kernels (one CTA per tile, and CTA pairs on 256-row tiles) over more
    tiles than fit one round, every epilogue: equal to the one-tile-per-CTA kernel bit for
    bit (the same order of K), and close to float64."""
    from ayaka_b200.kernels import gemm_tc
    a = _randn(m, k, seed=20, dtype=torch.bfloat16)
    w = _randn(n, k, seed=21, dtype=torch.bfloat16, scale=1 / math.sqrt(k))
    bias = _randn(n, seed=22)
    exact = a.double() @ w.double().t() + bias.double()
    for mode in ("bf16", "f32", "residual"):
        outs = []
        for tile in (128, tile_n):
            # three rows more than the product has: they must stay as they are
            if mode == "bf16":
                out = torch.full((m + 3, n), 7.0, dtype=torch.bfloat16, device=DEV)
                gemm_tc.linear_bf16(a, w, bias, out, m, 1, False, tile_n=tile)
            elif mode == "f32":
                out = torch.full((m + 3, n), 7.0, device=DEV)
                gemm_tc.linear_bf16(a, w, bias, out, m, 0, False, tile_n=tile)
            else:
                out = torch.ones(m + 3, n, device=DEV)
                gemm_tc.linear_bf16(a, w, bias, out, m, 0, True, tile_n=tile)
            assert bool((out[m:] == (1.0 if mode == "residual" else 7.0)).all())
            outs.append(out[:m])
        gemm_tc.check_status(a.device)
        assert torch.equal(outs[0], outs[1])
        if mode == "bf16":
            want = plain.gelu(exact, "gelu_new")
            torch.testing.assert_close(outs[1].double(), want, rtol=2e-2, atol=2e-2)
        if mode == "f32":
            torch.testing.assert_close(outs[1].double(), exact, rtol=1e-4, atol=1e-4)
        if mode == "residual":
            torch.testing.assert_close(outs[1].double(), exact + 1.0, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("ranks", [2, 4])
@pytest.mark.parametrize("m,n,k", [(288, 1280, 5120), (288, 1600, 1600), (65, 136, 200),
                                   (300, 712, 136), (129, 100, 72), (500, 333, 6400)])
def test_linear_tcgen05_k_split_over_a_cluster(ranks, m, n, k):
    """A few hundred rows: 128 x 128 tiles whose K range is split over a cluster of 2 or 4
    CTAs and reduced through distributed shared memory in rank order. Every epilogue, ragged
    edges in M, N and K, rows beyond the product untouched, and the same bits on a second
    run and whatever else is in the batch (the order of the sum is fixed)."""
    from ayaka_b200.kernels import gemm_tc
    if -(-k // 64) <= -(-(-(-k // 64)) // ranks) * (ranks - 1):
        pytest.skip("fewer blocks of K than ranks")
    code = 3000 + ranks
    a = _randn(m, k, seed=24, dtype=torch.bfloat16)
    w = _randn(n, k, seed=25, dtype=torch.bfloat16, scale=1 / math.sqrt(k))
    bias = _randn(n, seed=26)
    exact = a.double() @ w.double().t() + bias.double()
    out = torch.full((m + 3, n), 7.0, device=DEV)
    gemm_tc.linear_bf16(a, w, bias, out, m, 0, False, tile_n=code)
    gemm_tc.check_status(a.device)
    assert bool((out[m:] == 7.0).all())
    torch.testing.assert_close(out[:m].double(), exact, rtol=1e-4, atol=1e-4)
    again = torch.zeros(m, n, device=DEV)
    gemm_tc.linear_bf16(a, w, bias, again, m, 0, False, tile_n=code)
    assert torch.equal(again, out[:m])
    last = min(70, m - 1)
    fewer = torch.zeros(last, n, device=DEV)
    gemm_tc.linear_bf16(a[m - last:].contiguous(), w, bias, fewer, last, 0, False, tile_n=code)
    assert torch.equal(fewer, out[m - last:m])  # a row's sum does not depend on the batch
    half = torch.full((m + 3, n), 7.0, dtype=torch.bfloat16, device=DEV)
    gemm_tc.linear_bf16(a, w, bias, half, m, 1, False, tile_n=code)
    assert bool((half[m:] == 7.0).all())
    torch.testing.assert_close(half[:m].double(), plain.gelu(exact, "gelu_new"), rtol=2e-2,
                               atol=2e-2)
    acc = torch.ones(m + 3, n, device=DEV)
    gemm_tc.linear_bf16(a, w, bias, acc, m, 0, True, tile_n=code)
    assert bool((acc[m:] == 1.0).all())
    torch.testing.assert_close(acc[:m].double(), exact + 1.0, rtol=1e-4, atol=1e-4)
    gemm_tc.check_status(a.device)


@pytest.mark.parametrize("splits", [-100, -2, -4, -8, 0])
@pytest.mark.parametrize("m", [1, 2, 8, 16, 17, 24, 33, 40, 57, 64])
def test_linear_tcgen05_few_rows(m, splits):
    """The weight-streaming kernel of decode steps: every padded row count, every K split
    (a negative tile selects it: -100 one CTA per tile, -2/-4/-8 that many cluster CTAs)."""
    from ayaka_b200.kernels import gemm_tc
    for n, k in ((1600, 1600), (300, 6400), (50257, 160), (136, 72)):
        a = _randn(m, k, seed=30, dtype=torch.bfloat16)
        w = _randn(n, k, seed=31, dtype=torch.bfloat16, scale=1 / math.sqrt(k))
        bias = _randn(n, seed=32)
        exact = a.double() @ w.double().t() + bias.double()
        out = torch.full((m + 1, n), float("nan"), device=DEV)
        gemm_tc.linear_bf16(a, w, bias, out, m, 0, False, tile_n=splits)
        gemm_tc.check_status(a.device)
        torch.testing.assert_close(out[:m].double(), exact, rtol=1e-4, atol=1e-4)
        assert torch.isnan(out[m:]).all()
        base = _randn(m, n, seed=33)
        acc = base.clone()
        gemm_tc.linear_bf16(a, w, bias, acc, m, 0, True, tile_n=splits)
        torch.testing.assert_close(acc.double(), exact + base.double(), rtol=1e-4, atol=1e-4)
        half = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
        gemm_tc.linear_bf16(a, w, bias, half, m, 2, False, tile_n=splits)
        torch.testing.assert_close(half.double(), plain.gelu(exact, "gelu"), rtol=1e-2, atol=1e-2)
    gemm_tc.check_status(a.device)


def test_linear_wide_products_of_33_to_64_rows():
    """Products too wide for a K split (more than 32 tiles of 128 columns) take 64-column
    tiles with the rows as the 128-row operand from 33 rows on: the library's own choice at
    the row counts around that border, every epilogue."""
    from ayaka_b200.kernels import gemm_tc
    n, k = 4800, 1600
    w = _randn(n, k, seed=41, dtype=torch.bfloat16, scale=1 / math.sqrt(k))
    bias = _randn(n, seed=42)
    for m in (32, 33, 48, 64):
        a = _randn(m, k, seed=40 + m, dtype=torch.bfloat16)
        exact = a.double() @ w.double().t() + bias.double()
        out = torch.full((m + 1, n), float("nan"), device=DEV)
        gemm_tc.linear_bf16(a, w, bias, out, m, 0, False)
        torch.testing.assert_close(out[:m].double(), exact, rtol=1e-4, atol=1e-4)
        assert torch.isnan(out[m:]).all()
        base = _randn(m, n, seed=43)
        acc = base.clone()
        gemm_tc.linear_bf16(a, w, bias, acc, m, 0, True)
        torch.testing.assert_close(acc.double(), exact + base.double(), rtol=1e-4, atol=1e-4)
        half = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
        gemm_tc.linear_bf16(a, w, bias, half, m, 1, False)
        torch.testing.assert_close(half.double(), plain.gelu(exact, "gelu_new"),
                                   rtol=1e-2, atol=1e-2)
    gemm_tc.check_status(a.device)


@pytest.mark.parametrize("m", [1, 8, 40])
@pytest.mark.parametrize("n,k", [(300, 96), (136, 840)])
def test_linear_normed(m, n, k):
    """Norm, then product, then activation, with a gather of the rows: against float64."""
    ops = _ops()
    for dtype in (torch.float32, torch.bfloat16):
        x = _randn(m + 3, k, seed=40, scale=2.0) + 0.5
        gamma, beta = _randn(k, seed=41) * 0.2 + 1.0, _randn(k, seed=42) * 0.3
        w = _randn(n, k, seed=43, dtype=dtype, scale=1 / math.sqrt(k))
        bias = _randn(n, seed=44)
        index = torch.arange(m + 2, 2, -1, dtype=torch.int32, device=DEV)  # rows m+2 .. 3
        normed = plain.layer_norm(x.double()[index.long()], gamma.double(), beta.double(), 1e-5)
        exact = plain.gelu(normed.to(dtype).double() @ w.double().t() + bias.double(),
                           "gelu_new")
        out = torch.full((m + 1, n), float("nan"), device=DEV)
        scratch = torch.zeros(m, k, dtype=dtype, device=DEV)
        ops.linear_normed(x, gamma, beta, 1e-5, w, bias, out, scratch=scratch, count=m,
                          activation="gelu_tanh", row_index=index)
        tol = 1e-4 if dtype == torch.float32 else 2e-3
        torch.testing.assert_close(out[:m].double(), exact, rtol=tol, atol=tol)
        assert torch.isnan(out[m:]).all()


@pytest.mark.parametrize("code", [-201, -202])
@pytest.mark.parametrize("m", [1, 5, 8, 9, 16])
def test_linear_at_most_16_rows(m, code):
    """The kernel that holds its weights on chip before the rows arrive: one CTA per 16
    (tile code -201) or 32 columns (-202, without a K split), K over a cluster from 57 steps
    of 32 on (splits 1, 2, 4, 8), tails in every dimension, every epilogue; rows beyond the
    product stay as they are; both codes give the same bits."""
    from ayaka_b200.kernels import gemm_tc
    for n, k in ((1600, 1600), (300, 6400), (50257, 160), (136, 72), (77, 3200), (333, 14336),
                 (17, 8)):
        if code == -202 and k > 1792:
            continue
        a = _randn(m, k, seed=50, dtype=torch.bfloat16)
        w = _randn(n, k, seed=51, dtype=torch.bfloat16, scale=1 / math.sqrt(k))
        bias = _randn(n, seed=52)
        exact = a.double() @ w.double().t() + bias.double()
        out = torch.full((m + 1, n), float("nan"), device=DEV)
        gemm_tc.linear_bf16(a, w, bias, out, m, 0, False, tile_n=code)
        torch.testing.assert_close(out[:m].double(), exact, rtol=1e-4, atol=1e-4)
        assert torch.isnan(out[m:]).all()
        other = torch.zeros(m, n, device=DEV)
        gemm_tc.linear_bf16(a, w, bias, other, m, 0, False, tile_n=-201)
        assert torch.equal(other, out[:m])
        again = torch.zeros(m, n, device=DEV)
        gemm_tc.linear_bf16(a, w, bias, again, m, 0, False, tile_n=code)
        assert torch.equal(again, out[:m])
        base = _randn(m, n, seed=53)
        acc = base.clone()
        gemm_tc.linear_bf16(a, w, None, acc, m, 0, True, tile_n=code)
        torch.testing.assert_close(acc.double(), exact - bias.double() + base.double(),
                                   rtol=1e-4, atol=1e-4)
        half = torch.full((m + 1, n), 7.0, dtype=torch.bfloat16, device=DEV)
        gemm_tc.linear_bf16(a, w, bias, half, m, 1, False, tile_n=code)
        torch.testing.assert_close(half[:m].double(), plain.gelu(exact, "gelu_new"),
                                   rtol=1e-2, atol=1e-2)
        assert bool((half[m:] == 7.0).all())
        # a row's sums do not depend on the other rows of the step or on its place among them
        if m > 1:
            alone = torch.zeros(1, n, device=DEV)
            gemm_tc.linear_bf16(a[m - 1:].contiguous(), w, bias, alone, 1, 0, False, tile_n=code)
            assert torch.equal(alone[0], out[m - 1])
    gemm_tc.check_status(a.device)


def test_linear_at_most_16_rows_refuses_what_it_cannot_take():
    from ayaka_b200.errors import BackendError
    from ayaka_b200.kernels import gemm_tc
    w = _randn(64, 20480, seed=54, dtype=torch.bfloat16)
    for m, k in ((17, 64), (4, 20480)):  # too many rows; K beyond eight CTAs' shared memory
        a = _randn(m, k, seed=55, dtype=torch.bfloat16)
        out = torch.zeros(m, 64, device=DEV)
        with pytest.raises(BackendError):
            gemm_tc.linear_bf16(a, w[:, :k], None, out, m, 0, False, tile_n=-200)
    a = _randn(4, 3200, seed=55, dtype=torch.bfloat16)  # two column tiles and a K split
    with pytest.raises(BackendError):
        gemm_tc.linear_bf16(a, w[:, :3200], None, torch.zeros(4, 64, device=DEV), 4, 0, False,
                            tile_n=-202)
    # left to itself the library takes another kernel for them
    a = _randn(4, 20480, seed=56, dtype=torch.bfloat16)
    out = torch.zeros(4, 64, device=DEV)
    gemm_tc.linear_bf16(a, w, None, out, 4, 0, False)
    torch.testing.assert_close(out.double(), a.double() @ w.double().t(), rtol=1e-3, atol=1e-3)


def test_linear_tcgen05_few_rows_is_reproducible():
    from ayaka_b200.kernels import gemm_tc
    a = _randn(8, 6400, seed=34, dtype=torch.bfloat16)
    w = _randn(1600, 6400, seed=35, dtype=torch.bfloat16, scale=0.02)
    first = torch.zeros(8, 1600, device=DEV)
    gemm_tc.linear_bf16(a, w, None, first, 8, 0, False)
    for _ in range(5):
        again = torch.zeros(8, 1600, device=DEV)
        gemm_tc.linear_bf16(a, w, None, again, 8, 0, False)
        assert torch.equal(first, again)


def test_linear_bfloat16_unaligned_k_takes_the_cuda_core_kernel():
    ops = _ops()
    a = _randn(9, 700, seed=16, dtype=torch.bfloat16)
    w = _randn(40, 700, seed=17, dtype=torch.bfloat16, scale=0.05)
    out = torch.zeros(9, 40, device=DEV)
    ops.linear(a, w, None, out)  # 700 * 2 bytes is no multiple of 16: TMA cannot read it
    torch.testing.assert_close(out.double(), a.double() @ w.double().t(), rtol=1e-4, atol=1e-4)


def test_linear_batch_invariance():
    """A row's result does not depend on how many rows run with it."""
    ops = _ops()
    for dtype, kernel in ((torch.float32, "simt"), (torch.bfloat16, "tcgen05"),
                          (torch.bfloat16, "simt")):
        a = _randn(300, 320, seed=18, dtype=dtype)
        w = _randn(200, 320, seed=19, dtype=dtype, scale=0.05)
        whole = torch.zeros(300, 200, device=DEV)
        ops.linear(a, w, None, whole, kernel=kernel)
        for rows in (65, 70, 129):
            part = torch.zeros(rows, 200, device=DEV)
            ops.linear(a[:rows].contiguous(), w, None, part, kernel=kernel)
            assert torch.equal(part, whole[:rows])
        # up to 64 rows the bfloat16 tensor-core product splits K over a cluster, up to 16
        # rows over the warps of a CTA: the same sums in another order, equal within fp32
        # rounding and equal among the row counts of their class
        for most, fewer in ((64, (17, 33)), (16, (1, 7, 9))):
            small = torch.zeros(most, 200, device=DEV)
            ops.linear(a[:most].contiguous(), w, None, small, kernel=kernel)
            torch.testing.assert_close(small, whole[:most], rtol=1e-5, atol=1e-5)
            for rows in fewer:
                part = torch.zeros(rows, 200, device=DEV)
                ops.linear(a[:rows].contiguous(), w, None, part, kernel=kernel)
                assert torch.equal(part, small[:rows])


# ---------------------------------------------------------------------------------------------
def _paged_case(lengths, rows_per_request, heads, kv_heads, head_dim, page_size, dtype, seed,
                boost=None):
    """Random q/k/v for whole sequences; K/V scattered into NaN-poisoned pages handed out in
    reverse order; the step holds the last rows_per_request[b] rows of each request."""
    g = torch.Generator().manual_seed(seed)
    pages_needed = [-(-n // page_size) for n in lengths]
    num_pages = sum(pages_needed) + 3
    k_pages = torch.full((num_pages, kv_heads, page_size, head_dim), float("nan"))
    v_pages = torch.full_like(k_pages, float("nan"))
    free = list(range(num_pages - 1, 0, -1))
    width = max(pages_needed)
    table = torch.zeros(len(lengths), width, dtype=torch.int32)
    seqs = []
    for b, n in enumerate(lengths):
        q = torch.randn(n, heads, head_dim, generator=g)
        k = torch.randn(n, kv_heads, head_dim, generator=g)
        v = torch.randn(n, kv_heads, head_dim, generator=g)
        if boost is not None:
            row, key = boost
            if row < n:
                k[key] = q[row, ::heads // kv_heads] * 3.0  # one score stands out for every head
        q, k, v = (t.to(dtype).float() for t in (q, k, v))
        seqs.append((q, k, v))
        for i in range(pages_needed[b]):
            table[b, i] = free.pop(0)
        for t in range(n):
            page, slot = int(table[b, t // page_size]), t % page_size
            k_pages[page, :, slot] = k[t]
            v_pages[page, :, slot] = v[t]
    q_rows, req, pos = [], [], []
    for b, (n, r) in enumerate(zip(lengths, rows_per_request)):
        q_rows.append(seqs[b][0][n - r:].reshape(r, heads * head_dim))
        req += [b] * r
        pos += list(range(n - r, n))
    return (torch.cat(q_rows).to(dtype).to(DEV), k_pages.to(dtype).to(DEV),
            v_pages.to(dtype).to(DEV), table.to(DEV),
            torch.tensor(req, dtype=torch.int32, device=DEV),
            torch.tensor(pos, dtype=torch.int32, device=DEV), seqs)


def _attention_reference(seqs, lengths, rows_per_request, heads, kv_heads, scale, window):
    outs = []
    for (q, k, v), n, r in zip(seqs, lengths, rows_per_request):
        rep = heads // kv_heads
        full = plain.causal_attention(q.double(), k.double().repeat_interleave(rep, 1),
                                      v.double().repeat_interleave(rep, 1), scale, window)
        outs.append(full[n - r:].reshape(r, -1))
    return torch.cat(outs)


ATTN_CASES = [
    # lengths, rows, heads, kv_heads, head_dim, page, window
    ((5, 17, 32, 9), (5, 17, 32, 9), 4, 4, 16, 16, 0),
    ((1, 64, 130), (1, 1, 1), 3, 3, 32, 16, 0),
    ((40, 33, 70), (2, 33, 1), 6, 2, 48, 8, 0),
    ((300,), (300,), 2, 1, 128, 16, 0),
    ((90, 200), (17, 5), 2, 2, 256, 32, 0),
    ((100, 257), (30, 1), 5, 5, 64, 16, 24),
    ((67,), (67,), 3, 1, 80, 4, 5),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ATTN_CASES)
def test_attention_paged(dtype, case):
    ops = _ops()
    lengths, rows, heads, kv_heads, head_dim, page, window = case
    q, k_pages, v_pages, table, req, pos, seqs = _paged_case(
        lengths, rows, heads, kv_heads, head_dim, page, dtype, seed=20)
    out = torch.full((q.shape[0] + 2, heads * head_dim), float("nan"), dtype=dtype, device=DEV)
    scale = 0.7 / math.sqrt(head_dim)
    ops.attention(q, k_pages, v_pages, table, req, pos, out, num_heads=heads, scale=scale,
                  window=window, rows=q.shape[0])
    expected = _attention_reference(seqs, lengths, rows, heads, kv_heads, scale, window)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out[:q.shape[0]].double().cpu(), expected, **tol)
    assert torch.isnan(out[q.shape[0]:].float()).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_a_far_key_among_hundreds(dtype):
    """Row 699 of a 700-token request must find key 3 (first page); row 350 key 349."""
    ops = _ops()
    lengths, rows, heads, kv_heads, head_dim, page = (700,), (700,), 2, 2, 64, 16
    for boost in ((699, 3), (350, 349), (16, 15), (16, 0)):
        q, k_pages, v_pages, table, req, pos, seqs = _paged_case(
            lengths, rows, heads, kv_heads, head_dim, page, dtype, seed=21, boost=boost)
        out = torch.zeros(700, heads * head_dim, dtype=dtype, device=DEV)
        ops.attention(q, k_pages, v_pages, table, req, pos, out, num_heads=heads, scale=1.0)
        row, key = boost
        got = out[row].float().cpu().reshape(heads, head_dim)
        # the boosted key takes almost all the weight, so the output is that key's value
        torch.testing.assert_close(got, seqs[0][2][key], rtol=2e-2, atol=2e-2)
        expected = _attention_reference(seqs, lengths, rows, heads, kv_heads, 1.0, 0)
        tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=2e-2,
                                                                               atol=2e-2)
        torch.testing.assert_close(out.double().cpu(), expected, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,head_dim,page", [(25, 64, 16), (3, 12, 5), (2, 72, 8)])
def test_kv_store_scatters_rows(dtype, heads, head_dim, page):
    """Rows go to their slots and nowhere else, in 16-byte pieces where the shapes allow
    (and element by element where they do not: a head size of 12)."""
    ops = _ops()
    rows, pages = 300, 80
    width = heads * head_dim
    qkv = _randn(rows, 3 * width, seed=23, dtype=dtype)
    order = torch.randperm(pages * page, generator=torch.Generator().manual_seed(5))[:rows]
    order[::7] = -1  # some rows store nothing
    slots = order.to(torch.int32).to(DEV)
    k_pages = torch.full((pages, heads, page, head_dim), float("nan"), dtype=dtype, device=DEV)
    v_pages = torch.full_like(k_pages, float("nan"))
    ops.kv_store(qkv[:, width:2 * width], qkv[:, 2 * width:], slots, k_pages, v_pages)
    want_k = torch.full_like(k_pages, float("nan"))
    want_v = torch.full_like(v_pages, float("nan"))
    for r, slot in enumerate(order.tolist()):
        if slot >= 0:
            want_k[slot // page, :, slot % page] = qkv[r, width:2 * width].view(heads, head_dim)
            want_v[slot // page, :, slot % page] = qkv[r, 2 * width:].view(heads, head_dim)
    assert torch.equal(torch.nan_to_num(k_pages.float(), nan=-7.0),
                       torch.nan_to_num(want_k.float(), nan=-7.0))
    assert torch.equal(torch.nan_to_num(v_pages.float(), nan=-7.0),
                       torch.nan_to_num(want_v.float(), nan=-7.0))


@pytest.mark.parametrize("rows,width,heads,kv_heads,head_dim,page", [
    (2048, 1600, 25, 25, 64, 16),   # the persistent kernel, 192-wide tiles that straddle q | k
    (300, 136, 4, 2, 32, 8),        # one tile per CTA, grouped heads, a ragged last row tile
    (200, 72, 2, 1, 96, 8),         # queries 192 wide, one key/value head of 96
    (130, 200, 4, 2, 96, 4),        # a head size that is no power of two
    (65, 64, 2, 2, 32, 16),
])
def test_linear_that_also_stores_keys_and_values(rows, width, heads, kv_heads, head_dim, page):
    """The fused projection whose epilogue writes the key and value columns into the pages
    (and the query columns to its output) gives bit for bit what the product followed by the
    store gives, and stores nothing for rows without a slot. A product that cannot carry the store says so and does nothing."""
    ops = _ops()
    q_width, kv_width = heads * head_dim, kv_heads * head_dim
    n = q_width + 2 * kv_width
    a = _randn(rows + 3, width, seed=41, dtype=torch.bfloat16)
    w = (_randn(n, width, seed=42) * 0.1).bfloat16()
    bias = _randn(n, seed=43)
    pages = -(-rows // page) + 5
    order = torch.randperm(pages * page, generator=torch.Generator().manual_seed(6))[:rows + 3]
    order[::11] = -1
    slots = order.to(torch.int32).to(DEV)

    def empty_pages():
        return torch.full((pages, kv_heads, page, head_dim), float("nan"), dtype=torch.bfloat16,
                          device=DEV)

    out_a = torch.zeros(rows + 3, n, dtype=torch.bfloat16, device=DEV)
    k_a, v_a = empty_pages(), empty_pages()
    assert ops.linear_kv(a, w, bias, out_a, slots, k_a, v_a, q_width=q_width, rows=rows)
    from ayaka_b200.kernels import gemm_tc
    gemm_tc.check_status(a.device)
    out_b = torch.zeros_like(out_a)
    k_b, v_b = empty_pages(), empty_pages()
    ops.linear(a, w, bias, out_b, rows=rows)
    ops.kv_store(out_b[:, q_width:q_width + kv_width], out_b[:, q_width + kv_width:], slots,
                 k_b, v_b, rows=rows)
    assert torch.equal(out_a[:, :q_width], out_b[:, :q_width])
    assert not out_a[:, q_width:].any()  # keys and values went to the cache only
    for got, want in ((k_a, k_b), (v_a, v_b)):
        assert torch.equal(torch.nan_to_num(got.float(), nan=-7.0),
                           torch.nan_to_num(want.float(), nan=-7.0))
    assert int((~torch.isnan(k_a.float())).sum()) == int((order[:rows] >= 0).sum()) * kv_width
    # few rows: the weight-streaming kernel has no such epilogue
    assert not ops.linear_kv(a, w, bias, out_a, slots, k_a, v_a, q_width=q_width, rows=64)
    # float32: not this kernel's business
    assert not ops.linear_kv(a.float(), w.float(), bias, out_a.float(), slots, k_a.float(),
                             v_a.float(), q_width=q_width, rows=rows)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kv_store_then_attend(dtype):
    """The store writes exactly the slots it is given; a padding row stores nothing and a
    padding request's rows come out zero."""
    ops = _ops()
    heads, head_dim, page = 3, 32, 4
    k_pages = torch.full((6, heads, page, head_dim), float("nan"), dtype=dtype, device=DEV)
    v_pages = torch.full_like(k_pages, float("nan"))
    qkv = _randn(5, 3 * heads * head_dim, seed=22, dtype=dtype)
    width = heads * head_dim
    slots = torch.tensor([5 * page + 0, 5 * page + 1, 5 * page + 2, 2 * page + 3, -1],
                         dtype=torch.int32, device=DEV)
    ops.kv_store(qkv[:, width:2 * width], qkv[:, 2 * width:], slots, k_pages, v_pages)
    assert torch.equal(k_pages[5, :, 1], qkv[1, width:2 * width].reshape(heads, head_dim))
    assert torch.equal(v_pages[2, :, 3], qkv[3, 2 * width:].reshape(heads, head_dim))
    written = ~torch.isnan(k_pages.float())
    assert int(written.sum()) == 4 * heads * head_dim
    table = torch.tensor([[5, 0]], dtype=torch.int32, device=DEV)
    req = torch.tensor([0, 0, 0, -1], dtype=torch.int32, device=DEV)
    pos = torch.tensor([0, 1, 2, 0], dtype=torch.int32, device=DEV)
    out = torch.full((4, width), float("nan"), dtype=dtype, device=DEV)
    ops.attention(qkv[:4, :width], k_pages, v_pages, table, req, pos, out, num_heads=heads,
                  scale=0.2)
    q = qkv[:3, :width].float().cpu().reshape(3, heads, head_dim)
    k = qkv[:3, width:2 * width].float().cpu().reshape(3, heads, head_dim)
    v = qkv[:3, 2 * width:].float().cpu().reshape(3, heads, head_dim)
    expected = plain.causal_attention(q, k, v, 0.2).reshape(3, width)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out[:3].float().cpu(), expected, **tol)
    assert torch.equal(out[3].float(), torch.zeros(width, device=DEV))


@pytest.mark.parametrize("kernel", ["tcgen05", "mma"])
@pytest.mark.parametrize("case", ATTN_CASES + [
    ((1024, 1024), (1024, 1024), 25, 25, 64, 16, 0),
    ((700, 3, 200), (130, 3, 65), 4, 2, 32, 16, 0),
    ((500,), (250,), 2, 2, 64, 128, 100),
    ((700, 3, 200, 129), (130, 3, 65, 129), 6, 2, 64, 16, 0),
    ((3000,), (1500,), 2, 1, 64, 12, 0),
    ((900, 260), (513, 255), 3, 3, 64, 8, 300),
    ((600, 300), (600, 257), 2, 1, 64, 256, 0),   # pages larger than a block of keys
    ((700,), (300,), 2, 2, 64, 32, 150),
    ((515, 64), (515, 64), 1, 1, 64, 64, 0),
])
def test_attention_prefill_tensor_cores(case, kernel):
    """The bfloat16 flash kernels for prompt portions (tcgen05 for head size 64, tiles of 128
    rows; mma.sync for every head size, tiles of 64): every head size class, grouped heads,
    windows, requests of one row beside long ones, page sizes that are no power of two, pages
    in scrambled order."""
    ops = _ops()
    lengths, rows, heads, kv_heads, head_dim, page, window = case
    if head_dim % 16:
        pytest.skip("head sizes are multiples of 16")
    if kernel == "tcgen05" and head_dim != 64:
        pytest.skip("the tcgen05 kernel serves head size 64")
    q, k_pages, v_pages, table, req, pos, seqs = _paged_case(
        lengths, rows, heads, kv_heads, head_dim, page, torch.bfloat16, seed=25, boost=(699, 3))
    n = q.shape[0]
    starts = [0]
    for r in rows:
        starts.append(starts[-1] + r)
    row_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    kv_len = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    out = torch.full((n + 2, heads * head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    scale = 0.7 / math.sqrt(head_dim)
    ops.attention_prefill(q, k_pages, v_pages, table, row_start, kv_len, out, num_heads=heads,
                          scale=scale, host_rows=list(rows), window=window, kernel=kernel)
    from ayaka_b200.kernels import gemm_tc
    gemm_tc.check_status(q.device)
    expected = _attention_reference(seqs, lengths, rows, heads, kv_heads, scale, window)
    torch.testing.assert_close(out[:n].double().cpu(), expected, rtol=2e-2, atol=2e-2)
    assert torch.isnan(out[n:].float()).all()
    # the plain CUDA-core kernel agrees far more closely than either agrees with float64
    plain_out = torch.zeros(n, heads * head_dim, dtype=torch.bfloat16, device=DEV)
    ops.attention(q, k_pages, v_pages, table, req, pos, plain_out, num_heads=heads, scale=scale,
                  window=window)
    torch.testing.assert_close(out[:n].float(), plain_out.float(), rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("sign", [-1.0, 1.0, 0.0])
def test_attention_prefill_first_reference(sign):
    """The tcgen05 kernel takes 0 as a row's first reference when its first maximum is within
    2^8 of that and moves it otherwise: scores that are all far below zero (every probability
    would underflow against 0), all far above (they would overflow), and ordinary ones."""
    ops = _ops()
    n, heads, head_dim, page = 300, 2, 64, 16
    g = torch.Generator().manual_seed(31)
    unit = torch.nn.functional.normalize(torch.randn(head_dim, generator=g), dim=0)
    q = 0.3 * torch.randn(n, heads, head_dim, generator=g) + 6.0 * abs(sign) * unit
    k = 0.3 * torch.randn(n, heads, head_dim, generator=g) + 6.0 * sign * unit
    v = torch.randn(n, heads, head_dim, generator=g)
    q, k, v = (t.bfloat16().float() for t in (q, k, v))
    scale = 1.0  # scores near 36 * sign: e^-36 and e^36 against a reference of 0
    pages = -(-n // page)
    k_pages = torch.full((pages + 1, heads, page, head_dim), float("nan"))
    v_pages = torch.full_like(k_pages, float("nan"))
    for t in range(n):
        k_pages[1 + t // page, :, t % page] = k[t]
        v_pages[1 + t // page, :, t % page] = v[t]
    table = torch.arange(1, pages + 1, dtype=torch.int32).view(1, pages).to(DEV)
    out = torch.zeros(n, heads * head_dim, dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill(
        q.reshape(n, -1).bfloat16().to(DEV), k_pages.bfloat16().to(DEV),
        v_pages.bfloat16().to(DEV), table,
        torch.tensor([0, n], dtype=torch.int32, device=DEV),
        torch.tensor([n], dtype=torch.int32, device=DEV), out, num_heads=heads, scale=scale,
        host_rows=[n], kernel="tcgen05")
    from ayaka_b200.kernels import gemm_tc
    gemm_tc.check_status(out.device)
    expected = plain.causal_attention(q.double(), k.double(), v.double(), scale)
    torch.testing.assert_close(out.double().cpu(), expected.reshape(n, -1), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("splits", [1, 2, 5, 8, 16, -2, -7])
@pytest.mark.parametrize("case", [
    # lengths, heads, kv_heads, head_dim, page, window
    ((1, 64, 130, 700), 3, 3, 32, 16, 0),
    ((1000, 17), 25, 25, 64, 16, 0),
    ((40, 33, 70, 2), 6, 2, 48, 8, 0),
    ((300, 5), 2, 1, 128, 16, 0),
    ((90,), 2, 2, 256, 32, 0),
    ((100, 257, 3), 4, 4, 16, 16, 24),
    ((67, 400), 3, 1, 80, 4, 50),
])
def test_attention_decode_split_kv(dtype, splits, case):
    """One row per request, the keys split over several CTAs and merged by the last one;
    twice in a row on the same scratch, which the kernel must leave ready for reuse."""
    ops = _ops()
    ops.set_decode_tensor_cores(False)  # this kernel also where the other would be chosen
    try:
        _split_kv_case(ops, dtype, splits, case)
    finally:
        ops.set_decode_tensor_cores(True)


def _split_kv_case(ops, dtype, splits, case):
    lengths, heads, kv_heads, head_dim, page, window = case
    # a negative count: that many splits merged on chip by a thread-block cluster (no
    # scratch); positive: through the scratch buffers and a ticket
    on_chip, splits = splits < 0, abs(splits)
    rows = (1,) * len(lengths)
    q, k_pages, v_pages, table, req, pos, seqs = _paged_case(
        lengths, rows, heads, kv_heads, head_dim, page, dtype, seed=24, boost=(999, 2))
    n = q.shape[0]
    # a padding row in the middle of the batch
    q = torch.cat([q[:1], torch.full_like(q[:1], float("nan")), q[1:]])
    req = torch.cat([req[:1], torch.tensor([-1], dtype=torch.int32, device=DEV), req[1:]])
    pos = torch.cat([pos[:1], torch.zeros(1, dtype=torch.int32, device=DEV), pos[1:]])
    partial = torch.full(((n + 1) * heads * splits * (head_dim + 2),), float("nan"), device=DEV)
    tickets = torch.zeros((n + 1) * heads, dtype=torch.int32, device=DEV)
    if on_chip:
        partial = tickets = None
    scale = 0.9 / math.sqrt(head_dim)
    expected = _attention_reference(seqs, lengths, rows, heads, kv_heads, scale, window)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    for _ in range(2):
        out = torch.full((n + 1, heads * head_dim), float("nan"), dtype=dtype, device=DEV)
        ops.attention_decode(q, k_pages, v_pages, table, req, pos, out, num_heads=heads,
                             scale=scale, window=window, splits=splits, partial=partial,
                             tickets=tickets)
        got = torch.cat([out[:1], out[2:]]).double().cpu()
        torch.testing.assert_close(got, expected, **tol)
        assert torch.equal(out[1].float(), torch.zeros(heads * head_dim, device=DEV))
        assert tickets is None or int(tickets.abs().sum()) == 0
    # the fused KV store: wipe each row's own slot in the cache, hand its key and value in
    # from "this step's projection", and the kernel must both use and store them
    kv_width = kv_heads * head_dim
    k_new = torch.zeros(n + 1, kv_width, dtype=dtype, device=DEV)
    v_new = torch.zeros_like(k_new)
    wiped_k, wiped_v = k_pages.clone(), v_pages.clone()
    at = 0
    for b, length in enumerate(lengths):
        row = at if at == 0 else at + 1  # the padding row sits at index 1
        where, slot = int(table[b, (length - 1) // page]), (length - 1) % page
        k_new[row] = k_pages[where, :, slot].reshape(-1)
        v_new[row] = v_pages[where, :, slot].reshape(-1)
        wiped_k[where, :, slot] = float("nan")
        wiped_v[where, :, slot] = float("nan")
        at += 1
    out = torch.full((n + 1, heads * head_dim), float("nan"), dtype=dtype, device=DEV)
    ops.attention_decode(q, wiped_k, wiped_v, table, req, pos, out, num_heads=heads, scale=scale,
                         window=window, splits=splits, partial=partial, tickets=tickets,
                         k_new=k_new, v_new=v_new, store=True)
    got = torch.cat([out[:1], out[2:]]).double().cpu()
    torch.testing.assert_close(got, expected, **tol)
    assert torch.equal(wiped_k.nan_to_num(7.0), k_pages.nan_to_num(7.0))
    assert torch.equal(wiped_v.nan_to_num(7.0), v_pages.nan_to_num(7.0))


@pytest.mark.parametrize("case", [
    # lengths, heads, kv_heads, head_dim, page, window
    ((1000, 17), 25, 25, 64, 16, 0),
    ((300, 5), 2, 1, 128, 16, 0),
    ((1, 2, 16, 17, 33, 130), 4, 2, 64, 8, 0),
    ((100, 257, 3), 4, 4, 64, 16, 24),
    ((67, 400), 6, 2, 128, 4, 50),
    ((70, 31, 48), 3, 3, 64, 12, 0),
])
@pytest.mark.parametrize("ask", [-4, -8, -16])
def test_attention_decode_on_tensor_cores(case, ask):
    """The decode kernel for many rows (both products as warp-level MMAs over tiles of 16
    keys; ``splits=-4`` / ``-8`` ask for it with four / eight warps per (row, head) whatever
    the row count): against plain attention, with a
    padding row, twice in a row, then with each row's own key and value handed in from the
    projection and stored by the kernel."""
    ops = _ops()
    dtype = torch.bfloat16
    lengths, heads, kv_heads, head_dim, page, window = case
    if ask == -16 and head_dim > 64:
        pytest.skip("sixteen warps are for head size 64")
    rows = (1,) * len(lengths)
    q, k_pages, v_pages, table, req, pos, seqs = _paged_case(
        lengths, rows, heads, kv_heads, head_dim, page, dtype, seed=27, boost=(999, 2))
    n = q.shape[0]
    q = torch.cat([q[:1], torch.full_like(q[:1], float("nan")), q[1:]])
    req = torch.cat([req[:1], torch.tensor([-1], dtype=torch.int32, device=DEV), req[1:]])
    pos = torch.cat([pos[:1], torch.zeros(1, dtype=torch.int32, device=DEV), pos[1:]])
    scale = 0.9 / math.sqrt(head_dim)
    expected = _attention_reference(seqs, lengths, rows, heads, kv_heads, scale, window)
    tol = dict(rtol=2e-2, atol=2e-2)
    for _ in range(2):
        out = torch.full((n + 1, heads * head_dim), float("nan"), dtype=dtype, device=DEV)
        ops.attention_decode(q, k_pages, v_pages, table, req, pos, out, num_heads=heads,
                             scale=scale, window=window, splits=ask)
        got = torch.cat([out[:1], out[2:]]).double().cpu()
        torch.testing.assert_close(got, expected, **tol)
        assert torch.equal(out[1].float(), torch.zeros(heads * head_dim, device=DEV))
    kv_width = kv_heads * head_dim
    k_new = torch.zeros(n + 1, kv_width, dtype=dtype, device=DEV)
    v_new = torch.zeros_like(k_new)
    wiped_k, wiped_v = k_pages.clone(), v_pages.clone()
    for b, length in enumerate(lengths):
        row = b if b == 0 else b + 1  # the padding row sits at index 1
        where, slot = int(table[b, (length - 1) // page]), (length - 1) % page
        k_new[row] = k_pages[where, :, slot].reshape(-1)
        v_new[row] = v_pages[where, :, slot].reshape(-1)
        wiped_k[where, :, slot] = float("nan")
        wiped_v[where, :, slot] = float("nan")
    out = torch.full((n + 1, heads * head_dim), float("nan"), dtype=dtype, device=DEV)
    ops.attention_decode(q, wiped_k, wiped_v, table, req, pos, out, num_heads=heads, scale=scale,
                         window=window, splits=ask, k_new=k_new, v_new=v_new, store=True)
    got = torch.cat([out[:1], out[2:]]).double().cpu()
    torch.testing.assert_close(got, expected, **tol)
    assert torch.equal(wiped_k.nan_to_num(7.0), k_pages.nan_to_num(7.0))
    assert torch.equal(wiped_v.nan_to_num(7.0), v_pages.nan_to_num(7.0))


def test_attention_refuses_what_it_cannot_do():
    ops = _ops()
    from ayaka_b200.errors import BackendError
    q = torch.zeros(1, 24, device=DEV)
    pages = torch.zeros(2, 1, 4, 24, device=DEV)
    table = torch.ones(1, 1, dtype=torch.int32, device=DEV)
    zero = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(BackendError):
        ops.attention(q, pages[..., :20].contiguous(), pages[..., :20].contiguous(), table, zero,
                      zero, q[:, :20].contiguous(), num_heads=1, scale=1.0)  # head_dim 20


# ---------------------------------------------------------------------------------------------
def test_argmax_smallest_id_on_ties():
    ops = _ops()
    logits = _randn(6, 50257, seed=23)
    logits[0, 77] = logits[0, 40000] = 9.0
    logits[1, 50256] = 11.0
    logits[2, 0] = 12.0
    logits[3] = 1.5
    logits[4, 5] = float("nan")
    out = torch.full((6,), -1, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out)
    expected = [plain.argmax_smallest_id(torch.nan_to_num(row, nan=-1e30)) for row in logits.cpu()]
    assert out.tolist() == expected
    assert out.tolist()[:4] == [77, 50256, 0, 0]
    split = torch.full((6,), -1, dtype=torch.int32, device=DEV)
    scratch = torch.full((2 * 6 * ops.ARGMAX_PARTS,), float("nan"), device=DEV)
    ops.argmax(logits, split, scratch=scratch)  # the two-stage version
    assert split.tolist() == expected
    tiny = torch.tensor([[3.0, 5.0, 5.0]], device=DEV)  # fewer columns than parts
    ops.argmax(tiny, split, rows=1, scratch=scratch)
    assert int(split[0]) == 1


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows", [1, 8, 16])
def test_decode_chain_same_bits_with_and_without_dependent_launch(rows):
    """Kernels of a decode step start before the kernel ahead has finished (programmatic
    dependent launch) and read its output only after their wait, partly through L1. Over a
    chain of 48 decode layers of GPT-2 XL's sizes (large enough that several kernels wait on
    chip at once) nothing stale is ever read: the residual stream at the end has the same
    bits with dependent launch on and off, launched one by one and replayed from a graph."""
    ops = _ops()
    width, inner, heads, head_dim, page, context, layers = 1600, 6400, 25, 64, 16, 256, 4

    def weights(n, k, seed):
        return [_randn(n, k, seed=seed + i, dtype=torch.bfloat16, scale=0.02)
                for i in range(layers)]

    w_qkv, w_out = weights(3 * width, width, 100), weights(width, width, 110)
    w_up, w_down = weights(inner, width, 120), weights(width, inner, 130)
    b_qkv, b_out, b_up = _randn(3 * width, seed=140), _randn(width, seed=141), \
        _randn(inner, seed=142)
    gamma, beta = _randn(width, seed=143) * 0.1 + 1.0, _randn(width, seed=144) * 0.1
    start = _randn(rows, width, seed=145)
    residual = torch.zeros(rows, width, device=DEV)
    normed = torch.zeros(rows, width, dtype=torch.bfloat16, device=DEV)
    qkv = torch.zeros(rows, 3 * width, dtype=torch.bfloat16, device=DEV)
    attended = torch.zeros(rows, width, dtype=torch.bfloat16, device=DEV)
    hidden = torch.zeros(rows, inner, dtype=torch.bfloat16, device=DEV)
    pages = rows * context // page + 1
    k_pages = [_randn(pages, heads, page, head_dim, seed=150 + i, dtype=torch.bfloat16)
               for i in range(layers)]
    v_pages = [_randn(pages, heads, page, head_dim, seed=160 + i, dtype=torch.bfloat16)
               for i in range(layers)]
    table = torch.arange(1, 1 + rows * context // page, dtype=torch.int32,
                         device=DEV).view(rows, context // page)
    request = torch.arange(rows, dtype=torch.int32, device=DEV)
    position = torch.full((rows,), context - 1, dtype=torch.int32, device=DEV)
    splits = ops.decode_splits(rows, heads, context)

    def chain():
        for index in range(48):
            i = index % layers
            ops.layer_norm(residual, gamma, beta, 1e-5, normed, count=rows)
            ops.linear(normed, w_qkv[i], b_qkv, qkv, rows=rows)
            ops.attention_decode(qkv[:, :width], k_pages[i], v_pages[i], table, request,
                                 position, attended, num_heads=heads, scale=0.125, rows=rows,
                                 splits=splits, k_new=qkv[:, width:2 * width],
                                 v_new=qkv[:, 2 * width:], store=True)
            ops.linear(attended, w_out[i], b_out, residual, residual=True, rows=rows)
            ops.layer_norm(residual, gamma, beta, 1e-5, normed, count=rows)
            ops.linear(normed, w_up[i], b_up, hidden, activation="gelu_tanh", rows=rows)
            ops.linear(hidden, w_down[i], None, residual, residual=True, rows=rows)

    results = []
    try:
        for dependent_launch in (False, True):
            ops.set_pdl(dependent_launch)
            residual.copy_(start)
            chain()
            results.append(residual.clone())
            graph = torch.cuda.CUDAGraph()
            residual.copy_(start)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph):
                chain()
            for _ in range(2):
                residual.copy_(start)
                graph.replay()
                results.append(residual.clone())
    finally:
        ops.set_pdl(True)
    torch.cuda.synchronize()
    assert bool(torch.isfinite(results[0]).all())
    assert all(torch.equal(results[0], other) for other in results[1:])


def test_an_empty_kernel_boundary_costs_about_a_microsecond(tmp_path, capsys):
    """What a decode step pays for being ≈ 340 kernels and not one: a chain of empty kernels
    (``tests/csrc/null_chain.cu``: wait for the predecessor, release the successor) replayed
    from a CUDA graph, with the launch attribute the engine's kernels use and without it.
    The figures are printed (run with ``-s``); the assertion is only that a boundary stays
    well under the two microseconds a kernel's own dependent chain takes."""
    import ctypes
    import subprocess

    from ayaka_b200.kernels.build import CSRC, _nvcc

    out = tmp_path / "libnull_chain.so"
    subprocess.run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17",
                    "--shared", "-Xcompiler", "-fPIC", "-I", str(CSRC), "-o", str(out),
                    str(Path(__file__).resolve().parent / "csrc" / "null_chain.cu")], check=True)
    library = ctypes.CDLL(str(out))
    sink = torch.zeros(4, dtype=torch.int32, device=DEV)
    count = 340

    def per_kernel_us(blocks, threads, pdl):
        library.set_pdl(pdl)
        side = torch.cuda.Stream()

        def body():
            status = library.null_chain(count, blocks, threads, ctypes.c_void_p(sink.data_ptr()),
                                        0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert status == 0

        with torch.cuda.stream(side):
            body()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                body()
        graph.replay()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(10):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            stop.record()
            torch.cuda.synchronize()
            best = min(best, start.elapsed_time(stop))
        return best * 1000 / count

    with capsys.disabled():
        print()
        for blocks, threads in ((1, 32), (148, 256), (600, 256), (888, 256)):
            with_pdl, without = per_kernel_us(blocks, threads, 1), per_kernel_us(blocks, threads, 0)
            print(f"empty kernel, {blocks} CTAs x {threads}: {with_pdl:.2f} us with programmatic "
                  f"dependent launch, {without:.2f} us without")
            assert with_pdl < 2.0
