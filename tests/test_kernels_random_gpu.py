"""Random shapes through the attention kernels and the bfloat16 products, each against
float64. The cases of test_kernels_gpu.py are chosen; these are drawn: head sizes 16 to 128,
grouped heads, pages of 4 to 256 tokens (no powers of two among them), windows, requests of
one token beside long ones, products from 1 to 2,100 rows with widths and depths that are no
multiple of any tile, operands that are column ranges of wider buffers."""

from __future__ import annotations

import math
import random

import pytest
import torch

import plain_gpt2 as plain
import test_kernels_gpu as fixed

pytestmark = pytest.mark.gpu
DEV = "cuda"


def close(got: torch.Tensor, expected: torch.Tensor, tol: float, what: str) -> None:
    torch.testing.assert_close(got.double().cpu(), expected, rtol=tol, atol=tol,
                               msg=lambda text: f"{what}: {text}")


@pytest.mark.parametrize("seed", range(24))
def test_attention_kernels_on_random_cases(seed):
    from ayaka_b200.kernels import gemm_tc, ops

    rng = random.Random(f"attention-{seed}")
    head_dim = rng.choice([16, 32, 48, 64, 64, 64, 80, 128, 128])
    kv_heads, group = rng.choice([1, 2, 3]), rng.choice([1, 1, 2, 4])
    heads = kv_heads * group
    page = rng.choice([4, 8, 12, 16, 16, 32, 64, 128, 256])
    decode = rng.random() < 0.4
    lengths, rows = [], []
    for _ in range(rng.randint(1, 6)):
        n = rng.choice([rng.randint(1, 40), rng.randint(40, 400), rng.randint(400, 1400)])
        lengths.append(n)
        rows.append(1 if decode else
                    rng.choice([1, rng.randint(1, min(n, 8)), rng.randint(1, n), n]))
    window = rng.choice([0, 0, 0, rng.randint(1, 64), rng.randint(64, 700)])
    scale = rng.choice([0.5, 0.9, 1.3]) / math.sqrt(head_dim)
    case = f"{lengths} rows {rows} heads {heads}/{kv_heads} x {head_dim} page {page} window {window}"
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        q, k_pages, v_pages, table, req, pos, seqs = fixed._paged_case(
            lengths, rows, heads, kv_heads, head_dim, page, dtype, seed=seed)
        expected = fixed._attention_reference(seqs, lengths, rows, heads, kv_heads, scale, window)
        n = q.shape[0]

        def fresh() -> torch.Tensor:
            return torch.full((n + 1, heads * head_dim), float("nan"), dtype=dtype, device=DEV)

        out = fresh()
        ops.attention(q, k_pages, v_pages, table, req, pos, out, num_heads=heads, scale=scale,
                      window=window)
        close(out[:n], expected, tol, f"plain kernel {dtype} {case}")
        assert torch.isnan(out[n:].float()).all()
        if dtype == torch.bfloat16:
            starts = [0]
            for count in rows:
                starts.append(starts[-1] + count)
            row_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
            kv_len = torch.tensor(lengths, dtype=torch.int32, device=DEV)
            for kernel in ("mma", "tcgen05") if head_dim == 64 else ("mma",):
                out = fresh()
                ops.attention_prefill(q, k_pages, v_pages, table, row_start, kv_len, out,
                                      num_heads=heads, scale=scale, host_rows=list(rows),
                                      window=window, kernel=kernel)
                gemm_tc.check_status(q.device)
                close(out[:n], expected, tol, f"prompt kernel {kernel} {case}")
        if not decode:
            continue
        asks = [1, 2, 8, rng.randint(1, 8)]
        if dtype == torch.bfloat16 and head_dim in (64, 128):
            asks += [-1, -4, -8] + ([-16] if head_dim == 64 else [])
        kv_width = kv_heads * head_dim
        k_new = torch.zeros(n, kv_width, dtype=dtype, device=DEV)
        v_new = torch.zeros_like(k_new)
        wiped_k, wiped_v = k_pages.clone(), v_pages.clone()
        for b, length in enumerate(lengths):
            where, slot = int(table[b, (length - 1) // page]), (length - 1) % page
            k_new[b] = k_pages[where, :, slot].reshape(-1)
            v_new[b] = v_pages[where, :, slot].reshape(-1)
            wiped_k[where, :, slot] = float("nan")
            wiped_v[where, :, slot] = float("nan")
        for ask in asks:
            ops.set_decode_tensor_cores(ask < 0)  # a positive count: the split-KV kernel
            try:
                out = fresh()
                ops.attention_decode(q, k_pages, v_pages, table, req, pos, out, num_heads=heads,
                                     scale=scale, window=window, splits=ask)
                close(out[:n], expected, tol, f"decode kernel {ask} {dtype} {case}")
                out, into_k, into_v = fresh(), wiped_k.clone(), wiped_v.clone()
                ops.attention_decode(q, into_k, into_v, table, req, pos, out, num_heads=heads,
                                     scale=scale, window=window, splits=ask, k_new=k_new,
                                     v_new=v_new, store=True)
                close(out[:n], expected, tol, f"decode kernel {ask} with store {dtype} {case}")
                assert torch.equal(into_k.nan_to_num(7.0), k_pages.nan_to_num(7.0)), case
                assert torch.equal(into_v.nan_to_num(7.0), v_pages.nan_to_num(7.0)), case
            finally:
                ops.set_decode_tensor_cores(True)


ACTIVATIONS = {"none": None, "gelu_tanh": "gelu_new", "gelu_erf": "gelu"}


@pytest.mark.parametrize("seed", range(48))
def test_products_on_random_shapes(seed):
    """Through ``ops.linear``, so with the kernel and the tile the library picks itself."""
    from ayaka_b200.kernels import gemm_tc, ops

    rng = random.Random(f"product-{seed}")
    g = torch.Generator().manual_seed(seed)
    m = rng.choice([rng.randint(1, 16), rng.randint(17, 64), rng.randint(65, 300),
                    rng.randint(300, 2100)])
    n = rng.choice([rng.randint(1, 64), rng.randint(64, 700), rng.randint(700, 7000),
                    8 * rng.randint(1, 800)])
    k = 8 * rng.choice([rng.randint(1, 16), rng.randint(16, 250), rng.randint(250, 900)])
    wide = rng.random() < 0.3
    a_whole = torch.randn(m + 2, k * (3 if wide else 1), generator=g).to(torch.bfloat16).to(DEV)
    a = a_whole[:, k:2 * k] if wide else a_whole
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    bias = torch.randn(n, generator=g).to(DEV) if rng.random() < 0.7 else None
    exact = a[:m].double().cpu() @ w.double().cpu().t()
    if bias is not None:
        exact = exact + bias.double().cpu()
    mode = rng.choice(["bfloat16", "float32", "residual"])
    activation = "none" if mode == "residual" else rng.choice(list(ACTIVATIONS))
    what = f"{m} x {n} x {k} {mode} {activation} wide={wide} bias={bias is not None}"
    if ACTIVATIONS[activation] is not None:
        exact = plain.gelu(exact, ACTIVATIONS[activation])
    if mode == "residual":
        before = torch.randn(m + 2, n, generator=g).to(DEV)
        out = before.clone()
        ops.linear(a, w, bias, out, residual=True, rows=m)
        close(out[:m], exact + before[:m].double().cpu(), 2e-3, what)
        assert torch.equal(out[m:], before[m:]), what
    else:
        dtype = torch.bfloat16 if mode == "bfloat16" else torch.float32
        pad = rng.choice([0, 8])
        whole = torch.full((m + 2, n + pad), float("nan"), dtype=dtype, device=DEV)
        out = whole[:, :n]
        ops.linear(a, w, bias, out, activation=activation, rows=m)
        close(out[:m], exact, 1.2e-2 if mode == "bfloat16" else 2e-3, what)
        assert torch.isnan(whole[m:].float()).all(), what
        assert pad == 0 or torch.isnan(whole[:, n:].float()).all(), what
    gemm_tc.check_status(torch.device(DEV))
