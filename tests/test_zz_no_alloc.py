"""The decode-attention entry point that allocates nothing, called through its exported C
symbol, against the ordinary entry point that takes its scratch from the caller.

Some hosts of the library cannot allocate device memory when they need attention — a server
that gave every free byte to its own pools at start-up, or a loop that must not pay the
device synchronisation an allocation implies. For them the library keeps the kernel's scratch
in a fixed array of its own. This file runs last (pytest collects files by name), so a run
that stops at the first failure has already run everything else; the test passes alone in a
fresh process as well as after the others.
"""

from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_size_t, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(rows, heads, kv_heads, head_dim, page, context, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    pages_per_row = -(-context // page)
    num_pages = rows * pages_per_row + 1
    k_pages = torch.randn(num_pages, kv_heads, page, head_dim, generator=g).to(dtype).cuda()
    v_pages = torch.randn(num_pages, kv_heads, page, head_dim, generator=g).to(dtype).cuda()
    order = torch.randperm(num_pages - 1, generator=g) + 1  # page 0 is padding
    table = order.reshape(rows, pages_per_row).to(torch.int32).cuda()
    q = torch.randn(rows, heads * head_dim, generator=g).to(dtype).cuda()
    lengths = torch.randint(1, context + 1, (rows,), generator=g)
    positions = (lengths - 1).to(torch.int32).cuda()
    request_of_row = torch.arange(rows, dtype=torch.int32).cuda()
    return q, k_pages, v_pages, table, request_of_row, positions


def _call(entry, q, k_pages, v_pages, table, req, pos, out, rows, heads, kv_heads, head_dim,
          page, scale, splits, type_code, stream):
    return entry(c_void_p(q.data_ptr()), c_int(q.stride(0)), c_void_p(k_pages.data_ptr()),
                 c_void_p(v_pages.data_ptr()), c_void_p(table.data_ptr()),
                 c_int(table.stride(0)), c_void_p(req.data_ptr()), c_void_p(pos.data_ptr()),
                 c_void_p(out.data_ptr()), c_int(out.stride(0)), c_int(rows), c_int(heads),
                 c_int(kv_heads), c_int(head_dim), c_int(page), c_float(scale), c_int(0),
                 c_int(splits), c_int(type_code), stream)


def _plain_attention(q, k_pages, v_pages, table, positions, heads, scale):
    """Softmax attention of each row over its own keys, gathered page by page, in float64."""
    rows = q.shape[0]
    _, kv_heads, page, head_dim = k_pages.shape
    out = torch.zeros(rows, heads * head_dim, dtype=torch.float64)
    table, positions = table.cpu(), positions.cpu()
    k_pages, v_pages, q = k_pages.cpu().double(), v_pages.cpu().double(), q.cpu().double()
    for row in range(rows):
        length = int(positions[row]) + 1
        pages = table[row, :-(-length // page)].long()
        keys = k_pages[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, head_dim)[:, :length]
        values = v_pages[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, head_dim)[:, :length]
        for head in range(heads):
            kv = head // (heads // kv_heads)
            query = q[row, head * head_dim:(head + 1) * head_dim]
            weights = torch.softmax(keys[kv] @ query * scale, 0)
            out[row, head * head_dim:(head + 1) * head_dim] = weights @ values[kv]
    return out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row(dtype):
    from ayaka_b200.kernels import ops
    from ayaka_b200.kernels.lib import library

    lib = library("attention_decode")
    entry = lib.ayk_attention_decode_noalloc  # the exported C symbol
    entry.restype = c_int
    limit_floats, limit_tickets = c_size_t(), c_size_t()
    lib.ayk_attention_decode_noalloc_limits(ctypes.byref(limit_floats),
                                            ctypes.byref(limit_tickets))
    assert limit_floats.value == 1 << 20 and limit_tickets.value == 1 << 14
    type_code = 1 if dtype == torch.bfloat16 else 0
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)

    # two calls in a row on the shared array, of different shapes: the second must not be
    # disturbed by what the first left behind
    for rows, heads, kv_heads, head_dim, page, context, splits, seed in (
            (5, 6, 2, 64, 16, 300, 12, 1), (3, 4, 4, 32, 8, 700, 16, 2)):
        q, k_pages, v_pages, table, req, pos = _case(rows, heads, kv_heads, head_dim, page,
                                                     context, dtype, seed)
        scale = 1.0 / math.sqrt(head_dim)
        expected = torch.zeros_like(q)
        partial = torch.zeros(rows * heads * splits * (head_dim + 2), device="cuda")
        tickets = torch.zeros(rows * heads, dtype=torch.int32, device="cuda")
        ops.attention_decode(q, k_pages, v_pages, table, req, pos, expected, num_heads=heads,
                             scale=scale, splits=splits, partial=partial, tickets=tickets)
        got = torch.full_like(q, float("nan"))
        # the first call on a device is the set-up call (it looks up the array's address and
        # makes the driver load the library's device image); what must allocate nothing is
        # every call after it, so the free bytes the driver reports are compared around the
        # second call of this shape
        for attempt in range(2):
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info()
            status = _call(entry, q, k_pages, v_pages, table, req, pos, got, rows, heads,
                           kv_heads, head_dim, page, scale, splits, type_code, stream)
            assert status == 0
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before  # driver level: no cudaMalloc hid in the call
        torch.testing.assert_close(got.float(), expected.float(), **tol)
        plain = _plain_attention(q, k_pages, v_pages, table, pos, heads, scale)
        torch.testing.assert_close(got.double().cpu(), plain, **tol)

    # sizes beyond the fixed array are refused, and nothing is launched
    rows, heads, head_dim, splits = 64, 64, 256, 8  # 64 * 64 * 8 * 258 floats > 2^20
    dummy = torch.zeros(1, device="cuda")
    status = entry(c_void_p(dummy.data_ptr()), c_int(heads * head_dim),
                   c_void_p(dummy.data_ptr()), c_void_p(dummy.data_ptr()),
                   c_void_p(dummy.data_ptr()), c_int(1), c_void_p(dummy.data_ptr()),
                   c_void_p(dummy.data_ptr()), c_void_p(dummy.data_ptr()),
                   c_int(heads * head_dim), c_int(rows), c_int(heads), c_int(heads),
                   c_int(head_dim), c_int(16), c_float(1.0), c_int(0), c_int(splits),
                   c_int(type_code), stream)
    assert status == -3  # AYK_TOO_LARGE
    torch.cuda.synchronize()
