"""The bfloat16 tensor-core matrix product's Python side: argument rules, the status word."""

from __future__ import annotations

from ctypes import c_int, c_void_p

import torch

from ayaka_b200.errors import BackendError
from ayaka_b200.kernels import flags
from ayaka_b200.kernels.lib import check, entry, raw_stream

__all__ = ["check_status", "linear_bf16", "linear_bf16_kv", "status_word"]

#: what ``ayk_gemm_bf16_tc_kv`` returns when it does not serve the case (nothing ran)
NOT_TAKEN = -6

#: tile width (columns of the output per CTA) the next calls use; 0 lets the library choose.
TILE_N = 0


def status_word(device: torch.device) -> torch.Tensor:
    """One int32 per device that a kernel sets when a bounded wait ran out."""
    return flags.status_word(device)


def check_status(device: torch.device) -> None:
    """Read the status word (a device synchronisation) and raise if a kernel gave up."""
    word = status_word(device)
    value = int(word.item())
    if value:
        word.zero_()
        check(value, "tensor-core kernel")


def usable(a: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether TMA can read these operands: 16-byte aligned, row strides multiples of 8."""
    return (a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and a.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0)


def linear_bf16(a: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                out: torch.Tensor, rows: int, activation: int, residual: bool,
                tile_n: int | None = None) -> None:
    if not usable(a, weight):
        raise BackendError("linear: operands break the TMA rules (16-byte aligned, row strides "
                           "multiples of 8 elements)")
    n, k = weight.shape
    mode = 2 if residual else (0 if out.dtype == torch.bfloat16 else 1)
    from ayaka_b200.kernels import ops

    ops._launches += 1
    fn = entry("gemm_tc", "ayk_gemm_bf16_tc")
    status = fn(c_void_p(a.data_ptr()), c_int(a.stride(0)), c_void_p(weight.data_ptr()),
                c_int(weight.stride(0)), c_void_p(0 if bias is None else bias.data_ptr()),
                c_void_p(out.data_ptr()), c_int(out.stride(0)), c_int(rows), c_int(n), c_int(k),
                c_int(activation), c_int(mode), c_int(TILE_N if tile_n is None else tile_n),
                c_void_p(status_word(a.device).data_ptr()),
                c_void_p(raw_stream()))
    check(status, "linear (tcgen05)")


def linear_bf16_kv(a: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                   out: torch.Tensor, rows: int, slot_mapping: torch.Tensor,
                   k_pages: torch.Tensor, v_pages: torch.Tensor, q_width: int) -> bool:
    """The fused query/key/value projection with the key and value columns also stored into
    the cache pages (``[page, kv_head, slot, head_dim]``) at ``slot_mapping``. Returns False,
    having run nothing, when the library cannot carry the store with this product."""
    if not usable(a, weight):
        return False
    n, k = weight.shape
    _, kv_heads, page_size, head_dim = k_pages.shape
    from ayaka_b200.kernels import ops

    fn = entry("gemm_tc", "ayk_gemm_bf16_tc_kv")
    status = fn(c_void_p(a.data_ptr()), c_int(a.stride(0)), c_void_p(weight.data_ptr()),
                c_int(weight.stride(0)), c_void_p(0 if bias is None else bias.data_ptr()),
                c_void_p(out.data_ptr()), c_int(out.stride(0)), c_int(rows), c_int(n), c_int(k),
                c_void_p(slot_mapping.data_ptr()), c_void_p(k_pages.data_ptr()),
                c_void_p(v_pages.data_ptr()), c_int(q_width), c_int(kv_heads * head_dim),
                c_int(kv_heads), c_int(head_dim), c_int(page_size),
                c_void_p(status_word(a.device).data_ptr()),
                c_void_p(raw_stream()))
    if status == NOT_TAKEN:
        return False
    ops._launches += 1
    check(status, "linear with key/value store (tcgen05)")
    return True
