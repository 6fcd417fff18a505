"""The kernels as functions over torch tensors.

Every function writes into tensors the caller allocated and launches on torch's current
CUDA stream. Tensors are on one CUDA device; 2-D tensors may have any row stride but a unit
stride along the last dimension. Nothing here falls back to torch arithmetic: a missing
library or a refused argument raises :class:`~ayaka_b200.errors.BackendError`.
"""

from __future__ import annotations

import contextlib
from collections.abc import Iterator
from ctypes import c_float, c_int, c_void_p

import torch

from ayaka_b200.errors import BackendError
from ayaka_b200.kernels.lib import check, library, raw_stream

__all__ = [
    "ACTIVATIONS",
    "argmax",
    "attention",
    "attention_decode",
    "attention_prefill",
    "decode_splits",
    "embed_rows",
    "kv_store",
    "launch_count",
    "leaving_out",
    "layer_norm",
    "linear",
    "linear_normed",
    "logits_adjust",
    "logits_scale_cap",
    "sample",
    "set_decode_tensor_cores",
    "set_pdl",
    "sm_count",
    "timed",
]

ACTIVATIONS = {"none": 0, "gelu_tanh": 1, "gelu_erf": 2}
_TYPE = {torch.float32: 0, torch.bfloat16: 1}

#: Which bfloat16 matrix-product kernel :func:`linear` launches: ``"tcgen05"`` (the tensor
#: cores, the serving path) or ``"simt"`` (the CUDA-core reference); tests switch it.
BF16_GEMM = "tcgen05"


#: Whether parts that can hand a layer half (or a run of layers) to the C++ host code
#: (``csrc/step_host.cu``) do so; tests switch it off to compare the two paths bit by bit.
NATIVE_STEP = True

_launches = 0

#: Kernel classes that launch nothing while a measurement runs; empty in normal use. A
#: class is an operation's name, for matrix products with the weight's shape
#: (``"linear:4800x1600"``). ``bench.py`` times a step with and without each class inside
#: the same chain of dependent launches, which is what a kernel costs there; a step with a
#: class left out computes nothing meaningful.
_left_out: frozenset[str] = frozenset()


@contextlib.contextmanager
def leaving_out(*classes: str) -> Iterator[None]:
    """Within the block the named kernel classes are not launched (for measurements only)."""
    global _left_out
    before = _left_out
    _left_out = before | frozenset(classes)
    try:
        yield
    finally:
        _left_out = before


_TIMED = ("embed_rows", "layer_norm", "linear", "linear_kv", "kv_store", "attention",
          "attention_prefill", "attention_decode", "argmax", "sample")


@contextlib.contextmanager
def timed() -> Iterator[dict[str, list[tuple[torch.cuda.Event, torch.cuda.Event]]]]:
    """Within the block every launch through this module is bracketed by two CUDA events,
    gathered per kernel class (see ``leaving_out`` for the names); after a synchronisation
    ``start.elapsed_time(stop)`` of each pair is that kernel's own duration. The events keep
    a kernel from starting under its predecessor's tail, so this suits steps of large
    kernels (prompt portions), not decode chains. For measurements only."""
    module = globals()
    originals = {name: module[name] for name in _TIMED}
    record: dict[str, list[tuple[torch.cuda.Event, torch.cuda.Event]]] = {}

    def wrap(name: str, function):  # noqa: ANN001, ANN202
        def wrapped(*args, **kwargs):  # noqa: ANN002, ANN003, ANN202
            klass = name
            if name in ("linear", "linear_kv"):
                klass = f"linear:{args[1].shape[0]}x{args[1].shape[1]}"
            start = torch.cuda.Event(enable_timing=True)
            stop = torch.cuda.Event(enable_timing=True)
            start.record()
            result = function(*args, **kwargs)
            stop.record()
            record.setdefault(klass, []).append((start, stop))
            return result
        return wrapped

    for name, function in originals.items():
        module[name] = wrap(name, function)
    try:
        yield record
    finally:
        module.update(originals)


def set_pdl(enabled: bool) -> None:
    """Switch programmatic dependent launch on or off in every library (it is on by default;
    measurements switch it off to see what it buys). Graphs captured earlier keep their edges."""
    from ayaka_b200.kernels import lib

    lib.set_pdl(enabled)


def set_decode_tensor_cores(enabled: bool) -> None:
    """Let decode attention choose its tensor-core kernel where that serves the case (the
    default), or keep every call on the split-KV kernel (tests of that kernel at head sizes
    64 and 128 in bfloat16, and measurements of one kernel against the other)."""
    library("attention_decode").ayk_set_decode_tensor_cores(c_int(1 if enabled else 0))


def launch_count() -> int:
    """Kernels launched through this module since the process started (a graph capture
    counts the kernels it records)."""
    return _launches


def _status_word(device: torch.device) -> torch.Tensor:
    from ayaka_b200.kernels import gemm_tc

    return gemm_tc.status_word(device)


def _stream() -> c_void_p:
    global _launches
    _launches += 1
    return c_void_p(raw_stream())


def _ptr(tensor: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if tensor is None else tensor.data_ptr())


def _need(op: str, name: str, tensor: torch.Tensor, dtype: torch.dtype | None = None,
          ndim: int | None = None) -> None:
    if not tensor.is_cuda:
        raise BackendError(f"{op}: {name} must be on a CUDA device, it is on {tensor.device}")
    if dtype is not None and tensor.dtype != dtype:
        raise BackendError(f"{op}: {name} must be {dtype}, got {tensor.dtype}")
    if ndim is not None and tensor.ndim != ndim:
        raise BackendError(f"{op}: {name} must have {ndim} dimensions, got {tensor.ndim}")
    if tensor.ndim and tensor.numel() and tensor.stride(-1) != 1:
        raise BackendError(f"{op}: {name} must have a unit stride along its last dimension")


def embed_rows(table: torch.Tensor, index: torch.Tensor, out: torch.Tensor, *,
               add_table: torch.Tensor | None = None, add_index: torch.Tensor | None = None,
               bad_index: torch.Tensor, scale: float = 1.0) -> None:
    """``out[i] = scale * table[index[i]] (+ add_table[add_index[i]])`` as fp32 rows.

    ``bad_index`` is one int32 on the device that the kernel sets to 1 if an id is outside
    its table.
    """
    op = "embed_rows"
    if _left_out and op in _left_out:
        return
    _need(op, "table", table, ndim=2)
    _need(op, "index", index, torch.int32, 1)
    _need(op, "out", out, torch.float32, 2)
    _need(op, "bad_index", bad_index, torch.int32)
    if table.dtype not in _TYPE or not table.is_contiguous():
        raise BackendError(f"{op}: table must be contiguous float32 or bfloat16")
    rows, width = index.shape[0], table.shape[1]
    if out.shape[0] < rows or out.shape[1] != width:
        raise BackendError(f"{op}: out {list(out.shape)} does not hold [{rows}, {width}]")
    if add_table is not None:
        if add_index is None:
            raise BackendError(f"{op}: add_table needs add_index")
        _need(op, "add_table", add_table, table.dtype, 2)
        _need(op, "add_index", add_index, torch.int32, 1)
        if add_table.shape[1] != width or add_index.shape[0] != rows or \
                not add_table.is_contiguous():
            raise BackendError(f"{op}: add_table/add_index do not match the rows")
    name = "ayk_embed_rows_f32" if table.dtype == torch.float32 else "ayk_embed_rows_bf16"
    fn = getattr(library("embed"), name)
    status = fn(_ptr(table), _ptr(index), c_int(table.shape[0]), _ptr(add_table),
                _ptr(add_index), c_int(0 if add_table is None else add_table.shape[0]),
                _ptr(out), c_int(out.stride(0)), c_int(rows), c_int(width), c_float(scale),
                _ptr(bad_index), _stream())
    check(status, op)


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor | None, eps: float,
               out: torch.Tensor, *, rows: torch.Tensor | None = None,
               count: int | None = None) -> None:
    """LayerNorm of fp32 rows into ``out`` (float32 or bfloat16).

    With ``rows`` (int32), output row ``i`` normalises ``x[rows[i]]``. ``count`` limits the
    number of output rows (default: all of ``rows`` or of ``x``).
    """
    op = "layer_norm"
    if _left_out and op in _left_out:
        return
    _need(op, "x", x, torch.float32, 2)
    _need(op, "gamma", gamma, torch.float32, 1)
    if beta is not None:
        _need(op, "beta", beta, torch.float32, 1)
    _need(op, "out", out, ndim=2)
    if out.dtype not in _TYPE:
        raise BackendError(f"{op}: out must be float32 or bfloat16, got {out.dtype}")
    width = x.shape[1]
    if gamma.shape[0] != width or (beta is not None and beta.shape[0] != width) or \
            out.shape[1] != width:
        raise BackendError(f"{op}: widths differ")
    if rows is not None:
        _need(op, "rows", rows, torch.int32, 1)
    n = count if count is not None else (rows.shape[0] if rows is not None else x.shape[0])
    if n > out.shape[0] or (rows is None and n > x.shape[0]) or \
            (rows is not None and n > rows.shape[0]):
        raise BackendError(f"{op}: {n} rows do not fit the tensors")
    name = "ayk_layer_norm_f32" if out.dtype == torch.float32 else "ayk_layer_norm_bf16"
    fn = getattr(library("norm"), name)
    status = fn(_ptr(x), c_int(x.stride(0)), _ptr(rows), _ptr(gamma), _ptr(beta),
                c_float(eps), _ptr(out), c_int(out.stride(0)), c_int(n), c_int(width), _stream())
    check(status, op)


def linear(a: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor,
           *, activation: str = "none", residual: bool = False, rows: int | None = None,
           kernel: str | None = None) -> None:
    """``out = act(a @ weight.T + bias)``, or ``out += a @ weight.T + bias`` with ``residual``.

    ``a`` is ``[M, K]``, ``weight`` ``[N, K]`` (both float32, or both bfloat16), ``bias``
    float32 ``[N]``. ``out`` is ``[M, N]``: float32 always allowed (and required with
    ``residual``), bfloat16 for bfloat16 inputs. ``rows`` limits M. float32 inputs run on
    the CUDA cores with fp32 FMA (no reduced-precision matrix mode); bfloat16 inputs on the
    tensor cores unless ``kernel="simt"``.
    """
    op = "linear"
    if _left_out and f"linear:{weight.shape[0]}x{weight.shape[1]}" in _left_out:
        return
    _need(op, "a", a, ndim=2)
    _need(op, "weight", weight, a.dtype, 2)
    _need(op, "out", out, ndim=2)
    if a.dtype not in _TYPE or out.dtype not in _TYPE:
        raise BackendError(f"{op}: float32 and bfloat16 only, got {a.dtype} -> {out.dtype}")
    if bias is not None:
        _need(op, "bias", bias, torch.float32, 1)
    m = a.shape[0] if rows is None else rows
    n, k = weight.shape
    if a.shape[1] != k or m > a.shape[0] or m > out.shape[0] or out.shape[1] != n or \
            (bias is not None and bias.shape[0] != n):
        raise BackendError(
            f"{op}: shapes a{list(a.shape)} w{list(weight.shape)} out{list(out.shape)} "
            f"rows={m} do not fit")
    if activation not in ACTIVATIONS:
        raise BackendError(f"{op}: unknown activation {activation!r}")
    if residual and (out.dtype != torch.float32 or activation != "none"):
        raise BackendError(f"{op}: a residual sum is float32 and has no activation")
    if a.dtype == torch.float32 and out.dtype != torch.float32:
        raise BackendError(f"{op}: float32 inputs give float32 output")
    which = kernel or (BF16_GEMM if a.dtype == torch.bfloat16 else "simt")
    if which == "tcgen05" and a.dtype == torch.bfloat16:
        from ayaka_b200.kernels import gemm_tc

        # operands TMA cannot read (a row stride that is no multiple of 8 elements) go to
        # the CUDA-core kernel: slower, same result
        if kernel == "tcgen05" or gemm_tc.usable(a, weight):
            gemm_tc.linear_bf16(a, weight, bias, out, m, ACTIVATIONS[activation], residual)
            return
    fn = library("gemm_simt").ayk_gemm_simt
    status = fn(_ptr(a), c_int(a.stride(0)), _ptr(weight), c_int(weight.stride(0)), _ptr(bias),
                _ptr(out), c_int(out.stride(0)), c_int(m), c_int(n), c_int(k),
                c_int(ACTIVATIONS[activation]), c_int(1 if residual else 0),
                c_int(_TYPE[a.dtype]), c_int(_TYPE[out.dtype]), _stream())
    check(status, op)


def linear_kv(a: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
              out: torch.Tensor, slot_mapping: torch.Tensor, k_pages: torch.Tensor,
              v_pages: torch.Tensor, *, q_width: int, rows: int | None = None) -> bool:
    """``a @ weight.T + bias`` for a fused query/key/value projection (bfloat16): the query
    columns go to ``out[:, :q_width]``; the key and value columns (keys, then values) go into
    the cache pages at ``slot_mapping``, written by the product's own epilogue, and **not**
    to ``out`` (whose columns from ``q_width`` on keep what they held). Returns False, having
    done nothing, when that cannot be had (float32, few rows, sizes the kernel does not
    take): the caller then runs :func:`linear` and :func:`kv_store`."""
    op = "linear_kv"
    if _left_out and f"linear:{weight.shape[0]}x{weight.shape[1]}" in _left_out:
        return True
    if a.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or BF16_GEMM != "tcgen05":
        return False
    _need(op, "a", a, torch.bfloat16, 2)
    _need(op, "weight", weight, torch.bfloat16, 2)
    _need(op, "out", out, torch.bfloat16, 2)
    _need(op, "slot_mapping", slot_mapping, torch.int32, 1)
    _need(op, "k_pages", k_pages, torch.bfloat16, 4)
    _need(op, "v_pages", v_pages, torch.bfloat16, 4)
    if bias is not None:
        _need(op, "bias", bias, torch.float32, 1)
    m = a.shape[0] if rows is None else rows
    n, k = weight.shape
    _, kv_heads, _, head_dim = k_pages.shape
    if a.shape[1] != k or m > a.shape[0] or m > out.shape[0] or out.shape[1] != n or \
            m > slot_mapping.shape[0] or n != q_width + 2 * kv_heads * head_dim or \
            v_pages.shape != k_pages.shape or (bias is not None and bias.shape[0] != n):
        raise BackendError(f"{op}: shapes do not fit")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous pages only")
    from ayaka_b200.kernels import gemm_tc

    return gemm_tc.linear_bf16_kv(a, weight, bias, out, m, slot_mapping, k_pages, v_pages,
                                  q_width)


def linear_normed(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor | None, eps: float,
                  weight: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor, *,
                  scratch: torch.Tensor, count: int, activation: str = "none",
                  row_index: torch.Tensor | None = None) -> None:
    """``out = act(LayerNorm(x) @ weight.T + bias)`` for ``count`` rows (``x[row_index]`` with
    a gather index): the norm into ``scratch`` (``[>= count, K]`` in the weight's dtype), then
    the product. Two kernels on purpose. A variant that computed the norm inside the few-rows
    product's kernel (statistics carried along by the kernel that last wrote the rows) was
    measured on a B200 in a 48-layer decode chain and lost at every row count, 59.7 against
    53.8 microseconds a layer at 8 rows: with programmatic dependent launch a kernel boundary
    costs less than the extra dependent phases inside the product's kernel."""
    if activation not in ACTIVATIONS:
        raise BackendError(f"linear_normed: unknown activation {activation!r}")
    layer_norm(x, gamma, beta, eps, scratch, rows=row_index, count=count)
    linear(scratch, weight, bias, out, activation=activation, rows=count)


def kv_store(k: torch.Tensor, v: torch.Tensor, slot_mapping: torch.Tensor,
             k_pages: torch.Tensor, v_pages: torch.Tensor, *, rows: int | None = None) -> None:
    """Write this step's key and value rows ``[N, kv_heads * head_dim]`` into the pages.

    Pages are ``[page, kv_head, slot, head_dim]``; ``slot_mapping[i] = page * page_size +
    slot`` or negative for a row that stores nothing. ``k`` and ``v`` share a row stride (they
    are column ranges of one projection output).
    """
    op = "kv_store"
    if _left_out and op in _left_out:
        return
    _need(op, "k", k, ndim=2)
    _need(op, "v", v, k.dtype, 2)
    _need(op, "slot_mapping", slot_mapping, torch.int32, 1)
    _need(op, "k_pages", k_pages, k.dtype, 4)
    _need(op, "v_pages", v_pages, k.dtype, 4)
    if k.dtype not in _TYPE or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous float32 or bfloat16 pages only")
    _, kv_heads, page_size, head_dim = k_pages.shape
    n = k.shape[0] if rows is None else rows
    if k.shape[1] != kv_heads * head_dim or v.shape != k.shape or k.stride(0) != v.stride(0) \
            or v_pages.shape != k_pages.shape or n > k.shape[0] or n > slot_mapping.shape[0]:
        raise BackendError(f"{op}: shapes do not fit")
    fn = library("attention_simt").ayk_kv_store
    status = fn(_ptr(k), _ptr(v), c_int(k.stride(0)), _ptr(slot_mapping), _ptr(k_pages),
                _ptr(v_pages), c_int(n), c_int(kv_heads), c_int(head_dim), c_int(page_size),
                c_int(_TYPE[k.dtype]), _stream())
    check(status, op)


def attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
              block_table: torch.Tensor, request_of_row: torch.Tensor, positions: torch.Tensor,
              out: torch.Tensor, *, num_heads: int, scale: float, window: int = 0,
              rows: int | None = None) -> None:
    """Causal attention of query rows over their requests' cached keys and values.

    ``q`` and ``out`` are ``[N, num_heads * head_dim]``; row ``i`` belongs to request
    ``request_of_row[i]`` (a row of ``block_table``; negative = padding row, output zero) and
    sits at ``positions[i]``; it sees keys ``max(0, p - window + 1) .. p`` (``window`` 0 = all).
    The keys of the step's own rows must already be stored.
    """
    op = "attention"
    if _left_out and op in _left_out:
        return
    _need(op, "q", q, ndim=2)
    _need(op, "out", out, q.dtype, 2)
    _need(op, "k_pages", k_pages, q.dtype, 4)
    _need(op, "v_pages", v_pages, q.dtype, 4)
    _need(op, "block_table", block_table, torch.int32, 2)
    _need(op, "request_of_row", request_of_row, torch.int32, 1)
    _need(op, "positions", positions, torch.int32, 1)
    if q.dtype not in _TYPE or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous float32 or bfloat16 pages only")
    _, kv_heads, page_size, head_dim = k_pages.shape
    n = q.shape[0] if rows is None else rows
    if q.shape[1] != num_heads * head_dim or out.shape[1] != q.shape[1] or n > out.shape[0] \
            or n > request_of_row.shape[0] or n > positions.shape[0] or \
            v_pages.shape != k_pages.shape:
        raise BackendError(f"{op}: shapes do not fit")
    fn = library("attention_simt").ayk_attention_simt
    status = fn(_ptr(q), c_int(q.stride(0)), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                c_int(block_table.stride(0)), _ptr(request_of_row), _ptr(positions), _ptr(out),
                c_int(out.stride(0)), c_int(n), c_int(num_heads), c_int(kv_heads),
                c_int(head_dim), c_int(page_size), c_float(scale), c_int(window),
                c_int(_TYPE[q.dtype]), _stream())
    check(status, op)


#: Which kernel :func:`attention_prefill` launches for head size 64: ``"tcgen05"`` (both
#: products on the 5th-generation tensor cores, accumulators in tensor memory) or ``"mma"``
#: (the warp-level kernel that serves every other head size); tests switch it.
PREFILL_ATTENTION = "tcgen05"


def attention_prefill(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_table: torch.Tensor, row_start: torch.Tensor, kv_len: torch.Tensor,
                      out: torch.Tensor, *, num_heads: int, scale: float, host_rows: list[int],
                      window: int = 0, kernel: str | None = None) -> None:
    """Causal attention of prompt portions in bfloat16 on the tensor cores.

    Request ``b`` owns rows ``row_start[b] .. row_start[b + 1]`` of ``q`` and ``out``, which
    are the last rows of its ``kv_len[b]`` cached tokens; ``host_rows`` is the host copy of
    the row counts (the grid is sized from it). Head size 64 runs on tcgen05; the other head
    sizes on a warp-level kernel compiled for the head size (``kernel`` forces one of them).
    """
    op = "attention_prefill"
    if _left_out and op in _left_out:
        return
    _need(op, "q", q, torch.bfloat16, 2)
    _need(op, "out", out, torch.bfloat16, 2)
    _need(op, "k_pages", k_pages, torch.bfloat16, 4)
    _need(op, "v_pages", v_pages, torch.bfloat16, 4)
    _need(op, "block_table", block_table, torch.int32, 2)
    _need(op, "row_start", row_start, torch.int32, 1)
    _need(op, "kv_len", kv_len, torch.int32, 1)
    if not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous pages only")
    _, kv_heads, page_size, head_dim = k_pages.shape
    count = len(host_rows)
    if q.shape[1] != num_heads * head_dim or out.shape[1] != q.shape[1] or \
            row_start.shape[0] < count + 1 or kv_len.shape[0] < count or \
            block_table.shape[0] < count or v_pages.shape != k_pages.shape:
        raise BackendError(f"{op}: shapes do not fit")
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise BackendError(f"{op}: head_dim must be a multiple of 16 in [16, 256]")
    # the tcgen05 kernel works on tiles of 256 rows: a step of short portions only is better
    # served by the warp-level kernel's tiles of 64
    which = kernel or (PREFILL_ATTENTION if head_dim == 64 and scale > 0
                       and max(host_rows, default=0) >= 256 else "mma")
    if which == "tcgen05":
        if head_dim != 64:
            raise BackendError(f"{op}: the tcgen05 kernel serves head size 64, not {head_dim}")
        lib = library("attention_prefill_tc")
        tile_rows = lib.ayk_attention_prefill_tc_rows()
        tiles = sum(-(-rows // tile_rows) for rows in host_rows)
        status = lib.ayk_attention_prefill_tc(
            _ptr(q), c_int(q.stride(0)), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
            c_int(block_table.stride(0)), _ptr(row_start), _ptr(kv_len), _ptr(out),
            c_int(out.stride(0)), c_int(count), c_int(tiles), c_int(num_heads), c_int(kv_heads),
            c_int(head_dim), c_int(page_size), c_int(k_pages.shape[0]), c_float(scale),
            c_int(window), _ptr(_status_word(q.device)), _stream())
        check(status, op)
        return
    tiles = sum(-(-rows // 64) for rows in host_rows)
    fn = library("attention_prefill", AYK_HEAD_DIM=head_dim).ayk_attention_prefill
    status = fn(_ptr(q), c_int(q.stride(0)), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                c_int(block_table.stride(0)), _ptr(row_start), _ptr(kv_len), _ptr(out),
                c_int(out.stride(0)), c_int(count), c_int(tiles), c_int(num_heads),
                c_int(kv_heads), c_int(head_dim), c_int(page_size), c_float(scale),
                c_int(window), _stream())
    check(status, op)


#: CTAs of the decode attention kernel the grid aims at per SM: six are resident (32 KB of
#: shared memory each), and a little over one round measured best
DECODE_CTAS_PER_SM = 7
_sm_counts: dict[int, int] = {}


def sm_count(device: torch.device | None = None) -> int:
    """Streaming multiprocessors of ``device`` (the current one when absent), asked once."""
    index = torch.cuda.current_device() if device is None or device.index is None \
        else device.index
    found = _sm_counts.get(index)
    if found is None:
        found = torch.cuda.get_device_properties(index).multi_processor_count
        _sm_counts[index] = found
    return found


def decode_splits(num_rows: int, num_heads: int, max_kv_len: int,
                  device: torch.device | None = None) -> int:
    """How many CTAs share one (request, head) of a decode step: the grid should fill the
    device about once (``DECODE_CTAS_PER_SM`` CTAs per SM), a cluster merges up to 8 shares on
    chip, and a warp wants at least 32 keys."""
    fill = DECODE_CTAS_PER_SM * sm_count(device) // max(1, num_rows * num_heads)
    enough_keys = max(1, max_kv_len // 128)
    splits = max(1, min(fill, enough_keys, 8))
    while splits & (splits - 1):  # a power of two
        splits -= 1
    return splits


def attention_decode(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     block_table: torch.Tensor, request_of_row: torch.Tensor,
                     positions: torch.Tensor, out: torch.Tensor, *, num_heads: int, scale: float,
                     window: int = 0, rows: int | None = None, splits: int = 1,
                     partial: torch.Tensor | None = None,
                     tickets: torch.Tensor | None = None, k_new: torch.Tensor | None = None,
                     v_new: torch.Tensor | None = None, store: bool = False) -> None:
    """Attention for steps whose every request brings one row (same contract as
    :func:`attention`). ``splits`` CTAs share each (request, head). Up to 8 splits merge on
    chip (a thread-block cluster); given ``partial`` (float32, at least rows * heads * splits
    * (head_dim + 2)) and ``tickets`` (int32 zeros, at least rows * heads; left zero) the
    shares go through that scratch instead, which more than 8 splits require. With ``k_new``/``v_new``
    (``[rows, kv_heads * head_dim]``, column ranges of the projection output) each row's own
    key and value are taken from there, and with ``store`` the kernel also writes them into
    the row's cache slot, so no separate KV store runs."""
    op = "attention_decode"
    if _left_out and op in _left_out:
        return
    _need(op, "q", q, ndim=2)
    _need(op, "out", out, q.dtype, 2)
    _need(op, "k_pages", k_pages, q.dtype, 4)
    _need(op, "v_pages", v_pages, q.dtype, 4)
    _need(op, "block_table", block_table, torch.int32, 2)
    _need(op, "request_of_row", request_of_row, torch.int32, 1)
    _need(op, "positions", positions, torch.int32, 1)
    if q.dtype not in _TYPE or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous float32 or bfloat16 pages only")
    _, kv_heads, page_size, head_dim = k_pages.shape
    n = q.shape[0] if rows is None else rows
    if q.shape[1] != num_heads * head_dim or out.shape[1] != q.shape[1] or n > out.shape[0] \
            or n > request_of_row.shape[0] or n > positions.shape[0] or \
            v_pages.shape != k_pages.shape:
        raise BackendError(f"{op}: shapes do not fit")
    if splits > 8 and partial is None:
        raise BackendError(f"{op}: more than 8 splits need scratch")
    if (partial is None) != (tickets is None):
        raise BackendError(f"{op}: partial and tickets come together")
    if partial is not None and tickets is not None:
        _need(op, "partial", partial, torch.float32)
        _need(op, "tickets", tickets, torch.int32)
        if partial.numel() < n * num_heads * splits * (head_dim + 2) or \
                tickets.numel() < n * num_heads:
            raise BackendError(f"{op}: the scratch buffers are too small")
    if k_new is not None:
        if v_new is None:
            raise BackendError(f"{op}: k_new needs v_new")
        _need(op, "k_new", k_new, q.dtype, 2)
        _need(op, "v_new", v_new, q.dtype, 2)
        if k_new.shape[1] != kv_heads * head_dim or v_new.shape != k_new.shape or \
                k_new.stride(0) != v_new.stride(0) or k_new.shape[0] < n:
            raise BackendError(f"{op}: k_new/v_new do not fit")
    elif store:
        raise BackendError(f"{op}: store needs k_new and v_new")
    status = library("attention_decode").ayk_attention_decode(
        _ptr(q), c_int(q.stride(0)), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
        c_int(block_table.stride(0)), _ptr(request_of_row), _ptr(positions), _ptr(out),
        c_int(out.stride(0)), c_int(n), c_int(num_heads), c_int(kv_heads), c_int(head_dim),
        c_int(page_size), c_float(scale), c_int(window), c_int(splits), _ptr(partial),
        _ptr(tickets), _ptr(k_new), _ptr(v_new),
        c_int(0 if k_new is None else k_new.stride(0)), c_int(1 if store else 0),
        _ptr(_status_word(q.device)), c_int(_TYPE[q.dtype]), _stream(),
        c_int(k_pages.shape[0]))
    check(status, op)


ARGMAX_PARTS = 32


def argmax(logits: torch.Tensor, out: torch.Tensor, *, rows: int | None = None,
           scratch: torch.Tensor | None = None) -> None:
    """``out[i]`` = the id of row ``i``'s largest logit, the smallest id among equals.

    With ``scratch`` (float32, at least ``2 * rows * ARGMAX_PARTS`` elements) every row is
    split over ``ARGMAX_PARTS`` CTAs and folded by a second small kernel: faster for a few
    rows of a large vocabulary."""
    op = "argmax"
    if _left_out and op in _left_out:
        return
    _need(op, "logits", logits, torch.float32, 2)
    _need(op, "out", out, torch.int32, 1)
    n = logits.shape[0] if rows is None else rows
    if n > out.shape[0] or n > logits.shape[0]:
        raise BackendError(f"{op}: {n} rows do not fit")
    if scratch is not None:
        _need(op, "scratch", scratch, torch.float32)
        if scratch.numel() < 2 * n * ARGMAX_PARTS or not scratch.is_contiguous():
            raise BackendError(f"{op}: scratch is too small")
        flat = scratch.reshape(-1)
        values = flat[:n * ARGMAX_PARTS]
        ids = flat[n * ARGMAX_PARTS:2 * n * ARGMAX_PARTS].view(torch.int32)
        global _launches
        _launches += 1  # two kernels; _stream() below counts the other
        status = library("sampling").ayk_argmax_split(
            _ptr(logits), c_int(logits.stride(0)), c_int(n), c_int(logits.shape[1]),
            c_int(ARGMAX_PARTS), _ptr(values), _ptr(ids), _ptr(out), _stream())
        check(status, op)
        return
    status = library("sampling").ayk_argmax(_ptr(logits), c_int(logits.stride(0)), c_int(n),
                                            c_int(logits.shape[1]), _ptr(out), _stream())
    check(status, op)


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor | None,
           top_p: torch.Tensor | None, min_p: torch.Tensor | None, seeds: torch.Tensor,
           positions: torch.Tensor, out: torch.Tensor, *, rows: int | None = None) -> None:
    """One token per row of fp32 logits: temperature, top-k, top-p, min-p and the inverse CDF
    over the canonical order, the random number from Philox(seed, position) in the kernel.

    ``temperature`` float32 (a row below 1e-5 is greedy); ``top_k`` int32 (<= 0 off);
    ``top_p``/``min_p`` float32; ``seeds``/``positions`` int64 (position = index in the
    sequence of the token being produced); ``out`` int32.
    """
    op = "sample"
    _need(op, "logits", logits, torch.float32, 2)
    _need(op, "temperature", temperature, torch.float32, 1)
    _need(op, "seeds", seeds, torch.int64, 1)
    _need(op, "positions", positions, torch.int64, 1)
    _need(op, "out", out, torch.int32, 1)
    n = logits.shape[0] if rows is None else rows
    for name, tensor, dtype in (("top_k", top_k, torch.int32), ("top_p", top_p, torch.float32),
                                ("min_p", min_p, torch.float32)):
        if tensor is not None:
            _need(op, name, tensor, dtype, 1)
            if tensor.shape[0] < n:
                raise BackendError(f"{op}: {name} has fewer than {n} rows")
    if min(temperature.shape[0], seeds.shape[0], positions.shape[0], out.shape[0],
           logits.shape[0]) < n:
        raise BackendError(f"{op}: {n} rows do not fit the tensors")
    status = library("sampling").ayk_sample(
        _ptr(logits), c_int(logits.stride(0)), c_int(n), c_int(logits.shape[1]),
        _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(seeds), _ptr(positions),
        _ptr(out), _stream())
    check(status, op)


#: words of a row's header in the descriptor of :func:`logits_adjust`
ADJUST_WORDS = 16


def logits_scale_cap(logits: torch.Tensor, *, rows: int, scale: float = 1.0,
                     softcap: float = 0.0) -> None:
    """``x = scale * x`` and then, with ``softcap`` > 0, ``x = softcap * tanh(x / softcap)``
    on ``rows`` rows of fp32 ``logits`` in place (what some architectures do to the head's
    output; GPT-2 does neither and never launches this)."""
    op = "logits_scale_cap"
    _need(op, "logits", logits, torch.float32, 2)
    if rows < 0 or rows > logits.shape[0] or softcap < 0:
        raise BackendError(f"{op}: rows={rows}, softcap={softcap} do not fit")
    status = library("sampling").ayk_logits_scale_cap(
        _ptr(logits), c_int(logits.stride(0)), c_int(logits.shape[1]), c_int(rows),
        c_float(scale), c_float(softcap), _stream())
    check(status, op)


def logits_adjust(logits: torch.Tensor, desc: torch.Tensor, num_rows: int,
                  mask_scratch: torch.Tensor | None = None) -> None:
    """Adjust rows of fp32 ``logits`` in place before a token is chosen: allowed and banned
    ids, additive biases, repetition / frequency / presence penalties, in that order.

    ``desc`` (int32, on the device) holds ``num_rows`` headers of ``ADJUST_WORDS`` words
    followed by the lists they point to (offsets are word indices into ``desc``): row of
    ``logits``; history offset, history length, prompt length (the history is the request's
    prompt followed by its output); bias offset and count (ids, then as many float32 values);
    allowed offset and count (-1: no restriction); banned offset and count; repetition,
    frequency and presence as float32 bits. ``mask_scratch`` (int32, ``num_rows *
    ceil(vocab / 32)`` words) is needed when a row has an allowed list.
    """
    op = "logits_adjust"
    _need(op, "logits", logits, torch.float32, 2)
    _need(op, "desc", desc, torch.int32, 1)
    if num_rows < 0 or desc.shape[0] < num_rows * ADJUST_WORDS:
        raise BackendError(f"{op}: the descriptor does not hold {num_rows} rows")
    if mask_scratch is not None:
        _need(op, "mask_scratch", mask_scratch, torch.int32, 1)
        if mask_scratch.shape[0] < num_rows * ((logits.shape[1] + 31) // 32):
            raise BackendError(f"{op}: mask_scratch is too small")
    status = library("sampling").ayk_logits_adjust(
        _ptr(logits), c_int(logits.stride(0)), c_int(logits.shape[1]), _ptr(desc),
        c_int(num_rows), _ptr(mask_scratch), _stream())
    check(status, op)
