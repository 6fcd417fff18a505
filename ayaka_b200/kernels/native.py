"""The C++ host code of a step (``csrc/step_host.cu``) seen from Python.

The structures below mirror the C structs field by field (the library reports its sizes and
:func:`host_library` compares). A part packs its static arguments once
(:func:`attention_part`, :func:`mlp_part`); the runner packs a step's arguments once per step
(:class:`StepArgs`); then one call runs a layer half, or :func:`run_layers` a whole run of
layers. The kernels are reached through the addresses of the same exported entry points the
functions of ``kernels/ops.py`` call.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, byref, c_float, c_int, c_void_p, cast

import torch

from ayaka_b200.errors import BackendError
from ayaka_b200.kernels import flags, lib, ops

__all__ = ["LayerRuns", "StepArgs", "attention_part", "host_library", "mlp_part", "run_attention",
           "run_layers", "run_mlp", "step_args"]

_TYPE = {torch.float32: 0, torch.bfloat16: 1}


class GroupStep(Structure):
    _fields_ = [("block_table", c_void_p), ("slot_mapping", c_void_p), ("table_stride", c_int),
                ("page_size", c_int)]


class Step(Structure):
    _fields_ = [
        ("num_rows", c_int), ("num_requests", c_int), ("decode_only", c_int),
        ("max_kv_len", c_int), ("sm_count", c_int), ("decode_ctas_per_sm", c_int),
        ("bf16_gemm_simt", c_int), ("prefill_mma", c_int), ("tile_n", c_int),
        ("positions", c_void_p), ("request_of_row", c_void_p), ("row_start", c_void_p),
        ("kv_len", c_void_p), ("host_rows", c_void_p), ("status", c_void_p),
        ("stream", c_void_p),
        ("num_groups", c_int), ("launches", c_int), ("groups", GroupStep * 8),
    ]


class Kernels(Structure):
    _fields_ = [(name, c_void_p) for name in (
        "layer_norm_f32", "layer_norm_bf16", "gemm_tc", "gemm_tc_kv", "gemm_simt", "kv_store",
        "attention_decode", "attention_simt", "attention_prefill", "attention_prefill_tc",
        "attention_prefill_tc_rows")]


class AttentionPart(Structure):
    _fields_ = [
        ("k", Kernels), ("type", c_int), ("width", c_int), ("num_heads", c_int),
        ("num_kv_heads", c_int), ("head_dim", c_int), ("window", c_int), ("scale", c_float),
        ("eps", c_float), ("keys_as_projected", c_int), ("norm_weight", c_void_p),
        ("norm_bias", c_void_p), ("qkv_weight", c_void_p), ("qkv_bias", c_void_p),
        ("out_weight", c_void_p), ("out_bias", c_void_p), ("normed", c_void_p),
        ("qkv", c_void_p), ("attended", c_void_p),
    ]


class MlpPart(Structure):
    _fields_ = [
        ("k", Kernels), ("type", c_int), ("width", c_int), ("inner", c_int),
        ("activation", c_int), ("eps", c_float), ("norm_weight", c_void_p),
        ("norm_bias", c_void_p), ("up_weight", c_void_p), ("up_bias", c_void_p),
        ("down_weight", c_void_p), ("down_bias", c_void_p), ("normed", c_void_p),
        ("inner_buf", c_void_p),
    ]


class LayerRun(Structure):
    _fields_ = [("attention", POINTER(AttentionPart)), ("mlp", POINTER(MlpPart)),
                ("k_pages", c_void_p), ("v_pages", c_void_p), ("num_pages", c_int),
                ("group", c_int), ("writes", c_int), ("pad", c_int)]


_host: ctypes.CDLL | None = None


def host_library() -> ctypes.CDLL:
    """The library of ``csrc/step_host.cu``, checked against the structures above."""
    global _host
    if _host is None:
        found = lib.library("step_host")
        sizes = (c_int * 5)()
        found.ayk_host_sizes(sizes)
        mine = [ctypes.sizeof(kind) for kind in (Step, AttentionPart, MlpPart, LayerRun, Kernels)]
        if list(sizes) != mine:
            raise BackendError(f"the host library's structs {list(sizes)} do not match "
                               f"kernels/native.py's {mine}")
        found.ayk_host_attention.restype = c_int
        found.ayk_host_mlp.restype = c_int
        found.ayk_host_layers.restype = c_int
        _host = found
    return _host


def _address(library_name: str, symbol: str, **defines: int) -> int:
    function = getattr(lib.library(library_name, **defines), symbol)
    return cast(function, c_void_p).value or 0


def _kernels(dtype: torch.dtype, head_dim: int | None = None) -> Kernels:
    """The entry points a part of this dtype may reach. A float32 model never loads (or
    compiles) the tensor-core libraries."""
    table = Kernels()
    table.gemm_simt = _address("gemm_simt", "ayk_gemm_simt")
    if dtype == torch.bfloat16:
        table.layer_norm_bf16 = _address("norm", "ayk_layer_norm_bf16")
        table.gemm_tc = _address("gemm_tc", "ayk_gemm_bf16_tc")
        table.gemm_tc_kv = _address("gemm_tc", "ayk_gemm_bf16_tc_kv")
    else:
        table.layer_norm_f32 = _address("norm", "ayk_layer_norm_f32")
    if head_dim is not None:
        table.kv_store = _address("attention_simt", "ayk_kv_store")
        table.attention_decode = _address("attention_decode", "ayk_attention_decode")
        if dtype == torch.bfloat16:
            table.attention_prefill = _address("attention_prefill", "ayk_attention_prefill",
                                               AYK_HEAD_DIM=head_dim)
            if head_dim == 64:
                table.attention_prefill_tc = _address("attention_prefill_tc",
                                                      "ayk_attention_prefill_tc")
                table.attention_prefill_tc_rows = _address("attention_prefill_tc",
                                                           "ayk_attention_prefill_tc_rows")
        else:
            table.attention_simt = _address("attention_simt", "ayk_attention_simt")
    return table


def _ptr(tensor: torch.Tensor | None) -> int:
    return 0 if tensor is None else tensor.data_ptr()


def attention_part(*, dtype: torch.dtype, width: int, num_heads: int, num_kv_heads: int,
                   head_dim: int, window: int, scale: float, eps: float,
                   keys_as_projected: bool, norm_weight: torch.Tensor,
                   norm_bias: torch.Tensor | None, qkv_weight: torch.Tensor,
                   qkv_bias: torch.Tensor | None, out_weight: torch.Tensor,
                   out_bias: torch.Tensor | None, normed: torch.Tensor, qkv: torch.Tensor,
                   attended: torch.Tensor) -> AttentionPart:
    for name, tensor in (("qkv_weight", qkv_weight), ("out_weight", out_weight),
                         ("normed", normed), ("qkv", qkv), ("attended", attended)):
        if not tensor.is_contiguous():
            raise BackendError(f"native attention part: {name} must be contiguous")
    part = AttentionPart()
    part.k = _kernels(dtype, head_dim)
    part.type = _TYPE[dtype]
    part.width, part.num_heads, part.num_kv_heads = width, num_heads, num_kv_heads
    part.head_dim, part.window = head_dim, window
    part.scale, part.eps = scale, eps
    part.keys_as_projected = 1 if keys_as_projected else 0
    part.norm_weight, part.norm_bias = _ptr(norm_weight), _ptr(norm_bias)
    part.qkv_weight, part.qkv_bias = _ptr(qkv_weight), _ptr(qkv_bias)
    part.out_weight, part.out_bias = _ptr(out_weight), _ptr(out_bias)
    part.normed, part.qkv, part.attended = _ptr(normed), _ptr(qkv), _ptr(attended)
    return part


def mlp_part(*, dtype: torch.dtype, width: int, inner: int, activation: str, eps: float,
             norm_weight: torch.Tensor, norm_bias: torch.Tensor | None,
             up_weight: torch.Tensor, up_bias: torch.Tensor | None, down_weight: torch.Tensor,
             down_bias: torch.Tensor | None, normed: torch.Tensor,
             inner_buf: torch.Tensor) -> MlpPart:
    for name, tensor in (("up_weight", up_weight), ("down_weight", down_weight),
                         ("normed", normed), ("inner", inner_buf)):
        if not tensor.is_contiguous():
            raise BackendError(f"native feed-forward part: {name} must be contiguous")
    part = MlpPart()
    part.k = _kernels(dtype)
    part.type = _TYPE[dtype]
    part.width, part.inner, part.activation = width, inner, ops.ACTIVATIONS[activation]
    part.eps = eps
    part.norm_weight, part.norm_bias = _ptr(norm_weight), _ptr(norm_bias)
    part.up_weight, part.up_bias = _ptr(up_weight), _ptr(up_bias)
    part.down_weight, part.down_bias = _ptr(down_weight), _ptr(down_bias)
    part.normed, part.inner_buf = _ptr(normed), _ptr(inner_buf)
    return part


class StepArgs:
    """A step's arguments as the host library wants them; built once per step (or once per
    graph bucket) from a :class:`~ayaka_b200.parts.context.StepContext`."""

    __slots__ = ("step", "_keep", "_rows")

    def __init__(self, context, device: torch.device) -> None:  # noqa: ANN001
        from ayaka_b200.kernels import gemm_tc

        step = Step()
        rows = context.host_rows
        step.num_rows, step.num_requests = context.num_rows, context.num_requests
        step.decode_only = 1 if context.decode_only else 0
        step.max_kv_len = context.max_kv_len
        self._rows = (c_int * max(len(rows), 1))(*rows)
        step.host_rows = ctypes.addressof(self._rows)
        step.sm_count = ops.sm_count(device)
        step.decode_ctas_per_sm = ops.DECODE_CTAS_PER_SM
        step.bf16_gemm_simt = 1 if ops.BF16_GEMM != "tcgen05" else 0
        step.prefill_mma = 1 if ops.PREFILL_ATTENTION != "tcgen05" else 0
        step.tile_n = gemm_tc.TILE_N
        step.positions = context.positions.data_ptr()
        step.request_of_row = context.request_of_row.data_ptr()
        step.row_start = context.row_start.data_ptr()
        step.kv_len = context.kv_len.data_ptr()
        step.status = flags.status_word(device).data_ptr()
        step.stream = 0
        if len(context.groups) > 8:
            raise BackendError("the host library takes at most 8 cache groups")
        step.num_groups = len(context.groups)
        for index, group in enumerate(context.groups):
            step.groups[index].block_table = group.block_table.data_ptr()
            step.groups[index].slot_mapping = group.slot_mapping.data_ptr()
            step.groups[index].table_stride = group.block_table.stride(0) \
                if group.block_table.ndim == 2 and group.block_table.shape[0] else 1
            step.groups[index].page_size = group.page_size
        self.step = step
        self._keep = context  # the tensors whose addresses the struct holds

    def on_current_stream(self) -> Step:
        self.step.stream = lib.raw_stream()
        return self.step


def step_args(context, device: torch.device) -> StepArgs:  # noqa: ANN001
    """The step's arguments, packed the first time a part asks and kept with the step."""
    found = context.extra.get("native")
    if found is None:
        found = StepArgs(context, device)
        context.extra["native"] = found
    return found


def _done(status: int, step: Step, before: int, what: str) -> None:
    ops._launches += step.launches - before
    lib.check(status, what)


def run_attention(part: AttentionPart, args: StepArgs, residual: torch.Tensor, cache) -> None:  # noqa: ANN001
    step = args.on_current_stream()
    before = step.launches
    status = host_library().ayk_host_attention(
        byref(part), byref(step), c_void_p(residual.data_ptr()), c_void_p(_ptr(cache.k_pages)),
        c_void_p(_ptr(cache.v_pages)), c_int(cache.k_pages.shape[0]), c_int(cache.group),
        c_int(1 if cache.writes else 0))
    _done(status, step, before, "attention half of a layer (host library)")


def run_mlp(part: MlpPart, args: StepArgs, residual: torch.Tensor) -> None:
    step = args.on_current_stream()
    before = step.launches
    status = host_library().ayk_host_mlp(byref(part), byref(step),
                                         c_void_p(residual.data_ptr()))
    _done(status, step, before, "feed-forward half of a layer (host library)")


class LayerRuns:
    """The execution order as an array the host library walks in one call."""

    def __init__(self, entries: list[tuple[AttentionPart, MlpPart, object]]) -> None:
        self.count = len(entries)
        self.array = (LayerRun * max(self.count, 1))()
        self._keep = entries
        for index, (attention, mlp, cache) in enumerate(entries):
            run = self.array[index]
            run.attention = ctypes.pointer(attention)
            run.mlp = ctypes.pointer(mlp)
            run.k_pages, run.v_pages = _ptr(cache.k_pages), _ptr(cache.v_pages)
            run.num_pages = cache.k_pages.shape[0]
            run.group = cache.group
            run.writes = 1 if cache.writes else 0


def run_layers(runs: LayerRuns, args: StepArgs, residual: torch.Tensor) -> None:
    step = args.on_current_stream()
    before = step.launches
    failed_at = c_int(-1)
    status = host_library().ayk_host_layers(runs.array, c_int(runs.count), byref(step),
                                            c_void_p(residual.data_ptr()), byref(failed_at))
    _done(status, step, before, f"layer run {failed_at.value} (host library)")
