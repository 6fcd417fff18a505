"""Mixers: the parts that let a token see other tokens. Here: causal multi-head attention."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, CacheNeed, Part, StateNeed, register_part
from ayaka_b200.parts.context import LayerCache, StepContext, Workspace
from ayaka_b200.parts.embedding import PositionEncoding
from ayaka_b200.parts.spec import PartSpec

__all__ = ["Attention", "Mixer", "leading_single_rows"]


#: From this many leading single-row requests on, a step that also holds prompt portions
#: runs them through the decode attention kernel (``csrc/step_host.cu`` has the same rule).
LEADING_SINGLE_ROWS = 4


def leading_single_rows(host_rows: list[int]) -> int:
    """How many requests at the head of the step bring exactly one row, if at least
    ``LEADING_SINGLE_ROWS`` do and something else follows; else 0."""
    lead = 0
    for rows in host_rows:
        if rows != 1:
            break
        lead += 1
    return lead if LEADING_SINGLE_ROWS <= lead < len(host_rows) else 0


class Mixer(Part):
    """Interface of a mixer.

    ``cache_need()`` says which paged keys/values the mixer wants (or ``None``);
    ``state_need()`` which fixed-size per-request state (or ``None``). ``forward`` reads
    ``hidden`` (``[N, width]`` in the compute dtype: the normalised residual), and **adds**
    its result to ``residual`` (fp32 ``[N, width]``) in place. It may use ``cache`` as its
    needs say and ``step.workspace`` for scratch.

    Optional: ``forward_normed(norm, residual, step, cache)`` — the same, but the part applies
    ``norm`` (a norm part with ``weight``, ``bias``, ``eps``) to ``residual`` itself, which lets
    it fuse the norm into its first kernel. A block calls it when the part has it.
    """

    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                cache: LayerCache) -> None:
        raise NotImplementedError


@register_part("mixer", "attention")
class Attention(Mixer):
    """Causal attention with one fused query/key/value projection and an output projection.

    ``qkv = h @ Wqkv.T + b`` with columns ordered queries, keys, values; keys and values go
    to the cache before attending, so a row sees itself; ``scores = scale * q.k`` over keys
    ``max(0, p - window + 1) .. p``, softmax and the weighted sum in fp32; then
    ``residual += o @ Wout.T + b`` (the reference's ``python/ayaka/layers/attention/dense.py:
    101-125`` and ``python/ayaka/ops/attention.py:15-24, 133-137``).

    Spec parameters: ``width``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``
    (the factor on q.k, given by the architecture: this part has no default), ``window``
    (0 = none), ``bias`` (bool).
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext, position: Part | None = None) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.num_heads = int(spec.num_heads)  # type: ignore[arg-type]
        self.num_kv_heads = int(spec.num_kv_heads)  # type: ignore[arg-type]
        self.head_dim = int(spec.head_dim)  # type: ignore[arg-type]
        self.scale = float(spec.scale)  # type: ignore[arg-type]
        self.window = int(spec.get("window", 0))  # type: ignore[arg-type]
        self.position = position
        # keys go to the cache as projected unless the position encoding rewrites them first
        self._keys_as_projected = position is None or \
            type(position).on_query_key is PositionEncoding.on_query_key
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"num_kv_heads ({self.num_kv_heads}) must divide num_heads "
                             f"({self.num_heads})")
        if self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise ValueError(f"head_dim must be a multiple of 16 in [16, 256], got "
                             f"{self.head_dim}")
        bias = bool(spec.get("bias", True))
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        out_features = self.q_width + 2 * self.kv_width
        self.qkv_weight = self.add_param("qkv.weight", (out_features, self.width), "matrix")
        self.qkv_bias = self.add_param("qkv.bias", (out_features,), "vector") if bias else None
        self.out_weight = self.add_param("out.weight", (self.width, self.q_width), "matrix")
        self.out_bias = self.add_param("out.bias", (self.width,), "vector") if bias else None
        self._native: dict[tuple[int, int], object] = {}

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window)

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                cache: LayerCache) -> None:
        qkv = step.workspace.buffer("attention.qkv", self.q_width + 2 * self.kv_width,
                                    self.ctx.dtype)
        stored = self._project(hidden, qkv, step, cache)
        self._attend(qkv, residual, step, cache, stored)

    def native_part(self, norm: Part, workspace: Workspace):  # noqa: ANN201
        """This mixer with ``norm`` in front of it as the C++ host code takes it (packed once
        per workspace), or ``None`` when that code cannot run it: a position encoding that
        rewrites queries and keys is a Python hook."""
        if self.position is not None and not self._keys_as_projected:
            return None
        key = (id(norm), id(workspace))
        found = self._native.get(key)
        if found is None:
            from ayaka_b200.kernels import native

            dtype = self.ctx.dtype
            found = native.attention_part(
                dtype=dtype, width=self.width, num_heads=self.num_heads,
                num_kv_heads=self.num_kv_heads, head_dim=self.head_dim, window=self.window,
                scale=self.scale, eps=norm.eps, keys_as_projected=True,  # type: ignore
                norm_weight=norm.weight, norm_bias=norm.bias,  # type: ignore[attr-defined]
                qkv_weight=self.qkv_weight, qkv_bias=self.qkv_bias, out_weight=self.out_weight,
                out_bias=self.out_bias,
                normed=workspace.buffer("block.normed", self.width, dtype),
                qkv=workspace.buffer("attention.qkv", self.q_width + 2 * self.kv_width, dtype),
                attended=workspace.buffer("attention.out", self.q_width, dtype))
            self._native[key] = found
        return found

    def forward_normed(self, norm: Part, residual: torch.Tensor, step: StepContext,
                       cache: LayerCache) -> None:
        if ops.NATIVE_STEP and cache.k_pages is not None:
            part = self.native_part(norm, step.workspace)
            if part is not None:
                from ayaka_b200.kernels import native

                native.run_attention(part, native.step_args(step, residual.device), residual,
                                     cache)
                return
        qkv = step.workspace.buffer("attention.qkv", self.q_width + 2 * self.kv_width,
                                    self.ctx.dtype)
        scratch = step.workspace.buffer("block.normed", self.width, self.ctx.dtype)
        ops.layer_norm(residual, norm.weight, norm.bias, norm.eps,  # type: ignore
                       scratch, count=step.num_rows)
        stored = self._project(scratch, qkv, step, cache)
        self._attend(qkv, residual, step, cache, stored)

    def _project(self, hidden: torch.Tensor, qkv: torch.Tensor, step: StepContext,
                 cache: LayerCache) -> bool:
        """The fused projection; True if its epilogue also stored the keys and values of the
        step's rows into the cache (prompt portions in bfloat16, no position encoding that
        would change the keys first)."""
        if cache.writes and not step.decode_only and self._keys_as_projected:
            group = step.groups[cache.group]  # type: ignore[index]
            if ops.linear_kv(hidden, self.qkv_weight, self.qkv_bias, qkv, group.slot_mapping,
                             cache.k_pages, cache.v_pages, q_width=self.q_width,
                             rows=step.num_rows):
                return True
        ops.linear(hidden, self.qkv_weight, self.qkv_bias, qkv, rows=step.num_rows)
        return False

    def _attend(self, qkv: torch.Tensor, residual: torch.Tensor, step: StepContext,
                cache: LayerCache, stored: bool = False) -> None:
        n = step.num_rows
        group = step.groups[cache.group]  # type: ignore[index]
        q = qkv[:, :self.q_width]
        k = qkv[:, self.q_width:self.q_width + self.kv_width]
        v = qkv[:, self.q_width + self.kv_width:]
        if self.position is not None:
            self.position.on_query_key(q, k, step)  # type: ignore[attr-defined]
        if cache.writes and not step.decode_only and not stored:
            ops.kv_store(k, v, group.slot_mapping, cache.k_pages, cache.v_pages, rows=n)
        attended = step.workspace.buffer("attention.out", self.q_width, self.ctx.dtype)
        if step.decode_only:
            # one row per request: a decode kernel (which one, and how a pair's keys are
            # shared out, is the library's choice; `splits` is what the split-KV one takes)
            reach = min(step.max_kv_len, self.window) if self.window else step.max_kv_len
            # (at most 8: a cluster merges the shares on chip, no scratch)
            splits = ops.decode_splits(n, self.num_heads, reach, q.device)
            ops.attention_decode(q, cache.k_pages, cache.v_pages, group.block_table,
                                 step.request_of_row, step.positions, attended,
                                 num_heads=self.num_heads, scale=self.scale, window=self.window,
                                 rows=n, splits=splits,
                                 k_new=k if cache.writes else None,
                                 v_new=v if cache.writes else None, store=cache.writes)
        elif self.ctx.dtype == torch.bfloat16:
            # Prompt portions: tensor-core flash attention. The requests that lead the step
            # with a single row each (the scheduler puts decoding requests first) go to the
            # decode kernel instead: as tiles of a prompt kernel each would occupy a CTA
            # built for 64 or 256 rows. Their keys and values are in the cache by now.
            lead = leading_single_rows(step.host_rows)
            if lead:
                reach = min(step.max_kv_len, self.window) if self.window else step.max_kv_len
                ops.attention_decode(q, cache.k_pages, cache.v_pages, group.block_table,
                                     step.request_of_row, step.positions, attended,
                                     num_heads=self.num_heads, scale=self.scale,
                                     window=self.window, rows=lead,
                                     splits=ops.decode_splits(lead, self.num_heads, reach,
                                                              q.device))
            ops.attention_prefill(q, cache.k_pages, cache.v_pages, group.block_table[lead:],
                                  step.row_start[lead:], step.kv_len[lead:], attended,
                                  num_heads=self.num_heads, scale=self.scale,
                                  host_rows=step.host_rows[lead:], window=self.window)
        else:
            ops.attention(q, cache.k_pages, cache.v_pages, group.block_table,
                          step.request_of_row, step.positions, attended,
                          num_heads=self.num_heads, scale=self.scale, window=self.window, rows=n)
        ops.linear(attended, self.out_weight, self.out_bias, residual, residual=True, rows=n)
