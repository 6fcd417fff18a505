"""Feed-forward parts. Here: the dense two-matrix MLP."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, Part, register_part
from ayaka_b200.parts.context import StepContext, Workspace
from ayaka_b200.parts.spec import PartSpec

__all__ = ["DenseMLP", "FeedForward"]


class FeedForward(Part):
    """Interface of a feed-forward: read ``hidden`` (``[N, width]``, compute dtype) and **add**
    the result to ``residual`` (fp32 ``[N, width]``) in place. Optional:
    ``forward_normed(norm, residual, step)`` applies the norm itself (see ``Mixer``)."""

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext) -> None:
        raise NotImplementedError


@register_part("feed_forward", "dense")
class DenseMLP(FeedForward):
    """``residual += act(h @ Wup.T + b_up) @ Wdown.T + b_down`` with the activation evaluated
    in fp32 inside the first product's epilogue (``python/ayaka/layers/ffn/dense.py:22-57``).

    Spec parameters: ``width``, ``inner``, ``activation`` (``gelu_tanh`` or ``gelu_erf``),
    ``bias`` (bool).
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.inner = int(spec.inner)  # type: ignore[arg-type]
        self.activation = str(spec.activation)
        if self.activation not in ops.ACTIVATIONS or self.activation == "none":
            raise ValueError(f"unknown activation {self.activation!r}")
        bias = bool(spec.get("bias", True))
        self.up_weight = self.add_param("up.weight", (self.inner, self.width), "matrix")
        self.up_bias = self.add_param("up.bias", (self.inner,), "vector") if bias else None
        self.down_weight = self.add_param("down.weight", (self.width, self.inner), "matrix")
        self.down_bias = self.add_param("down.bias", (self.width,), "vector") if bias else None
        self._native: dict[tuple[int, int], object] = {}

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext) -> None:
        n = step.num_rows
        inner = step.workspace.buffer("feed_forward.inner", self.inner, self.ctx.dtype)
        ops.linear(hidden, self.up_weight, self.up_bias, inner, activation=self.activation,
                   rows=n)
        ops.linear(inner, self.down_weight, self.down_bias, residual, residual=True, rows=n)

    def native_part(self, norm: Part, workspace: Workspace):  # noqa: ANN201
        """This feed-forward with ``norm`` in front of it as the C++ host code takes it
        (packed once per workspace)."""
        key = (id(norm), id(workspace))
        found = self._native.get(key)
        if found is None:
            from ayaka_b200.kernels import native

            dtype = self.ctx.dtype
            found = native.mlp_part(
                dtype=dtype, width=self.width, inner=self.inner, activation=self.activation,
                eps=norm.eps, norm_weight=norm.weight, norm_bias=norm.bias,  # type: ignore
                up_weight=self.up_weight, up_bias=self.up_bias, down_weight=self.down_weight,
                down_bias=self.down_bias,
                normed=workspace.buffer("block.normed", self.width, dtype),
                inner_buf=workspace.buffer("feed_forward.inner", self.inner, dtype))
            self._native[key] = found
        return found

    def forward_normed(self, norm: Part, residual: torch.Tensor, step: StepContext) -> None:
        if ops.NATIVE_STEP:
            from ayaka_b200.kernels import native

            native.run_mlp(self.native_part(norm, step.workspace),
                           native.step_args(step, residual.device), residual)
            return
        n = step.num_rows
        inner = step.workspace.buffer("feed_forward.inner", self.inner, self.ctx.dtype)
        scratch = step.workspace.buffer("block.normed", self.width, self.ctx.dtype)
        ops.linear_normed(residual, norm.weight, norm.bias, norm.eps,  # type: ignore
                          self.up_weight, self.up_bias, inner, scratch=scratch, count=n,
                          activation=self.activation)
        ops.linear(inner, self.down_weight, self.down_bias, residual, residual=True, rows=n)
