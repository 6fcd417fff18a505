"""Feed-forward parts. Here: the dense two-matrix MLP."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, Part, register_part
from ayaka_b200.parts.context import StepContext
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

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext) -> None:
        n = step.num_rows
        inner = step.workspace.buffer("feed_forward.inner", self.inner, self.ctx.dtype)
        ops.linear(hidden, self.up_weight, self.up_bias, inner, activation=self.activation,
                   rows=n)
        ops.linear(inner, self.down_weight, self.down_bias, residual, residual=True, rows=n)

    def forward_normed(self, norm: Part, residual: torch.Tensor, step: StepContext) -> None:
        n = step.num_rows
        inner = step.workspace.buffer("feed_forward.inner", self.inner, self.ctx.dtype)
        scratch = step.workspace.buffer("block.normed", self.width, self.ctx.dtype)
        ops.linear_normed(residual, norm.weight, norm.bias, norm.eps,  # type: ignore
                          self.up_weight, self.up_bias, inner, scratch=scratch, count=n,
                          activation=self.activation)
        ops.linear(inner, self.down_weight, self.down_bias, residual, residual=True, rows=n)
