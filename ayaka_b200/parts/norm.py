"""Normalisation parts."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, Part, register_part
from ayaka_b200.parts.spec import PartSpec

__all__ = ["LayerNorm"]


@register_part("norm", "layer_norm")
class LayerNorm(Part):
    """``(x - mean) / sqrt(var + eps) * weight + bias`` over the last dimension, biased
    variance, computed in fp32 from the fp32 residual stream and rounded once to the output's
    dtype (formula: the reference's ``python/ayaka/layers/norm.py:59-100``).

    Spec parameters: ``width``, ``eps``, ``bias`` (bool).

    ``fusable_layer_norm``: a norm part sets this when it is exactly the formula above with
    the attributes ``weight``, ``bias`` (or ``None``) and ``eps``; a part whose first kernel
    can normalise its input itself (``forward_normed``) may then be handed the norm instead
    of its output. A norm part without the attribute is always applied on its own.
    """

    fusable_layer_norm = True

    def __init__(self, spec: PartSpec, ctx: BuildContext) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.eps = float(spec.eps)  # type: ignore[arg-type]
        self.weight = self.add_param("weight", (self.width,), "vector")
        self.bias = self.add_param("bias", (self.width,), "vector") if spec.get("bias", True) \
            else None

    def forward(self, x: torch.Tensor, out: torch.Tensor, *, count: int,
                rows: torch.Tensor | None = None) -> None:
        """Normalise ``count`` fp32 rows of ``x`` (gathered by ``rows`` if given) into ``out``."""
        ops.layer_norm(x, self.weight, self.bias, self.eps, out, rows=rows, count=count)
