"""Arrangements: how one layer wires its norms, its mixer and its feed-forward."""

from __future__ import annotations

import torch

from ayaka_b200.parts.base import BuildContext, Part, build_part, register_part
from ayaka_b200.parts.context import LayerCache, StepContext, Workspace
from ayaka_b200.parts.spec import LayerSpec

__all__ = ["Block", "PreNormBlock"]


class Block(Part):
    """Interface of an arrangement: ``forward(residual, step, cache)`` updates the fp32
    residual stream ``[N, width]`` in place. ``mixer`` is exposed for the cache planner."""

    mixer: Part

    def forward(self, residual: torch.Tensor, step: StepContext, cache: LayerCache) -> None:
        raise NotImplementedError


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """``x += mixer(norm(x)); x += feed_forward(norm(x))`` — GPT-2's block
    (``python/ayaka/models/gpt2.py:99-101``). The sums happen in fp32 inside the last matrix
    product of each half."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext, position: Part | None) -> None:
        super().__init__(ctx)
        self.mixer_norm = self.add_child(
            "mixer_norm", build_part("norm", spec.mixer_norm.kind, spec.mixer_norm, ctx))
        self.mixer = self.add_child(
            "mixer", build_part("mixer", spec.mixer.kind, spec.mixer, ctx, position))
        self.feed_forward_norm = self.add_child(
            "feed_forward_norm",
            build_part("norm", spec.feed_forward_norm.kind, spec.feed_forward_norm, ctx))
        self.feed_forward = self.add_child(
            "feed_forward",
            build_part("feed_forward", spec.feed_forward.kind, spec.feed_forward, ctx))
        self.width = int(spec.mixer_norm.width)  # type: ignore[arg-type]

    def native_run(self, workspace: Workspace):  # noqa: ANN201
        """``(attention part, feed-forward part)`` for the C++ host code when both halves of
        this layer can run there (fusable norms, parts that know how to pack themselves),
        else ``None``; see ``kernels/native.py``."""
        if not (_plain_norm(self.mixer_norm) and _plain_norm(self.feed_forward_norm)
                and hasattr(self.mixer, "native_part")
                and hasattr(self.feed_forward, "native_part")):
            return None
        attention = self.mixer.native_part(self.mixer_norm, workspace)  # type: ignore
        mlp = self.feed_forward.native_part(self.feed_forward_norm, workspace)  # type: ignore
        return None if attention is None or mlp is None else (attention, mlp)

    def forward(self, residual: torch.Tensor, step: StepContext, cache: LayerCache) -> None:
        n = step.num_rows
        hidden = step.workspace.buffer("block.normed", self.width, self.ctx.dtype)
        # a part that can apply the norm itself gets the residual and the norm part
        if hasattr(self.mixer, "forward_normed") and _plain_norm(self.mixer_norm):
            self.mixer.forward_normed(self.mixer_norm, residual, step, cache)  # type: ignore
        else:
            self.mixer_norm.forward(residual, hidden, count=n)  # type: ignore[attr-defined]
            self.mixer.forward(hidden, residual, step, cache)  # type: ignore[attr-defined]
        if hasattr(self.feed_forward, "forward_normed") and _plain_norm(self.feed_forward_norm):
            self.feed_forward.forward_normed(  # type: ignore[attr-defined]
                self.feed_forward_norm, residual, step)
        else:
            self.feed_forward_norm.forward(residual, hidden, count=n)  # type: ignore
            self.feed_forward.forward(hidden, residual, step)  # type: ignore[attr-defined]


def _plain_norm(norm: Part) -> bool:
    """Whether ``norm`` declares itself a LayerNorm that a fused kernel can apply from its
    (weight, bias, eps); see ``parts/norm.py``."""
    return bool(getattr(norm, "fusable_layer_norm", False))
