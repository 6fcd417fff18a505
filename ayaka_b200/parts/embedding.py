"""Token embedding, position encodings and the output head."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, Part, register_part
from ayaka_b200.parts.context import StepContext
from ayaka_b200.parts.spec import PartSpec

__all__ = ["LearnedPositions", "LinearHead", "NoPositions", "PositionEncoding", "TokenEmbedding"]


class PositionEncoding(Part):
    """Interface of a position encoding.

    ``added_rows(step)`` returns ``(table, index)`` for an encoding that adds one table row
    per token to the embedding (fused into the embedding kernel), or ``None``.
    ``on_query_key(q, k, step)`` lets an encoding change queries and keys in place before the
    keys are cached (a rotary encoding); the default does nothing.
    ``max_positions`` bounds a sequence, or is ``None``.
    """

    max_positions: int | None = None

    def added_rows(self, step: StepContext) -> tuple[torch.Tensor, torch.Tensor] | None:
        return None

    def on_query_key(self, q: torch.Tensor, k: torch.Tensor, step: StepContext) -> None:
        return None


@register_part("position", "learned")
class LearnedPositions(PositionEncoding):
    """A table ``[max_positions, width]`` whose row ``p`` is added to the token at position
    ``p`` (the reference's ``wpe``, ``python/ayaka/models/gpt2.py:147-149, 175``).

    Spec parameters: ``max_positions``, ``width``.
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext) -> None:
        super().__init__(ctx)
        self.max_positions = int(spec.max_positions)  # type: ignore[arg-type]
        self.weight = self.add_param(
            "weight", (self.max_positions, int(spec.width)), "table")  # type: ignore[arg-type]

    def added_rows(self, step: StepContext) -> tuple[torch.Tensor, torch.Tensor]:
        return self.weight, step.positions


@register_part("position", "none")
class NoPositions(PositionEncoding):
    """No position signal at all (for toy models in tests)."""

    def __init__(self, spec: PartSpec, ctx: BuildContext) -> None:
        super().__init__(ctx)


@register_part("embedding", "token")
class TokenEmbedding(Part):
    """Row gather from ``[vocab_size, width]`` into the fp32 residual stream, times ``scale``.

    Spec parameters: ``vocab_size``, ``width``, ``scale`` (a factor on the table's rows, in
    fp32 inside the kernel; 1 when absent, as for GPT-2).
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext) -> None:
        super().__init__(ctx)
        self.vocab_size = int(spec.vocab_size)  # type: ignore[arg-type]
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.scale = float(spec.get("scale", 1.0))  # type: ignore[arg-type]
        self.weight = self.add_param("weight", (self.vocab_size, self.width), "table")

    def forward(self, step: StepContext, out: torch.Tensor,
                added: tuple[torch.Tensor, torch.Tensor] | None) -> None:
        table, index = added if added is not None else (None, None)
        ops.embed_rows(self.weight, step.tokens[:step.num_rows], out,
                       add_table=table,
                       add_index=None if index is None else index[:step.num_rows],
                       bad_index=step.bad_index, scale=self.scale)


@register_part("head", "linear")
class LinearHead(Part):
    """``logits = hidden @ weight.T`` in fp32, no bias; ``weight`` is the embedding table when
    tied (``python/ayaka/layers/embedding/token.py:81-100``).

    Spec parameters: ``vocab_size``, ``width``, ``tied`` (bool); ``logit_scale`` (a factor on
    the logits, 1 when absent) and ``logit_softcap`` (``cap * tanh(x / cap)`` after the
    factor, off when absent or 0): GPT-2 has neither, and then nothing more is launched.
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext,
                 embedding: TokenEmbedding | None = None) -> None:
        super().__init__(ctx)
        self.vocab_size = int(spec.vocab_size)  # type: ignore[arg-type]
        self.tied = bool(spec.get("tied", True))
        self.logit_scale = float(spec.get("logit_scale", 1.0))  # type: ignore[arg-type]
        self.logit_softcap = float(spec.get("logit_softcap", 0.0))  # type: ignore[arg-type]
        if self.tied:
            if embedding is None:
                raise ValueError("a tied head needs the embedding it shares")
            self.weight = embedding.weight  # the same tensor, not declared twice
        else:
            self.weight = self.add_param(
                "weight", (self.vocab_size, int(spec.width)), "matrix")  # type: ignore[arg-type]

    def forward(self, hidden: torch.Tensor, logits: torch.Tensor, *, count: int) -> None:
        ops.linear(hidden, self.weight, None, logits, rows=count)
        self._finish(logits, count)

    def _finish(self, logits: torch.Tensor, count: int) -> None:
        if self.logit_scale != 1.0 or self.logit_softcap > 0.0:
            ops.logits_scale_cap(logits, rows=count, scale=self.logit_scale,
                                 softcap=self.logit_softcap)

    def forward_normed(self, norm: Part, residual: torch.Tensor, rows: torch.Tensor,
                       scratch: torch.Tensor, logits: torch.Tensor, *, count: int) -> None:
        """``logits = LayerNorm(residual[rows]) @ weight.T``: only the wanted rows are normed."""
        ops.linear_normed(residual, norm.weight, norm.bias, norm.eps,  # type: ignore
                          self.weight, None, logits, scratch=scratch, count=count,
                          row_index=rows)
        self._finish(logits, count)
