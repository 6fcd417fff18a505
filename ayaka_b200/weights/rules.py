"""How checkpoint tensors become model parameters, as data an architecture provides."""

from __future__ import annotations

import re
from dataclasses import dataclass, field

__all__ = ["RandomInit", "WeightRule", "WeightRules"]


@dataclass(frozen=True, slots=True)
class WeightRule:
    """Where one checkpoint tensor goes.

    The simplest rule fills a whole parameter, transposed on the way if the checkpoint stores
    it so. A parameter may also be *stacked* from several stored tensors (separate query, key
    and value matrices into one fused matrix; two feed-forward inputs into one), and a stored
    tensor may give only a *slice* of itself, or feed several parameters (a tuple of rules
    under one name). The reference describes the same with ``stored_parts``
    (``python/ayaka/models/base.py:169-177, 202-263``).

    Attributes:
        parameter: the model parameter this tensor (or slice) lands in.
        transposed: the checkpoint stores the transpose (Conv1D ``[in, out]``).
        dim: the dimension of the parameter along which ``offset`` and ``take`` count.
        offset: where along ``dim`` of the parameter the piece starts; ``None``: the piece is
            the whole parameter.
        take: ``(start, stop)`` along ``dim`` of the stored tensor (after transposition): only
            that slice is used; ``None``: all of it.
    """

    parameter: str
    transposed: bool = False
    dim: int = 0
    offset: int | None = None
    take: tuple[int, int] | None = None


@dataclass(frozen=True, slots=True)
class WeightRules:
    """Checkpoint name -> rule, names to ignore, and prefixes a checkpoint may carry.

    Attributes:
        rules: exact checkpoint names (without optional prefix) and their parameters.
        ignore: regular expressions (full match, after the prefix is stripped) of tensors
            that are in checkpoints but are not parameters (stored masks, a tied head).
        optional_prefixes: a name may start with one of these; it is stripped first.
    """

    rules: dict[str, WeightRule | tuple[WeightRule, ...]]
    ignore: tuple[str, ...] = ()
    optional_prefixes: tuple[str, ...] = ()
    _compiled: list[re.Pattern[str]] = field(default_factory=list, compare=False, repr=False)

    def of(self, stripped: str) -> tuple[WeightRule, ...]:
        """The rules of one checkpoint name (one stored tensor may feed several parameters)."""
        found = self.rules[stripped]
        return found if isinstance(found, tuple) else (found,)

    def strip(self, name: str) -> str:
        for prefix in self.optional_prefixes:
            if name.startswith(prefix):
                return name[len(prefix):]
        return name

    def ignored(self, stripped: str) -> bool:
        if not self._compiled and self.ignore:
            self._compiled.extend(re.compile(pattern) for pattern in self.ignore)
        return any(pattern.fullmatch(stripped) for pattern in self._compiled)


@dataclass(frozen=True, slots=True)
class RandomInit:
    """Distribution of random weights.

    Attributes:
        weight_std: standard deviation of matrices and tables (mean 0).
        scale_residual_projections: draw the projections that write to the residual stream
            with ``weight_std / sqrt(2 * n_layer)``.
        bias_std: standard deviation of biases (0: all zero).
        norm_std: norm scales are ``1 + N(0, norm_std)`` and norm biases ``N(0, norm_std)``
            (0: scale 1, bias 0).
    """

    weight_std: float = 0.02
    scale_residual_projections: bool = True
    bias_std: float = 0.0
    norm_std: float = 0.0
