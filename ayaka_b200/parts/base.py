"""What every part is made of: declared parameters, children, and the registries of kinds.

A part never allocates outside :meth:`Part.add_param` and never knows which model holds it.
Parameter storage follows one rule for all parts: matrices and lookup tables are kept in the
compute dtype (bfloat16 on the serving path, float32 on the 32-bit path), vectors (biases,
norm scales) in float32, integer tables in int32.
"""

from __future__ import annotations

from collections.abc import Callable, Iterator
from dataclasses import dataclass

import torch

from ayaka_b200.errors import ConfigError

__all__ = [
    "BuildContext",
    "CacheNeed",
    "Param",
    "Part",
    "StateNeed",
    "build_part",
    "register_part",
    "registered_kinds",
]


@dataclass(frozen=True, slots=True)
class BuildContext:
    """Where and in which dtype a model is built; ``meta`` builds shapes only."""

    dtype: torch.dtype
    device: torch.device


@dataclass(frozen=True, slots=True)
class CacheNeed:
    """Paged keys and values one mixer needs: its geometry and how far back it looks."""

    num_kv_heads: int
    head_dim: int
    window: int = 0  # 0: every earlier key; n > 0: the last n keys


@dataclass(frozen=True, slots=True)
class StateNeed:
    """Per-request state of fixed size one mixer needs (zeroed when a request starts)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(slots=True)
class Param:
    """One parameter tensor and how a checkpoint value becomes it."""

    tensor: torch.Tensor
    role: str  # "matrix" | "table" | "vector" | "int"


class Part:
    """Base of mixers, feed-forwards, norms, position encodings, blocks and models."""

    def __init__(self, ctx: BuildContext) -> None:
        self.ctx = ctx
        self._params: dict[str, Param] = {}
        self._children: dict[str, Part] = {}

    def add_param(self, name: str, shape: tuple[int, ...], role: str) -> torch.Tensor:
        dtype = {"matrix": self.ctx.dtype, "table": self.ctx.dtype,
                 "vector": torch.float32, "int": torch.int32}[role]
        tensor = torch.empty(shape, dtype=dtype, device=self.ctx.device)
        self._params[name] = Param(tensor, role)
        return tensor

    def share_param(self, name: str, param: Param) -> torch.Tensor:
        """Use another part's parameter under a name of this part (a tied head)."""
        self._params[name] = param
        return param.tensor

    def add_child(self, name: str, part: Part) -> Part:
        self._children[name] = part
        return part

    def named_params(self, prefix: str = "") -> Iterator[tuple[str, Param]]:
        for name, param in self._params.items():
            yield prefix + name, param
        for name, child in self._children.items():
            yield from child.named_params(f"{prefix}{name}.")

    def param(self, name: str) -> Param:
        return self._params[name]


_REGISTRIES: dict[str, dict[str, Callable[..., Part]]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}, "embedding": {},
    "head": {},
}


def register_part(family: str, kind: str) -> Callable[[Callable[..., Part]], Callable[..., Part]]:
    """Class decorator: make ``kind`` buildable in ``family`` (``mixer``, ``feed_forward``,
    ``norm``, ``position``, ``block``, ``embedding``, ``head``). Registering a kind again
    replaces it, so a test may define a toy part without touching the package."""
    if family not in _REGISTRIES:
        raise ConfigError("parts.family", "INVALID_CHOICE",
                          f"unknown family {family!r}; families are {sorted(_REGISTRIES)}")

    def decorate(factory: Callable[..., Part]) -> Callable[..., Part]:
        _REGISTRIES[family][kind] = factory
        return factory

    return decorate


def registered_kinds(family: str) -> list[str]:
    return sorted(_REGISTRIES[family])


def build_part(family: str, kind: str, *args: object, **kwargs: object) -> Part:
    """Build the registered ``kind`` of ``family``; the error lists what is registered."""
    try:
        factory = _REGISTRIES[family][kind]
    except KeyError:
        raise ConfigError(
            f"parts.{family}", "INVALID_CHOICE",
            f"no {family} of kind {kind!r} is registered; registered: "
            f"{registered_kinds(family)}") from None
    return factory(*args, **kwargs)
