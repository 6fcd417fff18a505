"""Descriptions of a model as data: parts with their sizes, layers, and the order they run in.

A :class:`PartSpec` names a registered kind of part and carries every size and constant that
part needs; nothing in a part reads a model's configuration. A :class:`LayerSpec` picks a
mixer, a feed-forward and norms for one layer and the arrangement that wires them. The
execution order is a list of :class:`Run` entries, which may name a layer twice or let a run
read the cache another run wrote.
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass, field

__all__ = ["LayerSpec", "ModelSpec", "PartSpec", "Run"]


class PartSpec:
    """A registered part kind and its parameters; immutable, hashable, attribute access."""

    __slots__ = ("_items", "kind")

    def __init__(self, kind: str, **params: object) -> None:
        object.__setattr__(self, "kind", kind)
        object.__setattr__(self, "_items", tuple(sorted(params.items())))

    def __getattr__(self, name: str) -> object:
        for key, value in object.__getattribute__(self, "_items"):
            if key == name:
                return value
        raise AttributeError(f"part {self.kind!r} has no parameter {name!r}")

    def __setattr__(self, name: str, value: object) -> None:
        raise AttributeError("a PartSpec cannot be changed")

    def get(self, name: str, default: object = None) -> object:
        for key, value in self._items:
            if key == name:
                return value
        return default

    @property
    def params(self) -> Mapping[str, object]:
        return dict(self._items)

    def __eq__(self, other: object) -> bool:
        return isinstance(other, PartSpec) and (self.kind, self._items) == (other.kind,
                                                                           other._items)

    def __hash__(self) -> int:
        return hash((self.kind, self._items))

    def __repr__(self) -> str:
        inner = ", ".join(f"{key}={value!r}" for key, value in self._items)
        return f"PartSpec({self.kind!r}, {inner})"


@dataclass(frozen=True, slots=True)
class LayerSpec:
    """One layer: the arrangement (a registered block kind) and the parts it wires."""

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True, slots=True)
class Run:
    """One entry of the execution order.

    Attributes:
        layer: index into ``ModelSpec.layers``; a layer may appear in several runs.
        reads_cache_of: index of an earlier entry of the order whose cache this run reads
            instead of writing one of its own, or ``None``.
    """

    layer: int
    reads_cache_of: int | None = None


@dataclass(frozen=True, slots=True)
class ModelSpec:
    """A whole decoder as data."""

    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    position: PartSpec
    layers: tuple[LayerSpec, ...]
    order: tuple[Run, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_id: int | None = None
    extra: Mapping[str, object] = field(default_factory=dict)
