"""One registry from the architecture name in ``config.json`` to everything that makes it run.

An :class:`Architecture` bundles four functions: parse the configuration, describe the
model as a :class:`~ayaka_b200.parts.spec.ModelSpec`, map checkpoint tensor names to the
model's parameters, and draw random weights in checkpoint layout. Adding an architecture is
registering one more of these; the engine, the cache, the scheduler and the replay program
take whatever the registry returns (the reference resolves names the same way,
``python/ayaka/models/registry.py:28-87``).
"""

from __future__ import annotations

from collections.abc import Callable, Iterator, Mapping
from dataclasses import dataclass

import torch

from ayaka_b200.errors import ModelLoadError
from ayaka_b200.parts.spec import ModelSpec
from ayaka_b200.weights.rules import RandomInit, WeightRules

__all__ = ["Architecture", "register_architecture", "resolve_architecture",
           "supported_architectures"]


@dataclass(frozen=True, slots=True)
class Architecture:
    """Everything architecture-specific, as functions of the parsed configuration."""

    name: str
    parse_config: Callable[[Mapping[str, object]], object]
    model_spec: Callable[[object], ModelSpec]
    weight_rules: Callable[[object], WeightRules]
    random_tensors: Callable[[object, int, RandomInit], Iterator[tuple[str, torch.Tensor]]]
    config_json: Callable[[object], dict[str, object]]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(architecture: Architecture) -> Architecture:
    _ARCHITECTURES[architecture.name] = architecture
    return architecture


def supported_architectures() -> list[str]:
    _builtin()
    return sorted(_ARCHITECTURES)


def resolve_architecture(name: object) -> Architecture:
    """The registered architecture called ``name``; the error lists the supported names."""
    _builtin()
    if not isinstance(name, str) or name not in _ARCHITECTURES:
        raise ModelLoadError(
            f"architecture {name!r} is not supported; supported: {sorted(_ARCHITECTURES)}",
            context={"architecture": name, "supported": tuple(sorted(_ARCHITECTURES))})
    return _ARCHITECTURES[name]


def architecture_of(config_json: Mapping[str, object]) -> Architecture:
    """The architecture a parsed ``config.json`` names in ``architectures[0]``."""
    names = config_json.get("architectures")
    if not isinstance(names, (list, tuple)) or not names:
        raise ModelLoadError("config.json has no 'architectures' list; cannot choose a model",
                             context={"missing": ("architecture",)})
    return resolve_architecture(names[0])


def _builtin() -> None:
    import ayaka_b200.models.gpt2  # noqa: F401  (registers itself)
