"""The parts a model is put together from, each registered under a kind name.

Importing this package registers the built-in kinds: mixer ``attention``; feed-forward
``dense``; norm ``layer_norm``; positions ``learned`` and ``none``; block ``pre_norm``;
embedding ``token``; head ``linear``.
"""

from ayaka_b200.parts import block, embedding, feed_forward, mixer, norm  # noqa: F401
from ayaka_b200.parts.base import (BuildContext, CacheNeed, Part, StateNeed, build_part,
                                   register_part, registered_kinds)
from ayaka_b200.parts.context import GroupStep, LayerCache, StepContext, Workspace
from ayaka_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, Run

__all__ = [
    "BuildContext", "CacheNeed", "GroupStep", "LayerCache", "LayerSpec", "ModelSpec", "Part",
    "PartSpec", "Run", "StateNeed", "StepContext", "Workspace", "build_part", "register_part",
    "registered_kinds",
]
