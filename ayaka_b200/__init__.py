"""ayaka_b200: a single-GPU GPT-2 inference engine written for NVIDIA B200 (sm_100a).

Public names are imported lazily so that ``import ayaka_b200`` never needs a GPU.
"""

from __future__ import annotations

__version__ = "0.1.0"

_LAZY = {
    "LLM": "ayaka_b200.engine.llm",
    "EngineConfig": "ayaka_b200.config.engine",
    "GPT2Config": "ayaka_b200.config.model",
    "SamplingParams": "ayaka_b200.sampling.params",
    "RequestOutput": "ayaka_b200.engine.outputs",
}

__all__ = ["__version__", *_LAZY]


def __getattr__(name: str) -> object:
    if name in _LAZY:
        import importlib

        return getattr(importlib.import_module(_LAZY[name]), name)
    raise AttributeError(f"module 'ayaka_b200' has no attribute {name!r}")
