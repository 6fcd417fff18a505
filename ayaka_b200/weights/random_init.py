"""Random-weights mode: a model folder written from a configuration and a seed.

The reference has the mode only as an enum member and refuses it
(``python/ayaka/model_loader/loader.py:172-183``); here it is the way tests and benchmarks
get models without a network. The tensors are drawn by the architecture under checkpoint
names and in checkpoint layout, so the folder loads like any other.
"""

from __future__ import annotations

import json
from collections.abc import Mapping
from pathlib import Path

import torch

from ayaka_b200.errors import ConfigError
from ayaka_b200.models.registry import architecture_of
from ayaka_b200.weights.rules import RandomInit
from ayaka_b200.weights.safetensors import write_safetensors

__all__ = ["random_state", "write_random_model"]

_STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def random_state(config_json: Mapping[str, object], seed: int,
                 init: RandomInit | None = None,
                 store_dtype: str = "float32") -> dict[str, torch.Tensor]:
    """Checkpoint-named random tensors for the architecture ``config_json`` names."""
    if store_dtype not in _STORE:
        raise ConfigError("random.store_dtype", "INVALID_CHOICE",
                          f"must be one of {sorted(_STORE)}, got {store_dtype!r}")
    architecture = architecture_of(config_json)
    config = architecture.parse_config(config_json)
    dtype = _STORE[store_dtype]
    return {name: tensor.to(dtype)
            for name, tensor in architecture.random_tensors(config, seed, init or RandomInit())}


def write_random_model(config_json: Mapping[str, object], folder: str | Path, seed: int,
                       init: RandomInit | None = None, store_dtype: str = "float32") -> Path:
    """Write ``folder/config.json`` and ``folder/model.safetensors`` and return the folder."""
    out = Path(folder)
    out.mkdir(parents=True, exist_ok=True)
    architecture = architecture_of(config_json)
    config = architecture.parse_config(config_json)
    state = random_state(config_json, seed, init, store_dtype)
    (out / "config.json").write_text(
        json.dumps(architecture.config_json(config), indent=2) + "\n", encoding="utf-8")
    write_safetensors(out / "model.safetensors", state,
                      metadata={"format": "pt", "seed": str(seed)})
    return out
