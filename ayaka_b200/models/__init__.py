"""Models: the registry of architectures, the generic decoder, and loading one from a folder."""

from __future__ import annotations

from collections.abc import Mapping
from pathlib import Path

import torch

from ayaka_b200.config.model import read_config_json
from ayaka_b200.models.decoder import DecoderModel
from ayaka_b200.models.registry import (Architecture, architecture_of, register_architecture,
                                        resolve_architecture, supported_architectures)
from ayaka_b200.parts.base import BuildContext
from ayaka_b200.weights.loader import TensorSource, load_into, open_model_dir

__all__ = ["Architecture", "DecoderModel", "architecture_of", "build_model", "load_model",
           "register_architecture", "resolve_architecture", "supported_architectures"]

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def build_model(config_json: Mapping[str, object], dtype: str,
                device: str | torch.device) -> tuple[DecoderModel, Architecture, object]:
    """Build (not load) the model a parsed ``config.json`` names."""
    architecture = architecture_of(config_json)
    config = architecture.parse_config(config_json)
    ctx = BuildContext(dtype=_DTYPES[dtype], device=torch.device(device))
    return DecoderModel(architecture.model_spec(config), ctx), architecture, config


def load_model(model_dir: str | Path, dtype: str, device: str | torch.device,
               tensors: Mapping[str, torch.Tensor] | None = None) -> tuple[DecoderModel, object]:
    """Build the model of ``model_dir/config.json`` and fill it from the folder's
    safetensors (or from ``tensors``, checkpoint-named, when given)."""
    config_json = read_config_json(model_dir)
    model, architecture, config = build_model(config_json, dtype, device)
    source = TensorSource(tensors=tensors) if tensors is not None else open_model_dir(model_dir)
    try:
        load_into(model, architecture.weight_rules(config), source)
    finally:
        source.close()
    return model, config
