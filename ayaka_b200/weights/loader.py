"""Filling a model's parameters from tensors found by name.

All problems of a checkpoint are collected and raised as one
:class:`~ayaka_b200.errors.ModelLoadError` that lists ``missing``, ``unexpected``,
``wrong_shape`` and ``unsupported_dtype`` (the reference reports the same categories at
once, ``python/ayaka/weights/mapping.py:131-174``); nothing is copied before the check
passes. Conversion: stored F64/F32/F16/BF16 values are converted to the parameter's dtype
(matrices and tables in the compute dtype, vectors float32, integer tables int32); Conv1D
weights are transposed while they are copied.
"""

from __future__ import annotations

import json
from collections.abc import Mapping
from pathlib import Path

import torch

from ayaka_b200.errors import ModelLoadError
from ayaka_b200.parts.base import Part
from ayaka_b200.weights.rules import WeightRules
from ayaka_b200.weights.safetensors import DTYPE_OF_TOKEN, SafetensorsFile

__all__ = ["TensorSource", "load_into", "open_model_dir"]

_FLOATS = (torch.float64, torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class TensorSource:
    """Tensors by name with their shapes and dtypes known before any value is read."""

    def __init__(self, files: list[SafetensorsFile] | None = None,
                 tensors: Mapping[str, torch.Tensor] | None = None) -> None:
        self._files = files or []
        self._tensors = dict(tensors or {})
        self._where: dict[str, SafetensorsFile] = {}
        for file in self._files:
            for name in file.names():
                if name in self._where:
                    raise ModelLoadError(f"tensor {name!r} is stored in two files")
                self._where[name] = file

    def names(self) -> list[str]:
        return [*self._where, *self._tensors]

    def describe(self, name: str) -> tuple[tuple[int, ...], torch.dtype]:
        if name in self._tensors:
            tensor = self._tensors[name]
            return tuple(tensor.shape), tensor.dtype
        entry = self._where[name].entries[name]
        return entry.shape, DTYPE_OF_TOKEN[entry.dtype]

    def tensor(self, name: str) -> torch.Tensor:
        if name in self._tensors:
            return self._tensors[name]
        return self._where[name].tensor(name)

    def close(self) -> None:
        for file in self._files:
            file.close()


def open_model_dir(model_dir: str | Path) -> TensorSource:
    """The tensors of a model folder: ``model.safetensors``, or the shards that
    ``model.safetensors.index.json`` lists, or every ``*.safetensors`` file in it."""
    folder = Path(model_dir)
    if not folder.is_dir():
        raise ModelLoadError(f"{folder} is not a folder", context={"path": str(folder)})
    index = folder / "model.safetensors.index.json"
    single = folder / "model.safetensors"
    if single.is_file():
        paths = [single]
    elif index.is_file():
        try:
            weight_map = json.loads(index.read_text(encoding="utf-8"))["weight_map"]
        except (json.JSONDecodeError, KeyError, TypeError) as error:
            raise ModelLoadError(f"{index} is malformed: {error}") from None
        paths = sorted({folder / shard for shard in weight_map.values()})
        files = [SafetensorsFile(path) for path in paths]
        source = TensorSource(files)
        listed, stored = set(weight_map), set(source.names())
        if listed != stored:
            raise ModelLoadError(
                f"{index} and the shards disagree: only in the index "
                f"{sorted(listed - stored)[:5]}, only in the shards {sorted(stored - listed)[:5]}")
        return source
    else:
        paths = sorted(folder.glob("*.safetensors"))
        if not paths:
            raise ModelLoadError(f"{folder} holds no safetensors file",
                                 context={"path": str(folder)})
    return TensorSource([SafetensorsFile(path) for path in paths])


def load_into(model: Part, rules: WeightRules, source: TensorSource) -> None:
    """Copy every checkpoint tensor of ``source`` into the parameter its rule names."""
    params = dict(model.named_params())
    missing_rules = [name for name, rule in rules.rules.items() if rule.parameter not in params]
    if missing_rules:
        raise ModelLoadError("weight rules name parameters the model does not have: "
                             + ", ".join(missing_rules[:8]))
    bound: dict[str, str] = {}  # stripped checkpoint name -> stored name
    unexpected: list[str] = []
    duplicated: list[str] = []
    for stored in source.names():
        stripped = rules.strip(stored)
        if stripped in rules.rules:
            if stripped in bound:
                duplicated.append(stored)
            bound[stripped] = stored
        elif not rules.ignored(stripped):
            unexpected.append(stored)
    missing = [name for name in rules.rules if name not in bound]
    wrong_shape: list[str] = []
    unsupported: list[str] = []
    for stripped, stored in bound.items():
        rule = rules.rules[stripped]
        param = params[rule.parameter]
        shape, dtype = source.describe(stored)
        expected = tuple(param.tensor.shape)
        if rule.transposed:
            expected = expected[::-1]
        if shape != expected:
            wrong_shape.append(f"{stored}: stored {list(shape)}, expected {list(expected)}")
        allowed = _INTS if param.role == "int" else _FLOATS
        if dtype not in allowed:
            unsupported.append(f"{stored}: {dtype}")
    claimed = {rule.parameter for rule in rules.rules.values()}
    unfilled = [name for name in params if name not in claimed]
    if missing or unexpected or wrong_shape or unsupported or duplicated or unfilled:
        parts = []
        for label, items in (("missing", missing), ("unexpected", unexpected),
                             ("wrong_shape", wrong_shape), ("unsupported_dtype", unsupported),
                             ("stored_twice", duplicated),
                             ("parameters_without_a_rule", unfilled)):
            if items:
                parts.append(f"{label} ({len(items)}): " + ", ".join(sorted(items)))
        raise ModelLoadError(
            "the checkpoint does not fit the model: " + "; ".join(parts),
            context={"missing": tuple(sorted(missing)), "unexpected": tuple(sorted(unexpected)),
                     "wrong_shape": tuple(sorted(wrong_shape)),
                     "unsupported_dtype": tuple(sorted(unsupported))})
    for stripped, stored in bound.items():
        rule = rules.rules[stripped]
        target = params[rule.parameter].tensor
        value = source.tensor(stored)
        if target.device.type != "meta":
            moved = value.to(target.device, non_blocking=False)
            target.copy_(moved.t() if rule.transposed else moved)
