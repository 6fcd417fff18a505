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
from ayaka_b200.weights.rules import WeightRule, WeightRules
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


def _piece_shape(rule: WeightRule, stored: tuple[int, ...]) -> tuple[int, ...] | str:
    """Shape of what ``rule`` takes out of a stored tensor (after transposition and slicing),
    or a sentence saying why it cannot."""
    shape = stored[::-1] if rule.transposed else stored
    if rule.take is None:
        return shape
    if not 0 <= rule.dim < len(shape):
        return f"has no dimension {rule.dim} to slice"
    start, stop = rule.take
    if not 0 <= start < stop <= shape[rule.dim]:
        return f"cannot give [{start}, {stop}) of its {shape[rule.dim]} along dimension {rule.dim}"
    return (*shape[:rule.dim], stop - start, *shape[rule.dim + 1:])


def load_into(model: Part, rules: WeightRules, source: TensorSource) -> None:
    """Copy every checkpoint tensor of ``source`` into the parameter (or the part of a
    parameter) its rules name. Nothing is copied unless everything fits: every stored tensor
    known and of the right shape and dtype, every parameter covered exactly once."""
    params = dict(model.named_params())
    missing_rules = [name for name in rules.rules
                     for rule in rules.of(name) if rule.parameter not in params]
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
    # parameter -> the [start, stop) ranges along the rule's dimension that pieces fill
    filled: dict[str, list[tuple[int, int, int]]] = {}
    whole: dict[str, int] = {}
    plan: list[tuple[str, WeightRule, int]] = []  # stored name, rule, length along dim
    for stripped, stored in bound.items():
        shape, dtype = source.describe(stored)
        for rule in rules.of(stripped):
            param = params[rule.parameter]
            expected = tuple(param.tensor.shape)
            piece = _piece_shape(rule, shape)
            if isinstance(piece, str):
                wrong_shape.append(f"{stored}: stored {list(shape)} {piece}")
                continue
            if rule.offset is None:
                fits = piece == expected
                whole[rule.parameter] = whole.get(rule.parameter, 0) + 1
                length = 0
            else:
                dim = rule.dim
                fits = (0 <= dim < len(expected) and len(piece) == len(expected)
                        and piece[:dim] == expected[:dim] and piece[dim + 1:] == expected[dim + 1:]
                        and 0 <= rule.offset and rule.offset + piece[dim] <= expected[dim])
                length = piece[dim] if fits else 0
                if fits:
                    filled.setdefault(rule.parameter, []).append(
                        (dim, rule.offset, rule.offset + length))
            if not fits:
                where = "" if rule.offset is None else \
                    f" at {rule.offset} along dimension {rule.dim}"
                stored_as = list(shape[::-1] if rule.transposed else shape)
                wrong_shape.append(
                    f"{stored}: stored {list(shape)}"
                    + (f" (transposed {stored_as})" if rule.transposed else "")
                    + (f", slice {list(rule.take)}" if rule.take else "")
                    + f", expected to fit {rule.parameter} {list(expected)}{where}")
            allowed = _INTS if param.role == "int" else _FLOATS
            if dtype not in allowed:
                unsupported.append(f"{stored}: {dtype}")
            plan.append((stored, rule, length))
    claimed = {rule.parameter for name in rules.rules for rule in rules.of(name)}
    unfilled = [name for name in params if name not in claimed]
    # a parameter built from pieces must be covered exactly once (judged only when all its
    # pieces are there and fit: otherwise "missing" or "wrong_shape" already says it)
    waiting = {rule.parameter for name in missing for rule in rules.of(name)}
    badly_covered: list[str] = []
    for name, count in whole.items():
        if count > 1 or name in filled:
            badly_covered.append(f"{name}: filled whole by more than one stored tensor")
    for name, ranges in filled.items():
        if name in waiting or name in whole or any(name in line for line in wrong_shape):
            continue
        dims = {dim for dim, _, _ in ranges}
        if len(dims) != 1:
            badly_covered.append(f"{name}: pieces along different dimensions")
            continue
        extent = params[name].tensor.shape[dims.pop()]
        at = 0
        for _, start, stop in sorted(ranges):
            if start != at:
                badly_covered.append(
                    f"{name}: pieces {'overlap' if start < at else 'leave a gap'} at {min(start, at)}")
                break
            at = stop
        else:
            if at != extent:
                badly_covered.append(f"{name}: pieces cover {at} of {extent}")
    if missing or unexpected or wrong_shape or unsupported or duplicated or unfilled or \
            badly_covered:
        parts = []
        for label, items in (("missing", missing), ("unexpected", unexpected),
                             ("wrong_shape", wrong_shape), ("unsupported_dtype", unsupported),
                             ("stored_twice", duplicated),
                             ("parameters_without_a_rule", unfilled),
                             ("parameters_badly_covered", badly_covered)):
            if items:
                parts.append(f"{label} ({len(items)}): " + ", ".join(sorted(items)))
        raise ModelLoadError(
            "the checkpoint does not fit the model: " + "; ".join(parts),
            context={"missing": tuple(sorted(missing)), "unexpected": tuple(sorted(unexpected)),
                     "wrong_shape": tuple(sorted(wrong_shape)),
                     "unsupported_dtype": tuple(sorted(unsupported)),
                     "badly_covered": tuple(sorted(badly_covered))})
    for stored, rule, length in plan:
        target = params[rule.parameter].tensor
        if target.device.type == "meta":
            continue
        # moved as stored, then transposed and cut on the device, where that costs nothing
        value = source.tensor(stored).to(target.device, non_blocking=False)
        if rule.transposed:
            value = value.t()
        if rule.take is not None:
            value = value.narrow(rule.dim, rule.take[0], rule.take[1] - rule.take[0])
        if rule.offset is not None:
            target = target.narrow(rule.dim, rule.offset, length)
        target.copy_(value)
