"""Reading and writing safetensors files without any library.

Layout: a little-endian ``u64`` header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` (plus an optional
``__metadata__``), then the payload. The header is validated before a byte of payload
is touched, as the reference does (``python/ayaka/weights/safetensors.py:154-295``):
length inside the file, no repeated name, known dtype, offsets inside the payload,
``end - begin == prod(shape) * itemsize``, no overlap. Tensors are read through one
memory map.
"""

from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import torch

from ayaka_b200.errors import ModelLoadError

__all__ = ["DTYPE_OF_TOKEN", "SafetensorsFile", "TensorEntry", "write_safetensors"]

_DTYPES: dict[str, torch.dtype] = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_TOKENS = {dtype: token for token, dtype in _DTYPES.items()}
DTYPE_OF_TOKEN = _DTYPES
_MAX_HEADER = 100 << 20


@dataclass(frozen=True, slots=True)
class TensorEntry:
    """One tensor of a file: its dtype token, shape and byte range in the payload."""

    name: str
    dtype: str
    shape: tuple[int, ...]
    begin: int
    end: int


def _strict_object(pairs: list[tuple[str, object]]) -> dict[str, object]:
    out: dict[str, object] = {}
    for key, value in pairs:
        if key in out:
            raise ModelLoadError(f"safetensors header repeats the name {key!r}")
        out[key] = value
    return out


class SafetensorsFile:
    """A validated safetensors file; ``tensor(name)`` returns a CPU tensor over the map."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        if not self.path.is_file():
            raise ModelLoadError(f"{self.path} does not exist", context={"path": str(self.path)})
        size = self.path.stat().st_size
        with open(self.path, "rb") as handle:
            head = handle.read(8)
            if len(head) != 8:
                raise ModelLoadError(f"{self.path} is too short to be a safetensors file")
            (header_len,) = struct.unpack("<Q", head)
            if header_len > _MAX_HEADER or 8 + header_len > size:
                raise ModelLoadError(
                    f"{self.path}: header length {header_len} does not fit a file of {size} bytes")
            raw = handle.read(header_len)
        try:
            header = json.loads(raw.decode("utf-8"), object_pairs_hook=_strict_object)
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise ModelLoadError(f"{self.path}: header is not valid JSON: {error}") from None
        if not isinstance(header, dict):
            raise ModelLoadError(f"{self.path}: header must be a JSON object")
        self._payload_start = 8 + header_len
        payload = size - self._payload_start
        self.metadata = header.pop("__metadata__", None)
        self.entries: dict[str, TensorEntry] = {}
        ranges: list[tuple[int, int, str]] = []
        for name, info in header.items():
            entry = self._entry(name, info, payload)
            self.entries[name] = entry
            if entry.end > entry.begin:
                ranges.append((entry.begin, entry.end, name))
        ranges.sort()
        for (_, end, first), (begin, _, second) in zip(ranges, ranges[1:]):
            if begin < end:
                raise ModelLoadError(f"{self.path}: tensors {first!r} and {second!r} overlap")
        self._map: mmap.mmap | None = None

    def _entry(self, name: str, info: object, payload: int) -> TensorEntry:
        where = f"{self.path}: tensor {name!r}"
        if not isinstance(info, dict):
            raise ModelLoadError(f"{where} has no description")
        dtype, shape, offsets = info.get("dtype"), info.get("shape"), info.get("data_offsets")
        if dtype not in _DTYPES:
            raise ModelLoadError(f"{where} has the unknown dtype {dtype!r}")
        if not isinstance(shape, list) or any(type(n) is not int or n < 0 for n in shape):
            raise ModelLoadError(f"{where} has a malformed shape {shape!r}")
        if (not isinstance(offsets, list) or len(offsets) != 2
                or any(type(n) is not int for n in offsets)):
            raise ModelLoadError(f"{where} has malformed data_offsets {offsets!r}")
        begin, end = offsets
        if not 0 <= begin <= end <= payload:
            raise ModelLoadError(f"{where}: bytes [{begin}, {end}) lie outside the payload")
        count = 1
        for n in shape:
            count *= n
        itemsize = torch.empty((), dtype=_DTYPES[dtype]).element_size()
        if end - begin != count * itemsize:
            raise ModelLoadError(
                f"{where}: {end - begin} bytes do not hold shape {shape} of {dtype}")
        return TensorEntry(name, dtype, tuple(shape), begin, end)

    def names(self) -> list[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor's values, a CPU tensor that aliases the file's memory map (read only)."""
        entry = self.entries[name]
        dtype = _DTYPES[entry.dtype]
        if entry.end == entry.begin:
            return torch.empty(entry.shape, dtype=dtype)
        if self._map is None:
            with open(self.path, "rb") as handle:
                self._map = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_READ)
        count = 1
        for n in entry.shape:
            count *= n
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            flat = torch.frombuffer(self._map, dtype=dtype, count=count,
                                    offset=self._payload_start + entry.begin)
        return flat.reshape(entry.shape)

    def close(self) -> None:
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:  # a tensor still aliases the map; the OS unmaps at exit
                pass
            self._map = None


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor],
                      metadata: dict[str, str] | None = None) -> None:
    """Write ``tensors`` (CPU or device, any listed dtype) as one safetensors file."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    ordered = list(tensors.items())
    for name, tensor in ordered:
        if tensor.dtype not in _TOKENS:
            raise ModelLoadError(f"cannot store dtype {tensor.dtype} of {name!r}")
        size = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _TOKENS[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + size]}
        offset += size
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-len(raw) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(raw)))
        handle.write(raw)
        for _, tensor in ordered:
            data = tensor.detach().to("cpu").contiguous()
            if data.numel():
                handle.write(data.reshape(-1).view(torch.uint8).numpy().data)
