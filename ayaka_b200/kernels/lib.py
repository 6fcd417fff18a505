"""Loading the CUDA libraries through ctypes and checking what their entry points return."""

from __future__ import annotations

import ctypes
import threading

import torch

from ayaka_b200.errors import BackendError
from ayaka_b200.kernels.build import ensure_built

__all__ = ["check", "entry", "library", "loaded_libraries", "raw_stream", "set_pdl"]

_REFUSALS = {
    -1: "an argument the kernel does not take (a size, a stride or a missing pointer)",
    -2: "a pointer or stride that breaks the kernel's alignment rule",
    -3: "a size beyond the kernel's stated maximum",
    -4: "a CUDA driver entry point is missing or failed",
    -5: "a device-side wait ran out; the kernel gave up and reported it",
}
_libraries: dict[str, ctypes.CDLL] = {}
_guard = threading.Lock()
_pdl = True


def set_pdl(enabled: bool) -> None:
    """Programmatic dependent launch on or off, in the libraries loaded so far and in those
    loaded later."""
    global _pdl
    with _guard:
        _pdl = bool(enabled)
        for found in _libraries.values():
            found.ayk_set_pdl(ctypes.c_int(1 if _pdl else 0))


def library(name: str, **defines: int) -> ctypes.CDLL:
    """The shared library built from ``csrc/<name>.cu`` (with the given macro definitions);
    built on first use, loaded once."""
    if not defines:  # the usual call, hundreds of times a step: no key to build, no lock
        found = _libraries.get(name)
        if found is not None:
            return found
    key = name + "".join(f"-{k}{v}" for k, v in sorted(defines.items()))
    with _guard:
        found = _libraries.get(key)
        if found is None:
            path = ensure_built(name, defines=defines or None)
            try:
                found = ctypes.CDLL(str(path))
            except OSError as error:
                raise BackendError(f"cannot load {path}: {error}") from None
            if not _pdl:
                found.ayk_set_pdl(ctypes.c_int(0))
            _libraries[key] = found
        return found


_entries: dict[tuple[str, str], object] = {}


def entry(name: str, symbol: str):  # noqa: ANN201 - a ctypes function pointer
    """The exported function ``symbol`` of ``csrc/<name>.cu``'s library, looked up once: a
    step launches hundreds of kernels and the look-up (a lock, a key, an attribute search)
    would otherwise be paid per launch."""
    found = _entries.get((name, symbol))
    if found is None:
        found = getattr(library(name), symbol)
        _entries[(name, symbol)] = found
    return found


try:  # torch's own accessors, without the Stream object the public call builds per call
    _raw_stream = torch._C._cuda_getCurrentRawStream
    _device_index = torch._C._cuda_getDevice
except AttributeError:  # pragma: no cover - other torch builds
    _raw_stream = _device_index = None


def raw_stream() -> int:
    """The handle of the current CUDA stream of the current device."""
    if _raw_stream is not None:
        return _raw_stream(_device_index())
    return torch.cuda.current_stream().cuda_stream


def loaded_libraries() -> list[str]:
    """Names of the libraries this process has loaded so far."""
    return sorted(_libraries)


def check(status: int, op: str) -> None:
    """Raise :class:`BackendError` unless an entry point returned 0."""
    if status == 0:
        return
    if status < 0:
        reason = _REFUSALS.get(status, f"refusal code {status}")
        raise BackendError(f"{op}: {reason}", context={"op": op, "status": status})
    raise BackendError(f"{op}: CUDA error {status} at launch", context={"op": op, "status": status})
