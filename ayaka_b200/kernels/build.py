"""Compiling the CUDA sources with nvcc, one shared library per ``.cu`` file.

Nothing is compiled at import. A library is built the first time a kernel of it is called
(so a float32 run never builds the bfloat16 tensor-core kernels) or all at once by
:func:`build_all`. Libraries are cached beside the sources in ``csrc/_build`` under a name
that carries a hash of the source, its headers and the flags; when that folder cannot be
written the cache goes to a per-user folder under the system's temporary directory. While
nvcc runs, a line goes to standard error every few seconds.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

from ayaka_b200.errors import BackendError

__all__ = ["CSRC", "build_all", "ensure_built", "library_names"]

CSRC = Path(__file__).resolve().parent.parent / "csrc"
_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
)
_locks: dict[str, threading.Lock] = {}
_locks_guard = threading.Lock()


def library_names() -> list[str]:
    """Every ``.cu`` file of the source folder, without its suffix."""
    return sorted(path.stem for path in CSRC.glob("*.cu"))


def _nvcc() -> str | None:
    found = shutil.which("nvcc")
    if found:
        return found
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and (Path(root) / "bin" / "nvcc").is_file():
            return str(Path(root) / "bin" / "nvcc")
    return None


#: Libraries compiled once per value of a macro, and the values :func:`build_all` prepares.
VARIANTS: dict[str, tuple[str, tuple[int, ...]]] = {
    "attention_prefill": ("AYK_HEAD_DIM", (16, 32, 48, 64, 128)),
}


def _defines(defines: dict[str, int] | None) -> list[str]:
    return [f"-D{key}={value}" for key, value in sorted((defines or {}).items())]


def _digest(name: str, defines: dict[str, int] | None = None) -> str:
    h = hashlib.sha256()
    h.update(" ".join([*_FLAGS, *_defines(defines)]).encode())
    h.update((CSRC / f"{name}.cu").read_bytes())
    for header in sorted([*CSRC.glob("*.cuh"), *CSRC.glob("*.h")]):
        h.update(header.name.encode())
        h.update(header.read_bytes())
    return h.hexdigest()[:16]


def _fallback_dir() -> Path:
    return Path(tempfile.gettempdir()) / f"ayaka_b200-build-{os.getuid()}"


def _writable_build_dir() -> Path:
    preferred = CSRC / "_build"
    try:
        preferred.mkdir(exist_ok=True)
        probe = preferred / f".write-test-{os.getpid()}-{threading.get_ident()}"
        probe.write_bytes(b"")
        probe.unlink()
        return preferred
    except OSError:
        fallback = _fallback_dir()
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def _say(text: str) -> None:
    print(f"ayaka_b200: {text}", file=sys.stderr, flush=True)


def _compile(name: str, filename: str, verbose: bool,
             defines: dict[str, int] | None = None) -> Path:
    nvcc = _nvcc()
    if nvcc is None:
        raise BackendError(
            f"the CUDA library of {name}.cu is not built and nvcc was not found; "
            "this engine has no fallback path")
    folder = _writable_build_dir()
    target = folder / filename
    partial = folder / f".{filename}.{os.getpid()}.{threading.get_ident()}.tmp"
    command = [nvcc, *_FLAGS, *_defines(defines), "-I", str(CSRC), "-o", str(partial),
               str(CSRC / f"{name}.cu")]
    label = name + "".join(f" {d[2:]}" for d in _defines(defines))
    if verbose:
        _say(f"compiling {label}.cu for sm_100a ...")
    started = time.monotonic()
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                               text=True, cwd=str(folder))
    finished = threading.Event()

    def heartbeat() -> None:
        while not finished.wait(10.0):
            _say(f"still compiling {name}.cu ({time.monotonic() - started:.0f} s)")

    if verbose:
        threading.Thread(target=heartbeat, daemon=True).start()
    output, _ = process.communicate()
    finished.set()
    if process.returncode != 0:
        partial.unlink(missing_ok=True)
        raise BackendError(f"nvcc failed on {name}.cu:\n{output}")
    os.replace(partial, target)
    tag = _tag(defines)
    for stale in folder.glob(f"libayk_{name}{tag}.*.so"):
        if stale != target and stale.name.count(".") == target.name.count("."):
            stale.unlink(missing_ok=True)
    if verbose:
        _say(f"compiled {label}.cu in {time.monotonic() - started:.1f} s")
    return target


def _tag(defines: dict[str, int] | None) -> str:
    return "".join(f"-{key.lower()}{value}" for key, value in sorted((defines or {}).items()))


def ensure_built(name: str, *, verbose: bool = True,
                 defines: dict[str, int] | None = None) -> Path:
    """Return the path of the shared library of ``csrc/<name>.cu`` (compiled with the given
    macro definitions), compiling it if needed."""
    if not (CSRC / f"{name}.cu").is_file():
        raise BackendError(f"no CUDA source {CSRC / (name + '.cu')}")
    key = name + _tag(defines)
    with _locks_guard:
        lock = _locks.setdefault(key, threading.Lock())
    with lock:
        filename = f"libayk_{key}.{_digest(name, defines)}.so"
        for folder in (CSRC / "_build", _fallback_dir()):
            if (folder / filename).is_file():
                return folder / filename
        return _compile(name, filename, verbose, defines)


def build_all(*, verbose: bool = True) -> list[Path]:
    """Compile every library, several nvcc processes at a time, and return their paths."""
    jobs: list[tuple[str, dict[str, int] | None]] = []
    for name in library_names():
        if name in VARIANTS:
            macro, values = VARIANTS[name]
            jobs.extend((name, {macro: value}) for value in values)
        else:
            jobs.append((name, None))
    with ThreadPoolExecutor(max_workers=max(1, min(os.cpu_count() or 1, len(jobs)))) as pool:
        return list(pool.map(
            lambda job: ensure_built(job[0], verbose=verbose, defines=job[1]), jobs))
