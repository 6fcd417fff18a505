"""Markers and shared fixtures. ``-m gpu`` tests need a CUDA device; everything else runs on
the CPU. Model folders are written under pytest's temporary folder, never into the tree."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for path in (ROOT, ROOT / "tests"):
    if str(path) not in sys.path:
        sys.path.insert(0, str(path))


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config: pytest.Config, items: list[pytest.Item]) -> None:
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter: pytest.TerminalReporter) -> None:
    """The largest engine-against-plain errors the run measured, per kind of test."""
    try:
        import engine_support
    except ImportError:
        return
    if engine_support.MEASURED:
        terminalreporter.write_sep("-", "largest errors, as a fraction of the largest |logit|")
        for name, value in sorted(engine_support.MEASURED.items()):
            terminalreporter.write_line(f"{name}\t{value:.2e}")
