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


@pytest.fixture(autouse=True, scope="session")
def _bf16_gemm_choice():
    """``AYK_TEST_BF16_GEMM=simt`` runs the bfloat16 engine tests on the CUDA-core matrix
    product (a development aid for telling a tensor-core fault from a cache fault)."""
    import os

    choice = os.environ.get("AYK_TEST_BF16_GEMM")
    if choice:
        from ayaka_b200.kernels import ops

        ops.BF16_GEMM = choice
    yield
