"""Shared pytest configuration: the ``gpu`` marker and common fixtures."""

from __future__ import annotations

import pathlib
import sys

import numpy as np
import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config: pytest.Config, items: list[pytest.Item]) -> None:
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden() -> dict[str, np.ndarray]:
    """Vectors generated from the reference's own test functions (tests/golden/make_golden.py)."""
    with np.load(ROOT / "tests" / "golden" / "reference_vectors.npz") as data:
        return {key: data[key] for key in data.files}
