"""Shared pytest configuration: the ``gpu`` marker and helpers used by several files."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on a B200")


@pytest.fixture(scope="session")
def golden_dir() -> Path:
    return ROOT / "tests" / "golden"


@pytest.fixture(scope="session")
def native_lib():
    """The built C-ABI library (built on demand; nvcc cross-compiles without a GPU)."""
    from fuseml_b200 import _native, build

    build.build()
    return _native.load()
