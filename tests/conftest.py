"""Shared test setup: repository root on sys.path, the ``gpu`` marker, and both native
libraries (the product's CUDA library and the CPU oracle) built before collection."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    # nvcc cross-compiles without a GPU; both builds are no-ops when the libraries are current.
    from kernel_pocs_b200 import build as product_build

    product_build.build()
    from oracle import oracle

    oracle.build()


@pytest.fixture(scope="session")
def golden_dir() -> Path:
    return ROOT / "tests" / "golden"
