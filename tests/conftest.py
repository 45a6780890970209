import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def golden_files(kind):
    names = sorted(n for n in os.listdir(GOLDEN) if n.endswith(".npz") and n.startswith(kind + "_"))
    return [os.path.join(GOLDEN, n) for n in names]


@pytest.fixture(scope="session")
def library_path():
    """Path of the built C-ABI library; built on demand with nvcc (cross-compiles without a GPU)."""
    from qutai_b200 import build

    return build.ensure_built()
