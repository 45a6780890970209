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


@pytest.fixture
def kernel_variant():
    """``kernel_variant(which)`` switches one kernel to its comparison form (``qmoe_test_select_variant``) for the
    rest of the test; every selector is back at its default afterwards."""
    from qutai_b200 import lib

    chosen = []

    def select(which, value=1):
        lib.call("qmoe_test_select_variant", which, value)
        chosen.append(which)

    yield select
    for which in chosen:
        lib.call("qmoe_test_select_variant", which, 0)
