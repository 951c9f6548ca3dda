import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from harness import CpuBackend
    return CpuBackend("oracle")


@pytest.fixture(scope="session")
def ref():
    from harness import CpuBackend, have_ref
    if not have_ref():
        pytest.skip("oracle/_ref/libplast_ref.so not built (reference sources absent)")
    return CpuBackend("ref")


@pytest.fixture(scope="session")
def cuda():
    from harness import CudaBackend
    return CudaBackend()


@pytest.fixture(scope="session")
def recipes():
    from harness import OracleRecipes
    return OracleRecipes()
