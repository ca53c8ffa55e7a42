import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def built_lib():
    """Builds (if stale) and returns the path of the C-ABI library; nvcc works without a GPU."""
    from tensorvia_b200 import build
    return build.build_libtvb()


@pytest.fixture(scope="session")
def tv(built_lib):
    import tensorvia_b200
    return tensorvia_b200
