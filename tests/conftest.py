import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def built_library():
    """The CUDA library and the CPU checker exist (built in-tree; nvcc cross-compiles without a GPU)."""
    from dooms_b200 import _lib
    if not _lib.LIB_PATH.exists():
        from dooms_b200.build import build
        build()
    from oracle import binding
    if not binding.ORACLE_SO.exists():
        binding.build()
    return _lib.lib()


@pytest.fixture(scope="session")
def model_dir(tmp_path_factory):
    return tmp_path_factory.mktemp("models")
