import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "tests") not in sys.path:      # helper modules beside the tests (gguf_cases)
    sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def lib():
    import mlcompiler_b200
    return mlcompiler_b200.load_library(build_if_missing=True)


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    oracle.build_port()
    return oracle


@pytest.fixture(scope="session")
def executor(lib):
    import mlcompiler_b200
    ex = mlcompiler_b200.Executor(0)
    yield ex
    ex.close()
