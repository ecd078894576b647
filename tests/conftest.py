"""Shared test plumbing: import paths, the `gpu` marker, and in-tree builds."""
import importlib.util
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]
PACKAGE_DIR = REPO / "flash-train_b200"
for entry in (str(REPO), str(PACKAGE_DIR / "python")):
    if entry not in sys.path:
        sys.path.insert(0, entry)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_build_module():
    spec = importlib.util.spec_from_file_location("ftrain_build", PACKAGE_DIR / "build.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


@pytest.fixture(scope="session")
def native_library():
    """libflash_train.so, rebuilt if a source is newer."""
    return load_build_module().build_library(verbose=False)


@pytest.fixture(scope="session")
def capi(native_library):
    from flash_train import capi as module

    return module


@pytest.fixture(scope="session")
def oracle():
    from oracle import build_oracle

    build_oracle.build_restatement()
    from oracle import oracle as module

    return module


@pytest.fixture(scope="session")
def reference_capi(capi, oracle):
    """The reference's own sources built for the CPU, behind the same ctypes
    declarations; None where the reference checkout (and a prebuilt copy) is absent."""
    from oracle import build_oracle

    try:
        path = build_oracle.build_reference()
    except Exception:
        path = None
    return capi.bind(str(path)) if path is not None else None
