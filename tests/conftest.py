import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu on the GPU box")


def _has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle.bindings import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The unmodified reference behind oracle/_ref, where that library was built."""
    from oracle.bindings import Reference
    if not Reference.available():
        pytest.skip("oracle/_ref/libcortexsdr_ref.so not built (reference tree absent)")
    return Reference()


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(os.path.join(GOLDEN, name), allow_pickle=False)
    return load


@pytest.fixture(scope="session")
def lib():
    from cortexsdr_b200 import _lib
    return _lib.load(build_if_missing=True)


@pytest.fixture(scope="session")
def ctx(lib):
    import cortexsdr_b200 as cs
    return cs.default_context()


def rel_err(y, ref):
    """(max-abs / max|ref|, relative L2): the two parity metrics of the matmul path."""
    y = np.asarray(y, np.float64)
    ref = np.asarray(ref, np.float64)
    den = max(np.abs(ref).max(), 1e-30)
    return np.abs(y - ref).max() / den, np.linalg.norm(y - ref) / max(np.linalg.norm(ref), 1e-30)
