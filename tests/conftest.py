import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def built_lib():
    """The CUDA library, compiled in-tree if it is stale (nvcc cross-compiles without a GPU)."""
    from tile_fusion_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def oracle(built_lib):
    from oracle.bindings import Oracle, build
    build(ref=True)
    return Oracle()


@pytest.fixture(scope="session")
def ref(oracle):
    from oracle.bindings import Ref
    if not Ref.available():
        pytest.skip("reference tree not present and oracle/_ref not built")
    return Ref()
