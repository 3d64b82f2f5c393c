"""Shared test set-up: import paths, the `gpu` marker and small seeded model directories."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "text-embeddings-inference_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


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
    """The built shared library; building it is cheap when nothing changed."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("tei_b200_build", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if not mod.LIB_PATH.exists():
        mod.build()
    from tei_b200 import _lib
    return _lib.load()


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Small seeded model directories of every family (head_dim 32, 64 and 128)."""
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import small_models
    return small_models.write_all(tmp_path_factory.mktemp("models"))
