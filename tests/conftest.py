import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def grab():
    return importlib.import_module("grab-anns_b200")


@pytest.fixture(scope="session")
def oracle():
    import oracle as o
    o.lib()
    return o


@pytest.fixture(scope="session")
def datasets():
    return importlib.import_module("grab-anns_b200.datasets")


def clustered(n, dim, n_centres, sigma, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    cen = rng.standard_normal((n_centres, dim)).astype(np.float32)
    idx = rng.integers(0, n_centres, size=n)
    return (cen[idx] + sigma * rng.standard_normal((n, dim))).astype(np.float32)
