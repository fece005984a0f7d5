import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    cache = {}

    def load(name):
        if name not in cache:
            cache[name] = torch.load(os.path.join(GOLDEN, name + ".pt"), weights_only=False)
        return cache[name]

    return load


@pytest.fixture(scope="session")
def lib():
    """The built C-ABI library (built on demand where nvcc exists)."""
    from sana_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.load()


def nmax_err(a: torch.Tensor, ref: torch.Tensor) -> float:
    """Normalised max error max|a-ref| / max|ref| (elementwise relative error is
    ill-conditioned here: outputs cross zero)."""
    a, ref = a.double().cpu(), ref.double().cpu()
    return ((a - ref).abs().max() / ref.abs().max().clamp(min=1e-30)).item()


def cosine(a: torch.Tensor, ref: torch.Tensor) -> float:
    a, ref = a.double().flatten().cpu(), ref.double().flatten().cpu()
    return (a @ ref / (a.norm() * ref.norm()).clamp(min=1e-30)).item()
