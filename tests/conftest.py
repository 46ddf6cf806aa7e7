"""Shared fixtures.  Tests marked ``gpu`` need a B200; everything else runs on CPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def _have_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _have_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def fa():
    """The package (ctypes binding over libfa_b200.so); builds the library if missing."""
    import __graft_entry__ as ge
    pkg = ge.load_package()
    if not os.path.exists(pkg.LIB_PATH):
        ge.build()
    return pkg


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.lib()
    return o


@pytest.fixture(scope="session")
def golden():
    return {name: np.load(os.path.join(GOLDEN, name + ".npz"))
            for name in ("demo_b1h4s256d64", "bench_gate", "normal_small")}


@pytest.fixture(params=["auto", "one_tile", "tile_pair", "cta_pair"])
def prefill_variant(request, fa):
    """Runs a test once per 16-bit prefill kernel (fa_set_prefill_variant) and once with the
    library's own choice."""
    fa.set_prefill_variant(request.param)
    yield request.param
    fa.set_prefill_variant("auto")


@pytest.fixture()
def dev(fa):
    import torch
    torch.cuda.set_device(0)
    fa.clear_device_status()
    yield torch.device("cuda:0")
    assert fa.device_status() == 0, "a kernel recorded an error status"
