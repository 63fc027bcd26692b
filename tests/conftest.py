import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import gqa_oracle

    gqa_oracle.build()
    return gqa_oracle


@pytest.fixture(scope="session")
def gqa_lib():
    """The C-ABI library; GPU tests fail loudly (not skip) when it has not been built."""
    from hopper_jeni_b200 import capi

    return capi.load_library()


@pytest.fixture(scope="session")
def selftest_lib(gqa_lib):
    """The diagnostics library (checker kernels, building-block and time-out self tests)."""
    from hopper_jeni_b200 import capi

    return capi.load_selftest_library()
