import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) device")


def pytest_collection_modifyitems(config, items):
    # The no-allocation entry point's test must run after every other test.
    items.sort(key=lambda it: 1 if "test_zz_" in it.nodeid else 0)


@pytest.fixture(scope="session")
def orc():
    from oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "linear_path.npz"))


@pytest.fixture(scope="session")
def lib():
    import gem16_b200.build as b
    if not os.path.exists(b.LIB):
        b.build()
    from gem16_b200 import load
    return load()


@pytest.fixture(scope="session")
def dev(lib):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    lib.gemb_device_check()
    return torch.device("cuda:0")
