"""Shared fixtures.  GPU tests carry the ``gpu`` marker; everything else runs on CPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name), allow_pickle=False)


@pytest.fixture(scope="session")
def g_const():
    return load_golden("constants_d128.npz")


@pytest.fixture(scope="session")
def g_polar():
    return load_golden("polar_d128.npz")


@pytest.fixture(scope="session")
def g_prod():
    return load_golden("prod_d128.npz")


@pytest.fixture(scope="session")
def g_qjl():
    return load_golden("qjl_d128.npz")


@pytest.fixture(scope="session")
def g_prim():
    return load_golden("primitives.npz")


@pytest.fixture(scope="session")
def g_outlier():
    return load_golden("outlier_d128.npz")


@pytest.fixture(scope="session")
def g_decay():
    return load_golden("temporal_decay.npz")


@pytest.fixture(scope="session")
def g_kv():
    return load_golden("kv_attention.npz")
