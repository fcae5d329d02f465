import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name))
    meta = json.loads(bytes(z["meta"]).decode())
    return meta, z


@pytest.fixture(scope="session")
def golden_recorded():
    return load_golden("recorded_calls.npz")


@pytest.fixture(scope="session")
def golden_sweep():
    return load_golden("sweep.npz")


@pytest.fixture(scope="session")
def golden_layers():
    return load_golden("layers.npz")


@pytest.fixture(scope="session")
def golden_layers2():
    return load_golden("layers2.npz")
