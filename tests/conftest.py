import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def port():
    from oracle.binding import Port
    return Port()


@pytest.fixture(scope="session")
def ref():
    from oracle.binding import Ref
    if not Ref.available():
        pytest.skip("oracle/_ref/liboracle_ref.so not built (needs the reference tree: make -C oracle ref)")
    r = Ref()
    r.set_gpu_index(-1)
    return r


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "xnor_ref_golden.npz")
    data = np.load(path)
    cases = json.loads(bytes(data["cases"]).decode())
    return cases, data
