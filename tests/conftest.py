import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "pytorch-window-matmul_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    data = np.load(os.path.join(ROOT, "tests", "golden", "reference_cpu.npz"))
    cases = {}
    for name in data["names"]:
        name = str(name)
        cases[name] = {k.split("/", 1)[1]: data[k] for k in data.files if k.startswith(name + "/")}
    return cases
