import glob
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_golden(name):
    """(source, function, kwargs, expected outputs) of one committed reference fixture."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"), allow_pickle=False)
    kwargs, expected = {}, {}
    for k in z.files:
        if k.startswith("in__"):
            v = z[k]
            kwargs[k[4:]] = v if v.ndim else v.item()
        elif k.startswith("out__"):
            expected[k[5:]] = z[k]
    return str(z["__source__"]), str(z["__function__"]), kwargs, expected


def golden_names():
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, "*.npz")))


@pytest.fixture(scope="session")
def build_lib():
    from ktir_cpu_b200.build import build
    return build()
