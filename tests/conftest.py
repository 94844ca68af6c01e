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


def golden_cases(prefix):
    """Names of the golden cases whose reference-Python file exists, e.g. prefix 'b_' or 'd_'."""
    names = sorted(f[len("pyref_"):-4] for f in os.listdir(GOLDEN) if f.startswith("pyref_" + prefix) and f.endswith(".npz"))
    return names


class Golden:
    """One golden case: inputs (float32), metadata and the expected float64 outputs of the reference."""

    def __init__(self, name, source="pyref"):
        f = np.load(os.path.join(GOLDEN, f"pyref_{name}.npz"))
        self.name = name
        self.inputs = {k[3:]: f[k] for k in f.files if k.startswith("in_")}
        self.meta = {k[5:]: f[k].item() for k in f.files if k.startswith("meta_")}
        self.expected = {k[4:]: f[k] for k in f.files if k.startswith("out_")}
        self.cuda = None
        path = os.path.join(GOLDEN, f"cudaref_{name}.npz")
        if os.path.exists(path):
            c = np.load(path)
            self.cuda = {k: c[k] for k in c.files}


def rel_err(got, want):
    """max|got - want| / max|want| (norm-relative error used throughout the parity tests)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


@pytest.fixture(scope="session")
def oracle():
    from oracle import c_oracle
    c_oracle.build()
    return c_oracle
