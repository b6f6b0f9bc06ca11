import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")
_ALL_CASES = sorted(f[:-4] for f in os.listdir(GOLDEN_DIR) if f.endswith(".npz"))
GOLDEN_CASES = [c for c in _ALL_CASES if not c.endswith("_f64")]       # T = float
GOLDEN_CASES_F64 = [c for c in _ALL_CASES if c.endswith("_f64")]       # T = double


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN_DIR, name + ".npz")))


def golden_positions(g, oracle):
    """Feature vectors of a golden case, rebuilt the way the op builds them."""
    inp = g["input"]
    sdims = list(inp.shape[:-1])
    if "positions" in g:
        return g["positions"]
    if bool(g["bilateral"]):
        ref = g["reference"]
        return oracle.compute_positions(ref.reshape(-1, ref.shape[-1]), sdims,
                                        float(g["theta_alpha"]), float(g["theta_beta"]),
                                        dtype=inp.dtype)
    return oracle.compute_positions(None, sdims, float(g["theta_gamma"]), -1.0, dtype=inp.dtype)


def sorted_rows(keys):
    order = np.lexsort(keys.T[::-1])
    return keys[order]


def bits(a):
    a = np.asarray(a)
    if a.dtype == np.float64:
        return np.ascontiguousarray(a).view(np.uint64)
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.fixture(scope="session")
def oracle():
    from oracle import cpu_oracle
    return cpu_oracle
