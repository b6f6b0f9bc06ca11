"""The product's per-point geometry (csrc/simplex.cuh), compiled for the host, against the oracle:
per-pixel simplex keys and barycentric weights bit-exact."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from conftest import GOLDEN_CASES, ROOT, bits, golden_positions, load_golden


@pytest.fixture(scope="module")
def shim(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("shim") / "libsimplex_host.so")
    subprocess.check_call([
        "g++", "-O2", "-std=c++17", "-ffp-contract=off", "-fPIC", "-shared", "-o", out,
        "-I", os.path.join(ROOT, "permutohedral_lattice_b200", "csrc"),
        os.path.join(ROOT, "tests", "helpers", "simplex_host_shim.cpp")])
    return ctypes.CDLL(out)


def run_shim(shim, pos, scale):
    n, pd = pos.shape
    keys = np.zeros((n, pd + 1, pd), np.int16)
    w = np.zeros((n, pd + 1), np.float32)
    fp = ctypes.POINTER(ctypes.c_float)
    rc = shim.simplex_host(pos.ctypes.data_as(fp), scale.ctypes.data_as(fp), n, pd,
                           keys.ctypes.data_as(ctypes.POINTER(ctypes.c_short)), w.ctypes.data_as(fp))
    assert rc == 0
    return keys, w


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_keys_and_weights_match_golden(case, shim, oracle):
    g = load_golden(case)
    pos = np.ascontiguousarray(golden_positions(g, oracle), np.float32)
    keys, w = run_shim(shim, pos, oracle.scale_factors(pos.shape[1]))
    assert np.array_equal(keys, g["pixel_keys"])
    assert np.array_equal(bits(w), bits(g["pixel_weights"]))


@pytest.mark.parametrize("pd", [2, 3, 4, 5, 16])
def test_keys_and_weights_match_oracle_random(pd, shim, oracle):
    rng = np.random.default_rng(pd)
    pos = (rng.standard_normal((20000, pd)) * rng.choice([0.1, 1.0, 10.0, 50.0], (20000, 1))
           ).astype(np.float32)
    pos[:100] = np.round(pos[:100])          # exact ties on lattice hyperplanes
    pos[100:200] = 0.0
    keys, w = run_shim(shim, pos, oracle.scale_factors(pd))
    res = oracle.filter(np.ones((len(pos), 1), np.float32), pos)
    assert np.array_equal(keys, res.pixel_keys())
    assert np.array_equal(bits(w), bits(res.pix_weight))
