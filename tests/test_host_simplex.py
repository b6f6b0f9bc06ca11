"""The product's per-point geometry (csrc/simplex.cuh), compiled for the host, against the oracle:
per-pixel simplex keys bit-exact, barycentric weights to the last bit or one unit off it."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from conftest import GOLDEN_CASES, GOLDEN_CASES_F64, ROOT, bits, golden_positions, load_golden


@pytest.fixture(scope="module")
def shim(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("shim") / "libsimplex_host.so")
    subprocess.check_call([
        "g++", "-O2", "-std=c++17", "-ffp-contract=off", "-fPIC", "-shared", "-o", out,
        "-I", os.path.join(ROOT, "permutohedral_lattice_b200", "csrc"),
        os.path.join(ROOT, "tests", "helpers", "simplex_host_shim.cpp")])
    return ctypes.CDLL(out)


def assert_weights_close(got, want):
    """Bit-exact up to the reference's double rounding: at most one unit in the last place of a weight
    near 1, and rare."""
    diff = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert diff.max() <= 2.0 ** -23
    assert (diff > 0).mean() <= 1e-4


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
    assert_weights_close(w, g["pixel_weights"])


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
    assert_weights_close(w, res.pix_weight)


def run_shim_f64(shim, pos, scale):
    n, pd = pos.shape
    keys = np.zeros((n, pd + 1, pd), np.int16)
    w = np.zeros((n, pd + 1), np.float64)
    dp = ctypes.POINTER(ctypes.c_double)
    rc = shim.simplex_host_f64(pos.ctypes.data_as(dp), scale.ctypes.data_as(dp), n, pd,
                               keys.ctypes.data_as(ctypes.POINTER(ctypes.c_short)), w.ctypes.data_as(dp))
    assert rc == 0
    return keys, w


@pytest.mark.parametrize("case", GOLDEN_CASES_F64)
def test_double_keys_and_weights_match_golden_bit_for_bit(case, shim, oracle):
    g = load_golden(case)
    pos = np.ascontiguousarray(golden_positions(g, oracle), np.float64)
    keys, w = run_shim_f64(shim, pos, oracle.scale_factors(pos.shape[1], np.float64))
    assert np.array_equal(keys, g["pixel_keys"])
    assert np.array_equal(bits(w), bits(g["pixel_weights"]))


@pytest.mark.parametrize("pd", [2, 3, 4, 5, 16])
def test_double_keys_and_weights_match_oracle_random(pd, shim, oracle):
    rng = np.random.default_rng(100 + pd)
    pos = rng.standard_normal((20000, pd)) * rng.choice([0.1, 1.0, 10.0, 50.0], (20000, 1))
    pos[:100] = np.round(pos[:100])
    pos[100:200] = 0.0
    keys, w = run_shim_f64(shim, pos, oracle.scale_factors(pd, np.float64))
    res = oracle.filter(np.ones((len(pos), 1)), pos, dtype=np.float64)
    assert np.array_equal(keys, res.pixel_keys())
    assert np.array_equal(bits(w), bits(res.pix_weight))


def test_reciprocal_division_is_the_ieee_quotient(shim):
    rng = np.random.default_rng(1)
    fp = ctypes.POINTER(ctypes.c_float)
    shim.small_int_to_float_host.restype = ctypes.c_float
    for c in (0, 1, 2, 511, 1023, 65535, 8388607):
        assert shim.small_int_to_float_host(c) == float(c)
    for b in (80.0, 0.0625, 8.0, 0.125, 16.0, 0.1, 5.0, 3.0, 0.2, 0.7, 1e-3, 123.456, 2.0 ** -20, 3e6):
        a = np.concatenate([np.arange(0, 4096, dtype=np.float32), rng.random(200000, dtype=np.float32),
                            (rng.standard_normal(200000) * 1000).astype(np.float32)])
        out = np.empty_like(a)
        shim.div_by_rcp_host(a.ctypes.data_as(fp), ctypes.c_float(b), len(a), out.ctypes.data_as(fp))
        assert np.array_equal(bits(out), bits(a / np.float32(b))), b
