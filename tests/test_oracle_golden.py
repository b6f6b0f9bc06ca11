"""The C restatement (oracle/pl_oracle.c) against fixtures produced by the unmodified reference
CPU implementation (tests/golden/make_golden.py): everything bit-exact."""
import numpy as np
import pytest

from conftest import (GOLDEN_CASES, GOLDEN_CASES_F64, bits, golden_positions, load_golden,
                      sorted_rows)


@pytest.mark.parametrize("case", GOLDEN_CASES + GOLDEN_CASES_F64)
def test_port_reproduces_reference_fixture(case, oracle):
    g = load_golden(case)
    inp = g["input"]
    assert inp.dtype == (np.float64 if case.endswith("_f64") else np.float32)
    c = inp.shape[-1]
    pos = golden_positions(g, oracle)
    fwd = oracle.filter(inp.reshape(-1, c), pos, reverse=False, dtype=inp.dtype)
    rev = oracle.filter(inp.reshape(-1, c), pos, reverse=True, structure=False, dtype=inp.dtype)
    assert fwd.out.dtype == inp.dtype and fwd.pix_weight.dtype == inp.dtype
    assert fwd.num_vertices == int(g["num_vertices"])
    assert np.array_equal(sorted_rows(fwd.keys), g["keys_sorted"])
    assert np.array_equal(fwd.pixel_keys(), g["pixel_keys"])
    assert np.array_equal(bits(fwd.pix_weight), bits(g["pixel_weights"]))
    assert np.array_equal(bits(fwd.out), bits(g["out_forward"].reshape(-1, c)))
    assert np.array_equal(bits(rev.out), bits(g["out_reverse"].reshape(-1, c)))


def test_scale_factors_formula(oracle):
    # (pd+1) sqrt(2/3) / sqrt((i+1)(i+2)), double arithmetic rounded to float
    # (src/PermutohedralLatticeCPU.h:209-214)
    for pd in (2, 3, 4, 5, 16):
        inv = np.float32((pd + 1) * np.sqrt(2.0 / 3))
        want = [np.float32(1.0 / np.sqrt(float((i + 1) * (i + 2))) * float(inv)) for i in range(pd)]
        assert np.array_equal(bits(oracle.scale_factors(pd)), bits(np.array(want, np.float32)))


def test_weights_sum_to_one_and_keys_sum_rule(oracle):
    g = load_golden("rgb_pd5_vd4")
    w = g["pixel_weights"].astype(np.float64)
    assert np.allclose(w.sum(1), 1.0, atol=1e-5)
    keys = g["pixel_keys"].astype(np.int64)           # [n, pd+1, pd]
    pd = keys.shape[-1]
    # remainder-r vertex: every stored coordinate is congruent to r modulo pd+1
    for r in range(pd + 1):
        assert np.all((keys[:, r, :] - r) % (pd + 1) == 0)


def test_empty_and_single_pixel(oracle):
    out = oracle.filter(np.zeros((0, 3), np.float32), np.zeros((0, 5), np.float32))
    assert out.out.shape == (0, 3) and out.num_vertices == 0
    one = oracle.filter(np.array([[0.25, 0.5, 0.75]], np.float32),
                        np.array([[1.5, -2.0, 0.3, 0.1, 7.0]], np.float32))
    # a lone pixel gets its own value back (weights normalise out)
    assert np.allclose(one.out, [[0.25, 0.5, 0.75]], atol=1e-6)
    assert one.num_vertices == 6
