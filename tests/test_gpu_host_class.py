"""The C++ host layer (include/LatticeFilterKernel.hpp: ComputeKernel / LatticeFilter functors and the
op class with the reference's parameter lists) on a GPU, checked against the CPU oracle."""
import os
import struct
import subprocess

import numpy as np
import pytest

from conftest import ROOT, rel_l2

pytestmark = pytest.mark.gpu

BIN = os.path.join(ROOT, "tests", "helpers", "host_class_test.bin")


@pytest.mark.parametrize("shape,c,r,bilateral,reverse", [
    ((2, 33, 47), 3, 3, True, False),
    ((1, 9, 10, 11), 2, 1, True, True),
    ((2, 25, 30), 21, 3, True, False),
    ((1, 40, 28), 4, 3, False, False),
])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_cpp_op_class_matches_oracle(shape, c, r, bilateral, reverse, dtype, tmp_path, oracle):
    if not os.path.exists(BIN):
        pytest.fail("tests/helpers/host_class_test.bin is not built (python -m permutohedral_lattice_b200.build)")
    rng = np.random.default_rng(17)
    inp = rng.random(shape + (c,)).astype(dtype)
    ref = rng.random(shape + (r,)).astype(dtype)
    ta, tb, tg = 5.0, float(np.float32(0.2)), 3.0   # float attributes of the op class
    sd = list(shape[1:]) + [0] * (3 - len(shape[1:]))
    src, dst = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(src, "wb") as f:
        f.write(struct.pack("<9i", shape[0], len(shape) - 1, sd[0], sd[1], sd[2], c, r, int(bilateral), int(reverse)))
        f.write(struct.pack("<3f", ta, tb, tg))
        f.write(inp.tobytes())
        f.write(ref.tobytes())
    f64 = dtype == np.float64
    res = subprocess.run([BIN, str(src), str(dst)] + (["f64"] if f64 else []), capture_output=True, text=True,
                         timeout=300)
    assert res.returncode == 0, res.stderr
    assert res.stdout.startswith("ok")
    # ComputeSized started from a bound of 64 entries and grew it until the lattice fitted
    fields = dict(kv.split("=") for kv in res.stdout.split()[1:])
    assert 64 < int(fields["sized_entries"]) <= int(fields["sized_bound"])
    got = np.fromfile(dst, dtype).reshape((2,) + inp.shape)
    want = oracle.lattice_filter(inp, ref, bilateral, ta, tb, tg, reverse, dtype=dtype)
    for which, name in ((0, "whole batch"), (1, "per item")):
        assert rel_l2(got[which], want) <= (1e-12 if f64 else 1e-5), name
        assert np.abs(got[which] - want).max() <= (1e-11 if f64 else 1e-4), name
