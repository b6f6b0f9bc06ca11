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
def test_cpp_op_class_matches_oracle(shape, c, r, bilateral, reverse, tmp_path, oracle):
    if not os.path.exists(BIN):
        pytest.fail("tests/helpers/host_class_test.bin is not built (python -m permutohedral_lattice_b200.build)")
    rng = np.random.default_rng(17)
    inp = rng.random(shape + (c,), dtype=np.float32)
    ref = rng.random(shape + (r,), dtype=np.float32)
    ta, tb, tg = 5.0, 0.2, 3.0
    sd = list(shape[1:]) + [0] * (3 - len(shape[1:]))
    src, dst = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(src, "wb") as f:
        f.write(struct.pack("<9i", shape[0], len(shape) - 1, sd[0], sd[1], sd[2], c, r, int(bilateral), int(reverse)))
        f.write(struct.pack("<3f", ta, tb, tg))
        f.write(inp.tobytes())
        f.write(ref.tobytes())
    res = subprocess.run([BIN, str(src), str(dst)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    assert res.stdout.startswith("ok")
    got = np.fromfile(dst, np.float32).reshape((2,) + inp.shape)
    want = oracle.lattice_filter(inp, ref, bilateral, ta, tb, tg, reverse)
    for which, name in ((0, "whole batch"), (1, "per item")):
        assert rel_l2(got[which], want) <= 1e-5, name
        assert np.abs(got[which] - want).max() <= 1e-4, name
