"""Spatial-only filters (bilateral=False, src/LatticeFilterKernel.cpp:137-142): the CUDA path locates
vertices by direct indexing instead of hashing.  Same bar as every other case: vertex count, key set,
per-point simplex keys and weights bit-exact against the CPU oracle, outputs within rel-L2 1e-5 /
max-abs 1e-4; and the hashed path (developer switch) must build the identical lattice."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import gpu_helpers
    return gpu_helpers


@pytest.fixture
def hashed_path():
    """Turns direct indexing off for one test and restores the previous setting afterwards."""
    from permutohedral_lattice_b200 import capi
    was = capi.lib().pl_debug_direct_index(0)
    yield
    capi.lib().pl_debug_direct_index(was)


# (spatial shape, channels, theta_gamma, direct indexing expected).  The last three are so small or so
# sparse that the dense index (whose bounds carry a fixed margin) outgrows the table region of the
# workspace: the call then hashes, and must give the same results.
CASES = [
    ((64, 48), 4, 3.0, True),        # 2-D image, the CRF smoothness kernel
    ((33, 17), 21, 1.0, True),       # theta_gamma 1: nearly one vertex per point, wide rows
    ((40, 56), 2, 8.0, True),        # coarse lattice
    ((24, 20, 22), 2, 2.0, True),    # volume, pd 3
    ((300,), 1, 5.0, True),          # 1-D signal, pd 1
    ((1, 1), 3, 3.0, True),          # a single point
    ((9, 10, 11), 2, 2.0, False),    # tiny volume
    ((3, 4, 5, 6), 2, 1.5, False),   # four spatial dimensions, a few points each
    ((50, 70), 3, 0.37, False),      # theta_gamma below one: vertices far sparser than the index
]


@pytest.mark.parametrize("shape,c,tg,direct", CASES)
def test_spatial_only_matches_oracle(shape, c, tg, direct, gpu, oracle):
    rng = np.random.default_rng(5)
    inp = rng.standard_normal((2,) + shape + (c,)).astype(np.float32)
    for reverse in (False, True):
        want, items = oracle.lattice_filter(inp, None, False, 1.0, 1.0, tg, reverse, structure=True)
        out, ws, call, x, r = gpu.run_op(inp, None, False, 1.0, 1.0, tg, reverse)
        st, (vk, vi, pv, pw) = gpu.export_op(ws, call, r)
        assert st.direct_index == int(direct)
        gpu.assert_structure_equal(vk, vi, pv, pw, items, str(shape))
        gpu.assert_outputs_close(out.cpu().numpy(), want, str(shape))


def test_bilateral_calls_keep_the_hash_table(gpu):
    rng = np.random.default_rng(6)
    inp = rng.standard_normal((1, 20, 20, 2)).astype(np.float32)
    ref = rng.random((1, 20, 20, 3), dtype=np.float32)
    out, ws, call, x, r = gpu.run_op(inp, ref, True, 4.0, 0.25, 1.0, False)
    st, _ = gpu.export_op(ws, call, r)
    assert st.direct_index == 0


def test_hashed_and_direct_paths_build_the_same_lattice(gpu, hashed_path):
    import permutohedral_lattice_b200 as plb
    from permutohedral_lattice_b200 import capi
    from conftest import bits, sorted_rows
    rng = np.random.default_rng(7)
    inp = rng.standard_normal((3, 45, 52, 5)).astype(np.float32)
    res = {}
    for name, enable in (("hashed", 0), ("direct", 1)):
        capi.lib().pl_debug_direct_index(enable)
        out, ws, call, x, r = gpu.run_op(inp, None, False, 1.0, 1.0, 2.5, False, mode="deterministic")
        st, (vk, vi, pv, pw) = gpu.export_op(ws, call, r)
        assert st.direct_index == enable
        vk, vi, pv, pw = (t.cpu().numpy() for t in (vk, vi, pv, pw))
        res[name] = (st.num_vertices, sorted_rows(np.concatenate([vi[:, None].astype(np.int16), vk], 1)),
                     vk[pv.reshape(-1)], bits(pw), bits(out.cpu().numpy()))
    assert res["hashed"][0] == res["direct"][0]
    for a, b in zip(res["hashed"][1:], res["direct"][1:]):
        assert np.array_equal(a, b)   # deterministic mode: outputs bit for bit as well


def test_small_table_falls_back_to_hashing(gpu, oracle):
    """max_entries shrinks the workspace's table region; when the dense index no longer fits, the call
    hashes, with the same results."""
    rng = np.random.default_rng(8)
    inp = rng.standard_normal((8, 16, 16, 2)).astype(np.float32)
    want = oracle.lattice_filter(inp, None, False, 1.0, 1.0, 16.0, False)
    for max_entries, direct in ((0, 1), (200, 0)):
        out, ws, call, x, r = gpu.run_op(inp, None, False, 1.0, 1.0, 16.0, False, max_entries=max_entries)
        st, _ = gpu.export_op(ws, call, r, max_entries=max_entries)
        assert st.direct_index == direct
        gpu.assert_outputs_close(out.cpu().numpy(), want, "max_entries %d" % max_entries)


def test_spatial_only_lattice_reuse(gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(9)
    inp = rng.standard_normal((2, 30, 41, 4)).astype(np.float32)
    lat = plb.Lattice(None, spatial_shape=(2, 30, 41), bilateral=False, theta_gamma=3.0, max_channels=4)
    assert lat.stats().direct_index == 1
    for reverse in (False, True):
        want = oracle.lattice_filter(inp, None, False, 1.0, 1.0, 3.0, reverse)
        got = lat.apply(torch.from_numpy(inp).cuda(), reverse=reverse)
        gpu.assert_outputs_close(got.cpu().numpy(), want, "reuse")
