"""pl_lattice_filter_f32_noalloc: the op for callers that may not allocate device memory (a plugin
inside an application whose pool already owns the GPU, a service that forbids allocation once it
runs).  Its scratch is an array inside the library, so the test drives it through the C ABI with
nothing but input and output pointers and checks it against the ordinary entry point, twice in a
row because the second call starts from the scratch the first one left behind.

Collected last on purpose: a failure here must not hide the other GPU tests."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-5
MAX_ABS_TOL = 1e-4


def _call_noalloc(x, ref, sdims, bilateral, ta, tb, tg, reverse, max_entries=0):
    import torch
    from permutohedral_lattice_b200 import capi
    out = torch.empty_like(x)
    rc = capi.lib().pl_lattice_filter_f32_noalloc(
        out.data_ptr(), x.data_ptr(), 0 if ref is None else ref.data_ptr(), x.shape[0], len(sdims),
        capi.int_array(sdims), x.shape[-1], 0 if ref is None else ref.shape[-1], int(bilateral), ta, tb, tg,
        int(reverse), max_entries, torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_noalloc_matches_workspace_entry_point_twice():
    import torch
    import permutohedral_lattice_b200 as plb
    from permutohedral_lattice_b200 import capi
    rng = np.random.default_rng(21)
    cases = [((2, 48, 40), 3, 21, 6.0, 0.125), ((1, 30, 50), 3, 3, 4.0, 0.2)]
    for round_ in range(2):           # two calls in a row per case, on the scratch the last call left
        for shape, r, c, ta, tb in cases:
            ref = torch.from_numpy(rng.random(shape + (r,), dtype=np.float32)).cuda()
            x = torch.from_numpy(rng.standard_normal(shape + (c,)).astype(np.float32)).cuda()
            for reverse in (False, True):
                want = plb.lattice_filter(x, ref, True, ta, tb, 1.0, reverse)
                rc, got = _call_noalloc(x, ref, list(shape[1:]), True, ta, tb, 1.0, reverse)
                assert rc == capi.PL_OK, capi.lib().pl_strerror(rc)
                torch.cuda.synchronize()
                w, g = want.cpu().numpy().astype(np.float64), got.cpu().numpy().astype(np.float64)
                assert np.isfinite(g).all()
                assert np.linalg.norm(g - w) / np.linalg.norm(w) <= REL_L2_TOL
                assert np.abs(g - w).max() <= MAX_ABS_TOL


def test_noalloc_refuses_sizes_beyond_its_scratch():
    import torch
    from permutohedral_lattice_b200 import capi
    x = torch.zeros((1, 1024, 1024, 3), device="cuda")
    rc, _ = _call_noalloc(x, x, [1024, 1024], True, 8.0, 0.125, 1.0, False)
    assert rc == capi.PL_WORKSPACE_TOO_SMALL
    assert b"built-in scratch" in capi.lib().pl_last_cuda_error()
    # the same image fits once the caller bounds the number of lattice entries
    rng = np.random.default_rng(3)
    blocks = np.repeat(np.repeat(rng.random((1, 16, 16, 3), dtype=np.float32), 16, 1), 16, 2)
    img = torch.from_numpy(np.ascontiguousarray(blocks)).cuda()
    import permutohedral_lattice_b200 as plb
    rc, out = _call_noalloc(img, img, [256, 256], True, 8.0, 0.125, 1.0, False, max_entries=200000)
    assert rc == capi.PL_OK
    # whether the lattice stayed within max_entries is known on the device only: the caller has no
    # workspace pointer, so the counters of the built-in scratch are read with a null workspace
    st = plb.lattice_stats(None)
    assert st.device_status == capi.PL_OK and 0 < st.num_vertices <= st.num_entries <= 200000
    want, ws, _ = plb.lattice_filter_raw(img, img, True, 8.0, 0.125, 1.0, False, max_entries=200000)
    assert plb.lattice_stats(ws).num_vertices == st.num_vertices
    w, g = want.cpu().numpy().astype(np.float64), out.cpu().numpy().astype(np.float64)
    assert np.isfinite(g).all()
    assert np.linalg.norm(g - w) / np.linalg.norm(w) <= REL_L2_TOL
    assert np.abs(g - w).max() <= MAX_ABS_TOL


def test_noalloc_reports_a_max_entries_that_was_too_small():
    """The call itself returns PL_OK (nothing is known on the host); the device sets a status bit, every
    later kernel of the call stands down, and the output is filled with NaN.  Nothing faults."""
    import torch
    import permutohedral_lattice_b200 as plb
    from permutohedral_lattice_b200 import capi
    rng = np.random.default_rng(5)
    img = torch.from_numpy(rng.random((1, 64, 64, 3), dtype=np.float32)).cuda()
    rc, out = _call_noalloc(img, img, [64, 64], True, 8.0, 0.125, 1.0, False, max_entries=100)
    assert rc == capi.PL_OK
    st = plb.lattice_stats(None)
    assert st.device_status == capi.PL_CAPACITY_EXCEEDED
    assert torch.isnan(out).all()
    # the scratch is usable again by the next call
    rc, out = _call_noalloc(img, img, [64, 64], True, 8.0, 0.125, 1.0, False)
    assert rc == capi.PL_OK
    assert plb.lattice_stats(None).device_status == capi.PL_OK
    assert torch.isfinite(out).all()
