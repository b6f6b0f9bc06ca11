"""T = double on the GPU against the CPU oracle in double and the reference-made fp64 fixtures:
lattice structure (vertex count, keys, per-point simplex keys, barycentric weights) bit-exact,
outputs within rel-L2 1e-12 / max-abs 1e-11 (the splat sums are double reductions in varying order)."""
import numpy as np
import pytest

from conftest import GOLDEN_CASES_F64, bits, load_golden, rel_l2, sorted_rows

pytestmark = pytest.mark.gpu

REL_L2_TOL_F64 = 1e-12
MAX_ABS_TOL_F64 = 1e-11


@pytest.fixture(scope="module")
def gpu():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import gpu_helpers
    return gpu_helpers


def close64(got, want, what=""):
    got = np.asarray(got)
    assert got.dtype == np.float64, what + ": output is not double"
    assert got.shape == want.shape
    assert np.isfinite(got).all(), what + ": non-finite output"
    r = rel_l2(got, want)
    m = float(np.abs(got - want).max()) if got.size else 0.0
    assert r <= REL_L2_TOL_F64, "%s: relative L2 %.3g" % (what, r)
    assert m <= MAX_ABS_TOL_F64 * max(1.0, float(np.abs(want).max())), "%s: max abs %.3g" % (what, m)


@pytest.mark.parametrize("case", GOLDEN_CASES_F64)
def test_golden_fixture_f64(case, gpu):
    import torch
    import permutohedral_lattice_b200 as plb
    g = load_golden(case)
    inp = g["input"]
    assert inp.dtype == np.float64
    c = inp.shape[-1]
    n = int(np.prod(inp.shape[:-1]))
    if "positions" in g:
        pos = torch.from_numpy(g["positions"]).cuda()
        x = torch.from_numpy(inp.reshape(n, c)).cuda()
        out_f, ws = plb.filter_positions(x, pos, reverse=False)
        st = plb.lattice_stats(ws)
        vk, vi, pv, pw = plb.export_lattice(ws, st, 1, n, pos.shape[1], c + 1, positions=pos)
        out_r, _ = plb.filter_positions(x, pos, reverse=True)
    else:
        ref = g["reference"][None] if "reference" in g else None
        args = (bool(g["bilateral"]), float(g["theta_alpha"]), float(g["theta_beta"]),
                float(g["theta_gamma"]))
        out_f, ws, call, x, r = gpu.run_op(inp[None], ref, *args, False)
        st = plb.lattice_stats(ws)
        vk, vi, pv, pw = plb.export_lattice(ws, st, call.batch, call.n, call.pd, call.vd, reference=r,
                                            sdims=call.sdims, spatial_std=call.spatial_std,
                                            feature_std=call.feature_std, dtype=torch.float64)
        out_r = gpu.run_op(inp[None], ref, *args, True)[0]
    assert st.device_status == 0
    assert st.num_vertices == int(g["num_vertices"])
    vk_n, pv_n = vk.cpu().numpy(), pv.cpu().numpy()
    assert np.array_equal(sorted_rows(vk_n), g["keys_sorted"])
    assert np.array_equal(vk_n[pv_n[0]], g["pixel_keys"])
    assert pw.dtype == torch.float64
    assert np.array_equal(bits(pw.cpu().numpy()[0]), bits(g["pixel_weights"]))
    close64(out_f.cpu().numpy().reshape(inp.shape), g["out_forward"], case + " fwd")
    close64(out_r.cpu().numpy().reshape(inp.shape), g["out_reverse"], case + " rev")


@pytest.mark.parametrize("shape,r,c", [
    ((40, 56), 3, 21),       # CRF-like: pd 5, vd 22
    ((33, 47), 3, 3),        # RGB, ragged tiles
    ((1, 1), 3, 3),          # a single point
    ((17, 33), 1, 40),       # more channels than a warp has lanes
    ((6, 9, 7), 1, 2),       # volume, pd 4
    ((300,), 1, 1),          # 1-D signal
])
def test_op_path_f64_matches_oracle(shape, r, c, gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(64)
    ref = rng.random((2,) + shape + (r,))
    inp = rng.standard_normal((2,) + shape + (c,))
    for reverse in (False, True):
        want, items = oracle.lattice_filter(inp, ref, True, 4.0, 0.2, 1.0, reverse, structure=True,
                                            dtype=np.float64)
        out, ws, call, x, rt = gpu.run_op(inp, ref, True, 4.0, 0.2, 1.0, reverse)
        st = plb.lattice_stats(ws)
        assert st.device_status == 0
        vk, vi, pv, pw = plb.export_lattice(ws, st, call.batch, call.n, call.pd, call.vd, reference=rt,
                                            sdims=call.sdims, spatial_std=call.spatial_std,
                                            feature_std=call.feature_std)
        gpu.assert_structure_equal(vk, vi, pv, pw, items, "f64 " + str(shape))
        close64(out.cpu().numpy(), want, "f64 " + str(shape))


@pytest.mark.parametrize("shape,tg", [((30, 41), 2.5), ((12, 14, 16), 1.5)])
def test_spatial_only_f64(shape, tg, gpu, oracle):
    """bilateral=False in double: vertices located by direct indexing, as in float."""
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(5)
    inp = rng.random((2,) + shape + (3,))
    for reverse in (False, True):
        want, items = oracle.lattice_filter(inp, None, False, 1.0, 1.0, tg, reverse, structure=True,
                                            dtype=np.float64)
        out, ws, call, x, rt = gpu.run_op(inp, None, False, 1.0, 1.0, tg, reverse)
        st = plb.lattice_stats(ws)
        assert st.device_status == 0 and st.direct_index == 1
        vk, vi, pv, pw = plb.export_lattice(ws, st, call.batch, call.n, call.pd, call.vd, reference=rt,
                                            sdims=call.sdims, spatial_std=call.spatial_std,
                                            feature_std=call.feature_std, dtype=torch.float64)
        gpu.assert_structure_equal(vk, vi, pv, pw, items, "spatial f64 " + str(shape))
        close64(out.cpu().numpy(), want, "spatial f64 " + str(shape))


def test_positions_path_f64_pd16(gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(16)
    b, n, c = 2, 900, 3
    pos = rng.standard_normal((b, n, 16)) * 1.5
    inp = rng.random((b, n, c))
    x, p = torch.from_numpy(inp).cuda(), torch.from_numpy(pos).cuda()
    out, ws = plb.filter_positions(x, p)
    st = plb.lattice_stats(ws)
    vk, vi, pv, pw = plb.export_lattice(ws, st, b, n, 16, c + 1, positions=p)
    items = [oracle.filter(inp[i], pos[i], dtype=np.float64) for i in range(b)]
    gpu.assert_structure_equal(vk, vi, pv, pw, items, "f64 pd16")
    close64(out.cpu().numpy(), np.stack([o.out for o in items]), "f64 pd16")


def test_compute_positions_f64_bit_exact(gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(3)
    ref = rng.random((13 * 7 * 5, 2))
    want = oracle.compute_positions(ref, [13, 7, 5], 3.0, 0.7, dtype=np.float64)
    got = plb.compute_positions(torch.from_numpy(ref).cuda(), [13, 7, 5], 3.0, 0.7)
    assert got.dtype == torch.float64
    assert np.array_equal(bits(got.cpu().numpy()), bits(want))


def test_autograd_f64_is_the_reverse_filter(gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(8)
    ref = rng.random((1, 24, 20, 3))
    inp = rng.standard_normal((1, 24, 20, 4))
    grad = rng.standard_normal((1, 24, 20, 4))
    x = torch.from_numpy(inp).cuda().requires_grad_(True)
    r = torch.from_numpy(ref).cuda()
    out = plb.lattice_filter(x, r, True, 5.0, 0.3)
    out.backward(torch.from_numpy(grad).cuda())
    # the op's thetas are float attributes, widened to double
    want = oracle.lattice_filter(grad, ref, True, 5.0, float(np.float32(0.3)), 1.0, True, dtype=np.float64)
    assert x.grad.dtype == torch.float64
    close64(x.grad.cpu().numpy(), want, "f64 gradient")


def test_f64_refusals(gpu):
    import torch
    import permutohedral_lattice_b200 as plb
    x64 = torch.zeros((1, 8, 8, 3), dtype=torch.float64, device="cuda")
    r32 = torch.zeros((1, 8, 8, 3), dtype=torch.float32, device="cuda")
    with pytest.raises(TypeError):
        plb.lattice_filter_raw(x64, r32)                         # mixed number types
    with pytest.raises(TypeError):
        plb.lattice_filter_raw(x64, x64, mode="deterministic")   # float32 only
    with pytest.raises(TypeError):
        plb.lattice_filter(x64, x64, reuse_lattice=True)         # float32 only
    with pytest.raises(TypeError):
        plb.lattice_filter_raw(x64.half(), x64.half())
