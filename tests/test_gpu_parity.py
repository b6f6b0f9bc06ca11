"""Parity of the CUDA path (through the C ABI) with the CPU oracle and the reference-made golden
fixtures: lattice structure bit-exact, fp32 outputs within rel-L2 1e-5 / max-abs 1e-4."""
import numpy as np
import pytest

from conftest import GOLDEN_CASES, load_golden

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import gpu_helpers
    return gpu_helpers


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_golden_fixture(case, gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    g = load_golden(case)
    inp = g["input"]
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
        st, (vk, vi, pv, pw) = gpu.export_op(ws, call, r)
        out_r = gpu.run_op(inp[None], ref, *args, True)[0]
    assert st.device_status == 0
    assert st.num_vertices == int(g["num_vertices"])
    vk_n, pv_n = vk.cpu().numpy(), pv.cpu().numpy()
    from conftest import bits, sorted_rows
    assert np.array_equal(sorted_rows(vk_n), g["keys_sorted"])
    assert np.array_equal(vk_n[pv_n[0]], g["pixel_keys"])
    assert np.array_equal(bits(pw.cpu().numpy()[0]), bits(g["pixel_weights"]))
    gpu.assert_outputs_close(out_f.cpu().numpy().reshape(inp.shape), g["out_forward"], case + " fwd")
    gpu.assert_outputs_close(out_r.cpu().numpy().reshape(inp.shape), g["out_reverse"], case + " rev")


@pytest.mark.parametrize("config", [0, 1, 2, 3])
def test_small_workload_op_path(config, gpu, oracle):
    from permutohedral_lattice_b200 import workloads
    w = workloads.small(config)
    want, items = oracle.lattice_filter(w.input, w.reference, True, w.theta_alpha, w.theta_beta,
                                        1.0, False, structure=True)
    out, ws, call, x, r = gpu.run_op(w.input, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, False)
    st, (vk, vi, pv, pw) = gpu.export_op(ws, call, r)
    gpu.assert_structure_equal(vk, vi, pv, pw, items, w.name)
    gpu.assert_outputs_close(out.cpu().numpy(), want, w.name + " fwd")
    if w.backward:
        want_b = oracle.lattice_filter(w.grad, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, True)
        got_b = gpu.run_op(w.grad, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, True)[0]
        gpu.assert_outputs_close(got_b.cpu().numpy(), want_b, w.name + " bwd")


def test_small_workload_positions_pd16(gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    from permutohedral_lattice_b200 import workloads
    w = workloads.small(4)
    b, n, c = w.batch, w.pixels_per_item, w.input.shape[-1]
    x = torch.from_numpy(w.input.reshape(b, n, c)).cuda()
    p = torch.from_numpy(w.positions).cuda()
    out, ws = plb.filter_positions(x, p)
    st = plb.lattice_stats(ws)
    vk, vi, pv, pw = plb.export_lattice(ws, st, b, n, 16, c + 1, positions=p)
    items = [oracle.filter(w.input[i].reshape(n, c), w.positions[i]) for i in range(b)]
    gpu.assert_structure_equal(vk, vi, pv, pw, items, w.name)
    want = np.stack([o.out for o in items])
    gpu.assert_outputs_close(out.cpu().numpy(), want, w.name)


@pytest.mark.parametrize("shape,r,c", [
    ((1, 1), 3, 3),          # a single point
    ((1, 37), 3, 2),         # one row
    ((53, 1), 3, 2),         # one column (narrow tiles)
    ((17, 33), 1, 1),        # one past the tile edge in both directions
    ((3, 5, 7), 2, 4),       # tiny volume, pd 5
    ((300,), 1, 1),          # 1-D signal
])
def test_ragged_shapes(shape, r, c, gpu, oracle):
    rng = np.random.default_rng(11)
    ref = rng.random((2,) + shape + (r,), dtype=np.float32)
    inp = rng.standard_normal((2,) + shape + (c,)).astype(np.float32)
    for reverse in (False, True):
        want, items = oracle.lattice_filter(inp, ref, True, 3.0, 0.25, 1.0, reverse, structure=True)
        out, ws, call, x, rt = gpu.run_op(inp, ref, True, 3.0, 0.25, 1.0, reverse)
        st, (vk, vi, pv, pw) = gpu.export_op(ws, call, rt)
        gpu.assert_structure_equal(vk, vi, pv, pw, items, str(shape))
        gpu.assert_outputs_close(out.cpu().numpy(), want, str(shape))


@pytest.mark.parametrize("shape,r,c,why", [
    ((40, 48), 3, 21, "wide rows, tile rows arrive by bulk copies and are spread out in place"),
    ((25, 30), 3, 21, "wide rows, row bytes x width not a multiple of 16: 4-byte copies to the padded rows"),
    ((37, 20), 3, 21, "wide rows, ragged last tile column (4 points) on the bulk path"),
    ((6, 9, 7), 1, 21, "wide rows in a volume (pd 4)"),
    ((33, 18), 3, 8, "vd 9: no compiled instantiation, generic lane-group kernels"),
    ((20, 24), 3, 31, "vd 32: generic kernels, eight float4 per row"),
    ((18, 22), 3, 40, "vd 41: generic kernels, eleven float4 per row"),
])
def test_value_widths_and_staging_paths(shape, r, c, why, gpu, oracle):
    rng = np.random.default_rng(23)
    ref = rng.random((2,) + shape + (r,), dtype=np.float32)
    inp = rng.standard_normal((2,) + shape + (c,)).astype(np.float32)
    for reverse in (False, True):
        want, items = oracle.lattice_filter(inp, ref, True, 4.0, 0.2, 1.0, reverse, structure=True)
        out, ws, call, x, rt = gpu.run_op(inp, ref, True, 4.0, 0.2, 1.0, reverse)
        st, (vk, vi, pv, pw) = gpu.export_op(ws, call, rt)
        gpu.assert_structure_equal(vk, vi, pv, pw, items, why)
        gpu.assert_outputs_close(out.cpu().numpy(), want, why)


def test_wide_rows_on_the_positions_path(gpu, oracle):
    """vd 22 with features given as positions (pd 16 and pd 5): tiles are runs of points, the input block
    goes to the padded rows by 4-byte copies."""
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(29)
    for pd, n in ((16, 700), (5, 1000)):
        pos = (rng.standard_normal((2, n, pd)) * 1.2).astype(np.float32)
        inp = rng.random((2, n, 21), dtype=np.float32)
        out, ws = plb.filter_positions(torch.from_numpy(inp).cuda(), torch.from_numpy(pos).cuda())
        want = np.stack([oracle.filter(inp[i], pos[i], structure=False).out for i in range(2)])
        gpu.assert_outputs_close(out.cpu().numpy(), want, "positions pd %d vd 22" % pd)


def test_empty_inputs(gpu):
    import torch
    import permutohedral_lattice_b200 as plb
    out = plb.lattice_filter(torch.zeros((0, 8, 8, 3), device="cuda"), torch.zeros((0, 8, 8, 3), device="cuda"))
    assert out.shape == (0, 8, 8, 3)
    out = plb.lattice_filter(torch.zeros((2, 0, 8, 3), device="cuda"), torch.zeros((2, 0, 8, 3), device="cuda"))
    assert out.shape == (2, 0, 8, 3)


def test_identical_points_collide_into_one_simplex(gpu, oracle):
    # every point has the same features: pd+1 vertices in total, output = mean of the inputs
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(2)
    x = rng.random((1, 1000, 3), dtype=np.float32)
    p = np.tile(np.array([[0.3, -1.2, 4.0, 0.01, 2.5]], np.float32), (1, 1000, 1))
    out, ws = plb.filter_positions(torch.from_numpy(x).cuda(), torch.from_numpy(p).cuda())
    st = plb.lattice_stats(ws)
    assert st.num_vertices == 6
    want = oracle.filter(x[0], p[0]).out
    gpu.assert_outputs_close(out.cpu().numpy()[0], want, "collide")
    assert np.allclose(out.cpu().numpy()[0], x[0].mean(0, keepdims=True), atol=1e-5)


def test_batch_items_are_independent(gpu):
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(4)
    ref = torch.from_numpy(rng.random((3, 20, 24, 3), dtype=np.float32)).cuda()
    inp = torch.from_numpy(rng.random((3, 20, 24, 5), dtype=np.float32)).cuda()
    whole = plb.lattice_filter(inp, ref, True, 4.0, 0.2)
    for b in range(3):
        one = plb.lattice_filter(inp[b:b + 1], ref[b:b + 1], True, 4.0, 0.2)
        gpu.assert_outputs_close(one.cpu().numpy(), whole[b:b + 1].cpu().numpy(), "item %d" % b)


def test_capacity_exceeded_is_reported_not_fatal(gpu):
    import torch
    import permutohedral_lattice_b200 as plb
    from permutohedral_lattice_b200 import capi
    rng = np.random.default_rng(5)
    ref = torch.from_numpy(rng.random((1, 64, 64, 3), dtype=np.float32)).cuda()
    inp = torch.from_numpy(rng.random((1, 64, 64, 3), dtype=np.float32)).cuda()
    with pytest.raises(capi.PlError) as e:
        plb.lattice_filter_raw(inp, ref, True, 1.0, 0.01, max_entries=100)
    assert e.value.status == capi.PL_CAPACITY_EXCEEDED
    # the context is still usable and a properly sized call succeeds
    out = plb.lattice_filter(inp, ref, True, 1.0, 0.01)
    assert torch.isfinite(out).all()


def test_unsupported_dims_and_bad_arguments(gpu):
    import torch
    import permutohedral_lattice_b200 as plb
    from permutohedral_lattice_b200 import capi
    with pytest.raises(capi.PlError) as e:   # pd = 2 + 9 = 11 has no instantiation
        plb.lattice_filter(torch.zeros((1, 4, 4, 2), device="cuda"), torch.zeros((1, 4, 4, 9), device="cuda"))
    assert e.value.status == capi.PL_UNSUPPORTED_DIMS
    with pytest.raises(ValueError):
        plb.lattice_filter(torch.zeros((1, 4, 4, 2), device="cuda"), torch.zeros((1, 4, 5, 3), device="cuda"))
    with pytest.raises(ValueError):
        plb.lattice_filter(torch.zeros((1, 4, 4, 2)), torch.zeros((1, 4, 4, 3)))
    ws = torch.empty(1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(capi.PlError) as e:
        plb.lattice_filter_raw(torch.zeros((1, 8, 8, 2), device="cuda"), torch.zeros((1, 8, 8, 3), device="cuda"),
                               workspace=ws)
    assert e.value.status == capi.PL_WORKSPACE_TOO_SMALL


def test_autograd_matches_reverse_filter(gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(6)
    ref_n = rng.random((1, 24, 20, 3), dtype=np.float32)
    inp_n = rng.random((1, 24, 20, 4), dtype=np.float32)
    grad_n = rng.standard_normal((1, 24, 20, 4)).astype(np.float32)
    ref = torch.from_numpy(ref_n).cuda().requires_grad_(True)
    inp = torch.from_numpy(inp_n).cuda().requires_grad_(True)
    out = plb.lattice_filter(inp, ref, True, 5.0, 0.2)
    out.backward(torch.from_numpy(grad_n).cuda())
    want = oracle.lattice_filter(grad_n, ref_n, True, 5.0, 0.2, 1.0, True)
    gpu.assert_outputs_close(inp.grad.cpu().numpy(), want, "autograd")
    assert torch.count_nonzero(ref.grad) == 0


def test_compute_positions_matches_oracle(gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    from conftest import bits
    rng = np.random.default_rng(8)
    ref = rng.random((6 * 7 * 5, 2), dtype=np.float32)
    got = plb.compute_positions(torch.from_numpy(ref).cuda(), [6, 7, 5], 80.0, 0.0625).cpu().numpy()
    want = oracle.compute_positions(ref, [6, 7, 5], 80.0, 0.0625)
    assert np.array_equal(bits(got), bits(want))
    got = plb.compute_positions(None, [9, 4], 3.0, 1.0).cpu().numpy()
    want = oracle.compute_positions(None, [9, 4], 3.0, -1.0)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("config", [0, 2, 3])
def test_deterministic_mode_is_bitwise_reproducible(config, gpu, oracle):
    from permutohedral_lattice_b200 import workloads
    from conftest import bits
    w = workloads.small(config)
    want = oracle.lattice_filter(w.input, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, False)
    runs = []
    for _ in range(3):
        out = gpu.run_op(w.input, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, False,
                         mode="deterministic")[0]
        runs.append(out.cpu().numpy())
    gpu.assert_outputs_close(runs[0], want, w.name + " deterministic")
    assert np.array_equal(bits(runs[0]), bits(runs[1]))
    assert np.array_equal(bits(runs[0]), bits(runs[2]))


def test_deterministic_mode_positions_path_and_large_values(gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    from conftest import bits
    rng = np.random.default_rng(12)
    x = (rng.standard_normal((2, 3000, 5)) * 1e4).astype(np.float32)       # values far from 1
    p = (rng.standard_normal((2, 3000, 4)) * 2).astype(np.float32)
    xt, pt = torch.from_numpy(x).cuda(), torch.from_numpy(p).cuda()
    a = plb.filter_positions(xt, pt, mode="deterministic")[0].cpu().numpy()
    b = plb.filter_positions(xt, pt, mode="deterministic")[0].cpu().numpy()
    assert np.array_equal(bits(a), bits(b))
    want = np.stack([oracle.filter(x[i], p[i], structure=False).out for i in range(2)])
    from conftest import rel_l2
    assert rel_l2(a, want) <= 1e-5


def test_host_pipeline_matches_device_call(gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(31)
    ref = torch.from_numpy(rng.random((5, 24, 40, 3), dtype=np.float32)).pin_memory()
    inp = torch.from_numpy(rng.random((5, 24, 40, 6), dtype=np.float32)).pin_memory()
    pipe = plb.HostPipeline(n_streams=3, chunk_items=2)
    for reverse in (False, True):
        got = pipe.filter(inp, ref, True, 5.0, 0.2, reverse=reverse).numpy()
        want = oracle.lattice_filter(inp.numpy(), ref.numpy(), True, 5.0, 0.2, 1.0, reverse)
        gpu.assert_outputs_close(got, want, "host pipeline")


def test_lattice_built_once_applied_many_times(gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    from conftest import bits
    rng = np.random.default_rng(41)
    ref_n = rng.random((2, 30, 26, 3), dtype=np.float32)
    ref = torch.from_numpy(ref_n).cuda()
    lat = plb.Lattice(ref, bilateral=True, theta_alpha=5.0, theta_beta=0.2, max_channels=6, mode="deterministic")
    for c, reverse in ((6, False), (2, True), (6, True), (1, False)):
        x_n = rng.standard_normal((2, 30, 26, c)).astype(np.float32)
        got = lat.apply(torch.from_numpy(x_n).cuda(), reverse=reverse).cpu().numpy()
        want = oracle.lattice_filter(x_n, ref_n, True, 5.0, 0.2, 1.0, reverse)
        gpu.assert_outputs_close(got, want, "apply c=%d reverse=%s" % (c, reverse))
    # deterministic mode: build + apply is bit-for-bit the one-call filter
    x = torch.from_numpy(rng.random((2, 30, 26, 6), dtype=np.float32)).cuda()
    a = lat.apply(x, mode="deterministic").cpu().numpy()
    b = plb.lattice_filter(x, ref, True, 5.0, 0.2, mode="deterministic").cpu().numpy()
    assert np.array_equal(bits(a), bits(b))
    # a workspace sized for the atomic mode has no room for the fixed-point sums: refused before any launch
    small = plb.Lattice(ref, bilateral=True, theta_alpha=5.0, theta_beta=0.2, max_channels=6)
    with pytest.raises(plb.PlError) as err:
        small.apply(x, mode="deterministic")
    assert err.value.status == 3   # PL_WORKSPACE_TOO_SMALL


@pytest.mark.parametrize("shape,r,channels", [
    ((2, 30, 26), 3, (21, 3, 21)),        # ragged tiles; 21 channels: quarter-warp splat, 3: thread-per-window splat
    ((1, 64, 48), 3, (21, 1)),
    ((1, 6, 20, 22), 1, (3, 21)),         # volume
    ((2, 40, 36), 0, (3, 21)),            # spatial only: one-word keys, vertices found by direct indexing
    ((1, 24, 20), 14, (3, 21)),           # pd 16: 128-point tiles, five-word keys
    ((2, 50), 1, (1, 3)),                 # 1-D signal, pd 2
])
def test_lattice_reuse_walks_the_sorted_splats(gpu, oracle, shape, r, channels):
    """A lattice built for reuse keeps every tile's splats sorted by entry; its splat kernels copy that list
    instead of sorting.  Checked against the oracle in the atomic mode, forward and reverse."""
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(47)
    bilateral = r > 0
    ref_n = rng.random(shape + (max(r, 1),), dtype=np.float32)
    ref = torch.from_numpy(ref_n).cuda()
    lat = plb.Lattice(ref if bilateral else None, shape, bilateral, theta_alpha=5.0, theta_beta=0.2, theta_gamma=3.0,
                      max_channels=max(channels))
    for k, c in enumerate(channels):
        reverse = bool(k & 1)
        x_n = rng.standard_normal(shape + (c,)).astype(np.float32)
        got = lat.apply(torch.from_numpy(x_n).cuda(), reverse=reverse).cpu().numpy()
        want = oracle.lattice_filter(x_n, ref_n, bilateral, 5.0, 0.2, 3.0, reverse)
        gpu.assert_outputs_close(got, want, "apply c=%d reverse=%s" % (c, reverse))
    assert lat.stats().device_status == 0


def test_apply_refuses_a_workspace_no_build_prepared(gpu):
    """pl_lattice_apply_f32 on the workspace a one-call filter left behind: that lattice has no sorted splats, the
    splat kernel says so through the device status and the output is NaN (nothing is read out of bounds)."""
    import torch
    import permutohedral_lattice_b200 as plb
    from permutohedral_lattice_b200 import capi
    rng = np.random.default_rng(48)
    ref = torch.from_numpy(rng.random((1, 32, 32, 3), dtype=np.float32)).cuda()
    x = torch.from_numpy(rng.random((1, 32, 32, 21), dtype=np.float32)).cuda()
    _, ws, call = plb.lattice_filter_raw(x, ref, True, 5.0, 0.2, 1.0, False, max_entries=0)
    out = torch.zeros_like(x)
    rc = capi.lib().pl_lattice_apply_f32(
        out.data_ptr(), x.data_ptr(), 21, 0, capi.PL_MODE_ATOMIC, 1, 32 * 32, call.pd, 2, capi.int_array([32, 32]),
        ws.data_ptr(), ws.numel(), 0, torch.cuda.current_stream().cuda_stream)
    assert rc == capi.PL_OK
    torch.cuda.synchronize()
    assert plb.lattice_stats(ws).device_status == capi.PL_INVALID_ARGUMENT
    assert bool(torch.isnan(out).all())


def test_back_to_back_calls_are_repeatable(gpu):
    """Several kernels of a call start while the kernel before them drains and wait on the device for it; calls
    issued back to back on one workspace must still see each other's results in order.  The deterministic mode
    gives the same bits every time, so any kernel that read too early would show."""
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(59)
    ref = torch.from_numpy(rng.random((3, 96, 80, 3), dtype=np.float32)).cuda()
    x = torch.from_numpy(rng.standard_normal((3, 96, 80, 21)).astype(np.float32)).cuda()
    outs = [plb.lattice_filter(x, ref, True, 6.0, 0.15, mode="deterministic") for _ in range(60)]
    torch.cuda.synchronize()
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    lat = plb.Lattice(ref, bilateral=True, theta_alpha=6.0, theta_beta=0.15, max_channels=21, mode="deterministic")
    outs = [lat.apply(x, reverse=bool(i & 1), mode="deterministic") for i in range(40)]
    torch.cuda.synchronize()
    assert all(torch.equal(outs[i & 1], o) for i, o in enumerate(outs))


def test_autograd_with_lattice_reuse(gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(43)
    ref_n = rng.random((1, 24, 20, 3), dtype=np.float32)
    inp_n = rng.random((1, 24, 20, 4), dtype=np.float32)
    grad_n = rng.standard_normal((1, 24, 20, 4)).astype(np.float32)
    ref = torch.from_numpy(ref_n).cuda()
    inp = torch.from_numpy(inp_n).cuda().requires_grad_(True)
    out = plb.lattice_filter(inp, ref, True, 5.0, 0.2, reuse_lattice=True)
    out.backward(torch.from_numpy(grad_n).cuda())
    gpu.assert_outputs_close(out.detach().cpu().numpy(), oracle.lattice_filter(inp_n, ref_n, True, 5.0, 0.2), "fwd")
    gpu.assert_outputs_close(inp.grad.cpu().numpy(), oracle.lattice_filter(grad_n, ref_n, True, 5.0, 0.2, 1.0, True),
                             "bwd")


def test_cuda_graph_replay_matches_plain_call(gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(51)
    ref_n = rng.random((2, 40, 36, 3), dtype=np.float32)
    gf = plb.GraphedLatticeFilter((2, 40, 36, 5), (2, 40, 36, 3), True, 6.0, 0.2)
    gf.reference.copy_(torch.from_numpy(ref_n))
    for _ in range(3):      # replays with new contents of the static tensors
        x_n = rng.standard_normal((2, 40, 36, 5)).astype(np.float32)
        gf.input.copy_(torch.from_numpy(x_n))
        got = gf.replay().cpu().numpy()
        gpu.assert_outputs_close(got, oracle.lattice_filter(x_n, ref_n, True, 6.0, 0.2), "graph replay")
