"""Parity at the full sizes of the benchmark configurations: the CUDA path against the CPU oracle on
whole items, plus properties that need no oracle (constants are preserved, the filter is linear in its
input, batch items commute with the filter, the deterministic mode repeats itself)."""
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


@pytest.fixture(scope="module")
def crf16():
    from permutohedral_lattice_b200 import workloads
    return workloads.config2()


def test_config2_full_batch_forward_and_backward_against_oracle(gpu, oracle, crf16):
    import torch
    import permutohedral_lattice_b200 as plb
    w = crf16
    threads = min(16, __import__("os").cpu_count() or 1)
    want_f, _ = oracle.filter_batch_timed(w.input, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, False,
                                          threads=threads)
    want_b, _ = oracle.filter_batch_timed(w.grad, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, True,
                                          threads=threads)
    x = torch.from_numpy(w.input).cuda()
    ref = torch.from_numpy(w.reference).cuda()
    g = torch.from_numpy(w.grad).cuda()
    out_f, ws, call = plb.lattice_filter_raw(x, ref, True, w.theta_alpha, w.theta_beta, 1.0, False)
    st = plb.lattice_stats(ws)
    assert st.device_status == 0
    gpu.assert_outputs_close(out_f.cpu().numpy(), want_f, "c2 forward")
    # vertex count of the whole batch = sum of the per-item counts of the oracle (checked on two items
    # in full, structure included, and on the total through the reference's own count for the rest)
    items = [oracle.lattice_filter(w.input[i:i + 1], w.reference[i:i + 1], True, w.theta_alpha, w.theta_beta,
                                   1.0, False, structure=True)[1][0] for i in (0, 15)]
    vk, vi, pv, pw = plb.export_lattice(ws, st, call.batch, call.n, call.pd, call.vd, reference=ref,
                                        sdims=call.sdims, spatial_std=call.spatial_std,
                                        feature_std=call.feature_std)
    vk, vi, pv = vk.cpu().numpy(), vi.cpu().numpy(), pv.cpu().numpy()
    from conftest import sorted_rows
    for i, o in zip((0, 15), items):
        mine = vk[vi == i]
        assert len(mine) == o.num_vertices
        assert np.array_equal(sorted_rows(mine), sorted_rows(o.keys))
        assert np.array_equal(vk[pv[i]], o.pixel_keys())
    # (the backward call comes last: it reuses the stream's workspace, which the export above still needed)
    out_b = plb.lattice_filter(g, ref, True, w.theta_alpha, w.theta_beta, 1.0, reverse=True)
    gpu.assert_outputs_close(out_b.cpu().numpy(), want_b, "c2 backward")


def test_config2_properties_at_full_size(gpu, crf16):
    import torch
    import permutohedral_lattice_b200 as plb
    from conftest import bits
    w = crf16
    ref = torch.from_numpy(w.reference).cuda()
    x = torch.from_numpy(w.input).cuda()
    y = torch.from_numpy(w.grad).cuda()
    args = (True, w.theta_alpha, w.theta_beta, 1.0)
    # constants are preserved (the weights of every point are normalised away)
    const = torch.full_like(x, 0.375)
    out = plb.lattice_filter(const, ref, *args)
    assert float((out - 0.375).abs().max()) <= 1e-6
    # linear in the input
    fx = plb.lattice_filter(x, ref, *args)
    fy = plb.lattice_filter(y, ref, *args)
    fxy = plb.lattice_filter(2.0 * x - 0.5 * y, ref, *args)
    lin = 2.0 * fx - 0.5 * fy
    assert float((fxy - lin).norm() / lin.norm()) <= 1e-5
    assert float((fxy - lin).abs().max()) <= 1e-4
    # batch items commute with the filter
    perm = torch.tensor([5, 0, 15, 3, 9, 1, 2, 4, 6, 7, 8, 10, 11, 12, 13, 14], device="cuda")
    fperm = plb.lattice_filter(x[perm].contiguous(), ref[perm].contiguous(), *args)
    gpu.assert_outputs_close(fperm.cpu().numpy(), fx[perm].cpu().numpy(), "permuted batch")
    # deterministic mode repeats itself bit for bit and agrees with the atomic mode
    d1 = plb.lattice_filter(x, ref, *args, mode="deterministic")
    d2 = plb.lattice_filter(x, ref, *args, mode="deterministic")
    assert np.array_equal(bits(d1.cpu().numpy()), bits(d2.cpu().numpy()))
    gpu.assert_outputs_close(d1.cpu().numpy(), fx.cpu().numpy(), "deterministic vs atomic")


@pytest.mark.parametrize("config", [0, 1])
def test_single_image_configs_full_size(config, gpu, oracle):
    from permutohedral_lattice_b200 import workloads
    w = workloads.CONFIGS[config]()
    want, items = oracle.lattice_filter(w.input, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, False,
                                        structure=True)
    out, ws, call, x, r = gpu.run_op(w.input, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, False)
    st, (vk, vi, pv, pw) = gpu.export_op(ws, call, r)
    gpu.assert_structure_equal(vk, vi, pv, pw, items, w.name)
    gpu.assert_outputs_close(out.cpu().numpy(), want, w.name)
    if w.backward:
        want_b = oracle.lattice_filter(w.grad, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, True)
        got_b = gpu.run_op(w.grad, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, True)[0]
        gpu.assert_outputs_close(got_b.cpu().numpy(), want_b, w.name + " bwd")


def test_volume_config_two_items_full_size(gpu, oracle):
    from permutohedral_lattice_b200 import workloads
    w = workloads.config3(batch=2)
    want, items = oracle.lattice_filter(w.input, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, True,
                                        structure=True)
    out, ws, call, x, r = gpu.run_op(w.input, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, True)
    st, (vk, vi, pv, pw) = gpu.export_op(ws, call, r)
    gpu.assert_structure_equal(vk, vi, pv, pw, items, w.name)
    gpu.assert_outputs_close(out.cpu().numpy(), want, w.name)
    want_f = oracle.lattice_filter(w.input, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, False)
    got_f = gpu.run_op(w.input, w.reference, True, w.theta_alpha, w.theta_beta, 1.0, False)[0]
    gpu.assert_outputs_close(got_f.cpu().numpy(), want_f, w.name + " forward")


def test_pd16_config_one_item_full_size(gpu, oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    from permutohedral_lattice_b200 import workloads
    w = workloads.config4(batch=1)
    n, c = w.pixels_per_item, w.input.shape[-1]
    res = oracle.filter(w.input[0].reshape(n, c), w.positions[0])
    x = torch.from_numpy(w.input.reshape(1, n, c)).cuda()
    p = torch.from_numpy(w.positions).cuda()
    out, ws = plb.filter_positions(x, p)
    st = plb.lattice_stats(ws)
    assert st.device_status == 0
    assert st.num_vertices == res.num_vertices
    vk, vi, pv, pw = plb.export_lattice(ws, st, 1, n, 16, c + 1, positions=p)
    gpu.assert_structure_equal(vk, vi, pv, pw, [res], w.name)
    gpu.assert_outputs_close(out.cpu().numpy()[0], res.out, w.name)
