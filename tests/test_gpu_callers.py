"""The callers either side of the op: the image-file demo with the reference program's command line, and
dense-CRF mean-field inference built on lattices that are constructed once per image."""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_bilateral_demo_command_line(tmp_path, oracle):
    from PIL import Image
    rng = np.random.default_rng(3)
    blocks = rng.integers(0, 256, (6, 8, 3))
    img = np.clip(np.kron(blocks, np.ones((8, 8, 1))) + rng.normal(0, 6, (48, 64, 3)), 0, 255).astype(np.uint8)
    src, dst = tmp_path / "in.bmp", tmp_path / "out.bmp"
    Image.fromarray(img).save(src)
    res = subprocess.run([sys.executable, "-m", "permutohedral_lattice_b200.bilateral_demo", str(src), str(dst),
                          "8", "0.125"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr
    assert res.stdout.count("Measured from function call") == 2
    got = np.array(Image.open(dst))
    x = (img / 255.0).astype(np.float32)[None]
    want = np.round(oracle.lattice_filter(x, x, True, 8.0, 0.125)[0] * 255).astype(np.uint8)
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 1e-3      # a value on a rounding boundary may tip over
    res = subprocess.run([sys.executable, "-m", "permutohedral_lattice_b200.bilateral_demo"], cwd=ROOT,
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 1 and "Usage" in res.stdout


def test_dense_crf_mean_field_matches_cpu_composition(oracle):
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(5)
    b, h, w, labels = 2, 40, 36, 5
    image = np.clip(np.kron(rng.random((b, 5, 6, 3)), np.ones((1, 8, 6, 1))) + rng.normal(0, 0.03, (b, h, w, 3)),
                    0, 1).astype(np.float32)
    unaries = (2.0 * rng.standard_normal((b, h, w, labels))).astype(np.float32)
    ta, tb, tg, wb, ws = 10.0, 0.1, 2.0, 1.5, 0.75
    crf = plb.DenseCRF(torch.from_numpy(image).cuda(), labels, ta, tb, tg, wb, ws)
    got = crf.infer(torch.from_numpy(unaries).cuda(), iterations=3).cpu().numpy()

    def softmax(z):
        e = np.exp(z - z.max(-1, keepdims=True))
        return e / e.sum(-1, keepdims=True)

    compat = 1.0 - np.eye(labels, dtype=np.float32)
    q = softmax(-unaries)
    for _ in range(3):
        qb = oracle.lattice_filter(q, image, True, ta, tb, 1.0)
        qs = oracle.lattice_filter(q, None, False, 1.0, 1.0, tg)
        q = softmax(-unaries - (wb * qb + ws * qs) @ compat).astype(np.float32)
    assert np.abs(got - q).max() <= 1e-4
    assert np.abs(got.sum(-1) - 1).max() <= 1e-5


@pytest.mark.parametrize("n_points,labels,potts", [
    (1000, 21, True),        # ragged last block, Potts model
    (777, 21, False),        # general compatibility matrix
    (256, 5, False),         # exactly one block
    (300, 40, False),        # more than 32 labels: the 128-thread form
    (1, 2, True),            # a single point
])
def test_crf_update_kernel_matches_torch(n_points, labels, potts):
    """pl_crf_update_f32 (through the C ABI) against the same update written with torch operations:
    softmax(-U - (wb Qb + ws Qs) @ compat), fp32, max-abs 1e-5."""
    import torch
    from permutohedral_lattice_b200 import capi
    g = torch.Generator(device="cpu").manual_seed(n_points + labels)
    qb = torch.rand((n_points, labels), generator=g).cuda()
    qs = torch.rand((n_points, labels), generator=g).cuda()
    u = (3.0 * torch.randn((n_points, labels), generator=g)).cuda()
    compat = None if potts else torch.randn((labels, labels), generator=g).cuda()
    wb, ws = 1.5, 0.75
    out = torch.full((n_points + 3, labels), 7.0, device="cuda")     # guard rows after the end
    capi.check(capi.lib().pl_crf_update_f32(
        out.data_ptr(), u.data_ptr(), qb.data_ptr(), qs.data_ptr(), 0 if potts else compat.data_ptr(), wb, ws,
        n_points, labels, torch.cuda.current_stream().cuda_stream), "pl_crf_update_f32")
    torch.cuda.synchronize()
    cm = (1.0 - torch.eye(labels, device="cuda")) if potts else compat
    msg = (wb * qb + ws * qs).double() @ cm.double()
    want = torch.softmax(-u.double() - msg, dim=-1).float()
    assert torch.all(out[n_points:] == 7.0), "wrote past the last point"
    assert float((out[:n_points] - want).abs().max()) <= 1e-5
    assert float((out[:n_points].sum(-1) - 1).abs().max()) <= 1e-5


def test_crf_update_rejects_bad_arguments():
    import torch
    from permutohedral_lattice_b200 import capi
    t = torch.zeros((4, 3), device="cuda")
    L = capi.lib()
    s = torch.cuda.current_stream().cuda_stream
    assert L.pl_crf_update_f32(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 0, 1.0, 1.0, 4, 0, s) \
        == capi.PL_INVALID_ARGUMENT
    assert L.pl_crf_update_f32(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 0, 1.0, 1.0, 4, 129, s) \
        == capi.PL_UNSUPPORTED_DIMS
    assert L.pl_crf_update_f32(0, t.data_ptr(), t.data_ptr(), t.data_ptr(), 0, 1.0, 1.0, 4, 3, s) \
        == capi.PL_INVALID_ARGUMENT
    assert L.pl_crf_update_f32(0, 0, 0, 0, 0, 1.0, 1.0, 0, 3, s) == capi.PL_OK      # nothing to do


def test_host_pipeline_forward_backward_through_one_lattice(oracle):
    """HostPipeline.filter_forward_backward: reference sent once, one lattice per chunk, against the CPU oracle's
    forward and reverse calls."""
    import torch
    import permutohedral_lattice_b200 as plb
    import gpu_helpers
    rng = np.random.default_rng(77)
    ref = rng.random((5, 28, 30, 3), dtype=np.float32)
    x = rng.standard_normal((5, 28, 30, 4)).astype(np.float32)
    g = rng.standard_normal((5, 28, 30, 4)).astype(np.float32)
    pipe = plb.HostPipeline(torch.device("cuda", 0), n_streams=3, chunk_items=2, edge_chunks=1)
    hx, hg, hr = (torch.from_numpy(a).pin_memory() for a in (x, g, ref))
    for _ in range(2):      # twice: the second pass reuses the slots' buffers
        out, gout = pipe.filter_forward_backward(hx, hg, hr, True, 5.0, 0.2)
        gpu_helpers.assert_outputs_close(out.numpy(), oracle.lattice_filter(x, ref, True, 5.0, 0.2, 1.0, False), "fwd")
        gpu_helpers.assert_outputs_close(gout.numpy(), oracle.lattice_filter(g, ref, True, 5.0, 0.2, 1.0, True), "bwd")
