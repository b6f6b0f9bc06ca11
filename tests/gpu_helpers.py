"""Shared code of the GPU parity tests: run the CUDA path through the C ABI and compare its
lattice structure and outputs with the CPU oracle."""
import numpy as np
import torch

import permutohedral_lattice_b200 as plb
from conftest import bits, rel_l2, sorted_rows

# forward / backward fp32 outputs against the CPU oracle
REL_L2_TOL = 1e-5
MAX_ABS_TOL = 1e-4


def assert_outputs_close(got, want, what=""):
    got = np.asarray(got, np.float32)
    want = np.asarray(want, np.float32)
    assert got.shape == want.shape
    assert np.isfinite(got).all(), what + ": non-finite output"
    r = rel_l2(got, want)
    m = float(np.abs(got.astype(np.float64) - want.astype(np.float64)).max()) if got.size else 0.0
    assert r <= REL_L2_TOL, "%s: relative L2 %.3g > %.1g" % (what, r, REL_L2_TOL)
    assert m <= MAX_ABS_TOL, "%s: max abs %.3g > %.1g" % (what, m, MAX_ABS_TOL)


def assert_structure_equal(vkeys, vitem, pv, pw, oracle_items, what=""):
    """vkeys [M, pd], vitem [M], pv / pw [B, n, pd+1] from the GPU; oracle_items: LatticeResult per item.
    Vertex count, vertex key set, per-point simplex keys: bit-exact.  Weights: within one ulp."""
    vkeys, vitem, pv, pw = (t.cpu().numpy() for t in (vkeys, vitem, pv, pw))
    assert len(vkeys) == sum(o.num_vertices for o in oracle_items), what + ": vertex count"
    for b, o in enumerate(oracle_items):
        mine = vkeys[vitem == b]
        assert len(mine) == o.num_vertices, "%s: item %d vertex count %d != %d" % (
            what, b, len(mine), o.num_vertices)
        assert np.array_equal(sorted_rows(mine), sorted_rows(o.keys)), what + ": vertex key set"
        assert np.all(vitem[pv[b]] == b), what + ": point refers to another item's vertex"
        assert np.array_equal(vkeys[pv[b]], o.pixel_keys()), what + ": per-point simplex keys"
        # Weights: the kernels form the reference's float(double(x) * (1 / (pd + 1))) products in float-float
        # arithmetic, which can differ from that double rounding in the last bit; one unit in the last place
        # is what the code promises (keys, which decide the structure, are exact).  Same-sign floats order
        # like their bit patterns, so the distance in ulps is the difference of the patterns.
        gb, ob = bits(pw[b]).astype(np.int64), bits(o.pix_weight).astype(np.int64)
        assert np.abs(gb - ob).max() <= 1, what + ": barycentric weights differ by more than one ulp"


def run_op(inp, ref, bilateral, ta, tb, tg, reverse, **kw):
    x = torch.from_numpy(np.ascontiguousarray(inp)).cuda()
    r = None if ref is None else torch.from_numpy(np.ascontiguousarray(ref)).cuda()
    out, ws, call = plb.lattice_filter_raw(x, r, bilateral, ta, tb, tg, reverse, **kw)
    torch.cuda.synchronize()
    return out, ws, call, x, r


def export_op(ws, call, r, max_entries=None):
    st = plb.lattice_stats(ws)
    assert st.device_status == 0, "device status %d" % st.device_status
    return st, plb.export_lattice(ws, st, call.batch, call.n, call.pd, call.vd, reference=r,
                                  sdims=call.sdims, spatial_std=call.spatial_std,
                                  feature_std=call.feature_std, max_entries=max_entries)
