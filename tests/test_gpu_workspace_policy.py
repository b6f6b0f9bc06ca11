"""How much workspace a call gets by default (sized from what its lattice needs instead of the bound that can
never overflow), and what happens when a lattice outgrows it: a call on a new reference image is verified and
repeated on the spot; a call on the reference a verified call just used runs with that call's bound; calls made
with verify="deferred" (HostPipeline) that do not fit fill their output with NaN, are reported by
check_pending() and repeated by the pipeline.  Nothing here faults the GPU: a bound that is too small only sets
a status bit on the device."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

KW = dict(bilateral=True, theta_alpha=5.0, theta_beta=0.2, theta_gamma=1.0)


def _data(seed, batch=2, shape=(48, 44), c=4, blocky=True):
    import torch
    rng = np.random.default_rng(seed)
    if blocky:   # few lattice entries per point, so a bound well below the worst case suffices
        blocks = rng.random((batch, (shape[0] + 7) // 8, (shape[1] + 7) // 8, 3), dtype=np.float32)
        ref_n = np.repeat(np.repeat(blocks, 8, 1), 8, 2)[:, :shape[0], :shape[1]]
    else:        # white noise: nearly every splat its own entry
        ref_n = rng.random((batch,) + shape + (3,), dtype=np.float32)
    ref = torch.from_numpy(np.ascontiguousarray(ref_n)).cuda()
    x = torch.from_numpy(rng.standard_normal((batch,) + shape + (c,)).astype(np.float32)).cuda()
    return x, ref


@pytest.fixture()
def policy():
    """A clean slate for the module's memory of earlier calls."""
    import permutohedral_lattice_b200 as plb
    import sys
    lf = sys.modules["permutohedral_lattice_b200.lattice_filter"]   # (the package re-exports a function of that name)
    saved = (dict(lf._entries_per_item), lf.FIRST_GUESS_DIVISOR)
    lf._entries_per_item.clear()
    lf._pending.clear()
    lf._verified.clear()
    plb.release_workspaces()
    yield lf
    lf._entries_per_item.clear()
    lf._entries_per_item.update(saved[0])
    lf.FIRST_GUESS_DIVISOR = saved[1]
    lf._pending.clear()
    lf._verified.clear()


def test_default_workspace_is_smaller_than_the_worst_case_and_results_agree(policy):
    import permutohedral_lattice_b200 as plb
    from conftest import bits
    x, ref = _data(1)
    want, ws0, call0 = plb.lattice_filter_raw(x, ref, mode="deterministic", max_entries=0, **KW)
    worst_bytes = call0.workspace_bytes(0, mode="deterministic")
    plb.release_workspaces()
    got, ws, call = plb.lattice_filter_raw(x, ref, mode="deterministic", **KW)     # first of its kind: verified
    assert 0 < call.max_entries < call.batch * call.n * (call.pd + 1)
    assert ws.numel() < worst_bytes
    assert np.array_equal(bits(got.cpu().numpy()), bits(want.cpu().numpy()))
    got2, ws2, call2 = plb.lattice_filter_raw(x, ref, mode="deterministic", **KW)  # same reference: same bound
    st = plb.lattice_stats(ws2)
    assert st.device_status == 0 and st.num_entries <= call2.max_entries == st.max_entries
    assert call2.max_entries == call.max_entries
    assert np.array_equal(bits(got2.cpu().numpy()), bits(want.cpu().numpy()))


def test_first_call_of_a_kind_is_repeated_until_the_lattice_fits(policy):
    import permutohedral_lattice_b200 as plb
    from conftest import bits
    x, ref = _data(2)
    want, _, _ = plb.lattice_filter_raw(x, ref, mode="deterministic", max_entries=0, **KW)
    policy.FIRST_GUESS_DIVISOR = 64          # a first guess far too small: several repeats
    policy._entries_per_item.clear()
    policy._verified.clear()
    got, ws, call = plb.lattice_filter_raw(x, ref, mode="deterministic", **KW)
    st = plb.lattice_stats(ws)
    assert st.device_status == 0 and st.num_entries <= st.max_entries
    assert np.array_equal(bits(got.cpu().numpy()), bits(want.cpu().numpy()))


def test_new_reference_is_verified_even_when_earlier_data_needed_far_less(policy):
    import torch
    import permutohedral_lattice_b200 as plb
    from conftest import bits
    x, ref = _data(3, blocky=False)
    want, _, call = plb.lattice_filter_raw(x, ref, mode="deterministic", max_entries=0, **KW)
    kind = policy._kind(x.device, call)
    policy._entries_per_item[kind] = 10.0     # as if earlier data of this kind had needed almost nothing
    out, ws, call = plb.lattice_filter_raw(x, ref, mode="deterministic", **KW)
    assert np.array_equal(bits(out.cpu().numpy()), bits(want.cpu().numpy()))
    assert policy._entries_per_item[kind] > 10.0
    # the same reference again (a backward call): the verified bound is reused as it is
    out2, ws2, call2 = plb.lattice_filter_raw(x, ref, mode="deterministic", reverse=True, **KW)
    assert call2.max_entries == call.max_entries
    assert plb.lattice_stats(ws2).device_status == 0
    # written to in place: no longer "the same lattice", verified again
    ref.mul_(0.5)
    policy._entries_per_item[kind] = 10.0
    want3 = plb.lattice_filter_raw(x, ref, mode="deterministic", max_entries=0, **KW)[0]
    out3 = plb.lattice_filter_raw(x, ref, mode="deterministic", **KW)[0]
    assert np.array_equal(bits(out3.cpu().numpy()), bits(want3.cpu().numpy()))


def test_deferred_call_that_does_not_fit_is_reported_and_succeeds_when_repeated(policy):
    import torch
    import permutohedral_lattice_b200 as plb
    from permutohedral_lattice_b200 import capi
    from conftest import bits
    x, ref = _data(3, blocky=False)
    want, _, call = plb.lattice_filter_raw(x, ref, mode="deterministic", max_entries=0, **KW)
    kind = policy._kind(x.device, call)
    policy._entries_per_item[kind] = 10.0
    out, ws, _ = plb.lattice_filter_raw(x, ref, mode="deterministic", verify="deferred", **KW)
    torch.cuda.synchronize()
    assert torch.isnan(out).all()             # a call that did not fit never leaves plausible values
    with pytest.raises(plb.PlError) as err:
        plb.check_pending()
    assert err.value.status == capi.PL_CAPACITY_EXCEEDED
    for _ in range(24):                       # every report raises the bound; the repeat ends up fitting
        out, ws, _ = plb.lattice_filter_raw(x, ref, mode="deterministic", verify="deferred", **KW)
        try:
            plb.check_pending()
            break
        except plb.PlError as e:
            assert e.status == capi.PL_CAPACITY_EXCEEDED
    assert np.array_equal(bits(out.cpu().numpy()), bits(want.cpu().numpy()))


def test_host_pipeline_repeats_chunks_that_did_not_fit(policy):
    import torch
    import permutohedral_lattice_b200 as plb
    x, ref = _data(4, batch=5, blocky=False)
    hx, href = x.cpu().pin_memory(), ref.cpu().pin_memory()
    want = plb.lattice_filter(x, ref, **KW).cpu().numpy()
    pipe = plb.HostPipeline(torch.device("cuda", 0), n_streams=2, chunk_items=2, edge_chunks=1)
    pipe.filter(hx, href, **KW)               # teaches the policy what a chunk of this kind needs
    from permutohedral_lattice_b200.lattice_filter import FilterCall
    for batch in (1, 2):
        call = FilterCall((batch,) + tuple(x.shape[1:]), (batch,) + tuple(ref.shape[1:]), True, 5.0, 0.2, 1.0)
        policy._entries_per_item[policy._kind(x.device, call)] = 10.0
    out = pipe.filter(hx, href, **KW)         # chunks overflow, synchronize() finds out and repeats them
    got = out.numpy()
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 1e-4


def test_host_pipeline_gives_back_its_workspaces_when_closed(policy):
    import torch
    import permutohedral_lattice_b200 as plb
    x, ref = _data(6, batch=3)
    pipe = plb.HostPipeline(torch.device("cuda", 0), n_streams=2)
    pipe.filter(x.cpu().pin_memory(), ref.cpu().pin_memory(), **KW)
    mine = [k for k in policy._workspaces if isinstance(k[1], tuple) and k[1][:2] == ("HostPipeline", id(pipe))]
    assert mine                                   # one workspace per stream slot that was used
    pipe.close()
    assert not [k for k in policy._workspaces if isinstance(k[1], tuple) and k[1][:2] == ("HostPipeline", id(pipe))]
