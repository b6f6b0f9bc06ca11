"""Batch sharding with the CUDA filter: a rank's slice equals the same items of the unsharded call, and the
slices gathered over NCCL equal the single-GPU result.  The two-GPU test skips on a one-GPU box."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _data(batch, seed=7):
    rng = np.random.default_rng(seed)
    ref = rng.random((batch, 40, 36, 3), dtype=np.float32)
    inp = np.clip(rng.standard_normal((batch, 40, 36, 5)), -3.5, 3.5).astype(np.float32)
    # The deterministic mode rounds onto a fixed-point grid chosen from max |input| of the CALL; giving every
    # item the same maximum makes that grid the same for any slicing of the batch, so results can be
    # compared bit for bit across slicings.
    inp[:, 0, 0, 0] = 4.0
    return inp, ref


KW = dict(bilateral=True, theta_alpha=6.0, theta_beta=0.125, theta_gamma=1.0)


def test_one_rank_sharded_call_is_the_unsharded_call():
    import torch
    import permutohedral_lattice_b200 as plb
    from permutohedral_lattice_b200.sharding import lattice_filter_sharded
    from conftest import bits
    inp, ref = _data(3)
    x, r = torch.from_numpy(inp).cuda(), torch.from_numpy(ref).cuda()
    want = plb.lattice_filter(x, r, mode="deterministic", **KW)
    got = lattice_filter_sharded(x, r, gather=True, mode="deterministic", **KW)
    assert np.array_equal(bits(got.cpu().numpy()), bits(want.cpu().numpy()))


def test_slices_of_the_batch_filter_independently():
    """What sharding relies on: filtering items [lo, hi) alone gives the same bits (deterministic mode) as
    those items of the whole-batch call."""
    import torch
    import permutohedral_lattice_b200 as plb
    from permutohedral_lattice_b200.sharding import shard_range
    from conftest import bits
    inp, ref = _data(5)
    x, r = torch.from_numpy(inp).cuda(), torch.from_numpy(ref).cuda()
    want = plb.lattice_filter(x, r, mode="deterministic", reverse=True, **KW).cpu().numpy()
    for world in (2, 3):
        for rank in range(world):
            lo, hi = shard_range(5, world, rank)
            got = plb.lattice_filter(x[lo:hi], r[lo:hi], mode="deterministic", reverse=True, **KW)
            assert np.array_equal(bits(got.cpu().numpy()), bits(want[lo:hi]))


def _worker(rank, world, port, batch, result_dir):
    import torch
    import torch.distributed as dist
    import permutohedral_lattice_b200 as plb
    from permutohedral_lattice_b200.sharding import lattice_filter_sharded
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    inp, ref = _data(batch)
    x, r = torch.from_numpy(inp).to(dev), torch.from_numpy(ref).to(dev)
    on_zero = lattice_filter_sharded(x, r, gather=True, dst=0, mode="deterministic", **KW)
    everywhere = lattice_filter_sharded(x, r, gather=True, mode="atomic", reverse=True, **KW)
    torch.cuda.synchronize()
    assert (on_zero is None) == (rank != 0)
    if rank == 0:
        want = plb.lattice_filter(x, r, mode="deterministic", **KW)
        np.save(os.path.join(result_dir, "gathered.npy"), on_zero.cpu().numpy())
        np.save(os.path.join(result_dir, "single.npy"), want.cpu().numpy())
    want_rev = plb.lattice_filter(x, r, mode="atomic", reverse=True, **KW)
    np.save(os.path.join(result_dir, "all_%d.npy" % rank), everywhere.cpu().numpy())
    np.save(os.path.join(result_dir, "all_want_%d.npy" % rank), want_rev.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("batch", [4, 3])
def test_two_gpu_shards_gathered_over_nccl_equal_the_single_gpu_result(batch, tmp_path):
    import torch
    import torch.multiprocessing as mp
    from conftest import bits
    import gpu_helpers
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, batch, str(tmp_path)), nprocs=2, join=True)
    gathered = np.load(tmp_path / "gathered.npy")
    single = np.load(tmp_path / "single.npy")
    assert gathered.shape == single.shape
    assert np.array_equal(bits(gathered), bits(single))        # deterministic mode: bit for bit
    for rank in range(2):
        gpu_helpers.assert_outputs_close(np.load(tmp_path / ("all_%d.npy" % rank)),
                                         np.load(tmp_path / ("all_want_%d.npy" % rank)), "all_gather rank %d" % rank)
