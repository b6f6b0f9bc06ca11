"""Batch sharding over ranks, exercised with two gloo ranks on CPU.  The per-rank filter is the CPU
oracle here (the CUDA filter needs a GPU); what is under test is the partition and the gather."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from permutohedral_lattice_b200.sharding import lattice_filter_sharded, shard_range


def test_shard_range_partitions_exactly():
    for batch in (0, 1, 2, 7, 16):
        for world in (1, 2, 3, 4, 8):
            covered = []
            for r in range(world):
                lo, hi = shard_range(batch, world, r)
                assert 0 <= lo <= hi <= batch
                covered += list(range(lo, hi))
            assert covered == list(range(batch))
            sizes = [shard_range(batch, world, r)[1] - shard_range(batch, world, r)[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _oracle_filter(inp, ref, **kw):
    from oracle import cpu_oracle as O
    if inp.shape[0] == 0:
        return inp.clone()
    return torch.from_numpy(O.lattice_filter(inp.numpy(), ref.numpy(), **kw))


def _worker(rank, world, port, batch, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)                       # same data on every rank
    ref = torch.from_numpy(rng.random((batch, 12, 10, 3), dtype=np.float32))
    inp = torch.from_numpy(rng.random((batch, 12, 10, 2), dtype=np.float32))
    kw = dict(bilateral=True, theta_alpha=4.0, theta_beta=0.25, theta_gamma=1.0, reverse=False)
    full = lattice_filter_sharded(inp, ref, filter_fn=_oracle_filter, gather=True, **kw)
    mine = lattice_filter_sharded(inp, ref, filter_fn=_oracle_filter, gather=False, **kw)
    on_one = lattice_filter_sharded(inp, ref, filter_fn=_oracle_filter, gather=True, dst=1, **kw)
    assert (on_one is None) == (rank != 1)
    if rank == 1:
        np.save(os.path.join(result_dir, "on_one.npy"), on_one.numpy())
    np.save(os.path.join(result_dir, "full_%d.npy" % rank), full.numpy())
    np.save(os.path.join(result_dir, "mine_%d.npy" % rank), mine.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("batch", [3, 4, 1])
def test_two_rank_sharded_filter_matches_single_process(batch, tmp_path):
    from oracle import cpu_oracle as O
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, batch, str(tmp_path)), nprocs=2, join=True)
    rng = np.random.default_rng(0)
    ref = rng.random((batch, 12, 10, 3), dtype=np.float32)
    inp = rng.random((batch, 12, 10, 2), dtype=np.float32)
    want = O.lattice_filter(inp, ref, True, 4.0, 0.25, 1.0, False)
    assert np.array_equal(np.load(tmp_path / "on_one.npy").view(np.uint32), want.view(np.uint32))
    for rank in range(2):
        full = np.load(tmp_path / ("full_%d.npy" % rank))
        assert np.array_equal(full.view(np.uint32), want.view(np.uint32))
        lo, hi = shard_range(batch, 2, rank)
        mine = np.load(tmp_path / ("mine_%d.npy" % rank))
        assert np.array_equal(mine.view(np.uint32), want[lo:hi].view(np.uint32))
