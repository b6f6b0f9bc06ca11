"""Batch sharding across ranks.  Every batch item is an independent lattice (the reference loops over
items serially with no shared state, src/LatticeFilterKernel.cpp:152-179), so ranks filter
contiguous slices of the batch with no collective in the data path; gathering the outputs is optional
and happens after the filter."""
import torch
import torch.distributed as dist


def shard_range(batch, world_size, rank):
    """Contiguous slice [lo, hi) of `batch` items for `rank`; sizes differ by at most one, earlier ranks
    take the larger shares, ranks beyond the batch get an empty slice."""
    if world_size < 1 or not (0 <= rank < world_size) or batch < 0:
        raise ValueError("bad shard request: batch=%r world_size=%r rank=%r" % (batch, world_size, rank))
    base, extra = divmod(batch, world_size)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo, hi


def lattice_filter_sharded(input_image, reference_image, *, filter_fn=None, gather=False, group=None,
                           **filter_kwargs):
    """Filters this rank's slice of a batch that every rank holds (or can index) in full.

    filter_fn(input_slice, reference_slice, **filter_kwargs) defaults to the CUDA `lattice_filter`.
    Returns the rank's output slice, or with gather=True the whole output on every rank
    (all_gather of equally padded slices)."""
    if filter_fn is None:
        from .lattice_filter import lattice_filter as filter_fn
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    batch = input_image.shape[0]
    lo, hi = shard_range(batch, world, rank)
    ref_slice = None if reference_image is None else reference_image[lo:hi]
    out = filter_fn(input_image[lo:hi], ref_slice, **filter_kwargs)
    if not gather or world == 1:
        return out
    per = -(-batch // world)                       # every rank contributes `per` rows, padded
    padded = torch.zeros((per,) + tuple(out.shape[1:]), dtype=out.dtype, device=out.device)
    padded[:hi - lo] = out
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    pieces = []
    for r in range(world):
        rlo, rhi = shard_range(batch, world, r)
        pieces.append(parts[r][:rhi - rlo])
    return torch.cat(pieces, 0)
