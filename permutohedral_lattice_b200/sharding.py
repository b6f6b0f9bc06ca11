"""Batch sharding across ranks.  Every batch item is an independent lattice (the reference loops over
items serially with no shared state, src/LatticeFilterKernel.cpp:152-179), so ranks filter
contiguous slices of the batch with no collective in the data path; gathering the outputs is optional
and happens after the filter (NCCL over NVLink when the ranks are GPUs: no kernel of this package is
ever handed another GPU's memory)."""
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


def _world(group):
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


class OutputGather:
    """Collects the ranks' output slices of a `batch`-item tensor, either on every rank
    (`dst=None`, all_gather) or on one rank (`dst=r`, gather).  Buffers are allocated once and reused,
    so a gather inside a timed loop does no allocation.  Slices are padded to the largest share, so
    any batch size works with any number of ranks."""

    def __init__(self, batch, item_shape, dtype, device, dst=None, group=None):
        self.batch, self.group, self.dst = int(batch), group, dst
        self.world, self.rank = _world(group)
        self.per = -(-self.batch // self.world) if self.batch else 0
        self.lo, self.hi = shard_range(self.batch, self.world, self.rank)
        shape = (self.per,) + tuple(item_shape)
        self.even = self.batch == self.per * self.world          # every share is exactly `per` items
        self.padded = None if self.even else torch.zeros(shape, dtype=dtype, device=device)
        self.receives = dst is None or dst == self.rank
        self.full = None
        if self.receives:
            self.full = torch.empty((self.per * self.world,) + tuple(item_shape), dtype=dtype, device=device)

    def __call__(self, out_slice):
        """out_slice: this rank's [hi - lo, ...] output.  Returns the whole [batch, ...] output on the
        receiving rank(s), None elsewhere.  Runs on the current stream."""
        if self.world == 1:
            return out_slice
        src = out_slice
        if not self.even:
            self.padded[:self.hi - self.lo].copy_(out_slice)
            src = self.padded
        src = src.contiguous()
        if self.dst is None:
            dist.all_gather_into_tensor(self.full, src, group=self.group)
        else:
            parts = list(self.full.view((self.world, self.per) + tuple(self.full.shape[1:])).unbind(0)) \
                if self.receives else None
            dist.gather(src, parts, dst=self.dst, group=self.group)
        if not self.receives:
            return None
        if self.even:
            return self.full
        pieces = []
        for r in range(self.world):
            rlo, rhi = shard_range(self.batch, self.world, r)
            pieces.append(self.full[r * self.per:r * self.per + (rhi - rlo)])
        return torch.cat(pieces, 0)


def lattice_filter_sharded(input_image, reference_image, *, filter_fn=None, gather=False, dst=None, group=None,
                           **filter_kwargs):
    """Filters this rank's slice of a batch that every rank holds (or can index) in full.

    filter_fn(input_slice, reference_slice, **filter_kwargs) defaults to the CUDA `lattice_filter`.
    Returns the rank's output slice; with gather=True the whole output, on every rank (dst=None) or on
    rank `dst` only (None on the others)."""
    if filter_fn is None:
        from .lattice_filter import lattice_filter as filter_fn
    world, rank = _world(group)
    batch = input_image.shape[0]
    lo, hi = shard_range(batch, world, rank)
    ref_slice = None if reference_image is None else reference_image[lo:hi]
    out = filter_fn(input_image[lo:hi], ref_slice, **filter_kwargs)
    if not gather or world == 1:
        return out
    collect = OutputGather(batch, tuple(out.shape[1:]), out.dtype, out.device, dst=dst, group=group)
    return collect(out)
