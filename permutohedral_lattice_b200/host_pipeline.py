"""The op on HOST buffers: host -> device copies, filter and device -> host copies of consecutive
batch chunks overlap on a few CUDA streams (both copy engines and the SMs busy at once).  Each batch
item is an independent lattice, so chunking the batch changes no result.

The step is bound by the two copy directions (for the dense-CRF benchmark 0.8 GB in and 0.7 GB out
against 2 ms of kernels; the link carries about 47 GB/s each way when both directions run).  What the
pipeline can win or lose is the ramp: nothing flows back before the first chunk has arrived and been
filtered, nothing flows in while the last chunk's result leaves.  So the first and last chunks of a call
are single items and the ones between are larger (two items measured best: single items everywhere cost
more in small launches than they save).  Calls queued back to back (forward, then backward) share the
streams, so the flow of copies does not stop at the call boundary."""
import torch

from . import capi
from .lattice_filter import check_pending, lattice_filter_raw


class HostPipeline:
    """Reusable pipeline for one device.  `filter` takes pinned host tensors [B, *S, C] / [B, *S, R]
    and writes a pinned host tensor of the input's shape; it returns when the result is complete.
    Every stream slot owns its device buffers and its workspace."""

    def __init__(self, device=None, n_streams=4, chunk_items=2, edge_chunks=2):
        """chunk_items: items per chunk; edge_chunks: how many chunks at each end of a call are single items."""
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.streams = [torch.cuda.Stream(self.device) for _ in range(max(1, n_streams))]
        self.chunk_items = max(1, chunk_items)
        self.edge_chunks = max(0, edge_chunks)
        self._bufs = {}
        self._next_slot = 0
        self._queued = []    # calls since the last synchronize(), kept until their workspaces are known to have sufficed

    def _buf(self, slot, name, shape, dtype=torch.float32):
        key = (slot, name)
        t = self._bufs.get(key)
        if t is None or tuple(t.shape[1:]) != tuple(shape[1:]) or t.shape[0] < shape[0] or t.dtype != dtype:
            t = torch.empty(shape, dtype=dtype, device=self.device)
            self._bufs[key] = t
        return t[:shape[0]]

    def filter(self, input_host, reference_host, bilateral=True, theta_alpha=1.0, theta_beta=1.0,
               theta_gamma=1.0, reverse=False, mode="atomic", out_host=None, wait=True, copy_only=False,
               max_entries=None):
        """wait=False returns as soon as the work is queued; call `synchronize()` before reading
        out_host.  Consecutive calls may be queued back to back: they share the streams, so their
        copies and kernels keep overlapping across the call boundary.
        copy_only=True queues the same copies on the same streams without the filter between them
        (what the host link alone allows for this call; out_host then receives unspecified values).
        max_entries as in lattice_filter_raw.  With the default (workspaces sized from earlier calls) a chunk
        whose lattice outgrows its workspace is found in synchronize(), which then repeats the queued calls
        with worst-case workspaces before it returns."""
        for t, name in ((input_host, "input_host"), (reference_host, "reference_host")):
            if t is not None and (t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous()):
                raise ValueError("%s must be a contiguous float32 host tensor" % name)
        if bilateral and reference_host is None:
            raise ValueError("bilateral filtering needs reference_host")
        if out_host is None:
            out_host = torch.empty_like(input_host).pin_memory()
        batch = input_host.shape[0]
        if not copy_only and max_entries is None:
            self._queued.append((input_host, reference_host, bilateral, theta_alpha, theta_beta, theta_gamma, reverse,
                                 mode, out_host))
        main = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(main)
        for lo, hi in self.chunks(batch):
            slot = self._next_slot
            self._next_slot = (slot + 1) % len(self.streams)
            stream = self.streams[slot]
            stream.wait_event(ready)
            with torch.cuda.stream(stream):
                dx = self._buf(slot, "x", (hi - lo,) + tuple(input_host.shape[1:]))
                dx.copy_(input_host[lo:hi], non_blocking=True)
                dr = None
                if bilateral:
                    dr = self._buf(slot, "r", (hi - lo,) + tuple(reference_host.shape[1:]))
                    dr.copy_(reference_host[lo:hi], non_blocking=True)
                do = self._buf(slot, "o", (hi - lo,) + tuple(input_host.shape[1:]))
                if not copy_only:
                    lattice_filter_raw(dx, dr, bilateral, theta_alpha, theta_beta, theta_gamma, reverse, mode,
                                       out=do, max_entries=max_entries, check=False, verify="deferred",
                                       workspace_owner=("HostPipeline", id(self), slot))
                out_host[lo:hi].copy_(do, non_blocking=True)
        if wait:
            self.synchronize()
        return out_host

    def filter_forward_backward(self, input_host, grad_host, reference_host, bilateral=True, theta_alpha=1.0,
                                theta_beta=1.0, theta_gamma=1.0, mode="atomic", out_host=None, grad_out_host=None,
                                wait=True):
        """A layer's forward and backward through ONE lattice per chunk: the reference image travels to the
        device once, the lattice is built once and applied to `input_host` (reverse=False) and to `grad_host`
        (reverse=True).  Same results as two `filter` calls; the reference's own op rebuilds its lattice in
        the backward call, this is the form for callers that hold both tensors at once.
        Returns (out_host, grad_out_host)."""
        from .lattice_filter import Lattice
        for t, name in ((input_host, "input_host"), (grad_host, "grad_host"), (reference_host, "reference_host")):
            if t is not None and (t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous()):
                raise ValueError("%s must be a contiguous float32 host tensor" % name)
        if bilateral and reference_host is None:
            raise ValueError("bilateral filtering needs reference_host")
        if tuple(grad_host.shape) != tuple(input_host.shape):
            raise ValueError("grad_host must have input_host's shape")
        if out_host is None:
            out_host = torch.empty_like(input_host).pin_memory()
        if grad_out_host is None:
            grad_out_host = torch.empty_like(input_host).pin_memory()
        batch = input_host.shape[0]
        main = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(main)
        for lo, hi in self.chunks(batch):
            slot = self._next_slot
            self._next_slot = (slot + 1) % len(self.streams)
            stream = self.streams[slot]
            stream.wait_event(ready)
            shape = (hi - lo,) + tuple(input_host.shape[1:])
            with torch.cuda.stream(stream):
                dr = None
                if bilateral:
                    dr = self._buf(slot, "r", (hi - lo,) + tuple(reference_host.shape[1:]))
                    dr.copy_(reference_host[lo:hi], non_blocking=True)
                dx = self._buf(slot, "x", shape)
                dx.copy_(input_host[lo:hi], non_blocking=True)
                # worst-case workspace: building must not synchronise here (the chunks overlap)
                lattice = Lattice(dr, shape[:-1], bilateral, theta_alpha, theta_beta, theta_gamma,
                                  max_channels=shape[-1], max_entries=0, mode=mode)
                do = self._buf(slot, "o", shape)
                lattice.apply(dx, False, mode, out=do)
                out_host[lo:hi].copy_(do, non_blocking=True)
                dg = self._buf(slot, "g", shape)
                dg.copy_(grad_host[lo:hi], non_blocking=True)
                dgo = self._buf(slot, "go", shape)
                lattice.apply(dg, True, mode, out=dgo)
                grad_out_host[lo:hi].copy_(dgo, non_blocking=True)
                lattice.workspace.record_stream(stream)
        if wait:
            self.synchronize()
        return out_host, grad_out_host

    def chunks(self, batch):
        """[lo, hi) of every chunk of a `batch`-item call, in order."""
        head = min(self.edge_chunks, batch)
        tail = min(self.edge_chunks, batch - head)
        cuts = list(range(0, head)) + list(range(head, batch - tail, self.chunk_items)) + \
            list(range(batch - tail, batch)) + [batch]
        return [(cuts[i], cuts[i + 1]) for i in range(len(cuts) - 1)]

    def close(self):
        """Gives back the device buffers and the workspaces kept for this pipeline's stream slots."""
        import sys
        # (the package attribute "lattice_filter" is the function of that name: the module comes from sys.modules)
        cache = sys.modules[__package__ + ".lattice_filter"]._workspaces
        for key in [k for k in cache if isinstance(k[1], tuple) and k[1][:2] == ("HostPipeline", id(self))]:
            del cache[key]
        self._bufs.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def synchronize(self):
        for stream in self.streams:
            stream.synchronize()
        queued, self._queued = self._queued, []
        if not queued:
            return
        try:
            check_pending(wait=True)
        except capi.PlError as e:
            if e.status != capi.PL_CAPACITY_EXCEEDED:
                raise
            # some chunk's lattice did not fit the workspace sized from earlier calls (its result is NaN):
            # the calls since the last synchronize() run again with workspaces that cannot overflow
            for (x, r, bilateral, ta, tb, tg, reverse, mode, out_host) in queued:
                self.filter(x, r, bilateral, ta, tb, tg, reverse, mode, out_host=out_host, wait=False, max_entries=0)
            for stream in self.streams:
                stream.synchronize()
