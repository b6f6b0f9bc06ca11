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

from .lattice_filter import FilterCall, lattice_filter_raw


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

    def _buf(self, slot, name, shape, dtype=torch.float32):
        key = (slot, name)
        t = self._bufs.get(key)
        if t is None or tuple(t.shape[1:]) != tuple(shape[1:]) or t.shape[0] < shape[0] or t.dtype != dtype:
            t = torch.empty(shape, dtype=dtype, device=self.device)
            self._bufs[key] = t
        return t[:shape[0]]

    def _workspace(self, slot, call, mode):
        need = call.workspace_bytes(mode=mode)
        ws = self._bufs.get((slot, "ws"))
        if ws is None or ws.numel() < need:
            ws = torch.empty(need, dtype=torch.uint8, device=self.device)
            self._bufs[(slot, "ws")] = ws
        return ws

    def filter(self, input_host, reference_host, bilateral=True, theta_alpha=1.0, theta_beta=1.0,
               theta_gamma=1.0, reverse=False, mode="atomic", out_host=None, wait=True, copy_only=False):
        """wait=False returns as soon as the work is queued; call `synchronize()` before reading
        out_host.  Consecutive calls may be queued back to back: they share the streams, so their
        copies and kernels keep overlapping across the call boundary.
        copy_only=True queues the same copies on the same streams without the filter between them
        (what the host link alone allows for this call; out_host then receives unspecified values)."""
        for t, name in ((input_host, "input_host"), (reference_host, "reference_host")):
            if t is not None and (t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous()):
                raise ValueError("%s must be a contiguous float32 host tensor" % name)
        if bilateral and reference_host is None:
            raise ValueError("bilateral filtering needs reference_host")
        if out_host is None:
            out_host = torch.empty_like(input_host).pin_memory()
        batch = input_host.shape[0]
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
                    call = FilterCall(tuple(dx.shape), None if dr is None else tuple(dr.shape), bilateral,
                                      theta_alpha, theta_beta, theta_gamma)
                    lattice_filter_raw(dx, dr, bilateral, theta_alpha, theta_beta, theta_gamma, reverse, mode,
                                       out=do, workspace=self._workspace(slot, call, mode))
                out_host[lo:hi].copy_(do, non_blocking=True)
        if wait:
            self.synchronize()
        return out_host

    def chunks(self, batch):
        """[lo, hi) of every chunk of a `batch`-item call, in order."""
        head = min(self.edge_chunks, batch)
        tail = min(self.edge_chunks, batch - head)
        cuts = list(range(0, head)) + list(range(head, batch - tail, self.chunk_items)) + \
            list(range(batch - tail, batch)) + [batch]
        return [(cuts[i], cuts[i + 1]) for i in range(len(cuts) - 1)]

    def synchronize(self):
        for stream in self.streams:
            stream.synchronize()
