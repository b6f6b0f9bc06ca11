"""The op captured once in a CUDA graph and replayed: for small problems the dozen kernel launches of
a call cost more than the kernels, and a graph replay issues them with one launch."""
import torch

from .lattice_filter import FilterCall, lattice_filter_raw


class GraphedLatticeFilter:
    """Fixed shapes and parameters; `input`, `reference` and `output` are static device tensors the
    caller fills and reads, `replay()` runs the captured call on the current stream."""

    def __init__(self, input_shape, reference_shape=None, bilateral=True, theta_alpha=1.0, theta_beta=1.0,
                 theta_gamma=1.0, reverse=False, mode="atomic", device=None):
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.input = torch.zeros(tuple(input_shape), dtype=torch.float32, device=device)
        self.reference = None if reference_shape is None else torch.zeros(tuple(reference_shape),
                                                                          dtype=torch.float32, device=device)
        self.output = torch.empty_like(self.input)
        args = (bilateral, theta_alpha, theta_beta, theta_gamma, reverse, mode)
        # The graph owns its workspace: the addresses baked into the captured launches must never be
        # handed to another caller, as a workspace taken from the shared per-stream cache could be.
        call = FilterCall(tuple(input_shape), None if reference_shape is None else tuple(reference_shape), bilateral,
                          theta_alpha, theta_beta, theta_gamma)
        with torch.cuda.device(device):
            self._workspace = torch.empty(max(1, call.workspace_bytes(mode=mode)), dtype=torch.uint8, device=device)
        # one ordinary call first: sets kernel attributes outside the capture
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            lattice_filter_raw(self.input, self.reference, *args, out=self.output, workspace=self._workspace)
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            lattice_filter_raw(self.input, self.reference, *args, out=self.output, workspace=self._workspace)

    def replay(self):
        self.graph.replay()
        return self.output
