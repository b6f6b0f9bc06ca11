"""Host-side mirror of the reference operator on torch CUDA tensors.

`lattice_filter(input_image, reference_image, bilateral, theta_alpha, theta_beta, theta_gamma,
reverse)` has the arguments, defaults, shapes and gradient of the `LatticeFilter` op
(src/LatticeFilterKernel.cpp:30-43, gradient lattice_filter_op_loader.py:32-54); torch supplies
device memory and streams only, every computation happens in libpl_lattice.so through its C ABI.
"""
import ctypes

import torch

from . import capi

_workspaces = {}   # (device index, owner) -> uint8 tensor, grown on demand; owner: a stream handle or a caller's key


def _workspace(device, owner, nbytes):
    key = (device.index, owner)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def release_workspaces():
    _workspaces.clear()
    _pending.clear()
    _verified.clear()


# ---------------------------------------------------------------------------------------------------
# How much workspace a call gets.  Everything indexed by lattice entry or by vertex is sized from
# `max_entries`; the bound that can never overflow, batch * points * (pd + 1), is 1.5 to 40 times what the
# benchmark configurations use.  So by default (max_entries=None) a call is sized from what the lattice needs:
#   * a call whose reference image (or positions) is the tensor a VERIFIED call of the same kind just used
#     - same memory, same version counter, same shape: a layer's backward call, the next iteration on the same
#     image - builds the same lattice, so it runs with that call's bound and nothing needs checking;
#   * any other call is VERIFIED: it runs with 1.5 x the largest entry count per item seen for its kind (a
#     quarter of the worst case the first time), the stream is synchronised and the device status read, and
#     the call is repeated with four times the bound as long as the lattice did not fit.  One
#     synchronisation per new reference image.
# Callers that own a synchronisation point of their own (HostPipeline) ask for verify="deferred" instead: the
# call's counters are copied to pinned host memory behind it and looked at in check_pending(); a call that did
# not fit has filled its output with NaN, and the caller repeats it.
# max_entries=0 asks for the worst case (never overflows, never synchronises), max_entries > 0 for that bound.
# ---------------------------------------------------------------------------------------------------
_entries_per_item = {}   # kind of call -> largest num_entries / batch seen
_verified = {}           # kind of call -> (identity of the reference it ran on, the bound that sufficed)
_pending = {}            # kind of call -> list of (event, pinned int32[3] = entries, vertices, status bits, bound, batch)
_pinned_words = []       # pinned int32[3] buffers waiting to be used again (allocating pinned memory is slow)
FIRST_GUESS_DIVISOR = 4
HEADROOM = 1.5


def _kind(device, call, from_positions=False):
    return (device.index, tuple(call.sdims), call.pd, call.bilateral, call.theta, bool(from_positions))


def _identity(t, batch):
    """What makes two calls build the same lattice, as far as the host can tell: the same tensor (memory,
    shape) that no torch operation has written to in between (version counter)."""
    if t is None:
        return ("grid", batch)
    return (t.data_ptr(), t._version, tuple(t.shape), t.dtype)


def _status_code(bits):
    code = capi.PL_OK
    for c in range(capi.PL_INVALID_ARGUMENT, capi.PL_INTERNAL_ERROR + 1):
        if bits & (1 << c):
            code = c
    return code


def _look_at(kind, entry):
    """Takes a finished call's counters into account; raises if that call did not fit its bound."""
    _, host, bound, batch = entry
    entries, _, bits = (int(v) for v in host.tolist())
    _pinned_words.append(host)
    code = _status_code(bits)
    if code == capi.PL_CAPACITY_EXCEEDED:
        # the count stops at the first tile that did not fit: all that is known is "more than the bound"
        _entries_per_item[kind] = max(_entries_per_item.get(kind, 0.0), 2.0 * bound / max(batch, 1))
        raise capi.PlError(code, "a lattice filter call outgrew its workspace (bound %d entries); its output holds "
                                 "NaN.  The bound has been raised: repeat the call" % bound)
    if code != capi.PL_OK:
        raise capi.PlError(code, "a lattice filter call (device)")
    _entries_per_item[kind] = max(_entries_per_item.get(kind, 0.0), entries / max(batch, 1))


def check_pending(wait=True):
    """Looks at the counters of every call made with verify="deferred" that has not been looked at yet;
    wait=True synchronises with those calls first.  Raises PlError if one of them outgrew its workspace."""
    first_error = None
    for kind in list(_pending):
        keep = []
        for entry in _pending[kind]:
            if wait:
                entry[0].synchronize()
            if entry[0].query():
                try:
                    _look_at(kind, entry)
                except capi.PlError as e:
                    first_error = first_error or e
            else:
                keep.append(entry)
        _pending[kind] = keep
    if first_error is not None:
        raise first_error


def _guess_bound(kind, batch, worst, floor=0):
    """max_entries for a call whose lattice is not known yet; `floor`: a bound below which the call would lose
    something else (the direct index of a spatial-only call).  0 = the worst case."""
    per_item = _entries_per_item.get(kind)
    if per_item is None:
        bound = max(worst // FIRST_GUESS_DIVISOR, min(worst, 4096), floor)
    else:
        bound = max(int(HEADROOM * per_item * batch) + 4096, floor)
    return 0 if bound >= worst else bound


def _direct_index_floor(call):
    """Spatial-only calls index their vertices directly when the dense index fits the workspace's table
    region, whose size follows max_entries: the bound below which such a call would fall back to hashing."""
    if call.bilateral:
        return 0
    need = ctypes.c_int64(0)
    capi.check(capi.lib().pl_direct_index_min_entries(call.batch, len(call.sdims), capi.int_array(call.sdims),
                                                      call.spatial_std, ctypes.byref(need)),
               "pl_direct_index_min_entries")
    return int(need.value)


def _note_call(kind, ws, bound, batch, device):
    """Queues the copy of the call's counters (first 12 bytes of the workspace) behind it."""
    host = _pinned_words.pop() if _pinned_words else torch.empty(3, dtype=torch.int32).pin_memory()
    host.copy_(ws[:12].view(torch.int32), non_blocking=True)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(device))
    _pending.setdefault(kind, []).append((ev, host, bound, batch))


def _run_sized(kind, identity, batch, worst, device, stream, launch, verify="auto", floor=0):
    """Runs launch(max_entries) -> workspace under the default sizing policy.  Returns (workspace, max_entries)."""
    if verify == "deferred":
        max_entries = _guess_bound(kind, batch, worst, floor)
        ws = launch(max_entries)
        if max_entries:
            _note_call(kind, ws, max_entries, batch, device)
        return ws, max_entries
    known = _verified.get(kind)
    if known is not None and known[0] == identity:
        return launch(known[1]), known[1]          # the same lattice as a call that fitted this bound
    max_entries = _guess_bound(kind, batch, worst, floor)
    repeated = False
    while True:
        ws = launch(max_entries)
        if max_entries == 0:                       # the worst case cannot overflow: nothing to verify
            if repeated:                           # (but what the lattice needed is worth knowing for the next call)
                st = lattice_stats(ws, stream)
                _entries_per_item[kind] = max(_entries_per_item.get(kind, 0.0), st.num_entries / max(batch, 1))
            break
        repeated = True
        st = lattice_stats(ws, stream)
        if st.device_status == capi.PL_CAPACITY_EXCEEDED:
            grown = max_entries * FIRST_GUESS_DIVISOR
            max_entries = 0 if grown >= worst else grown
            continue
        if st.device_status != capi.PL_OK:
            raise capi.PlError(st.device_status, "lattice filter (device)")
        _entries_per_item[kind] = max(_entries_per_item.get(kind, 0.0), st.num_entries / max(batch, 1))
        break
    _verified[kind] = (identity, max_entries)
    return ws, max_entries


def _stream_handle(device):
    return torch.cuda.current_stream(device).cuda_stream


def _check_tensor(t, name, dtype=None):
    """float32 or float64 (the two types the reference registers its op for,
    src/LatticeFilterKernel.cpp:196-197,207-208); `dtype` pins it to another tensor's."""
    if not t.is_cuda:
        raise ValueError("%s must be a CUDA tensor (there is no CPU path in this package)" % name)
    if t.dtype not in (torch.float32, torch.float64):
        raise TypeError("%s must be float32 or float64" % name)
    if dtype is not None and t.dtype != dtype:
        raise TypeError("%s must have dtype %s like the other operand" % (name, dtype))


def _float32_only(t, what):
    if t is not None and t.dtype != torch.float32:
        raise TypeError("%s is available for float32 only" % what)


class FilterCall:
    """Geometry of one op call; keeps what pl_export_lattice needs to be given again."""

    def __init__(self, input_shape, reference_shape, bilateral, theta_alpha, theta_beta,
                 theta_gamma):
        if len(input_shape) < 3:
            raise ValueError("input_image must be [batch, *spatial, channels]")
        self.batch = int(input_shape[0])
        self.sdims = [int(s) for s in input_shape[1:-1]]
        self.n = 1
        for s in self.sdims:
            self.n *= s
        self.c = int(input_shape[-1])
        self.bilateral = bool(bilateral)
        if self.bilateral:
            if reference_shape is None or list(reference_shape[:-1]) != list(input_shape[:-1]):
                raise ValueError("reference_image must match input_image in batch and spatial dims")
            self.r = int(reference_shape[-1])
            self.spatial_std, self.feature_std = float(theta_alpha), float(theta_beta)
        else:
            self.r = 0
            self.spatial_std, self.feature_std = float(theta_gamma), -1.0
        self.pd = len(self.sdims) + self.r
        self.vd = self.c + 1
        self.theta = (float(theta_alpha), float(theta_beta), float(theta_gamma))
        self.max_entries = 0   # the bound the last call on this geometry ran with (0: worst case)

    def workspace_bytes(self, max_entries=0, dtype=torch.float32, mode="atomic"):
        nbytes = ctypes.c_size_t(0)
        head = (self.batch, self.n, self.pd, self.vd, len(self.sdims), capi.int_array(self.sdims), int(max_entries))
        if dtype == torch.float64:
            rc = capi.lib().pl_workspace_bytes_f64(*head, ctypes.byref(nbytes))
        else:
            rc = capi.lib().pl_workspace_bytes(*head, capi.MODES[mode], ctypes.byref(nbytes))
        capi.check(rc, "pl_workspace_bytes")
        return nbytes.value


def lattice_filter_raw(input_image, reference_image, bilateral=True, theta_alpha=1.0,
                       theta_beta=1.0, theta_gamma=1.0, reverse=False, mode="atomic",
                       max_entries=None, check=None, workspace=None, out=None, workspace_owner=None,
                       verify="auto"):
    """One call of pl_lattice_filter_f32 (or _f64, by the tensors' dtype) on the current stream.
    Returns (output, workspace, call).  max_entries: None sizes the workspace from what the lattice needs
    (see above; verify="deferred" for callers that check later), 0 for the worst case, > 0 is the caller's
    own bound (verified: synchronises).  workspace: a buffer of the caller's (worst case unless max_entries
    says otherwise); workspace_owner: a key under which this caller's workspace is kept apart from everybody
    else's (default: the stream).  The workspace returned holds this call's lattice until the next call that
    uses it (pl_lattice_stats, export_lattice)."""
    _check_tensor(input_image, "input_image")
    x = input_image.contiguous()
    f64 = x.dtype == torch.float64
    if f64 and mode != "atomic":
        raise TypeError("mode=%r is available for float32 only" % mode)
    ref = None
    if bilateral:
        _check_tensor(reference_image, "reference_image", x.dtype)
        ref = reference_image.contiguous()
    call = FilterCall(tuple(x.shape), None if ref is None else tuple(ref.shape), bilateral,
                      theta_alpha, theta_beta, theta_gamma)
    if not capi.lib().pl_supported(call.pd, call.vd):
        raise capi.PlError(capi.PL_UNSUPPORTED_DIMS, "lattice_filter(pd=%d, vd=%d)" % (call.pd, call.vd))
    if out is None:
        out = torch.empty_like(x)
    if call.batch == 0 or call.n == 0:
        return out, None, call
    stream = _stream_handle(x.device)
    owner = stream if workspace_owner is None else workspace_owner
    worst = call.batch * call.n * (call.pd + 1)

    def launch(bound):
        nbytes = call.workspace_bytes(bound, x.dtype, mode)
        ws = workspace if workspace is not None else _workspace(x.device, owner, nbytes)
        head = (out.data_ptr(), x.data_ptr(), 0 if ref is None else ref.data_ptr(), call.batch,
                len(call.sdims), capi.int_array(call.sdims), call.c, call.r, int(call.bilateral),
                call.theta[0], call.theta[1], call.theta[2], int(bool(reverse)), ws.data_ptr(),
                ws.numel(), int(bound))
        if f64:
            capi.check(capi.lib().pl_lattice_filter_f64(*head, stream), "pl_lattice_filter_f64")
        else:
            capi.check(capi.lib().pl_lattice_filter_f32(*head, capi.MODES[mode], stream),
                       "pl_lattice_filter_f32")
        return ws

    with torch.cuda.device(x.device):
        if max_entries is None and workspace is None:
            ws, max_entries = _run_sized(_kind(x.device, call), _identity(reference_image if bilateral else None,
                                                                          call.batch),
                                         call.batch, worst, x.device, stream, launch, verify=verify,
                                         floor=_direct_index_floor(call))
        else:
            max_entries = int(max_entries or 0)
            ws = launch(max_entries)
            if check is None:
                check = max_entries > 0
            if check:
                st = lattice_stats(ws, stream)
                if st.device_status != capi.PL_OK:
                    raise capi.PlError(st.device_status, "lattice_filter (device)")
    call.max_entries = max_entries     # what pl_export_lattice must be told again
    return out, ws, call


def lattice_stats(workspace, stream=None, device=None):
    """Counters of the last call that used `workspace` (synchronises the stream).  workspace=None reads
    those of the last pl_lattice_filter_f32_noalloc call on `device` (default: the current one)."""
    st = capi.PlStats()
    if workspace is not None:
        device = workspace.device
    elif device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if stream is None:
        stream = _stream_handle(device)
    with torch.cuda.device(device):
        capi.check(capi.lib().pl_lattice_stats(0 if workspace is None else workspace.data_ptr(),
                                               ctypes.byref(st), stream), "pl_lattice_stats")
    return st


class Lattice:
    """A lattice built once and applied many times (pl_lattice_build_f32 / pl_lattice_apply_f32).

    The reference rebuilds its lattice on every call; its main user, CRF mean-field inference, filters
    many tensors through the same reference image (forward, backward, every iteration).  `Lattice`
    keeps the structure (entries, vertices, neighbour table, per-point records) in a workspace of its
    own and only splats, blurs and slices per call."""

    def __init__(self, reference_image, spatial_shape=None, bilateral=True, theta_alpha=1.0, theta_beta=1.0,
                 theta_gamma=1.0, max_channels=1, max_entries=None, mode="atomic"):
        """reference_image [B, *S, R] (bilateral) — or None with spatial_shape = (B, *S) for a purely
        spatial kernel.  max_channels: the widest input that will be applied.  mode: "deterministic"
        sizes the workspace for `apply(..., mode="deterministic")` too (it then serves both modes).
        max_entries: None sizes the workspace from what the lattice needs and verifies that it fits (building
        synchronises once per reference image; a lattice that does not fit is rebuilt with a larger bound), 0
        is the worst case (never synchronises), > 0 the caller's own bound (verified)."""
        _float32_only(reference_image, "Lattice (build once, apply many times)")
        if bilateral:
            _check_tensor(reference_image, "reference_image")
            ref = reference_image.contiguous()
            shape = tuple(ref.shape[:-1])
            device = ref.device
        else:
            ref = None
            shape = tuple(spatial_shape if spatial_shape is not None else reference_image.shape[:-1])
            device = reference_image.device if reference_image is not None else torch.device(
                "cuda", torch.cuda.current_device())
        self.call = FilterCall(shape + (int(max_channels),), None if ref is None else tuple(ref.shape), bilateral,
                               theta_alpha, theta_beta, theta_gamma)
        self.device = device
        call = self.call
        if not capi.lib().pl_supported(call.pd, call.vd):
            raise capi.PlError(capi.PL_UNSUPPORTED_DIMS, "Lattice(pd=%d, vd=%d)" % (call.pd, call.vd))
        self.workspace = None
        self.max_entries = int(max_entries or 0)
        if call.batch == 0 or call.n == 0:
            return
        stream = _stream_handle(device)

        def build(bound):
            ws = torch.empty(call.workspace_bytes(bound, mode=mode), dtype=torch.uint8, device=device)
            capi.check(capi.lib().pl_lattice_build_f32(
                0 if ref is None else ref.data_ptr(), call.batch, len(call.sdims), capi.int_array(call.sdims),
                call.r, int(call.bilateral), call.theta[0], call.theta[1], call.theta[2], call.vd,
                ws.data_ptr(), ws.numel(), int(bound), stream), "pl_lattice_build_f32")
            return ws

        with torch.cuda.device(device):
            if max_entries is None:
                worst = call.batch * call.n * (call.pd + 1)
                # verified like a filter call: once per reference image, not again for a lattice rebuilt on it
                self.workspace, self.max_entries = _run_sized(
                    ("Lattice",) + _kind(device, call), _identity(reference_image if bilateral else None, call.batch),
                    call.batch, worst, device, stream, build, floor=_direct_index_floor(call))
            else:
                self.workspace = build(self.max_entries)
                if self.max_entries > 0:   # a bound chosen by the caller may be too small: known on the device only
                    st = lattice_stats(self.workspace)
                    if st.device_status != capi.PL_OK:
                        raise capi.PlError(st.device_status, "Lattice (device, max_entries=%d)" % self.max_entries)
        call.max_entries = self.max_entries

    def apply(self, input_image, reverse=False, mode="atomic", out=None):
        """Filters input_image [B, *S, C] (C <= max_channels) through the lattice."""
        _check_tensor(input_image, "input_image")
        _float32_only(input_image, "Lattice (build once, apply many times)")
        x = input_image.contiguous()
        call = self.call
        if tuple(x.shape[:-1]) != (call.batch,) + tuple(call.sdims):
            raise ValueError("input_image does not have the lattice's batch and spatial shape")
        if x.shape[-1] + 1 > call.vd:
            raise ValueError("input_image has more channels than the lattice was built for")
        if out is None:
            out = torch.empty_like(x)
        if self.workspace is None:
            return out
        with torch.cuda.device(self.device):
            capi.check(capi.lib().pl_lattice_apply_f32(
                out.data_ptr(), x.data_ptr(), x.shape[-1], int(bool(reverse)), capi.MODES[mode], call.batch,
                call.n, call.pd, len(call.sdims), capi.int_array(call.sdims), self.workspace.data_ptr(),
                self.workspace.numel(), self.max_entries, _stream_handle(self.device)), "pl_lattice_apply_f32")
        return out

    def stats(self):
        return lattice_stats(self.workspace)


class _LatticeFilterReuseFunction(torch.autograd.Function):
    """forward builds the lattice and keeps it for backward, which only applies it (reverse=True)."""

    @staticmethod
    def forward(ctx, input_image, reference_image, bilateral, theta_alpha, theta_beta, theta_gamma, reverse,
                mode):
        lattice = Lattice(reference_image, tuple(input_image.shape[:-1]), bilateral, theta_alpha, theta_beta,
                          theta_gamma, max_channels=input_image.shape[-1], mode=mode)
        ctx.lattice, ctx.mode = lattice, mode
        ctx.save_for_backward(reference_image)   # autograd's version check guards against in-place edits
        return lattice.apply(input_image, reverse, mode)

    @staticmethod
    def backward(ctx, grad):
        (reference_image,) = ctx.saved_tensors
        g = ctx.lattice.apply(grad, True, ctx.mode)
        ref_grad = torch.zeros_like(reference_image) if reference_image is not None else None
        return g, ref_grad, None, None, None, None, None, None


class _LatticeFilterFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input_image, reference_image, bilateral, theta_alpha, theta_beta, theta_gamma,
                reverse, mode):
        ctx.args = (bilateral, theta_alpha, theta_beta, theta_gamma, mode)
        ctx.save_for_backward(reference_image)
        out, _, _ = lattice_filter_raw(input_image, reference_image, bilateral, theta_alpha,
                                       theta_beta, theta_gamma, reverse, mode)
        return out

    @staticmethod
    def backward(ctx, grad):
        # lattice_filter_op_loader.py:32-54: the gradient w.r.t. the input is the same filter applied
        # to the upstream gradient with reverse=True; the reference image gets zeros.
        (reference_image,) = ctx.saved_tensors
        bilateral, theta_alpha, theta_beta, theta_gamma, mode = ctx.args
        g, _, _ = lattice_filter_raw(grad, reference_image, bilateral, theta_alpha, theta_beta,
                                     theta_gamma, True, mode)
        ref_grad = torch.zeros_like(reference_image) if reference_image is not None else None
        return g, ref_grad, None, None, None, None, None, None


def lattice_filter(input_image, reference_image, bilateral=True, theta_alpha=1.0, theta_beta=1.0,
                   theta_gamma=1.0, reverse=False, mode="atomic", reuse_lattice=False):
    """output[B, *S, C] = permutohedral-lattice filter of input_image[B, *S, C] guided by
    reference_image[B, *S, R] (bilateral) or by position only (bilateral=False, theta_gamma).
    reuse_lattice=True keeps the lattice built in forward for the backward pass instead of rebuilding
    it there (same results; the reference always rebuilds).
    The thetas are float attributes of the op (src/LatticeFilterKernel.cpp:36-38): they are rounded to
    float32 here and widened again for float64 tensors, as the reference does (:131-142)."""
    fn = _LatticeFilterReuseFunction if reuse_lattice else _LatticeFilterFunction
    as_attr = lambda v: ctypes.c_float(float(v)).value
    return fn.apply(input_image, reference_image, bool(bilateral), as_attr(theta_alpha), as_attr(theta_beta),
                    as_attr(theta_gamma), bool(reverse), mode)


def compute_positions(reference_image, spatial_dims, spatial_std, feature_std, dtype=None):
    """positions[n, n_sdims + R] for one item: the ComputeKernel functor
    (src/LatticeFilterKernel.h:40-54).  reference_image [n, R] or None; dtype (default: the reference
    image's, else float32) selects the float or double functor."""
    sdims = [int(s) for s in spatial_dims]
    n = 1
    for s in sdims:
        n *= s
    if reference_image is not None:
        _check_tensor(reference_image, "reference_image")
        ref = reference_image.contiguous().view(n, -1)
        r, device = ref.shape[1], ref.device
        dtype = ref.dtype if dtype is None else dtype
        _check_tensor(ref, "reference_image", dtype)
    else:
        ref, r, device = None, 0, torch.device("cuda", torch.cuda.current_device())
        dtype = torch.float32 if dtype is None else dtype
    pos = torch.empty((n, len(sdims) + r), dtype=dtype, device=device)
    fn = capi.lib().pl_compute_positions_f64 if dtype == torch.float64 else capi.lib().pl_compute_positions_f32
    with torch.cuda.device(device):
        capi.check(fn(0 if ref is None else ref.data_ptr(), pos.data_ptr(), n, r, len(sdims),
                      capi.int_array(sdims), float(spatial_std), float(feature_std), _stream_handle(device)),
                   "pl_compute_positions")
    return pos


def filter_positions(input_values, positions, reverse=False, mode="atomic", max_entries=None,
                     check=None, workspace=None, out=None, info=None):
    """The LatticeFilter functor (src/LatticeFilterKernel.h:28-38) on [batch, n, C] values at
    [batch, n, pd] positions (2-D tensors are taken as batch 1).  Returns (output, workspace).
    max_entries as in lattice_filter_raw; `info`, a dict, receives the bound the call ran with
    (info["max_entries"], to be given again to export_lattice)."""
    _check_tensor(input_values, "input_values")
    _check_tensor(positions, "positions", input_values.dtype)
    f64 = input_values.dtype == torch.float64
    if f64 and mode != "atomic":
        raise TypeError("mode=%r is available for float32 only" % mode)
    squeeze = input_values.dim() == 2
    x = input_values.contiguous().view((1,) + tuple(input_values.shape)) if squeeze else input_values.contiguous()
    p = positions.contiguous().view((1,) + tuple(positions.shape)) if squeeze else positions.contiguous()
    batch, n, c = x.shape
    pd = p.shape[-1]
    if tuple(p.shape[:2]) != (batch, n):
        raise ValueError("positions must be [batch, n, pd] matching input_values")
    vd = c + 1
    if out is None:
        out = torch.empty_like(x)
    elif tuple(out.shape) != tuple(x.shape) or out.dtype != x.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous tensor of the input's shape and dtype")
    ws = None
    if batch and n:
        stream = _stream_handle(x.device)

        def launch(bound):
            nbytes = ctypes.c_size_t(0)
            if f64:
                rc = capi.lib().pl_workspace_bytes_f64(batch, n, pd, vd, 0, None, int(bound), ctypes.byref(nbytes))
            else:
                rc = capi.lib().pl_workspace_bytes(batch, n, pd, vd, 0, None, int(bound), capi.MODES[mode],
                                                   ctypes.byref(nbytes))
            capi.check(rc, "pl_workspace_bytes")
            w = workspace if workspace is not None else _workspace(x.device, stream, nbytes.value)
            head = (out.data_ptr(), x.data_ptr(), p.data_ptr(), batch, n, pd, vd, int(bool(reverse)),
                    w.data_ptr(), w.numel(), int(bound))
            if f64:
                capi.check(capi.lib().pl_filter_f64(*head, stream), "pl_filter_f64")
            else:
                capi.check(capi.lib().pl_filter_f32(*head, capi.MODES[mode], stream), "pl_filter_f32")
            return w

        with torch.cuda.device(x.device):
            if max_entries is None and workspace is None:
                kind = (x.device.index, "positions", n, pd)
                ws, max_entries = _run_sized(kind, _identity(positions, batch), batch, batch * n * (pd + 1), x.device,
                                             stream, launch)
            else:
                max_entries = int(max_entries or 0)
                ws = launch(max_entries)
                if check is None:
                    check = max_entries > 0
                if check:
                    st = lattice_stats(ws, stream)
                    if st.device_status != capi.PL_OK:
                        raise capi.PlError(st.device_status, "filter_positions (device)")
        if info is not None:
            info["max_entries"] = max_entries
    return (out[0] if squeeze else out), ws


def export_lattice(workspace, stats, batch, n, pd, vd, positions=None, reference=None, sdims=None,
                   spatial_std=1.0, feature_std=1.0, max_entries=None, dtype=None):
    """Lattice structure of the last call on `workspace` as torch tensors:
    (vertex_keys [M, pd] int16, vertex_item [M] int32, pixel_vertex [batch, n, pd+1] int32,
    pixel_weight [batch, n, pd+1] in the call's number type).  dtype: that call's number type; by
    default the one of positions / reference, else float32."""
    device = workspace.device
    if max_entries is None:
        max_entries = int(stats.max_entries)   # the bound that call ran with (the workspace's layout depends on it)
    if dtype is None:
        given = positions if positions is not None else reference
        dtype = given.dtype if given is not None else torch.float32
    fn = capi.lib().pl_export_lattice_f64 if dtype == torch.float64 else capi.lib().pl_export_lattice
    m = int(stats.num_vertices)
    vkeys = torch.zeros((m, pd), dtype=torch.int16, device=device)
    vitem = torch.zeros((m,), dtype=torch.int32, device=device)
    pv = torch.zeros((batch, n, pd + 1), dtype=torch.int32, device=device)
    pw = torch.zeros((batch, n, pd + 1), dtype=dtype, device=device)
    with torch.cuda.device(device):
        if positions is not None:
            rc = fn(workspace.data_ptr(), positions.contiguous().data_ptr(), 0,
                    batch, n, pd, vd, 0, None, 0, 1.0, 1.0, int(max_entries),
                    m, vkeys.data_ptr(), vitem.data_ptr(), pv.data_ptr(),
                    pw.data_ptr(), _stream_handle(device))
        else:
            r = pd - len(sdims)
            rc = fn(workspace.data_ptr(), 0,
                    0 if reference is None else reference.contiguous().data_ptr(),
                    batch, n, pd, vd, len(sdims), capi.int_array(sdims), r,
                    float(spatial_std), float(feature_std), int(max_entries),
                    m, vkeys.data_ptr(), vitem.data_ptr(), pv.data_ptr(),
                    pw.data_ptr(), _stream_handle(device))
        capi.check(rc, "pl_export_lattice")
    return vkeys, vitem, pv, pw
