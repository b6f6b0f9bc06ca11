"""ctypes front end of the test-only CPU oracles (checker and timed CPU baseline).

Two interchangeable implementations behind one interface:
  impl="port"       oracle/libpl_oracle.so, the C restatement (always available)
  impl="reference"  oracle/_ref/libpl_ref.so, the unmodified reference header behind a shim
                    (available where it was built; its hash table is pre-sized so it never grows,
                    unless as_shipped=True)

Only tests, the smoke check and the benchmark's CPU-baseline legs may import this module.
"""
import ctypes
import os
from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import build as _build

_c_float_p = ctypes.POINTER(ctypes.c_float)
_c_double_p = ctypes.POINTER(ctypes.c_double)
_c_int_p = ctypes.POINTER(ctypes.c_int)
_c_short_p = ctypes.POINTER(ctypes.c_short)
_libs = {}


def _kind(dtype):
    """(numpy dtype, symbol suffix, ctypes pointer type, ctypes scalar type) of a number type."""
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return dtype, "", _c_float_p, ctypes.c_float
    if dtype == np.float64:
        return dtype, "_f64", _c_double_p, ctypes.c_double
    raise TypeError(f"oracle: unsupported dtype {dtype}")


def _fp(a):
    return a.ctypes.data_as(_c_double_p if a.dtype == np.float64 else _c_float_p)


def _declare(lib, pre, reference):
    """argtypes of one library's entry points, float and double."""
    for dtype in (np.float32, np.float64):
        _, sfx, ptr, scalar = _kind(dtype)
        f = getattr(lib, f"{pre}_filter{sfx}")
        f.restype = ctypes.c_void_p
        f.argtypes = [ptr, ptr, ptr, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int] + (
            [ctypes.c_longlong] if reference else [])
        getattr(lib, f"{pre}_num_vertices{sfx}").argtypes = [ctypes.c_void_p]
        getattr(lib, f"{pre}_keys{sfx}").argtypes = [ctypes.c_void_p, _c_short_p]
        getattr(lib, f"{pre}_matrix{sfx}").argtypes = [ctypes.c_void_p, _c_int_p, ptr]
        getattr(lib, f"{pre}_free{sfx}").argtypes = [ctypes.c_void_p]
        getattr(lib, f"{pre}_compute_positions{sfx}").argtypes = [
            ptr, ptr, ctypes.c_int, ctypes.c_int, ctypes.c_int, _c_int_p, scalar, scalar]
        f = getattr(lib, f"{pre}_filter_batch{sfx}")
        f.restype = ctypes.c_double
        f.argtypes = [ptr, ptr, ptr, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                      ctypes.c_int, _c_int_p, scalar, scalar, ctypes.c_int] + (
            [ctypes.c_longlong] if reference else []) + [ctypes.c_int]
        if reference:
            getattr(lib, f"{pre}_never_grew{sfx}").argtypes = [ctypes.c_void_p]
        else:
            getattr(lib, f"{pre}_scale_factors{sfx}").argtypes = [ctypes.c_int, ptr]


def _load_port():
    if "port" not in _libs:
        so = _build.ORACLE_SO
        if not os.path.exists(so):
            so = _build.build_oracle()
        lib = ctypes.CDLL(so)
        _declare(lib, "plo", reference=False)
        _libs["port"] = lib
    return _libs["port"]


def reference_available() -> bool:
    return os.path.exists(_build.REF_SO) or _build.reference_root() is not None


def _load_reference():
    if "reference" not in _libs:
        so = _build.REF_SO if os.path.exists(_build.REF_SO) else _build.build_reference()
        if so is None:
            raise RuntimeError("reference oracle library is not built and the reference tree is absent")
        lib = ctypes.CDLL(so)
        _declare(lib, "plref", reference=True)
        _libs["reference"] = lib
    return _libs["reference"]


@dataclass
class LatticeResult:
    out: np.ndarray                      # [n, C], the call's number type
    num_vertices: int = 0                # distinct lattice vertices
    keys: Optional[np.ndarray] = None    # [M, pd] int16, creation order
    pix_vertex: Optional[np.ndarray] = None  # [n, pd+1] int32
    pix_weight: Optional[np.ndarray] = None  # [n, pd+1], the call's number type

    def pixel_keys(self):
        """[n, pd+1, pd] int16: the keys of each pixel's enclosing-simplex vertices."""
        return self.keys[self.pix_vertex]


def scale_factors(pd: int, dtype=np.float32) -> np.ndarray:
    dtype, sfx, _, _ = _kind(dtype)
    out = np.zeros(pd, dtype)
    getattr(_load_port(), "plo_scale_factors" + sfx)(pd, _fp(out))
    return out


def compute_positions(reference, sdims, spatial_std, feature_std, impl="port", dtype=np.float32):
    """Feature vectors [n, n_sdims + R]; reference is [n, R] (R may be 0) or None."""
    dtype, sfx, _, _ = _kind(dtype)
    sdims = np.ascontiguousarray(sdims, np.int32)
    n = int(np.prod(sdims))
    if reference is None:
        reference = np.zeros((n, 0), dtype)
    reference = np.ascontiguousarray(reference, dtype).reshape(n, -1)
    r = reference.shape[1]
    pos = np.empty((n, len(sdims) + r), dtype)
    sd = sdims.ctypes.data_as(_c_int_p)
    if impl == "port":
        fn = getattr(_load_port(), "plo_compute_positions" + sfx)
    else:
        fn = getattr(_load_reference(), "plref_compute_positions" + sfx)
    fn(_fp(reference), _fp(pos), n, r, len(sdims), sd, spatial_std, feature_std)
    return pos


def filter(inp, positions, reverse=False, structure=True, impl="port", as_shipped=False,
           dtype=np.float32):
    """One lattice filter call on [n, C] values at [n, pd] positions."""
    dtype, sfx, _, _ = _kind(dtype)
    inp = np.ascontiguousarray(inp, dtype)
    positions = np.ascontiguousarray(positions, dtype)
    n, c = inp.shape
    pd = positions.shape[1]
    assert positions.shape[0] == n
    vd = c + 1
    out = np.empty((n, c), dtype)
    if impl == "port":
        lib = _load_port()
        h = getattr(lib, "plo_filter" + sfx)(_fp(out), _fp(inp), _fp(positions), n, pd, vd,
                                             int(reverse))
        if not h:
            raise ValueError("oracle: unsupported sizes")
        pre = "plo"
    else:
        lib = _load_reference()
        pre = "plref"
        run = getattr(lib, "plref_filter" + sfx)
        if as_shipped:
            h = run(_fp(out), _fp(inp), _fp(positions), n, pd, vd, int(reverse), 0)
        else:
            # first pass as shipped only to bound the vertex count, second pass pre-sized
            h0 = run(_fp(out), _fp(inp), _fp(positions), n, pd, vd, int(reverse), 0)
            bound = getattr(lib, "plref_num_vertices" + sfx)(h0)
            getattr(lib, "plref_free" + sfx)(h0)
            h = run(_fp(out), _fp(inp), _fp(positions), n, pd, vd, int(reverse), bound + 2)
            if not h:
                raise RuntimeError("reference oracle: pre-sized table grew")
            assert getattr(lib, "plref_never_grew" + sfx)(h)
    res = LatticeResult(out=out)
    res.num_vertices = getattr(lib, pre + "_num_vertices" + sfx)(h)
    if structure:
        m = res.num_vertices
        res.keys = np.empty((m, pd), np.int16)
        res.pix_vertex = np.empty((n, pd + 1), np.int32)
        res.pix_weight = np.empty((n, pd + 1), dtype)
        getattr(lib, pre + "_keys" + sfx)(h, res.keys.ctypes.data_as(_c_short_p))
        getattr(lib, pre + "_matrix" + sfx)(h, res.pix_vertex.ctypes.data_as(_c_int_p),
                                            _fp(res.pix_weight))
    getattr(lib, pre + "_free" + sfx)(h)
    return res


def op_geometry(input_shape, reference_shape, bilateral, theta_alpha, theta_beta, theta_gamma):
    """(batch, sdims, C, R, pd, vd, spatial_std, feature_std) as the op derives them
    (src/LatticeFilterKernel.cpp:112-142)."""
    batch = int(input_shape[0])
    sdims = [int(s) for s in input_shape[1:-1]]
    c = int(input_shape[-1])
    if bilateral:
        r = int(reference_shape[-1])
        return batch, sdims, c, r, r + len(sdims), c + 1, float(theta_alpha), float(theta_beta)
    return batch, sdims, c, 0, len(sdims), c + 1, float(theta_gamma), -1.0


def lattice_filter(input_image, reference_image, bilateral=True, theta_alpha=1.0, theta_beta=1.0,
                   theta_gamma=1.0, reverse=False, impl="port", structure=False, dtype=np.float32):
    """The op's semantics on numpy arrays [B, *S, C] / [B, *S, R].  Returns the output array, or
    (output, [LatticeResult per item]) when structure=True."""
    dtype = np.dtype(dtype)
    input_image = np.ascontiguousarray(input_image, dtype)
    batch, sdims, c, r, pd, vd, s_std, f_std = op_geometry(
        input_image.shape, None if reference_image is None else reference_image.shape, bilateral,
        theta_alpha, theta_beta, theta_gamma)
    n = int(np.prod(sdims))
    out = np.empty_like(input_image)
    results = []
    for b in range(batch):
        ref_b = None
        if r > 0:
            ref_b = np.ascontiguousarray(reference_image[b], dtype).reshape(n, r)
        pos = compute_positions(ref_b, sdims, s_std, f_std, impl=impl, dtype=dtype)
        res = filter(input_image[b].reshape(n, c), pos, reverse=reverse, structure=structure,
                     impl=impl, dtype=dtype)
        out[b] = res.out.reshape(input_image[b].shape)
        results.append(res)
    return (out, results) if structure else out


def filter_batch_timed(input_image, reference_image, bilateral=True, theta_alpha=1.0,
                       theta_beta=1.0, theta_gamma=1.0, reverse=False, impl="port", threads=1,
                       min_vertices=0, dtype=np.float32):
    """Runs the whole batch inside the C library on `threads` host threads and returns
    (output, wall seconds).  impl="reference" needs min_vertices > 0 (an upper bound on the
    per-item vertex count) to run with the never-growing table, 0 runs it as shipped."""
    dtype, sfx, _, _ = _kind(dtype)
    input_image = np.ascontiguousarray(input_image, dtype)
    batch, sdims, c, r, pd, vd, s_std, f_std = op_geometry(
        input_image.shape, None if reference_image is None else reference_image.shape, bilateral,
        theta_alpha, theta_beta, theta_gamma)
    n = int(np.prod(sdims))
    sd = np.ascontiguousarray(sdims, np.int32)
    out = np.empty_like(input_image)
    ref_p = None
    if r > 0:
        reference_image = np.ascontiguousarray(reference_image, dtype)
        ref_p = _fp(reference_image)
    if impl == "port":
        secs = getattr(_load_port(), "plo_filter_batch" + sfx)(
            _fp(out), _fp(input_image), ref_p, batch, n, c, r, len(sdims),
            sd.ctypes.data_as(_c_int_p), s_std, f_std, int(reverse), threads)
    else:
        secs = getattr(_load_reference(), "plref_filter_batch" + sfx)(
            _fp(out), _fp(input_image), ref_p, batch, n, c, r, len(sdims),
            sd.ctypes.data_as(_c_int_p), s_std, f_std, int(reverse), int(min_vertices), threads)
    if secs < 0:
        raise RuntimeError("CPU baseline run failed (table grew or bad sizes)")
    return out, secs
