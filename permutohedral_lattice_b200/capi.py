"""ctypes binding of the C ABI in include/pl_lattice.h (libpl_lattice.so, built in-tree by
permutohedral_lattice_b200/build.py).  There is no fallback: importing this module without the
compiled library raises."""
import ctypes
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# PL_LATTICE_LIB names another build of the same library (a variant under test); default: the in-tree one
LIB_PATH = os.environ.get("PL_LATTICE_LIB") or os.path.join(PKG, "libpl_lattice.so")

PL_OK = 0
PL_INVALID_ARGUMENT = 1
PL_UNSUPPORTED_DIMS = 2
PL_WORKSPACE_TOO_SMALL = 3
PL_CAPACITY_EXCEEDED = 4
PL_CUDA_ERROR = 5
PL_INTERNAL_ERROR = 6

PL_MODE_ATOMIC = 0
PL_MODE_DETERMINISTIC = 1
MODES = {"atomic": PL_MODE_ATOMIC, "deterministic": PL_MODE_DETERMINISTIC}

EXPORTED_SYMBOLS = [
    "pl_supported", "pl_strerror", "pl_last_cuda_error", "pl_workspace_bytes",
    "pl_compute_positions_f32", "pl_filter_f32", "pl_lattice_filter_f32", "pl_lattice_stats",
    "pl_export_lattice", "pl_profile_next_call", "pl_lattice_filter_f32_noalloc",
    "pl_lattice_build_f32", "pl_lattice_build_positions_f32", "pl_lattice_apply_f32",
    "pl_workspace_bytes_f64", "pl_compute_positions_f64", "pl_filter_f64", "pl_lattice_filter_f64",
    "pl_export_lattice_f64", "pl_debug_direct_index", "pl_crf_update_f32", "pl_launch_count",
    "pl_direct_index_min_entries",
]
STATIC_SCRATCH_BYTES = 64 << 20
NUM_STAGE_EVENTS = 6
STAGE_NAMES = ["build", "index", "splat", "blur", "slice"]


class PlStats(ctypes.Structure):
    _fields_ = [("num_vertices", ctypes.c_int64), ("num_entries", ctypes.c_int64),
                ("table_slots", ctypes.c_int64), ("device_status", ctypes.c_int32),
                ("direct_index", ctypes.c_int32), ("max_entries", ctypes.c_int64)]


class PlError(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        msg = "%s: %s" % (where, lib().pl_strerror(status).decode())
        if status == PL_CUDA_ERROR:
            msg += " (%s)" % lib().pl_last_cuda_error().decode()
        super().__init__(msg)


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "%s is missing: build it with `python -m permutohedral_lattice_b200.build` "
                "(there is no CPU or PyTorch fallback)" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        vp, i, i64, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
        ip = ctypes.POINTER(ctypes.c_int)
        L.pl_supported.argtypes = [i, i]
        L.pl_strerror.argtypes = [i]
        L.pl_strerror.restype = ctypes.c_char_p
        L.pl_last_cuda_error.restype = ctypes.c_char_p
        L.pl_workspace_bytes.argtypes = [i, i, i, i, i, ip, i64, i, ctypes.POINTER(ctypes.c_size_t)]
        L.pl_compute_positions_f32.argtypes = [vp, vp, i, i, i, ip, f, f, vp]
        L.pl_filter_f32.argtypes = [vp, vp, vp, i, i, i, i, i, vp, ctypes.c_size_t, i64, i, vp]
        L.pl_lattice_filter_f32.argtypes = [vp, vp, vp, i, i, ip, i, i, i, f, f, f, i, vp,
                                            ctypes.c_size_t, i64, i, vp]
        L.pl_lattice_stats.argtypes = [vp, ctypes.POINTER(PlStats), vp]
        L.pl_export_lattice.argtypes = [vp, vp, vp, i, i, i, i, i, ip, i, f, f, i64, i64, vp, vp, vp,
                                        vp, vp]
        L.pl_lattice_filter_f32_noalloc.argtypes = [vp, vp, vp, i, i, ip, i, i, i, f, f, f, i, i64, vp]
        L.pl_lattice_build_f32.argtypes = [vp, i, i, ip, i, i, f, f, f, i, vp, ctypes.c_size_t, i64, vp]
        L.pl_lattice_build_positions_f32.argtypes = [vp, i, i, i, i, vp, ctypes.c_size_t, i64, vp]
        L.pl_lattice_apply_f32.argtypes = [vp, vp, i, i, i, i, i, i, i, ip, vp, ctypes.c_size_t, i64, vp]
        d = ctypes.c_double
        L.pl_workspace_bytes_f64.argtypes = [i, i, i, i, i, ip, i64, ctypes.POINTER(ctypes.c_size_t)]
        L.pl_compute_positions_f64.argtypes = [vp, vp, i, i, i, ip, d, d, vp]
        L.pl_filter_f64.argtypes = [vp, vp, vp, i, i, i, i, i, vp, ctypes.c_size_t, i64, vp]
        L.pl_lattice_filter_f64.argtypes = [vp, vp, vp, i, i, ip, i, i, i, d, d, d, i, vp, ctypes.c_size_t,
                                            i64, vp]
        L.pl_export_lattice_f64.argtypes = [vp, vp, vp, i, i, i, i, i, ip, i, d, d, i64, i64, vp, vp, vp,
                                            vp, vp]
        L.pl_debug_direct_index.argtypes = [i]
        L.pl_direct_index_min_entries.argtypes = [i, i, ip, f, ctypes.POINTER(ctypes.c_int64)]
        L.pl_crf_update_f32.argtypes = [vp, vp, vp, vp, vp, f, f, i64, i, vp]
        L.pl_profile_next_call.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
        L.pl_launch_count.argtypes = []
        L.pl_launch_count.restype = ctypes.c_ulonglong
        _lib = L
    return _lib


def check(status, where):
    if status != PL_OK:
        raise PlError(status, where)


def int_array(values):
    return (ctypes.c_int * len(values))(*[int(v) for v in values])
