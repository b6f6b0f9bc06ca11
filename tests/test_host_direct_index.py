"""The dense index that spatial-only calls use instead of a hash table (csrc/direct_bounds.h), compiled
for the host: every vertex key the CPU oracle creates on a grid must fall inside the index, and two
different keys must never share a slot."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def shim(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("direct") / "libdirect_bounds_host.so")
    subprocess.check_call([
        "g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-o", out,
        "-I", os.path.join(ROOT, "permutohedral_lattice_b200", "csrc"),
        os.path.join(ROOT, "tests", "helpers", "direct_bounds_shim.cpp")])
    return ctypes.CDLL(out)


def _ptr(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


@pytest.mark.parametrize("shape,tg", [
    ((64, 48), 3.0), ((33, 17), 1.0), ((40, 56), 8.0), ((50, 70), 0.37), ((120, 90), 2.2),
    ((24, 20, 22), 2.0), ((9, 10, 11), 0.8), ((300,), 5.0), ((1, 1), 3.0), ((3, 4, 5, 6), 1.5),
    ((7, 200), 0.5), ((200, 7), 11.0),
])
def test_oracle_keys_fall_inside_the_index_and_never_collide(shape, tg, shim, oracle):
    pd = len(shape)
    n = int(np.prod(shape))
    pos = oracle.compute_positions(None, list(shape), tg, -1.0)
    res = oracle.filter(np.ones((n, 1), np.float32), pos, structure=True)
    keys = np.ascontiguousarray(res.keys, np.int16)                       # every vertex the grid creates
    sdims = np.asarray(shape, np.int32)
    scale = np.ascontiguousarray(oracle.scale_factors(pd), np.float32)
    # the vertices themselves, and their +-1 neighbours along every axis (looked up by the blur's
    # neighbour table: inside or outside, but never on another key's slot)
    nb = [keys]
    for a in range(pd + 1):
        step = np.ones(pd, np.int16)
        if a < pd:
            step[a] = -pd
        nb += [keys + step, keys - step]
    allk = np.unique(np.concatenate(nb), axis=0)
    slots = np.zeros(len(allk), np.uint64)
    outside = shim.direct_slots_host(pd, _ptr(sdims, ctypes.c_int), ctypes.c_float(tg), _ptr(scale, ctypes.c_float),
                                     _ptr(np.ascontiguousarray(allk), ctypes.c_short), len(allk),
                                     _ptr(slots, ctypes.c_ulonglong))
    assert outside >= 0, "the index was refused for this grid"
    own = np.zeros(len(keys), np.uint64)
    assert shim.direct_slots_host(pd, _ptr(sdims, ctypes.c_int), ctypes.c_float(tg), _ptr(scale, ctypes.c_float),
                                  _ptr(keys, ctypes.c_short), len(keys), _ptr(own, ctypes.c_ulonglong)) == 0
    assert len(np.unique(own)) == len(keys)
    # distinct keys, distinct slots (outside keys are never looked up, their slot value is unused)
    lo0 = ctypes.c_int()
    dlo = (ctypes.c_int * 8)()
    ext = (ctypes.c_uint * 8)()
    cells = ctypes.c_ulonglong()
    assert shim.direct_bounds_host(pd, _ptr(sdims, ctypes.c_int), ctypes.c_float(tg), _ptr(scale, ctypes.c_float), 1,
                                   ctypes.c_ulonglong(2 ** 62), ctypes.byref(lo0), dlo, ext, ctypes.byref(cells))
    k0 = allk[:, 0].astype(np.int64)
    inside = (k0 - lo0.value >= 0) & (k0 - lo0.value < ext[0])
    for i in range(1, pd):
        di = (allk[:, i].astype(np.int64) - k0) // (pd + 1)
        inside &= (di - dlo[i] >= 0) & (di - dlo[i] < ext[i])
    assert int((~inside).sum()) == outside
    assert len(np.unique(slots[inside])) == int(inside.sum())
    assert slots[inside].max() < cells.value


def test_index_is_refused_when_it_cannot_be_used(shim, oracle):
    scale = np.ascontiguousarray(oracle.scale_factors(2), np.float32)
    out = (ctypes.byref(ctypes.c_int()), (ctypes.c_int * 8)(), (ctypes.c_uint * 8)(),
           ctypes.byref(ctypes.c_ulonglong()))

    def ok(shape, tg, batch=1, max_slots=2 ** 40):
        sd = np.asarray(shape, np.int32)
        return shim.direct_bounds_host(len(shape), _ptr(sd, ctypes.c_int), ctypes.c_float(tg),
                                       _ptr(scale, ctypes.c_float), batch, ctypes.c_ulonglong(max_slots), *out)

    assert ok((64, 64), 3.0) == 1
    assert ok((64, 64), 3.0, max_slots=100) == 0          # does not fit the table region
    assert ok((64, 64), 0.0) == 0 and ok((64, 64), -1.0) == 0 and ok((64, 64), float("nan")) == 0
    assert ok((60000, 64), 1.0) == 0                      # coordinates beyond 16 bits
    assert ok((4096, 4096), 0.25, batch=64) == 0          # more slots than 32-bit entry numbers
