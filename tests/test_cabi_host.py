"""Host-side checks that need no GPU: the library loads, exports every symbol the header declares,
and validates arguments before touching the device."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def capi():
    from permutohedral_lattice_b200 import build, capi as c
    build.build()
    return c


def declared_functions():
    text = open(os.path.join(ROOT, "include", "pl_lattice.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pl_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(capi):
    names = declared_functions()
    assert "pl_lattice_filter_f32" in names and len(names) >= 10
    lib = capi.lib()
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(capi.EXPORTED_SYMBOLS) == names


def test_every_entry_point_cites_the_reference_or_says_it_has_no_counterpart():
    text = open(os.path.join(ROOT, "include", "pl_lattice.h")).read()
    for name in declared_functions():
        if name in ("pl_strerror", "pl_last_cuda_error"):
            continue
        idx = text.index(name + "(")
        comment = text[text.rfind("/*", 0, idx):idx]
        assert re.search(r"src/|Tests/|counterpart in the reference", comment), name


def test_supported_dims(capi):
    lib = capi.lib()
    for pd in (1, 2, 3, 4, 5, 6, 7, 8, 16):
        assert lib.pl_supported(pd, 22) == 1
    for pd in (0, 9, 15, 17, -1):
        assert lib.pl_supported(pd, 4) == 0
    assert lib.pl_supported(5, 1) == 0


def test_workspace_bytes_and_argument_checks(capi):
    lib = capi.lib()
    b = ctypes.c_size_t(0)
    sd = capi.int_array([512, 512])
    assert lib.pl_workspace_bytes(16, 512 * 512, 5, 22, 2, sd, 0, 0, ctypes.byref(b)) == capi.PL_OK
    worst = b.value
    assert lib.pl_workspace_bytes(16, 512 * 512, 5, 22, 2, sd, 4_000_000, 0, ctypes.byref(b)) == capi.PL_OK
    assert 0 < b.value < worst
    assert lib.pl_workspace_bytes(1, 512 * 512, 5, 22, 2, capi.int_array([512, 500]), 0, 0,
                                  ctypes.byref(b)) == capi.PL_INVALID_ARGUMENT
    assert lib.pl_workspace_bytes(1, 100, 11, 4, 0, None, 0, 0, ctypes.byref(b)) == capi.PL_UNSUPPORTED_DIMS
    assert lib.pl_workspace_bytes(1, 100, 5, 4, 0, None, 0, 0, None) == capi.PL_INVALID_ARGUMENT
    # more than 2^31 splats cannot be indexed
    assert lib.pl_workspace_bytes(65535, 1 << 20, 5, 4, 0, None, 0, 0, ctypes.byref(b)) == capi.PL_INVALID_ARGUMENT


def test_null_pointers_are_rejected_before_any_launch(capi):
    lib = capi.lib()
    sd = capi.int_array([8, 8])
    rc = lib.pl_lattice_filter_f32(None, None, None, 1, 2, sd, 3, 3, 1, 1.0, 1.0, 1.0, 0, None, 0, 0, 0, None)
    assert rc == capi.PL_INVALID_ARGUMENT
    rc = lib.pl_filter_f32(None, None, None, 1, 64, 5, 4, 0, None, 0, 0, 0, None)
    assert rc == capi.PL_INVALID_ARGUMENT
    rc = lib.pl_filter_f32(None, None, None, 1, 64, 12, 4, 0, None, 0, 0, 0, None)
    assert rc == capi.PL_UNSUPPORTED_DIMS
    rc = lib.pl_compute_positions_f32(None, None, 64, 3, 2, sd, 1.0, 1.0, None)
    assert rc == capi.PL_INVALID_ARGUMENT
    # empty problems succeed without a device
    assert lib.pl_filter_f32(None, None, None, 0, 64, 5, 4, 0, None, 0, 0, 0, None) == capi.PL_OK
    assert lib.pl_strerror(capi.PL_CAPACITY_EXCEEDED).decode().startswith("lattice entries")


def test_python_mirror_rejects_cpu_tensors(capi):
    import torch
    import permutohedral_lattice_b200 as plb
    with pytest.raises(ValueError):
        plb.lattice_filter(torch.zeros((1, 4, 4, 3)), torch.zeros((1, 4, 4, 3)))
