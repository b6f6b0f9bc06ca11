"""Compiles the CUDA library in-tree: permutohedral_lattice_b200/libpl_lattice.so (sm_100a only).

    python -m permutohedral_lattice_b200.build [--force] [--verbose]

-fmad=false: no multiply-add contraction anywhere in the translation unit; the lattice geometry must
round every operation separately to select the same simplices as the reference CPU code.
"""
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libpl_lattice.so")
SOURCES = [os.path.join(CSRC, "pl_lattice.cu")]
HEADERS = [os.path.join(CSRC, h) for h in ("simplex.cuh", "common.cuh", "lattice_build.cuh", "splat.cuh",
                                             "blur_slice.cuh", "export.cuh", "fp64.cuh", "direct_index.cuh", "direct_bounds.h", "crf.cuh")] + [
    os.path.join(ROOT, "include", "pl_lattice.h")]


def nvcc_path():
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "bin", "nvcc")):
            return os.path.join(cand, "bin", "nvcc")
    return "nvcc"


def build(force=False, verbose=False):
    deps = SOURCES + HEADERS
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(d) for d in deps):
        return LIB
    cmd = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-fmad=false", "-Xcompiler", "-fPIC", "-shared", "-o", LIB] + SOURCES
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))


HOST_TEST_SRC = os.path.join(ROOT, "tests", "helpers", "host_class_test.cpp")
HOST_TEST_BIN = os.path.join(ROOT, "tests", "helpers", "host_class_test.bin")


def build_host_class_test(force=False):
    """C++ program over include/LatticeFilterKernel.hpp used by the GPU tests (built here, runs on the
    GPU box)."""
    deps = [HOST_TEST_SRC, os.path.join(ROOT, "include", "LatticeFilterKernel.hpp"), LIB]
    if not force and os.path.exists(HOST_TEST_BIN) and all(
            os.path.getmtime(HOST_TEST_BIN) >= os.path.getmtime(d) for d in deps):
        return HOST_TEST_BIN
    cuda = os.path.dirname(os.path.dirname(nvcc_path())) if os.path.sep in nvcc_path() else "/usr/local/cuda"
    cmd = ["g++", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
           HOST_TEST_SRC, "-o", HOST_TEST_BIN, "-L", PKG, "-lpl_lattice", "-L", os.path.join(cuda, "lib64"),
           "-lcudart", "-Wl,-rpath,$ORIGIN/../../permutohedral_lattice_b200",
           "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    subprocess.check_call(cmd)
    return HOST_TEST_BIN
