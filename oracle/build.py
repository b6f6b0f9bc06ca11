"""Build recipe for the test-only CPU oracle libraries (checker and timed CPU baseline).

  oracle/libpl_oracle.so    C restatement of the reference CPU path (oracle/pl_oracle.c)
  oracle/_ref/libpl_ref.so  the UNMODIFIED reference header behind a C shim (oracle/ref_shim.cpp),
                            built only where the reference tree is present; the header is compiled
                            from where it lies and never copied.

Flags follow the parity-critical ones of the reference CPU build: -O2, no FMA contraction
(-ffp-contract=off), no -ffast-math, no -march=native.

Run:  python oracle/build.py [--force]
The reference tree (a checkout of MiguelMonteiro/permutohedral_lattice) is searched in $PL_REFERENCE_DIR,
then in a directory named "reference" beside this repository.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libpl_oracle.so")
REF_DIR_OUT = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR_OUT, "libpl_ref.so")
SIBLING_REFERENCE_DIR = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def reference_root():
    for cand in (os.environ.get("PL_REFERENCE_DIR"), SIBLING_REFERENCE_DIR):
        if cand and os.path.isfile(os.path.join(cand, "src", "PermutohedralLatticeCPU.h")):
            return cand
    return None


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "pl_oracle.c")
    if force or _stale(ORACLE_SO, [src, os.path.join(HERE, "pl_oracle_impl.h")]):
        cmd = ["gcc", "-O2", "-std=c99", "-D_POSIX_C_SOURCE=200809L", "-ffp-contract=off", "-fPIC",
               "-shared", "-o", ORACLE_SO, src, "-lm", "-lpthread"]
        subprocess.check_call(cmd)
    return ORACLE_SO


def build_reference(force=False):
    """Returns the path of libpl_ref.so, or None when the reference tree is absent and no prebuilt
    library exists."""
    root = reference_root()
    src = os.path.join(HERE, "ref_shim.cpp")
    if root is None:
        return REF_SO if os.path.exists(REF_SO) else None
    hdr = os.path.join(root, "src", "PermutohedralLatticeCPU.h")
    if force or _stale(REF_SO, [src, hdr]):
        os.makedirs(REF_DIR_OUT, exist_ok=True)
        cmd = ["g++", "-O2", "-std=c++11", "-ffp-contract=off", "-fPIC", "-shared", "-w",
               "-I", os.path.join(root, "src"), "-o", REF_SO, src, "-lpthread"]
        subprocess.check_call(cmd)
    return REF_SO


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_reference(force))
