"""Build recipe for the checkers (test infrastructure, not product code).

* ``liborc.so``   -- the plain-C restatement in ``q4_oracle.c`` (gcc, OpenMP).
* ``_ref/libtlref.so`` -- the reference itself: ``ref_shim.cpp`` compiled against
  the reference's own headers where they lie (``$TL_REFERENCE_DIR`` or the
  default mount).  Built only when that tree is present; the output directory is
  git-ignored so reference-derived binaries never enter history.

Usage: ``python oracle/build.py [--force]``.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.environ.get("TL_REFERENCE_DIR", "/root/reference")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_port(force=False):
    src = os.path.join(HERE, "q4_oracle.c")
    out = os.path.join(HERE, "liborc.so")
    if force or _stale(out, [src]):
        subprocess.check_call(["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-std=c11",
                               src, "-o", out, "-lm"])
    return out


def build_reference(force=False):
    inc = os.path.join(REF_DIR, "include")
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libtlref.so")
    if not os.path.isfile(os.path.join(inc, "tensorlib.h")):
        return out if os.path.exists(out) else None
    src = os.path.join(HERE, "ref_shim.cpp")
    if force or _stale(out, [src]):
        os.makedirs(out_dir, exist_ok=True)
        # -fno-access-control: read a q4 array's packed bytes out of its private
        # storage without modifying the reference sources.  No -march flag: the
        # reference picks its AVX2 microkernel at run time.
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-fPIC", "-shared",
                               "-fno-access-control", "-I", inc, src, "-o", out,
                               "-lpthread"])
    return out


def build_all(force=False):
    return build_port(force), build_reference(force)


if __name__ == "__main__":
    print(build_all("--force" in sys.argv))
