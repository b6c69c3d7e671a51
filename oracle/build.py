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


# The reference's OWN test / check programs, compiled unmodified against this
# repository's seam headers (include/gpu.h, include/cuda.h shadow the reference's
# by include order) so they exercise libtlb200.so through tl::use_gpu().
REFERENCE_CHECKS = {
    "ref_test_array": ["test/test_array.cpp", "test/test_basic.cpp"],
    "ref_check_llm_decode": ["bench/cuda/check/check_llm_decode.cpp"],
    "ref_check_llm_block": ["bench/shared/check/check_llm_block.cpp"],
    "ref_check_attn64": ["bench/cuda/check/check_attn64.cpp"],
    "ref_bench_q4_gemv": ["bench/cuda/speed/bench_q4_gemv.cpp"],
    "ref_bench_attn_decode": ["bench/cuda/speed/bench_attn_decode.cpp"],
}


def build_reference_checks(force=False):
    inc = os.path.join(REF_DIR, "include")
    if not os.path.isfile(os.path.join(inc, "tensorlib.h")):
        return []
    seam = os.path.join(HERE, "..", "include")
    out_dir = os.path.join(HERE, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    deps = [os.path.join(seam, "cuda.h"), os.path.join(seam, "gpu.h")]
    built, procs = [], []
    for name, srcs in REFERENCE_CHECKS.items():
        out = os.path.join(out_dir, name)
        paths = [os.path.join(REF_DIR, s) for s in srcs]
        built.append(out)
        if force or _stale(out, paths + deps):
            procs.append(subprocess.Popen(
                ["g++", "-std=c++17", "-O2", "-DTENSORLIB_CUDA", "-I", seam, "-I", inc,
                 "-I", os.path.join(REF_DIR, "test")] + paths + ["-o", out, "-ldl", "-lpthread"]))
    # this repository's own check of the runtime-hook executor (include/tlb200_executor.h),
    # a consumer of the reference's public tl::array API built in its TL_RUNTIME_HOOKS mode
    exe = os.path.join(out_dir, "check_executor")
    src = os.path.join(HERE, "..", "tests", "cpp", "check_executor.cpp")
    built.append(exe)
    if force or _stale(exe, [src, os.path.join(seam, "tlb200_executor.h")] + deps):
        procs.append(subprocess.Popen(
            ["g++", "-std=c++17", "-O2", "-DTENSORLIB_CUDA", "-DTL_RUNTIME_HOOKS", "-I", seam, "-I", inc,
             src, "-o", exe, "-ldl", "-lpthread"]))
    for p in procs:
        if p.wait():
            raise RuntimeError("compiling a reference check against the seam headers failed")
    return built


def build_reference_gpu(force=False):
    """The reference's OWN CUDA backend, for timing its kernels on the same GPU: its kernel
    source compiled to PTX the way its CMakeLists does (``nvcc -arch=sm_80 -ptx``; the driver
    JIT-compiles that PTX for the device it finds), the PTX turned into the byte-list include
    its ``include/cuda.h`` embeds (what ``cmake/bin2c.cmake`` writes: ``0x..,`` per byte and a
    closing ``0x00``), and ``ref_gpu_bench.cpp`` -- a small timing driver over the reference's
    public ``tl::cuda::`` facade -- compiled against the REFERENCE's headers, not this
    repository's seam.  Outputs only under ``oracle/_ref/``; nothing is copied."""
    inc = os.path.join(REF_DIR, "include")
    cu = os.path.join(REF_DIR, "kernels", "tensorlib_cuda.cu")
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "ref_gpu_bench")
    if not (os.path.isfile(os.path.join(inc, "tensorlib.h")) and os.path.isfile(cu)):
        return out if os.path.exists(out) else None
    src = os.path.join(HERE, "ref_gpu_bench.cpp")
    if force or _stale(out, [src, cu]):
        gen = os.path.join(out_dir, "gen")
        os.makedirs(gen, exist_ok=True)
        ptx = os.path.join(gen, "tensorlib_cuda.ptx")
        nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
        subprocess.check_call([nvcc, "-arch=sm_80", "-ptx", "-Wno-deprecated-gpu-targets", cu, "-o", ptx])
        with open(ptx, "rb") as f:
            data = f.read()
        with open(os.path.join(gen, "tensorlib_cuda_ptx.inc"), "w") as f:
            f.write("".join("0x%02x," % b for b in data) + " 0x00\n")
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-DTENSORLIB_CUDA", "-I", gen, "-I", inc,
                               src, "-o", out, "-ldl", "-lpthread"])
    return out


def build_all(force=False):
    return (build_port(force), build_reference(force), build_reference_checks(force),
            build_reference_gpu(force))


if __name__ == "__main__":
    print(build_all("--force" in sys.argv))
