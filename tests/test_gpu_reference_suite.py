"""The reference's OWN test and check programs, compiled unmodified against this
repository's seam headers (include/gpu.h + include/cuda.h shadow the reference's by
include order, see oracle/build.py) and run under tl::use_gpu() on top of
libtlb200.so.  Skipped where the binaries were never built (no reference tree)."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")


def run(name, *args, timeout=600):
    exe = os.path.join(REF, name)
    if not os.path.exists(exe):
        pytest.skip(f"{name} not built (needs the reference tree at build time)")
    env = dict(os.environ, TLB200_LIB=os.path.join(ROOT, "cpp_tensorlib_b200", "libtlb200.so"))
    r = subprocess.run([exe, *args], env=env, capture_output=True, text=True, timeout=timeout)
    return r.returncode, r.stdout + r.stderr


@pytest.mark.parametrize("mode", ["--gpu", "--auto"])
def test_reference_doctest_suite(mode):
    """test/test_array.cpp + test_basic.cpp: q4 decode dot + widen fallback (:809-856),
    fused decode attention (:763-807), epilogue fusion, GPU/CPU hand-offs."""
    rc, out = run("ref_test_array", mode)
    assert rc == 0 and "Status: SUCCESS" in out, out[-2000:]


def test_reference_llm_decode_loop():
    """bench/cuda/check/check_llm_decode.cpp: logits maxrel < 2e-3 and greedy ids equal."""
    rc, out = run("ref_check_llm_decode")
    assert "no CUDA device" not in out, "the backend did not come up"
    assert rc == 0 and "ALL OK" in out and "MATCH" in out, out[-2000:]


def test_reference_llm_block():
    rc, out = run("ref_check_llm_block")
    assert rc == 0 and "ALL OK" in out, out[-2000:]


def test_reference_attn64_decode_dpos_and_prefill():
    """bench/cuda/check/check_attn64.cpp: cache grown to 2047 tokens across the split
    boundary, attn_dpos bit-equal to attn, and the batched / chunked prefill sections
    (kv_cache::prefill -> kv_fill + attn_prefill) against its CPU causal attention."""
    rc, out = run("ref_check_attn64")
    lines = [l for l in out.splitlines() if "kv cache grow" in l or "attn_dpos" in l]
    assert len(lines) == 2 and all(l.rstrip().endswith("OK") for l in lines), out[-2000:]
    assert rc == 0 and "FAIL" not in out, out[-2000:]


def test_reference_q4_gemv_bench_correctness():
    """bench/cuda/speed/bench_q4_gemv.cpp:93-104: GEMV vs a double-precision host
    dequant-dot on every 17th row, llama-7B shapes."""
    rc, out = run("ref_bench_q4_gemv")
    rows = [l.split() for l in out.splitlines() if l and l.split()[0] in
            ("qkv_proj", "attn_out", "ffn_gate_up", "ffn_down", "lm_head")]
    assert len(rows) == 5, out[-2000:]
    assert all(float(r[-1]) < 1e-4 for r in rows), rows
