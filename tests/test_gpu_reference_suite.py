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
    # the program is a process of its own on the same GPU: hand back what this process's
    # allocator only caches, and keep the diagnostic switches of other tests out of it
    for k in [k for k in env if k.startswith("TLB_")]:
        env.pop(k)
    try:
        import gc
        import torch
        gc.collect()
        torch.cuda.empty_cache()
    except Exception:
        pass
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


def test_reference_attn_decode_bench_correctness_sections():
    """bench/cuda/speed/bench_attn_decode.cpp through the seam: the f32-vs-CPU maxrel column of
    its llama-shape table (:100-133; the bf16 run's error is the cache's rounding, ~1e-3), and
    the three 1e-4 correctness sections at D=128, 32 q / 8 kv heads -- the cache grown token by
    token across the split boundary (:197-298), the batched prefill at T=500 (:324-398) and the
    decode step that continues it (:400-453)."""
    rc, out = run("ref_bench_attn_decode", timeout=900)
    assert "no CUDA device" not in out, "the backend did not come up"
    assert rc == 0 and "FAIL" not in out, out[-3000:]
    want = ("grew to", "prefill T=", "decode step at pos=")
    for w in want:
        lines = [l for l in out.splitlines() if w in l]
        assert lines and all(" OK" in l for l in lines), (w, out[-3000:])


def test_reference_own_cuda_kernels_run_on_this_gpu():
    """oracle/_ref/ref_gpu_bench: the reference's OWN kernels (its PTX JIT-compiled by the driver
    for this GPU, reached through its own include/cuda.h, none of this repository's code on the
    path) on the BASELINE shapes.  Here only their sanity column is asserted (each kernel's
    result against a double-precision host loop); the timings are what bench.py's reference
    arm reports beside this build's."""
    import json
    exe = os.path.join(REF, "ref_gpu_bench")
    if not os.path.exists(exe):
        pytest.skip("ref_gpu_bench not built (needs the reference tree and nvcc at build time)")
    r = subprocess.run([exe, "--quick"], capture_output=True, text=True, timeout=600)
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert r.returncode == 0 and rows and "error" not in rows[0], r.stdout[-2000:] + r.stderr[-2000:]
    assert {x["name"] for x in rows} >= {"cfg1", "7b_qkv", "7b_o", "7b_gate_up", "7b_down", "cfg2_ctx4096"}
    for x in rows:
        assert x["us"] > 0 and x["maxrel"] < 1e-3, x


def test_runtime_hook_executor_keeps_the_hot_path_on_the_device():
    """tests/cpp/check_executor.cpp: the executor installed through the reference's runtime hooks
    (include/array.h:190-195, 2525-2532) evaluates BASELINE config 4 -- X.dot(Wq) * 0.5f + 1.0f at
    M in {1, 8, 64, 512} -- as one int4 launch per dot with the epilogue in the kernel and no host
    dequantisation, recognises the RMSNorm / SwiGLU compositions (array.h:2429-2439), and matches
    the reference's CPU evaluation (1e-4 / 1e-5)."""
    rc, out = run("check_executor", timeout=900)
    assert "no CUDA device" not in out, "the backend did not come up"
    if not (rc == 0 and "ALL OK" in out):
        # one of its checks compares wall-clock times (device evaluation against a host
        # dequantisation): run once more before calling it a failure, and show both outputs
        rc2, out2 = run("check_executor", timeout=900)
        assert rc2 == 0 and "ALL OK" in out2, "first run:\n" + out[-2000:] + "\nsecond run:\n" + out2[-2000:]
