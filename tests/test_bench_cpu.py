"""Host-side arithmetic of bench.py (no GPU): the byte counts the roofline figures rest on."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_token_bytes_of_baseline_config_5():
    """BASELINE config 5 (7B shape): 7.07 G int4 weights in the linears = 4.42 GB at 0.625 byte
    per weight, and 470 MB of f32 KV at ctx 4096 (28 layers x 2 x 4 heads x 4096 x 128 x 4)."""
    b = load_bench()
    wbytes, kv, params = b.token_bytes(b.QWEN7, 4096)
    sh = b.linear_shapes(b.QWEN7)
    assert sh["wqkv"] == (3584, 4608) and sh["wgu"] == (3584, 37888) and sh["wd"] == (18944, 3584)
    assert params == 28 * (3584 * 4608 + 3584 * 3584 + 3584 * 37888 + 18944 * 3584) + 3584 * 152064
    assert abs(wbytes - 4.42e9) < 0.02e9
    assert kv == 28 * 2 * 4 * 4096 * 128 * 4


def test_traffic_factors_cover_every_matrix_of_the_sweep():
    b = load_bench()
    assert set(b.TRAFFIC_FACTORS) == set(b.linear_shapes(b.QWEN7))
    assert all(1.0 <= f < 1.1 for f in b.TRAFFIC_FACTORS.values())


def test_config_block_names_the_workload_and_no_model_keys():
    b = load_bench()
    c = b.config_block(4)
    assert c["parallelism"] == "tp4" and "workload" in c and "model" not in c
