"""Input definitions shared by the golden-vector generator and the tests, so both
sides build byte-identical inputs from the same seeds."""
import numpy as np

import synth

# bench/cuda/check/check_llm_decode.cpp:24-27 shape family (GQA, hd 128), with
# the Qwen2.5 extras this build's decoder has (q/k/v biases, fused qkv / gate|up).
TINY = dict(hidden=512, layers=3, n_q=4, n_kv=2, hd=128, ff=1024, vocab=48, eps=1e-5,
            rope_base=10000.0)
# head_dim 64 family (Qwen2.5-0.5B-like ratios, scaled down): 14 q / 2 kv heads.
TINY64 = dict(hidden=896, layers=2, n_q=14, n_kv=2, hd=64, ff=1024, vocab=320, eps=1e-6,
              rope_base=1e6)
QWEN05 = dict(hidden=896, layers=24, n_q=14, n_kv=2, hd=64, ff=4864, vocab=151936, eps=1e-6,
              rope_base=1e6)
QWEN7 = dict(hidden=3584, layers=28, n_q=28, n_kv=4, hd=128, ff=18944, vocab=152064, eps=1e-6,
             rope_base=1e6)


def ref_q4_case():
    """test/test_array.cpp:809-856: K=256, N=48, LCG seed 5; a then w, then a2 [2,K]."""
    K, N = 256, 48
    s = synth.lcg_uniform(5, K + K * N + 2 * K)
    return s[:K].reshape(1, K), s[K:K + K * N].reshape(K, N), s[K + K * N:].reshape(2, K)


def ref_attn_case():
    """test/test_array.cpp:763-781: H=2, D=128, ctx=5, LCG seeds 1,2,3."""
    H, D, Cc = 2, 128, 5
    return (synth.lcg_uniform(1, H * D).reshape(H, D), synth.lcg_uniform(2, H * Cc * D).reshape(H, Cc, D),
            synth.lcg_uniform(3, H * Cc * D).reshape(H, Cc, D), 1.0 / np.sqrt(np.float32(D)))


def cfg1():
    """BASELINE config 1: W [K=896, N=4864] ~ N(0, 0.02) seed 0, x [1, 896] ~ N(0,1)."""
    return synth.normal(0, 1, (896, 4864), 0.02), synth.normal(0, 2, (1, 896))


def cfg2(ctx, H=28, D=128):
    """BASELINE config 2: q [28,128], K, V [28,ctx,128] ~ N(0,1) seed 1."""
    return (synth.normal(1, 1, (H, D)), synth.normal(1, 2, (H, ctx, D)), synth.normal(1, 3, (H, ctx, D)),
            1.0 / np.sqrt(np.float32(D)))


def cfg4(M, K=3584, N=18944):
    """BASELINE config 4: X [M, 3584] ~ N(0,1), W [3584, 18944] ~ N(0, 0.02), seed 3."""
    return synth.normal(3, 10 + M, (M, K)), synth.normal(3, 1, (K, N), 0.02)


def decoder_weights(cfg, seed):
    """Random-init decoder: linears N(0, 0.02) (quantised to q4 by the consumer),
    embeddings N(0, 0.02), norm weights 1 + N(0, 0.02), q/k/v biases N(0, 0.02)."""
    E, HD, NQ, NKV, FF, V = cfg["hidden"], cfg["hd"], cfg["n_q"], cfg["n_kv"], cfg["ff"], cfg["vocab"]
    w = {"embed": synth.normal(seed, 1, (V, E), 0.02),
         "onorm": 1 + synth.normal(seed, 2, (E,), 0.02),
         "lm_head": synth.normal(seed, 3, (E, V), 0.02), "layers": []}
    for l in range(cfg["layers"]):
        b = 100 + 20 * l
        w["layers"].append(dict(
            wqkv=synth.normal(seed, b + 1, (E, (NQ + 2 * NKV) * HD), 0.02),
            wo=synth.normal(seed, b + 2, (NQ * HD, E), 0.02),
            wgu=synth.normal(seed, b + 3, (E, 2 * FF), 0.02),
            wd=synth.normal(seed, b + 4, (FF, E), 0.02),
            bq=synth.normal(seed, b + 5, (NQ * HD,), 0.02),
            bk=synth.normal(seed, b + 6, (NKV * HD,), 0.02),
            bv=synth.normal(seed, b + 7, (NKV * HD,), 0.02),
            an=1 + synth.normal(seed, b + 8, (E,), 0.02),
            fn=1 + synth.normal(seed, b + 9, (E,), 0.02)))
    return w


LINEAR_IDS = dict(wqkv=0, wo=1, wgu=2, wd=3)
VECTOR_IDS = dict(an=0, fn=1, bq=2, bk=3, bv=4)
