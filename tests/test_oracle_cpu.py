"""CPU suite: pins the C restatement (oracle port) against the committed golden
vectors produced by the reference, and -- where the reference shim is built --
against the reference itself.  No GPU."""
import hashlib

import numpy as np
import pytest

import cases
import oracle
import synth


def relerr(a, b):
    """The reference's metric |got-ref| / (1+|ref|) (bench/cuda/check/check_llm_decode.cpp:253)."""
    return float(np.max(np.abs(a.astype(np.float64) - b) / (1.0 + np.abs(b))))


def test_q4_small_matches_reference_bytes(port, golden):
    a, w, a2 = cases.ref_q4_case()
    g = golden("q4_small")
    q4 = port.to_q4(w)
    assert np.array_equal(q4, g["q4"])                      # int4 layout: bit exact
    assert np.array_equal(port.q4_to_f32(q4, 256, 48), g["deq"])
    assert np.abs(g["deq"] - w).max() < 0.2                 # test/test_array.cpp:841-845
    assert relerr(port.gemm_q4(a, q4, 48), g["y1"]) < 1e-4
    assert relerr(port.gemm_q4(a2, q4, 48), g["y2"]) < 1e-4
    assert relerr(g["y1_shipped"], g["y1"]) < 1e-4          # shipped funnel == dequantised-f32 ref


def test_cfg1_matches_reference(port, golden):
    W, x = cases.cfg1()
    g = golden("cfg1")
    q4 = port.to_q4(W)
    assert np.array_equal(np.frombuffer(hashlib.sha256(q4.tobytes()).digest(), np.uint8), g["q4_sha"])
    assert np.array_equal(q4[:4096], g["q4_head"])
    assert relerr(port.gemm_q4(x, q4, 4864), g["y"]) < 1e-4
    assert relerr(port.gemm_q4(x, q4, 4864, 0.5, 1.0), g["y_affine"]) < 1e-4


def test_q4_rejects_bad_k(port):
    with pytest.raises(ValueError):
        port.to_q4(np.zeros((48, 4), np.float32))


def test_attention_matches_reference(port, golden):
    q, K, V, sc = cases.ref_attn_case()
    assert relerr(port.attn_decode(q, K, V, sc), golden("attn_small")["out"]) < 1e-4
    for ctx in (512, 2048):
        q, K, V, sc = cases.cfg2(ctx)
        assert relerr(port.attn_decode(q, K, V, sc), golden(f"cfg2_ctx{ctx}")["out"]) < 1e-4


def test_attention_gqa_prefix(port):
    # GQA + cache prefix addressing (include/cuda.h:966-984) against an explicit softmax
    q, K, V = synth.normal(31, 1, (4, 64)), synth.normal(31, 2, (2, 40, 64)), synth.normal(31, 3, (2, 40, 64))
    got = port.attn_decode(q, K, V, 0.125, ctx=17)
    for h in range(4):
        s = (K[h // 2, :17] @ q[h]) * 0.125
        p = np.exp(s - s.max()); p /= p.sum()
        assert np.allclose(got[h], p @ V[h // 2, :17], atol=1e-5)


def test_row_ops_match_reference(port, golden):
    xr1, xr2, x64 = synth.normal(11, 1, (4, 128)), synth.normal(11, 2, (4, 5, 128)), synth.normal(11, 3, (14, 64))
    g = golden("rope")
    assert np.array_equal(port.rope(xr1, 7, 10000.0), g["o1"])
    assert np.array_equal(port.rope(xr2, 7, 10000.0), g["o2"])
    assert np.array_equal(port.rope(x64, 4200, 1e6), g["o3"])
    xn, wn = synth.normal(12, 1, (6, 512)), 1 + synth.normal(12, 2, (512,), 0.1)
    assert relerr(port.rmsnorm(xn, wn, 1e-5), golden("rmsnorm")["o"]) < 2e-6
    gg, u = synth.normal(13, 1, (3, 1024)), synth.normal(13, 2, (3, 1024))
    assert relerr(port.swiglu(np.concatenate([gg, u], 1), 1024), golden("swiglu")["o"]) < 2e-6
    xo, ho = port.add_rmsnorm(xn, xn * 0.5, wn, 1e-5)
    assert np.allclose(xo, xn * 1.5) and relerr(ho, port.rmsnorm(xn * 1.5, wn, 1e-5)) < 1e-6


def test_argmax_first_maximum(port):
    v = np.array([1, 5, 3, 5, 5, -2], np.float32)
    assert port.argmax(v) == 1


def test_cfg4_reduced_matches_reference(port, golden):
    for M in (1, 8):
        X, Wf = cases.cfg4(M, N=512)
        y = port.gemm_q4(X, port.to_q4(Wf), 512, 0.5, 1.0)
        assert relerr(y, golden(f"cfg4_M{M}_N512")["y"]) < 1e-4


def _port_decoder(port, cfg, seed, max_ctx):
    wts = cases.decoder_weights(cfg, seed)
    d = oracle.PortDecoder(port, cfg, max_ctx)
    d.set_embed(wts["embed"]); d.set_vector(0, 5, wts["onorm"]); d.set_linear(0, 4, port.to_q4(wts["lm_head"]))
    for l, L in enumerate(wts["layers"]):
        for k, i in cases.LINEAR_IDS.items():
            d.set_linear(l, i, port.to_q4(L[k]))
        for k, i in cases.VECTOR_IDS.items():
            d.set_vector(l, i, L[k])
    return d


@pytest.mark.parametrize("name,cfg,seed", [("dec_tiny", cases.TINY, 21), ("dec_tiny64", cases.TINY64, 22)])
def test_decoder_matches_reference(port, golden, name, cfg, seed):
    """bench/cuda/check/check_llm_decode.cpp:241-277: logits maxrel < 2e-3 and
    greedy ids equal, here against the decoder assembled from reference ops."""
    g = golden(name)
    d = _port_decoder(port, cfg, seed, 64)
    prompt = list(g["prompt"])
    nxt = 0
    for i in range(len(g["next_tokens"])):
        tid = prompt[i] if i < len(prompt) else nxt
        nxt, lg = d.step(int(tid), i)
        assert relerr(lg, g["logits"][i]) < 2e-3
        assert nxt == int(g["next_tokens"][i])
    d.close()


def test_port_against_live_reference(port, ref):
    """Fresh inputs through both the restatement and the reference compiled from
    its own headers (skipped where the reference tree was never available)."""
    if ref is None:
        pytest.skip("reference shim not built (no reference tree on this machine)")
    W, x = synth.normal(41, 1, (384, 200), 0.05), synth.normal(41, 2, (3, 384))
    assert np.array_equal(port.to_q4(W), ref.to_q4(W))
    assert relerr(port.gemm_q4(x, port.to_q4(W), 200, 0.5, 1.0), ref.dot_q4(x, W, 0.5, 1.0)[0]) < 1e-4
    q, K, V = synth.normal(42, 1, (3, 64)), synth.normal(42, 2, (3, 77, 64)), synth.normal(42, 3, (3, 77, 64))
    assert relerr(port.attn_decode(q, K, V, 0.125), ref.attn_decode(q, K, V, 0.125)[0]) < 1e-5
    xr = synth.normal(43, 1, (6, 3, 64))
    assert np.array_equal(port.rope(xr, 123, 1e6), ref.rope(xr, 123, 1e6))


def test_port_bf16_cache_rounding_matches_torch(port):
    """The oracle's bf16-cache mode rounds stored rows to nearest even like kv_st
    (kernels/tensorlib_cuda.cu:831): checked against torch's f32 -> bf16 -> f32 on values that
    include exact ties, and on a decoder step whose logits must differ from the f32-cache run by
    no more than the rounding allows."""
    import torch
    import cases
    import oracle
    cfg = cases.TINY64
    wts = cases.decoder_weights(cfg, 22)

    def build(bf):
        o = oracle.PortDecoder(port, cfg, 16, kv_bf16=bf)
        o.set_embed(wts["embed"]); o.set_vector(0, 5, wts["onorm"]); o.set_linear(0, 4, port.to_q4(wts["lm_head"]))
        for l, L in enumerate(wts["layers"]):
            for k, i in cases.LINEAR_IDS.items():
                o.set_linear(l, i, port.to_q4(L[k]))
            for k, i in cases.VECTOR_IDS.items():
                o.set_vector(l, i, L[k])
        return o
    a, b = build(False), build(True)
    # fill_kv goes through the same store: read it back through one attention step
    import synth
    v = np.concatenate([np.array([1.0, 1.00390625, 1.01171875, -3.0e-5, 0.0, -0.0, 3.3e38, 1e-40], np.float32),
                        synth.normal(9, 1, (4096,), 3.0)])
    want = torch.from_numpy(v).to(torch.bfloat16).float().numpy()
    assert want[1] == 1.0 and want[2] == np.float32(1.015625)                 # ties go to even
    assert np.array_equal(port.bf16_round(v).view(np.uint32), want.view(np.uint32))
    la = lb = None
    tok = 3
    for pos in range(4):
        ta, la = a.step(tok, pos)
        tb, lb = b.step(tok, pos)
        tok = ta
    assert not np.array_equal(la, lb)                     # the rounding is really applied
    assert np.max(np.abs(la - lb)) < 5e-2
    a.close(); b.close()
