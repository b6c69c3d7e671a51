"""Generate the committed golden vectors from THE REFERENCE ITSELF (the shim built
from the reference's own headers, see oracle/build.py).  Run in a container that
has the reference tree:  python tests/golden/make_golden.py
Inputs are rebuilt by the tests from the same seeds (tests/cases.py); only the
reference's outputs (and small inputs) are stored here.
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import cases  # noqa: E402
import oracle  # noqa: E402
import synth  # noqa: E402


def sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), np.uint8)


def main():
    r = oracle.load_ref()
    assert r is not None, "build the reference shim first: python oracle/build.py"
    out = {}

    a, w, a2 = cases.ref_q4_case()
    q4 = r.to_q4(w)
    out["q4_small"] = dict(q4=q4, deq=r.q4_roundtrip_f32(w), y1=r.dot_q4(a, w)[0], y2=r.dot_q4(a2, w)[0],
                           y1_shipped=r.dot_q4(a, w, predequant=False)[0])

    W, x = cases.cfg1()
    q4 = r.to_q4(W)
    out["cfg1"] = dict(q4_sha=sha(q4), q4_head=q4[:4096].copy(), scales_head=q4[896 * 4864 // 2:][:4096].copy(),
                       y=r.dot_q4(x, W)[0], y_affine=r.dot_q4(x, W, 0.5, 1.0)[0])

    q, K, V, sc = cases.ref_attn_case()
    out["attn_small"] = dict(out=r.attn_decode(q, K, V, sc)[0])
    for ctx in (512, 2048):
        q, K, V, sc = cases.cfg2(ctx)
        out[f"cfg2_ctx{ctx}"] = dict(out=r.attn_decode(q, K, V, sc)[0])

    # bench/shared/check/check_llm_block.cpp shapes: rope [4,128] and [4,5,128] at pos 7
    xr1, xr2 = synth.normal(11, 1, (4, 128)), synth.normal(11, 2, (4, 5, 128))
    x64 = synth.normal(11, 3, (14, 64))
    out["rope"] = dict(o1=r.rope(xr1, 7, 10000.0), o2=r.rope(xr2, 7, 10000.0),
                       o3=r.rope(x64, 4200, 1e6))
    xn, wn = synth.normal(12, 1, (6, 512)), 1 + synth.normal(12, 2, (512,), 0.1)
    out["rmsnorm"] = dict(o=r.rmsnorm(xn, wn, 1e-5))
    g, u = synth.normal(13, 1, (3, 1024)), synth.normal(13, 2, (3, 1024))
    out["swiglu"] = dict(o=r.swiglu(g, u))

    # cfg4 at M = 1 and 8 on a reduced N (first 512 columns keep the file small;
    # K is the full 3584 so the accumulation length is the real one)
    for M in (1, 8):
        X, Wf = cases.cfg4(M, N=512)
        out[f"cfg4_M{M}_N512"] = dict(y=r.dot_q4(X, Wf, 0.5, 1.0)[0])

    for name, cfg, seed, prompt, ngen in (("dec_tiny", cases.TINY, 21, [1, 7, 3, 9, 2, 5], 6),
                                          ("dec_tiny64", cases.TINY64, 22, [5, 300, 17, 42], 8)):
        wts = cases.decoder_weights(cfg, seed)
        d = oracle.RefDecoder(r, cfg, 64)
        d.set_embed(wts["embed"]); d.set_vector(0, 5, wts["onorm"]); d.set_linear(0, 4, wts["lm_head"])
        for l, L in enumerate(wts["layers"]):
            for k, i in cases.LINEAR_IDS.items():
                d.set_linear(l, i, L[k])
            for k, i in cases.VECTOR_IDS.items():
                d.set_vector(l, i, L[k])
        toks, logits, nxt = [], [], 0
        for i in range(len(prompt) + ngen):
            tid = prompt[i] if i < len(prompt) else nxt
            nxt, lg = d.step(tid, i)
            toks.append(nxt); logits.append(lg)
        d.close()
        out[name] = dict(prompt=np.array(prompt), next_tokens=np.array(toks), logits=np.stack(logits))

    for name, d in out.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **d)
        print(name, {k: v.shape for k, v in d.items()})


if __name__ == "__main__":
    main()
