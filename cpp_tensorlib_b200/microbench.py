"""Single-kernel micro-benchmarks of the hot path (CUDA events, HBM-cold rotation).

  python -m cpp_tensorlib_b200.microbench gemv --N 37888 --K 3584 [--M 1] [--packed 1] [--copies 4] [--iters 20]
  python -m cpp_tensorlib_b200.microbench attn --heads 28 --kv-heads 28 --ctx 4096 --D 128

Distinct weight / cache copies are cycled so that the working set exceeds L2 and
the figure is an HBM figure; one pass over the copies is recorded into a CUDA
graph so host launch cost does not gate the GPU.  Prints one JSON line.
"""
import argparse
import json

import torch

from . import cuda as tl


def _time_graph(fn, iters):
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            fn()
    torch.cuda.synchronize()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def gemv(a):
    gen = torch.Generator(device="cuda").manual_seed(0)
    if a.bf16:
        Ws = [(torch.randn((a.N, a.K), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
              for _ in range(a.copies)]
        xv, yv = torch.randn(a.K, generator=gen, device="cuda"), torch.empty(a.N, device="cuda")

        def one_pass():
            for w in Ws:
                tl.gemv_bf16_row(xv, w, y=yv)
        ms = _time_graph(one_pass, a.iters) / a.copies
        nbytes = a.N * a.K * 2 + 4 * a.K + 4 * a.N
        print(json.dumps(dict(op="gemv_bf16_row", N=a.N, K=a.K, us_per_launch=ms * 1e3,
                              algorithmic_bytes=nbytes, GBps=nbytes / ms / 1e6)))
        return
    ws = [tl.to_q4(torch.randn((a.K, a.N), generator=gen, device="cuda") * 0.02) for _ in range(a.copies)]
    x = torch.randn((a.M, a.K), generator=gen, device="cuda")
    y = torch.empty((a.M, a.N), device="cuda")

    if a.packed:
        if a.M != 1:
            raise SystemExit("--packed is the M = 1 decode path")
        ps = [tl.Q4Packed(w) for w in ws]
        ws = None
        xv, yv = x.reshape(-1), y.reshape(-1)

        def one_pass():
            for w in ps:
                tl.gemv_q4p(xv, w, y=yv)
    else:
        def one_pass():
            for w in ws:
                tl.gemm_q4(x, w, y=y)
    ms = _time_graph(one_pass, a.iters) / a.copies
    nbytes = a.N * a.K * 0.625 + 4 * a.M * a.K + 4 * a.M * a.N
    print(json.dumps(dict(op="gemv_q4p" if a.packed else "gemv_q4", N=a.N, K=a.K, M=a.M, us_per_launch=ms * 1e3,
                          algorithmic_bytes=nbytes, GBps=nbytes / ms / 1e6,
                          TFLOPs=2.0 * a.M * a.N * a.K / ms / 1e9,
                          working_set_MB=a.copies * a.N * a.K * 0.625 / 1e6)))


def attn(a):
    gen = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn((a.heads, a.D), generator=gen, device="cuda")
    Ks = [torch.randn((a.kv_heads, a.ctx, a.D), generator=gen, device="cuda") for _ in range(a.copies)]
    Vs = [torch.randn((a.kv_heads, a.ctx, a.D), generator=gen, device="cuda") for _ in range(a.copies)]
    elt = 4
    if a.kv_bf16:
        Ks, Vs, elt = [k.to(torch.bfloat16) for k in Ks], [v.to(torch.bfloat16) for v in Vs], 2
    out = torch.empty_like(q)
    sc = a.D ** -0.5
    tl.attn_decode(q, Ks[0], Vs[0], sc, out=out)      # grows the library scratch before capture

    def one_pass():
        for K, V in zip(Ks, Vs):
            tl.attn_decode(q, K, V, sc, out=out)
    ms = _time_graph(one_pass, a.iters) / a.copies
    nbytes = 2 * a.kv_heads * a.ctx * a.D * elt + 2 * a.heads * a.D * 4
    print(json.dumps(dict(op="attn_decode_bf16kv" if a.kv_bf16 else "attn_decode", heads=a.heads, kv_heads=a.kv_heads, ctx=a.ctx, D=a.D,
                          us_per_launch=ms * 1e3, algorithmic_bytes=nbytes, GBps=nbytes / ms / 1e6,
                          working_set_MB=a.copies * nbytes / 1e6)))


def rmsnorm(a):
    x = torch.randn((1, a.n), device="cuda")
    w = torch.ones(a.n, device="cuda")
    out = torch.empty_like(x)

    def one_pass():
        for _ in range(a.copies):
            tl.rmsnorm(x, w, 1e-6, out=out)
    ms = _time_graph(one_pass, a.iters) / a.copies
    print(json.dumps(dict(op="rmsnorm", n=a.n, us_per_launch=ms * 1e3, pdl=a.pdl)))


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="op", required=True)
    g = sub.add_parser("gemv")
    g.add_argument("--N", type=int, default=37888)
    g.add_argument("--K", type=int, default=3584)
    g.add_argument("--M", type=int, default=1)
    g.add_argument("--packed", type=int, default=0, help="1: tile-packed weights (tlb_gemv_q4p)")
    g.add_argument("--bf16", type=int, default=0, help="1: bf16 row-major weights (tlb_gemv_bf16_row)")
    t = sub.add_parser("attn")
    t.add_argument("--heads", type=int, default=28)
    t.add_argument("--kv-heads", type=int, default=28)
    t.add_argument("--ctx", type=int, default=4096)
    t.add_argument("--D", type=int, default=128)
    t.add_argument("--kv-bf16", type=int, default=0, help="1: bf16 KV cache")
    r = sub.add_parser("rmsnorm")
    r.add_argument("--n", type=int, default=3584)
    for p in (g, t, r):
        p.add_argument("--copies", type=int, default=4)
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--pdl", type=int, default=1, help="programmatic dependent launch on/off")
    a = ap.parse_args()
    from ._lib import check, lib
    check(lib().tlb_set_pdl(a.pdl))
    {"gemv": gemv, "attn": attn, "rmsnorm": rmsnorm}[a.op](a)


if __name__ == "__main__":
    main()
