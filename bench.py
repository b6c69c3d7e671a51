#!/usr/bin/env python
"""Benchmark of the quantized-decode hot path on B200.

Headline workload (BASELINE config 5): Qwen2.5-7B-architecture int4 decoder,
random-init from seed 4, batch 1, KV cache pre-filled to ctx 4096 with N(0,1),
greedy decode; one step = one token.  N GPUs = tensor parallel (strong scaling:
the same model is split N ways), one process per GPU.

  python bench.py --gpus 1 --steps K --warmup W          # this build, CUDA path
  python bench.py --impl reference ...                    # reference CPU path, same metric
Prints ONE JSON line.  `value` is device-resident greedy decoding (token ids feed
back on the GPU, one CUDA-graph replay per token), `e2e` goes through the host-
buffer C-ABI call (token id H2D, next id D2H, every step).  `roofline` is the int4
GEMV kernel over one token's 113 weight matrices, timed with CUDA events in this
process.  `cpu_baseline` is the reference's own CPU code on a bounded sample.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN7 = dict(hidden=3584, layers=28, n_q=28, n_kv=4, hd=128, ff=18944, vocab=152064, eps=1e-6,
             rope_base=1e6)
CTX0 = 4096
SEED = 4
# DRAM read+write bytes per algorithmic byte of the int4 GEMV, from ncu captures of single
# launches (profiles/gemv_q4p_gate_up_7b.md, profiles/gemv_q4p_qkv_7b_small_launch.md): 1.036 on
# the 85 MB gate|up matrix, 1.001 on the down projection, 1.005 on qkv.  Constants taken from
# those captures and applied to each matrix of the sweep by its bytes (o like qkv, the lm_head
# like gate|up: same kernel mode), not a per-run measurement.
TRAFFIC_FACTORS = dict(wgu=1.036, lm_head=1.036, wd=1.001, wqkv=1.005, wo=1.005)
TRAFFIC_NOTE = ("ncu captures of single launches: dram read+write / algorithmic bytes = 1.036 (gate|up), "
                "1.001 (down), 1.005 (qkv); o taken as qkv, lm_head as gate|up; applied per matrix by bytes")


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def linear_shapes(cfg):
    E, HD = cfg["hidden"], cfg["hd"]
    return dict(wqkv=(E, (cfg["n_q"] + 2 * cfg["n_kv"]) * HD), wo=(cfg["n_q"] * HD, E),
                wgu=(E, 2 * cfg["ff"]), wd=(cfg["ff"], E), lm_head=(E, cfg["vocab"]))


def token_bytes(cfg, ctx):
    """Algorithmic HBM bytes of one decoded token: every q4 linear once (0.625 B per
    weight) plus the f32 KV prefix of every layer."""
    sh = linear_shapes(cfg)
    per_layer = sum(sh[n][0] * sh[n][1] for n in ("wqkv", "wo", "wgu", "wd"))
    params = cfg["layers"] * per_layer + sh["lm_head"][0] * sh["lm_head"][1]
    kv = cfg["layers"] * 2 * cfg["n_kv"] * ctx * cfg["hd"] * 4
    return params * 0.625, kv, params


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 50 ms during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            self.t.join(2)

    def summary(self):
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=reasons, samples=len(sm))


# ----------------------------------------------------------------------------- CUDA arm
def build_decoder(cfg, max_ctx, rank, world, ctx0):
    import torch
    from cpp_tensorlib_b200.decoder import Q4Decoder
    d = Q4Decoder(cfg, max_ctx, rank, world)
    sh = linear_shapes(cfg)

    def rnd(tag, shape, std, mean=0.0):
        g = torch.Generator(device="cuda").manual_seed(SEED * 1000003 + tag)
        return torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * std + mean
    d.set_vector_full(0, "embed", rnd(1, (cfg["vocab"], cfg["hidden"]), 0.02))
    d.set_vector_full(0, "onorm", rnd(2, (cfg["hidden"],), 0.02, 1.0))
    d.set_linear_full(0, "lm_head", rnd(3, sh["lm_head"], 0.02))
    HD = cfg["hd"]
    for l in range(cfg["layers"]):
        b = 100 + 20 * l
        for i, n in enumerate(("wqkv", "wo", "wgu", "wd")):
            d.set_linear_full(l, n, rnd(b + i, sh[n], 0.02))
        d.set_vector_full(l, "bq", rnd(b + 5, (cfg["n_q"] * HD,), 0.02))
        d.set_vector_full(l, "bk", rnd(b + 6, (cfg["n_kv"] * HD,), 0.02))
        d.set_vector_full(l, "bv", rnd(b + 7, (cfg["n_kv"] * HD,), 0.02))
        d.set_vector_full(l, "an", rnd(b + 8, (cfg["hidden"],), 0.02, 1.0))
        d.set_vector_full(l, "fn", rnd(b + 9, (cfg["hidden"],), 0.02, 1.0))
        if ctx0:
            d.fill_kv(l, rnd(b + 10, (cfg["n_kv"], ctx0, HD), 1.0), rnd(b + 11, (cfg["n_kv"], ctx0, HD), 1.0))
    torch.cuda.synchronize()
    return d


def gemv_sweep(cfg, dec, reps):
    """The packed int4 GEMV kernel alone over one token's weight matrices (28 x {qkv, o,
    gate|up, down} + lm_head = 4.42 GB at 7B, HBM-cold because the set is far larger
    than L2), launched back to back eagerly and bracketed by CUDA events on the
    launching stream.  Returns (bytes per pass, ms per pass, launches per pass, estimated DRAM
    traffic per pass)."""
    import torch
    from cpp_tensorlib_b200 import cuda as tlc
    names = ("wqkv", "wo", "wgu", "wd")
    keys = [(l, n) for l in range(cfg["layers"]) for n in names] + [(0, "lm_head")]
    ws = [dec._keep[k] for k in keys]
    xs = {w.K: torch.randn(w.K, device="cuda") for w in ws}
    ys = {w.N: torch.empty(w.N, device="cuda") for w in ws}
    one = lambda w: w.N * w.K * 0.625 + 4 * w.K + 4 * w.N
    nbytes = sum(one(w) for w in ws)
    traffic = sum(one(w) * TRAFFIC_FACTORS[k[1]] for k, w in zip(keys, ws))
    ws = [tlc.Q4Packed(w) for w in ws]          # the layout the decoder's linears stream
    for w in ws:
        tlc.gemv_q4p(xs[w.K], w, y=ys[w.N])
    torch.cuda.synchronize()
    # one pass recorded into a CUDA graph so host launch cost does not gate the GPU
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for w in ws:
                tlc.gemv_q4p(xs[w.K], w, y=ys[w.N])
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return nbytes, e0.elapsed_time(e1) / reps, len(ws), traffic


def cpu_sample(cfg, steps, warmup, note, layers=1):
    """The reference's own CPU code (compiled from its headers into oracle/_ref) --
    or the C restatement when that was never built -- on a bounded sample: `layers`
    of the model's layers at the 7B shape (+ a 1024-row lm_head), cache pre-filled to
    ctx 4096.  One sample step = one token through that slice.  Returns the measured
    per-step seconds and what is needed to extrapolate to the full model."""
    import numpy as np
    import oracle
    ref = oracle.load_ref()
    one = dict(cfg, layers=layers, vocab=1024)
    rng = np.random.default_rng(SEED)
    f = lambda *s: (rng.standard_normal(s, dtype=np.float32) * 0.02)
    sh = linear_shapes(one)
    total = CTX0 + steps + warmup + 1
    if ref is not None:
        d, kind, cores = oracle.RefDecoder(ref, one, total), "reference", ref.threads()
        lin = lambda w: w
    else:
        port = oracle.load_port()
        d, kind, cores = oracle.PortDecoder(port, one, total), "port", os.cpu_count()
        lin = port.to_q4
    d.set_embed(f(one["vocab"], one["hidden"]))
    d.set_vector(0, 5, 1 + f(one["hidden"]))
    d.set_linear(0, 4, lin(f(*sh["lm_head"])))
    HD = one["hd"]
    for l in range(layers):
        for i, n in enumerate(("wqkv", "wo", "wgu", "wd")):
            d.set_linear(l, i, lin(f(*sh[n])))
        for i, n in ((0, one["hidden"]), (1, one["hidden"]), (2, one["n_q"] * HD), (3, one["n_kv"] * HD), (4, one["n_kv"] * HD)):
            d.set_vector(l, i, (1 if i < 2 else 0) + f(n))
        d.fill_kv(l, rng.standard_normal((one["n_kv"], CTX0, HD), dtype=np.float32),
                  rng.standard_normal((one["n_kv"], CTX0, HD), dtype=np.float32))
    tok, times = 1, []
    for s in range(warmup + steps):
        t0 = time.perf_counter()
        tok, _ = d.step(tok, CTX0 + s, want_logits=False)
        times.append(time.perf_counter() - t0)
    d.close()
    _, _, params = token_bytes(cfg, CTX0)
    sample_params = layers * sum(sh[n][0] * sh[n][1] for n in ("wqkv", "wo", "wgu", "wd")) + \
        sh["lm_head"][0] * sh["lm_head"][1]
    return dict(times=times[warmup:], factor=params / sample_params, kind=kind, cores=cores,
                what=f"{layers} of {cfg['layers']} layers (+1024-row lm_head) at the 7B shape, ctx 4096; {note}")


def cpu_baseline_block(cfg, steps, warmup, note):
    r = cpu_sample(cfg, steps, warmup, note)
    t = min(r["times"])
    return dict(value=1.0 / (t * r["factor"]), unit="tokens/s", cores=r["cores"], kind=r["kind"],
                sample=f"{r['what']}; {steps} sample tokens, min {t * 1e3:.0f} ms per sample token, "
                       f"extrapolated to the model by parameter count ({r['factor']:.1f}x)")


def gpu_reference_rows(quick):
    """The reference's OWN CUDA kernels (its PTX JIT-compiled for this GPU, reached through its
    own headers: oracle/_ref/ref_gpu_bench) on the BASELINE shapes: microseconds and GB/s per
    launch, HBM-cold.  None where the binary was never built."""
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_gpu_bench")
    if not os.path.exists(exe):
        return None
    try:
        r = subprocess.run([exe] + (["--quick"] if quick else []), capture_output=True, text=True, timeout=600)
    except Exception as e:
        return dict(error=str(e))
    rows = []
    for l in r.stdout.splitlines():
        if l.startswith("{"):
            try:
                rows.append(json.loads(l))
            except ValueError:
                pass
    return dict(rows=rows, what="reference kernels (tl_gemv_q4, tl_attn_decode_split + tl_attn_combine) "
                                "JIT-compiled from the reference's PTX on this GPU, one CUDA graph of rotating "
                                "operand copies per shape, wall clock / launches, median of 7")


def run_reference(args, rank):
    """Reference arm: the reference's own CPU implementation of the path on this box's host
    cores.  A step is ONE token through a bounded slice of the workload (1 of the 28 layers
    at the 7B shape + a 1024-row lm_head, cache at ctx 4096); exactly --steps of them are
    timed after --warmup untimed ones.  `ms_per_step` is that MEASURED sample step; `value`
    is the full-model tokens/s extrapolated from it by parameter count, and says so."""
    if rank != 0:
        return
    note = ("pool = hardware_concurrency threads, but the M=1 SGEMM and the attention / dequant loops "
            "of the reference are single-threaded")
    K, W = max(1, args.steps), max(0, args.warmup)
    r = cpu_sample(QWEN7, K, W, note)
    ms = statistics.mean(r["times"]) * 1e3
    value = 1e3 / (ms * r["factor"])
    # is the cost per layer linear?  Two layers, three tokens.
    r2 = cpu_sample(QWEN7, 3, 1, note, layers=2)
    base = dict(value=value, unit="tokens/s", cores=r["cores"], kind=r["kind"],
                sample=f"{r['what']}; {K} sample tokens timed after {W} warm-up, mean {ms:.0f} ms per sample token")
    line = dict(impl="reference", metric="7B-shape int4 decode tok/s", value=value, unit="tokens/s",
                n_gpus=args.gpus, steps=K, warmup=W, ms_per_step=ms,
                higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f32 compute on int4 weights",
                data="synthetic", config=config_block(args.gpus), cpu_baseline=base,
                extrapolated_from=r["what"], factor=r["factor"],
                ms_per_token_full_model_extrapolated=ms * r["factor"],
                linearity_check=dict(one_layer_ms=min(r["times"]) * 1e3, two_layer_ms=min(r2["times"]) * 1e3,
                                     note="sample token through 1 and through 2 layers (+ the same 1024-row lm_head)"),
                e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_reference=gpu_reference_rows(quick=False))
    print(json.dumps(line), flush=True)


def config_block(n):
    return dict(workload="Qwen2.5-7B-architecture int4 decoder (BASELINE config 5): hidden 3584, 28 layers, "
                         "28q/4kv heads, head_dim 128, ff 18944, vocab 152064, batch 1, KV pre-filled to ctx 4096, "
                         "greedy decode, seed 4",
                parallelism=f"tp{n}", ctx=CTX0,
                l2="inputs larger than L2 (4.4 GB of weights streamed per token vs 126 MB L2)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="diagnostic: fewer layers (line is marked invalid)")
    ap.add_argument("--prefill", type=int, default=0,
                    help="diagnostic: time the batched prompt pass over this many tokens and exit")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank)

    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from cpp_tensorlib_b200 import check, lib
    check(lib().tlb_init(local))
    cfg = dict(QWEN7)
    if args.layers:
        cfg["layers"] = args.layers
    K, W = args.steps, max(3, args.warmup)
    max_ctx = CTX0 + max(128, K + W) + 8      # every region restarts at ctx 4096
    dec = build_decoder(cfg, max_ctx, rank, world, CTX0)
    dec.connect()
    if args.prefill:
        # diagnostic, not the bench line: the batched prompt pass (tensor-core int4 GEMM for
        # the projections, tiled causal attention) from an empty cache, single GPU
        T = args.prefill
        ids = [int(v) for v in torch.randint(0, cfg["vocab"], (T,), generator=torch.Generator().manual_seed(SEED))]
        times = []
        for _ in range(3):
            dec.set_pos(0)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            dec.prefill(ids)
            times.append(time.perf_counter() - t0)
        best = min(times)
        print(json.dumps(dict(diagnostic="batched prefill", T=T, layers=cfg["layers"], ms=best * 1e3,
                              tokens_per_s=T / best, ms_per_layer=best * 1e3 / cfg["layers"])), flush=True)
        dec.close()
        return
    dec.set_pos(CTX0)
    dec.set_token(1)
    dec.capture()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident greedy decoding: W warm-up tokens, then REPEATS timed regions of
    # exactly K tokens each (every region restarts at ctx 4096 from token 1, so all regions
    # do the same work; each is bracketed by barrier + synchronize on both sides and timed
    # with CUDA events on the launching stream, max over ranks).  The line reports the
    # median region; min and max are given beside it so that a change of 1-2 % can be told
    # from noise.
    REPEATS = 5
    barrier()
    dec.run(W)
    barrier()
    region_ms = []
    with ClockSampler(local) as clk:
        for _ in range(REPEATS):
            dec.set_pos(CTX0)
            dec.set_token(1)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dec.run(K)
            e1.record()
            barrier()
            ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            region_ms.append(float(ms.item()))
    ms_total = statistics.median(region_ms)
    last = dec.last_token()

    # ---- end to end through the host-buffer call: id H2D, graph, id D2H, per token
    dec.set_pos(CTX0)
    tok = 1
    for _ in range(3):
        tok = dec.step(tok)
    dec.set_pos(CTX0)
    barrier()
    t0 = time.perf_counter()
    tok, ids = 1, []
    for _ in range(K):
        tok = dec.step(tok)
        ids.append(tok)
    torch.cuda.synchronize()
    e2e_s = torch.tensor([time.perf_counter() - t0], device="cuda")
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_tps = K / float(e2e_s.item())
    import hashlib
    import struct
    ids_sha = hashlib.sha256(struct.pack(f"<{len(ids)}i", *ids)).hexdigest()[:16]

    # ---- roofline of the dominant kernel (per rank: its own shards)
    peak, peak_src = measured_peaks()
    gbytes, gms, glaunch, gtraffic = gemv_sweep(cfg, dec, 5)
    wbytes, kvbytes, _ = token_bytes(cfg, CTX0)
    achieved = gbytes / (gms * 1e-3) / 1e9
    tok_bytes = (wbytes + kvbytes) / world
    tok_ach = tok_bytes / (ms_total / K * 1e-3) / 1e9

    st = (__import__("ctypes").c_int * 2)()
    status = lib().tlb_device_status(st, 0)
    launches = dec.launches_per_token() * K
    dec.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        line = dict(metric="7B-shape int4 decode tok/s", value=K / (ms_total * 1e-3), unit="tokens/s",
                    n_gpus=world, steps=K, warmup=W, ms_per_step=ms_total / K, higher_is_better=True,
                    scaling="strong", vs_baseline=None, dtype="f32 compute on int4 weights",
                    data="synthetic", config=config_block(world), clocks=clk.summary(),
                    repeats=dict(n=REPEATS, statistic="median", ms_per_step_min=min(region_ms) / K,
                                 ms_per_step_max=max(region_ms) / K),
                    e2e=dict(value=e2e_tps, unit="tokens/s", h2d_bytes_per_step=4, d2h_bytes_per_step=4),
                    gpu_launches=launches,
                    roofline=dict(bound="hbm", achieved=achieved, peak=peak, unit="GB/s", frac=achieved / peak,
                                  traffic=gtraffic, peak_source=peak_src, kernel="gemv_q4p_kernel",
                                  traffic_factors=TRAFFIC_FACTORS, traffic_note=TRAFFIC_NOTE,
                                  what=f"{glaunch} int4 GEMV launches of one token ({gbytes / 1e9:.2f} GB algorithmic), "
                                       f"{gms:.3f} ms per pass, CUDA events"),
                    token_roofline=dict(bound="hbm", achieved=tok_ach, peak=peak, frac=tok_ach / peak, unit="GB/s",
                                        bytes_per_token_per_gpu=tok_bytes),
                    last_token=last, decoded_ids_sha=ids_sha, decoded_ids_head=ids[:8], device_status=int(status))
        # The line is only a measurement if the decode was right: the device-resident loop and
        # the host-buffer loop start from the same token and position, so they must end on the
        # same token, and no bounded wait may have expired.
        if ids[-1] != last:
            line["invalid"] = f"device-resident loop ended on token {last}, host-buffer loop on {ids[-1]}"
        elif status != 0:
            line["invalid"] = f"device status {int(status)} (where = {st[1]})"
        if args.layers:
            line["invalid"] = "diagnostic run with fewer layers than the named config"
        # CPU baseline: at N = 1 only, after the GPU work is done and the process group is gone
        if world == 1 and not args.no_cpu_baseline:
            try:
                line["cpu_baseline"] = cpu_baseline_block(QWEN7, 3, 1, "M=1 path of the reference is single-threaded")
            except Exception as e:  # the checker is optional at run time; say so instead of dying
                line["cpu_baseline"] = dict(value=None, unit="tokens/s", cores=0, kind="unavailable", sample=str(e))
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
