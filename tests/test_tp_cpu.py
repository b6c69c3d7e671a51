"""Host-side tensor-parallel logic on CPU: the shard plan, q4 shard slicing, and
the sharded decoder arithmetic -- in-process for tp 2/4/8 (uneven heads, replicated
KV heads) and as two gloo ranks."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
import oracle
import tp_emul
from cpp_tensorlib_b200 import decoder as dec

# 28 q / 4 kv heads like the 7B shape (so tp 8 exercises 4+3 q heads per KV head), small dims
TP_CFG = dict(hidden=256, layers=2, n_q=28, n_kv=4, hd=64, ff=1024, vocab=200, eps=1e-6, rope_base=1e6)


def test_shard_plan_covers_everything():
    for cfg in (cases.QWEN7, cases.QWEN05, TP_CFG):
        for tp in (1, 2, 4, 8):
            if cfg is cases.QWEN05 and tp > 2 and (tp % cfg["n_kv"] or cfg["n_q"] // cfg["n_kv"] < tp // cfg["n_kv"]):
                continue
            plans = [dec.shard_plan(cfg, tp, r) for r in range(tp)]
            assert sum(p["n_q"] for p in plans) == cfg["n_q"]
            q = sorted(p["q"] for p in plans)
            assert q[0][0] == 0 and q[-1][1] == cfg["n_q"] and all(a[1] == b[0] for a, b in zip(q, q[1:]))
            f = [p["ff"] for p in plans]
            assert f[0][0] == 0 and f[-1][1] == cfg["ff"] and all(a[1] == b[0] for a, b in zip(f, f[1:]))
            assert all((b - a) % 32 == 0 for a, b in f)
            v = [p["vocab"] for p in plans]
            assert v[0][0] == 0 and v[-1][1] == cfg["vocab"]
            grp = cfg["n_q"] // cfg["n_kv"]
            for p in plans:                      # every local q head reads a local KV head
                assert p["q"][0] // grp >= p["kv"][0] and (p["q"][1] - 1) // grp < p["kv"][1]
                assert p["n_q"] % p["n_kv"] == 0
    p8 = [dec.shard_plan(cases.QWEN7, 8, r) for r in range(8)]
    assert [p["n_q"] for p in p8] == [4, 3, 4, 3, 4, 3, 4, 3]
    assert [p["ff_local"] for p in p8] == [2432] * 4 + [2304] * 4
    with pytest.raises(ValueError):
        dec.shard_plan(dict(cases.QWEN7, n_kv=3, n_q=27), 2, 0)


def test_q4_slices_dequantise_to_slices_of_the_full_matrix(port):
    import synth
    K, N = 256, 96
    w = synth.normal(80, 1, (K, N), 0.05)
    wq = tp_emul.q4_cpu(port, w)
    full = port.q4_to_f32(wq.buf.numpy(), K, N)
    rows = dec.slice_q4_rows(wq, [(8, 24), (40, 41), (90, 96)])
    got = port.q4_to_f32(rows.buf.numpy(), K, rows.N)
    assert np.array_equal(got, np.concatenate([full[:, 8:24], full[:, 40:41], full[:, 90:96]], 1))
    ks = dec.slice_q4_k(wq, [(32, 96), (224, 256)])
    got = port.q4_to_f32(ks.buf.numpy(), ks.K, N)
    assert np.array_equal(got, np.concatenate([full[32:96], full[224:256]], 0))
    with pytest.raises(ValueError):
        dec.slice_q4_k(wq, [(16, 64)])


def _reference_run(port, cfg, weights, prompt, max_ctx):
    d = oracle.PortDecoder(port, cfg, max_ctx)
    d.set_embed(weights["embed"]); d.set_vector(0, 5, weights["onorm"])
    d.set_linear(0, 4, port.to_q4(weights["lm_head"]))
    for l, L in enumerate(weights["layers"]):
        for k, i in cases.LINEAR_IDS.items():
            d.set_linear(l, i, port.to_q4(L[k]))
        for k, i in cases.VECTOR_IDS.items():
            d.set_vector(l, i, L[k])
    out = [d.step(t, i) for i, t in enumerate(prompt)]
    d.close()
    return out


@pytest.mark.parametrize("tp", [2, 4, 8])
def test_sharded_decoder_matches_unsharded(port, tp):
    weights = cases.decoder_weights(TP_CFG, 33)
    prompt = [3, 150, 42, 7]
    want = _reference_run(port, TP_CFG, weights, prompt, 16)
    ranks = [tp_emul.RankState(port, TP_CFG, weights, tp, r, 16) for r in range(tp)]
    ar = lambda parts: np.sum(np.stack(parts).astype(np.float32), axis=0, dtype=np.float32)
    for i, t in enumerate(prompt):
        lg = tp_emul.full_logits(tp_emul.tp_step(ranks, t, i, ar))
        assert np.allclose(lg, want[i][1], rtol=1e-3, atol=1e-3)
        assert int(np.argmax(lg)) == want[i][0]


def _gloo_worker(rank, world, port_file, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port_file))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    port = oracle.load_port()
    weights = cases.decoder_weights(TP_CFG, 33)
    R = tp_emul.RankState(port, TP_CFG, weights, world, rank, 16)

    def ar(parts):
        t = torch.from_numpy(parts[0].copy())
        dist.all_reduce(t)
        return t.numpy()
    toks = []
    for i, tkn in enumerate([3, 150, 42, 7]):
        off, lg = tp_emul.tp_step([R], tkn, i, ar)[0]
        # vocabulary-parallel argmax: exchange (value, global index) pairs
        best = torch.tensor([float(lg.max()), float(off + int(np.argmax(lg)))], dtype=torch.float64)
        allb = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(allb, best)
        toks.append(int(max(allb, key=lambda b: (b[0].item(), -b[1].item()))[1].item()))
    if rank == 0:
        q.put(toks)
    dist.destroy_process_group()


def test_two_gloo_ranks_agree_with_unsharded(port):
    want = [t for t, _ in _reference_run(port, TP_CFG, cases.decoder_weights(TP_CFG, 33), [3, 150, 42, 7], 16)]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); prt = s.getsockname()[1]; s.close()
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, prt, q)) for r in range(2)]
    [p.start() for p in procs]
    got = q.get(timeout=120)
    [p.join(60) for p in procs]
    assert got == want


def test_host_barrier_reports_the_missing_rank():
    """Failure detection on the host (no GPU involved): the ranks that arrive learn, after the
    timeout, which rank did not, instead of launching kernels that would wait for it."""
    import threading
    from cpp_tensorlib_b200 import TlbError
    store = dist.HashStore()
    with pytest.raises(TlbError, match=r"rank\(s\) \[1\] of 2"):
        dec.host_barrier(store, "lonely", 0, 2, timeout_s=0.3)
    # everybody arrives: both return
    errs = []

    def arrive(r):
        try:
            dec.host_barrier(store, "full", r, 3, timeout_s=20.0)
        except Exception as e:  # pragma: no cover - reported below
            errs.append(e)
    ts = [threading.Thread(target=arrive, args=(r,)) for r in range(3)]
    [t.start() for t in ts]
    [t.join(30) for t in ts]
    assert not errs


def _barrier_worker(rank, world, prt, q):
    from datetime import timedelta
    store = dist.TCPStore("127.0.0.1", prt, world, is_master=(rank == 0), timeout=timedelta(seconds=30))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
    dist.barrier()                       # both ranks are alive here
    if rank == 1:
        # the rank fails on the host between steps: it raises and never reaches the next exchange
        q.put(("rank1", "left"))
        q.close(); q.join_thread()
        os._exit(0)
    try:
        dec.host_barrier(store, "step2", rank, world, timeout_s=1.0)
        q.put(("rank0", "no error"))
    except Exception as e:
        q.put(("rank0", str(e)))
    q.close(); q.join_thread()
    os._exit(0)


def test_gloo_rank_that_leaves_is_detected_by_the_host_barrier():
    import socket
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    s = socket.socket(); s.bind(("127.0.0.1", 0)); prt = s.getsockname()[1]; s.close()
    procs = [ctx.Process(target=_barrier_worker, args=(r, 2, prt, q)) for r in range(2)]
    [p.start() for p in procs]
    got = dict(q.get(timeout=120) for _ in range(2))
    [p.join(60) for p in procs]
    assert got["rank1"] == "left"
    assert "rank(s) [1] of 2 did not arrive" in got["rank0"], got
