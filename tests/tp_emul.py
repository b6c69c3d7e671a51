"""Tensor-parallel decoder step on the host, built from the oracle port's ops and
the product's shard plan / q4 slicing.  It lets the CPU suite check the sharding
arithmetic (which rows and K-slices each rank owns, uneven head splits, vocabulary
offsets) with any all-reduce: an in-process rank loop or gloo ranks."""
import numpy as np
import torch

import cases
from cpp_tensorlib_b200 import decoder as dec
from cpp_tensorlib_b200.cuda import Q4Weight


def q4_cpu(port, w_kn):
    K, N = w_kn.shape
    return Q4Weight(torch.from_numpy(port.to_q4(w_kn)), K, N)


class RankState:
    """One rank's shards (numpy q4 bytes) and KV cache."""

    def __init__(self, port, cfg, weights, tp_size, rank, max_ctx):
        self.port, self.cfg, self.rank, self.tp = port, cfg, rank, tp_size
        self.plan = p = dec.shard_plan(cfg, tp_size, rank)
        self.embed, self.onorm = weights["embed"], weights["onorm"]
        sh = lambda name, w: dec.shard_linear(name, q4_cpu(port, w), cfg, p) if tp_size > 1 else q4_cpu(port, w)
        self.lm = sh("lm_head", weights["lm_head"])
        self.layers = []
        for L in weights["layers"]:
            d = {n: sh(n, L[n]) for n in ("wqkv", "wo", "wgu", "wd")}
            for n in ("bq", "bk", "bv", "an", "fn"):
                d[n] = dec.shard_vector(n, torch.from_numpy(L[n]), cfg, p).numpy()
            d["K"] = np.zeros((p["n_kv"], max_ctx, cfg["hd"]), np.float32)
            d["V"] = np.zeros_like(d["K"])
            self.layers.append(d)

    def mv(self, x, wq):
        return self.port.gemm_q4(x.reshape(1, -1), wq.buf.numpy(), wq.N)[0]


def tp_step(ranks, token, pos, allreduce):
    """ranks: the RankState objects this process simulates.  allreduce(list of
    partial vectors, one per simulated rank) -> the summed vector (rank order)."""
    cfg, port = ranks[0].cfg, ranks[0].port
    HD = cfg["hd"]
    x = ranks[0].embed[token].copy()
    hb = port.rmsnorm(x, ranks[0].layers[0]["an"], cfg["eps"])
    for l in range(cfg["layers"]):
        parts = []
        for R in ranks:
            L, p = R.layers[l], R.plan
            qkv = R.mv(hb, L["wqkv"])
            nq, nkv = p["n_q"], p["n_kv"]
            q = port.rope(qkv[:nq * HD].reshape(nq, HD), pos, cfg["rope_base"], bias=L["bq"].reshape(nq, HD))
            k = port.rope(qkv[nq * HD:(nq + nkv) * HD].reshape(nkv, HD), pos, cfg["rope_base"],
                          bias=L["bk"].reshape(nkv, HD))
            v = qkv[(nq + nkv) * HD:] + L["bv"]
            L["K"][:, pos], L["V"][:, pos] = k, v.reshape(nkv, HD)
            att = port.attn_decode(q, L["K"], L["V"], 1.0 / np.sqrt(np.float32(HD)), ctx=pos + 1)
            parts.append(R.mv(att.reshape(-1), L["wo"]))
        x, hb = port.add_rmsnorm(x, allreduce(parts), ranks[0].layers[l]["fn"], cfg["eps"])
        parts = []
        for R in ranks:
            L, p = R.layers[l], R.plan
            gu = R.mv(hb, L["wgu"])
            parts.append(R.mv(port.swiglu(gu, p["ff_local"])[0], L["wd"]))
        nextw = ranks[0].layers[l + 1]["an"] if l + 1 < cfg["layers"] else ranks[0].onorm
        x, hb = port.add_rmsnorm(x, allreduce(parts), nextw, cfg["eps"])
    logits = [(R.plan["vocab"][0], R.mv(hb, R.lm)) for R in ranks]
    return logits


def full_logits(local):
    """Concatenate (offset, shard) pairs gathered from all ranks."""
    return np.concatenate([s for _, s in sorted(local, key=lambda t: t[0])])
