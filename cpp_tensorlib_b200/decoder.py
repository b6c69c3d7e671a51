"""Host side of the Qwen2.5-architecture int4 decoder: the shard plan for tensor
parallelism, q4 shard slicing, and a thin handle on the native driver
(``tlb_decoder_*`` in include/tlb200.h).

Structure follows the reference's model driver (bench/cuda/qwen_model.h: fused
QKV and gate|up weights by concatenation :85-142, Layer/Scratch/Model :175-308,
run_layers_ :673-740, captured_decoder :791-905); the reference is single-device,
so the shard plan and the exchange wiring have no counterpart there.
"""
import ctypes as C
import time

import numpy as np
import torch

from ._lib import TlbError, check, lib
from .cuda import Q4Weight, q4_bytes, to_q4

LINEAR = dict(wqkv=0, wo=1, wgu=2, wd=3, lm_head=4)
VECTOR = dict(an=0, fn=1, bq=2, bk=3, bv=4, onorm=5, embed=6)


def _split_even(total, parts, unit=1):
    """Split `total` (a multiple of `unit`) into `parts` contiguous ranges whose
    sizes are multiples of `unit` and differ by at most one unit."""
    assert total % unit == 0
    blocks = total // unit
    out, start = [], 0
    for r in range(parts):
        n = blocks // parts + (1 if r < blocks % parts else 0)
        out.append((start * unit, (start + n) * unit))
        start += n
    return out


def shard_plan(cfg, tp_size, rank):
    """Which slice of the model a rank owns.

    Column-parallel (split the output dim): q/k/v projections by heads, gate|up by
    ff columns, lm_head by vocabulary.  Row-parallel (split the input dim): wo by
    the rank's q heads, down by the rank's ff range.  When there are fewer KV heads
    than ranks each KV head (and its cache) is replicated on the tp_size/n_kv ranks
    that share it and that group's q heads are divided among them (28 q / 4 kv on 8
    ranks -> 4,3,4,3,...).  ff ranges are multiples of 128 so every K-slice keeps
    the 16-byte row alignment the TMA path needs.
    """
    NQ, NKV, FF, V = cfg["n_q"], cfg["n_kv"], cfg["ff"], cfg["vocab"]
    grp = NQ // NKV
    if tp_size <= NKV:
        if NKV % tp_size:
            raise ValueError("n_kv must be divisible by tp_size when tp_size <= n_kv")
        kv0, kv1 = _split_even(NKV, tp_size)[rank]
        q0, q1 = kv0 * grp, kv1 * grp
    else:
        if tp_size % NKV:
            raise ValueError("tp_size must be a multiple of n_kv when tp_size > n_kv")
        rep = tp_size // NKV
        kvh, sub = rank // rep, rank % rep
        if grp < rep:
            raise ValueError("more ranks per KV head than q heads in its group")
        a, b = _split_even(grp, rep)[sub]
        kv0, kv1 = kvh, kvh + 1
        q0, q1 = kvh * grp + a, kvh * grp + b
    ff_unit = 128 if FF % 128 == 0 else 32
    f0, f1 = _split_even(FF, tp_size, ff_unit)[rank]
    v0, v1 = _split_even(V, tp_size)[rank]
    return dict(q=(q0, q1), kv=(kv0, kv1), ff=(f0, f1), vocab=(v0, v1),
                n_q=q1 - q0, n_kv=kv1 - kv0, ff_local=f1 - f0, vocab_local=v1 - v0)


def _views(wq):
    K, N = wq.K, wq.N
    packed = wq.buf[:N * K // 2].view(N, K // 2)
    scales = wq.buf[N * K // 2:].view(N, K // 8)   # bytes of the f32 scales
    return packed, scales


def slice_q4_rows(wq, ranges):
    """Column-parallel shard: keep output rows [a,b) for each range, in order.
    Quantise-then-slice, so the shard dequantises to the same values as the full
    matrix (groups run along K and are untouched)."""
    packed, scales = _views(wq)
    p = torch.cat([packed[a:b] for a, b in ranges]).contiguous().view(-1)
    s = torch.cat([scales[a:b] for a, b in ranges]).contiguous().view(-1)
    n = sum(b - a for a, b in ranges)
    return Q4Weight(torch.cat([p, s]), wq.K, n)


def slice_q4_k(wq, ranges):
    """Row-parallel shard: keep input columns [k0,k1) (multiples of 32) of every
    output row, repacked contiguously."""
    packed, scales = _views(wq)
    for a, b in ranges:
        if a % 32 or b % 32:
            raise ValueError("K-slices must be multiples of the q4 group (32)")
    p = torch.cat([packed[:, a // 2:b // 2] for a, b in ranges], dim=1).contiguous().view(-1)
    s = torch.cat([scales[:, a // 8:b // 8] for a, b in ranges], dim=1).contiguous().view(-1)
    k = sum(b - a for a, b in ranges)
    return Q4Weight(torch.cat([p, s]), k, wq.N)


def shard_linear(name, wq, cfg, plan):
    """The rank's shard of one full-model q4 linear (logical [K, N])."""
    HD, NQ, NKV, FF = cfg["hd"], cfg["n_q"], cfg["n_kv"], cfg["ff"]
    (q0, q1), (k0, k1), (f0, f1), (v0, v1) = plan["q"], plan["kv"], plan["ff"], plan["vocab"]
    if name == "wqkv":
        ko, vo = NQ * HD, (NQ + NKV) * HD
        return slice_q4_rows(wq, [(q0 * HD, q1 * HD), (ko + k0 * HD, ko + k1 * HD),
                                  (vo + k0 * HD, vo + k1 * HD)])
    if name == "wo":
        return slice_q4_k(wq, [(q0 * HD, q1 * HD)])
    if name == "wgu":
        return slice_q4_rows(wq, [(f0, f1), (FF + f0, FF + f1)])
    if name == "wd":
        return slice_q4_k(wq, [(f0, f1)])
    if name == "lm_head":
        return slice_q4_rows(wq, [(v0, v1)])
    raise KeyError(name)


def shard_vector(name, v, cfg, plan):
    HD = cfg["hd"]
    if name == "bq":
        return v[plan["q"][0] * HD:plan["q"][1] * HD].contiguous()
    if name in ("bk", "bv"):
        return v[plan["kv"][0] * HD:plan["kv"][1] * HD].contiguous()
    return v


def host_barrier(store, name, rank, world, timeout_s=60.0, poll_s=0.01):
    """Arrival check of the tensor-parallel ranks on the HOST, before anything that would make
    their GPUs wait for one another is launched: every rank posts a key in the c10d store and
    polls for the others'.  A rank that died, hung or never started is reported by the ranks
    that did arrive as a ``TlbError`` naming it, after `timeout_s`, instead of a device-side
    spin on a peer that will never write.  (The device-side waits are bounded too; this check
    keeps them from being reached.)"""
    store.set(f"{name}/{rank}", b"1")
    deadline = time.monotonic() + timeout_s
    while True:
        missing = [r for r in range(world) if not store.check([f"{name}/{r}"])]
        if not missing:
            return
        if time.monotonic() > deadline:
            raise TlbError(f"host barrier '{name}': rank(s) {missing} of {world} did not arrive "
                           f"within {timeout_s:.1f} s")
        time.sleep(poll_s)


class Q4Decoder:
    """Handle on the native decoder.  Weights are device tensors kept alive here
    (the native side borrows their pointers)."""

    def __init__(self, cfg, max_ctx, tp_rank=0, tp_size=1, kv_dtype="f32"):
        """kv_dtype "bf16": the KV caches hold bf16 (kv_cache::init with dtype::bf16,
        include/cuda.h:1336-1346): half the KV stream, rows rounded to nearest even on append."""
        if kv_dtype not in ("f32", "bf16"):
            raise ValueError("kv_dtype must be 'f32' or 'bf16'")
        self.kv_bf16 = kv_dtype == "bf16"
        self.cfg, self.max_ctx, self.tp_rank, self.tp_size = dict(cfg), max_ctx, tp_rank, tp_size
        self.plan = shard_plan(cfg, tp_size, tp_rank)
        p = self.plan
        arr = (C.c_int64 * 13)(cfg["hidden"], cfg["layers"], p["n_q"], p["n_kv"], cfg["hd"],
                               p["ff_local"], p["vocab_local"], max_ctx, tp_rank, tp_size,
                               p["vocab"][0], cfg["vocab"], 1 if self.kv_bf16 else 0)
        self.h = C.c_void_p()
        check(lib().tlb_decoder_create(arr, 13, cfg["eps"], cfg["rope_base"], C.byref(self.h)))
        self._keep = {}
        self.captured = False

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    # ---- weights ---------------------------------------------------------------
    def set_linear_full(self, layer, name, w):
        """w: full-model weight, either f32 [K, N] on the device (quantised here with
        to_q4) or a Q4Weight; sharded for this rank and installed."""
        wq = w if isinstance(w, Q4Weight) else to_q4(w)
        sh = shard_linear(name, wq, self.cfg, self.plan) if self.tp_size > 1 else wq
        self._keep[(layer, name)] = sh
        check(lib().tlb_decoder_set_linear(self.h, layer, LINEAR[name], sh.qw_ptr, sh.K, sh.N))

    def set_vector_full(self, layer, name, v):
        sh = shard_vector(name, v, self.cfg, self.plan).contiguous()
        self._keep[(layer, name)] = sh
        check(lib().tlb_decoder_set_vector(self.h, layer, VECTOR[name], C.c_void_p(sh.data_ptr())))

    def load(self, weights):
        """weights: dict as built by tests/cases.decoder_weights (numpy or torch)."""
        dev = lambda a: a if torch.is_tensor(a) else torch.from_numpy(np.ascontiguousarray(a)).cuda()
        self.set_vector_full(0, "embed", dev(weights["embed"]))
        self.set_vector_full(0, "onorm", dev(weights["onorm"]))
        self.set_linear_full(0, "lm_head", dev(weights["lm_head"]))
        for l, L in enumerate(weights["layers"]):
            for n in ("wqkv", "wo", "wgu", "wd"):
                self.set_linear_full(l, n, dev(L[n]))
            for n in ("an", "fn", "bq", "bk", "bv"):
                self.set_vector_full(l, n, dev(L[n]))

    def kv(self, layer):
        """The layer's K and V caches as torch views [n_kv_local, max_ctx, hd]."""
        K, V = C.c_void_p(), C.c_void_p()
        check(lib().tlb_decoder_kv(self.h, layer, C.byref(K), C.byref(V)))
        shape = (self.plan["n_kv"], self.max_ctx, self.cfg["hd"])
        if self.kv_bf16:
            return (_as_tensor(K.value, shape, "<u2").view(torch.bfloat16),
                    _as_tensor(V.value, shape, "<u2").view(torch.bfloat16))
        return _as_tensor(K.value, shape), _as_tensor(V.value, shape)

    def fill_kv(self, layer, K, V):
        """Pre-fill rows [0, n) of a layer's cache from full-model K, V [n_kv, n, hd]."""
        a, b = self.plan["kv"]
        Kc, Vc = self.kv(layer)
        n = K.shape[1]
        Kc[:, :n].copy_(K[a:b])
        Vc[:, :n].copy_(V[a:b])

    def logits(self):
        p = C.c_void_p()
        check(lib().tlb_decoder_logits(self.h, C.byref(p)))
        return _as_tensor(p.value, (self.plan["vocab_local"],))

    # ---- tensor-parallel wiring ------------------------------------------------
    def connect(self, group=None, store=None, timeout_s=60.0):
        """Exchange the ranks' 128-byte records over torch.distributed and open the
        peers' exchange buffers.  With a c10d `store` the ranks first meet in a host
        barrier with a timeout (`host_barrier`), so a missing rank is an error here and
        not a hang in the collective."""
        if self.tp_size == 1:
            return
        import torch.distributed as dist
        if store is not None:
            host_barrier(store, "tlb_connect", self.tp_rank, self.tp_size, timeout_s)
        rec = (C.c_ubyte * 128)()
        check(lib().tlb_decoder_ipc_export(self.h, rec))
        mine = torch.tensor(list(bytes(rec)), dtype=torch.uint8, device="cuda")
        allr = [torch.empty_like(mine) for _ in range(self.tp_size)]
        dist.all_gather(allr, mine, group=group)
        blob = b"".join(bytes(t.cpu().numpy().tobytes()) for t in allr)
        check(lib().tlb_decoder_ipc_open(self.h, blob))
        dist.barrier(group=group)

    # ---- running ---------------------------------------------------------------
    def set_pos(self, pos):
        check(lib().tlb_decoder_set_pos(self.h, pos, self._stream()))

    def set_token(self, tok):
        check(lib().tlb_decoder_set_token(self.h, int(tok), self._stream()))

    def forward(self):
        check(lib().tlb_decoder_forward(self.h, self._stream()))

    def capture(self):
        check(lib().tlb_decoder_capture(self.h))
        self.captured = True

    def run(self, n):
        check(lib().tlb_decoder_run(self.h, n, self._stream()))

    def step(self, token=None):
        """One token end to end with host buffers: id in, next id out."""
        tin = C.c_int32(-1 if token is None else int(token))
        tout = C.c_int32(0)
        check(lib().tlb_decoder_step(self.h, C.byref(tin), C.byref(tout), self._stream()))
        return int(tout.value)

    def prefill(self, tokens):
        """prefill_batched (bench/cuda/qwen_model.h:423-442): the whole prompt as row-batched
        GEMMs + tiled causal attention from the current position; returns the greedy next
        token, which is also left on the device for run()."""
        ids = (C.c_int32 * len(tokens))(*[int(t) for t in tokens])
        tout = C.c_int32(0)
        check(lib().tlb_decoder_prefill(self.h, ids, len(tokens), C.byref(tout), self._stream()))
        return int(tout.value)

    def last_token(self):
        t = C.c_int32(0)
        check(lib().tlb_decoder_last_token(self.h, C.byref(t), self._stream()))
        return int(t.value)

    def launches_per_token(self):
        return int(lib().tlb_decoder_launches_per_token(self.h))

    def close(self):
        if self.h:
            check(lib().tlb_decoder_destroy(self.h))
            self.h = None
            self._keep.clear()


class _Ext:
    """Wrap a raw device pointer for torch through the CUDA array interface."""

    def __init__(self, ptr, shape, typestr="<f4"):
        self.__cuda_array_interface__ = dict(shape=tuple(shape), typestr=typestr, data=(ptr, False),
                                             version=2)


def _as_tensor(ptr, shape, typestr="<f4"):
    return torch.as_tensor(_Ext(ptr, shape, typestr), device="cuda")
