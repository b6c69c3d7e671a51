"""ctypes bindings for the checkers (TEST INFRASTRUCTURE ONLY).

``port``  -- the plain-C restatement (``liborc.so`` from ``q4_oracle.c``).
``ref``   -- the reference itself compiled from its own headers
             (``_ref/libtlref.so``), or ``None`` where it was never built.

Only the tests, the smoke test and the CPU-baseline / reference legs of the
benchmark import this package; the product package never does.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_i64 = C.c_int64


def q4_bytes(N, K):
    return N * K // 2 + N * (K // 32) * 4


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Port:
    """Plain-C restatement of the reference algorithms."""

    def __init__(self, path):
        L = self.lib = C.CDLL(path)
        L.orc_to_q4.argtypes = [_f32p, _i64, _i64, _u8p]
        L.orc_to_q4.restype = C.c_int
        L.orc_q4_to_f32.argtypes = [_u8p, _i64, _i64, _f32p]
        L.orc_gemm_q4.argtypes = [_f32p, _i64, _i64, _u8p, _i64, C.c_float, C.c_float, _f32p]
        L.orc_attn_decode.argtypes = [_f32p, _f32p, _f32p, _i64, _i64, _i64, _i64, _i64,
                                      C.c_float, _f32p]
        L.orc_rope.argtypes = [_f32p, C.c_void_p, _i64, _i64, _i64, _i64, C.c_float, _f32p]
        L.orc_rmsnorm.argtypes = [_f32p, _f32p, _i64, _i64, C.c_float, _f32p]
        L.orc_add_rmsnorm.argtypes = [_f32p, _f32p, _f32p, _i64, _i64, C.c_float, _f32p, _f32p]
        L.orc_swiglu.argtypes = [_f32p, _i64, _i64, _f32p]
        L.orc_argmax.argtypes = [_f32p, _i64]
        L.orc_argmax.restype = _i64
        L.orc_decoder_create.argtypes = [_i64] * 8 + [C.c_float, C.c_float]
        L.orc_decoder_create.restype = C.c_void_p
        L.orc_decoder_destroy.argtypes = [C.c_void_p]
        L.orc_decoder_set_linear.argtypes = [C.c_void_p, _i64, C.c_int, _u8p]
        L.orc_decoder_set_vector.argtypes = [C.c_void_p, _i64, C.c_int, _f32p]
        L.orc_decoder_set_embed.argtypes = [C.c_void_p, _f32p]
        L.orc_decoder_fill_kv.argtypes = [C.c_void_p, _i64, _f32p, _f32p, _i64]
        L.orc_decoder_step.argtypes = [C.c_void_p, _i64, _i64, C.c_void_p]
        L.orc_decoder_step.restype = _i64
        L.orc_decoder_set_kv_bf16.argtypes = [C.c_void_p, C.c_int]
        L.orc_bf16_round_array.argtypes = [_f32p, _i64, _f32p]

    def to_q4(self, w_kn):
        w = _f(w_kn)
        K, N = w.shape
        out = np.empty(q4_bytes(N, K), np.uint8)
        if self.lib.orc_to_q4(w, K, N, out):
            raise ValueError("to_q4: K must be a multiple of 32")
        return out

    def q4_to_f32(self, q4, K, N):
        out = np.empty((K, N), np.float32)
        self.lib.orc_q4_to_f32(q4, K, N, out)
        return out

    def gemm_q4(self, x, q4, N, alpha=1.0, beta=0.0):
        x = _f(x).reshape(-1, x.shape[-1])
        M, K = x.shape
        out = np.empty((M, N), np.float32)
        self.lib.orc_gemm_q4(x, M, K, q4, N, alpha, beta, out)
        return out

    def attn_decode(self, q, K, V, scale, ctx=None):
        q, K, V = _f(q), _f(K), _f(V)
        Hq, D = q.shape
        Hkv, kv_max, _ = K.shape
        ctx = kv_max if ctx is None else ctx
        out = np.empty((Hq, D), np.float32)
        self.lib.orc_attn_decode(q, K, V, Hq, Hkv, ctx, kv_max, D, scale, out)
        return out

    def rope(self, x, pos, base, bias=None):
        x = _f(x)
        D = x.shape[-1]
        T = x.shape[1] if x.ndim == 3 else 1
        rows = x.size // D
        out = np.empty_like(x)
        b = None if bias is None else _f(bias)
        self.lib.orc_rope(x, None if b is None else b.ctypes.data, rows, T, D, pos, base, out)
        return out

    def rmsnorm(self, x, w, eps):
        x = _f(x)
        n = x.shape[-1]
        out = np.empty_like(x)
        self.lib.orc_rmsnorm(x, _f(w), x.size // n, n, eps, out)
        return out

    def add_rmsnorm(self, a, b, w, eps):
        a = _f(a)
        n = a.shape[-1]
        xo, ho = np.empty_like(a), np.empty_like(a)
        self.lib.orc_add_rmsnorm(a, _f(b), _f(w), a.size // n, n, eps, xo, ho)
        return xo, ho

    def swiglu(self, gu, ff):
        gu = _f(gu).reshape(-1, 2 * ff)
        out = np.empty((gu.shape[0], ff), np.float32)
        self.lib.orc_swiglu(gu, gu.shape[0], ff, out)
        return out

    def argmax(self, v):
        v = _f(v).ravel()
        return int(self.lib.orc_argmax(v, v.size))

    def bf16_round(self, v):
        v = _f(v)
        out = np.empty_like(v)
        self.lib.orc_bf16_round_array(v.ravel(), v.size, out.ravel())
        return out


class PortDecoder:
    """Qwen2.5-block decoder on the host with q4 linears (borrowed buffers kept alive here)."""

    def __init__(self, port, cfg, max_ctx, kv_bf16=False):
        self.p, self.cfg, self.max_ctx = port, cfg, max_ctx
        self._keep = []
        self.h = port.lib.orc_decoder_create(cfg["hidden"], cfg["layers"], cfg["n_q"], cfg["n_kv"],
                                             cfg["hd"], cfg["ff"], cfg["vocab"], max_ctx,
                                             cfg["eps"], cfg["rope_base"])
        if kv_bf16:
            port.lib.orc_decoder_set_kv_bf16(self.h, 1)

    def set_linear(self, layer, which, q4):
        q4 = np.ascontiguousarray(q4, np.uint8)
        self._keep.append(q4)
        self.p.lib.orc_decoder_set_linear(self.h, layer, which, q4)

    def set_vector(self, layer, which, v):
        v = _f(v)
        self._keep.append(v)
        self.p.lib.orc_decoder_set_vector(self.h, layer, which, v)

    def set_embed(self, e):
        e = _f(e)
        self._keep.append(e)
        self.p.lib.orc_decoder_set_embed(self.h, e)

    def fill_kv(self, layer, K, V):
        K, V = _f(K), _f(V)
        self.p.lib.orc_decoder_fill_kv(self.h, layer, K, V, K.shape[1])

    def step(self, token, pos, want_logits=True):
        lg = np.empty(self.cfg["vocab"], np.float32) if want_logits else None
        t = self.p.lib.orc_decoder_step(self.h, token, pos, None if lg is None else lg.ctypes.data)
        return int(t), lg

    def close(self):
        if self.h:
            self.p.lib.orc_decoder_destroy(self.h)
            self.h = None


class Ref:
    """The reference's own CPU implementation (compiled from its headers)."""

    def __init__(self, path):
        L = self.lib = C.CDLL(path)
        L.ref_threads.restype = C.c_int
        L.ref_to_q4.argtypes = [_f32p, _i64, _i64, _u8p]
        L.ref_q4_roundtrip_f32.argtypes = [_f32p, _i64, _i64, _f32p]
        L.ref_dot_q4.argtypes = [_f32p, _i64, _i64, _f32p, _i64, C.c_float, C.c_float, C.c_int,
                                 C.c_int, _f32p, C.POINTER(C.c_double)]
        L.ref_attn_decode.argtypes = [_f32p, _f32p, _f32p, _i64, _i64, _i64, C.c_float, C.c_int,
                                      _f32p, C.POINTER(C.c_double)]
        L.ref_rope.argtypes = [_f32p, _i64, _i64, _i64, _i64, C.c_float, _f32p]
        L.ref_rmsnorm.argtypes = [_f32p, _f32p, _i64, _i64, C.c_float, _f32p]
        L.ref_swiglu.argtypes = [_f32p, _f32p, _i64, _i64, _f32p]
        L.ref_argmax.argtypes = [_f32p, _i64]
        L.ref_argmax.restype = _i64
        L.ref_decoder_create.argtypes = [_i64] * 8 + [C.c_float, C.c_float]
        L.ref_decoder_create.restype = C.c_void_p
        L.ref_decoder_destroy.argtypes = [C.c_void_p]
        L.ref_decoder_set_linear.argtypes = [C.c_void_p, _i64, C.c_int, _f32p, _i64, _i64]
        L.ref_decoder_set_vector.argtypes = [C.c_void_p, _i64, C.c_int, _f32p, _i64]
        L.ref_decoder_set_embed.argtypes = [C.c_void_p, _f32p]
        L.ref_decoder_fill_kv.argtypes = [C.c_void_p, _i64, _f32p, _f32p, _i64]
        L.ref_decoder_step.argtypes = [C.c_void_p, _i64, _i64, C.c_void_p]
        L.ref_decoder_step.restype = _i64

    def threads(self):
        return int(self.lib.ref_threads())

    def to_q4(self, w_kn):
        w = _f(w_kn)
        K, N = w.shape
        out = np.empty(q4_bytes(N, K), np.uint8)
        if self.lib.ref_to_q4(w, K, N, out):
            raise ValueError("reference to_q4 raised")
        return out

    def q4_roundtrip_f32(self, w_kn):
        w = _f(w_kn)
        out = np.empty_like(w)
        if self.lib.ref_q4_roundtrip_f32(w, w.shape[0], w.shape[1], out):
            raise ValueError("reference to_q4/to_f32 raised")
        return out

    def dot_q4(self, x, w_kn, alpha=1.0, beta=0.0, predequant=True, reps=1):
        x, w = _f(x), _f(w_kn)
        x = x.reshape(-1, x.shape[-1])
        M, K = x.shape
        N = w.shape[1]
        out = np.empty((M, N), np.float32)
        sec = C.c_double(0)
        if self.lib.ref_dot_q4(x, M, K, w, N, alpha, beta, int(predequant), reps, out,
                               C.byref(sec)):
            raise ValueError("reference dot raised")
        return out, sec.value

    def attn_decode(self, q, K, V, scale, reps=1):
        q, K, V = _f(q), _f(K), _f(V)
        H, D = q.shape
        out = np.empty((H, D), np.float32)
        sec = C.c_double(0)
        if self.lib.ref_attn_decode(q, K, V, H, K.shape[1], D, scale, reps, out, C.byref(sec)):
            raise ValueError("reference attn_decode raised")
        return out, sec.value

    def rope(self, x, pos, base):
        x = _f(x)
        D = x.shape[-1]
        T = x.shape[1] if x.ndim == 3 else 1
        out = np.empty_like(x)
        if self.lib.ref_rope(x, x.shape[0], T, D, pos, base, out):
            raise ValueError("reference rope raised")
        return out

    def rmsnorm(self, x, w, eps):
        x = _f(x).reshape(-1, x.shape[-1])
        out = np.empty_like(x)
        if self.lib.ref_rmsnorm(x, _f(w), x.shape[0], x.shape[1], eps, out):
            raise ValueError("reference rmsnorm raised")
        return out

    def swiglu(self, g, u):
        g, u = _f(g).reshape(-1, g.shape[-1]), _f(u).reshape(-1, u.shape[-1])
        out = np.empty_like(g)
        if self.lib.ref_swiglu(g, u, g.shape[0], g.shape[1], out):
            raise ValueError("reference swiglu raised")
        return out

    def argmax(self, v):
        v = _f(v).ravel()
        return int(self.lib.ref_argmax(v, v.size))


class RefDecoder:
    def __init__(self, ref, cfg, max_ctx):
        self.r, self.cfg = ref, cfg
        self.h = ref.lib.ref_decoder_create(cfg["hidden"], cfg["layers"], cfg["n_q"], cfg["n_kv"],
                                            cfg["hd"], cfg["ff"], cfg["vocab"], max_ctx,
                                            cfg["eps"], cfg["rope_base"])

    def set_linear(self, layer, which, w_kn):
        w = _f(w_kn)
        if self.r.lib.ref_decoder_set_linear(self.h, layer, which, w, w.shape[0], w.shape[1]):
            raise ValueError("reference set_linear raised")

    def set_vector(self, layer, which, v):
        v = _f(v)
        self.r.lib.ref_decoder_set_vector(self.h, layer, which, v, v.size)

    def set_embed(self, e):
        self.r.lib.ref_decoder_set_embed(self.h, _f(e))

    def fill_kv(self, layer, K, V):
        K, V = _f(K), _f(V)
        self.r.lib.ref_decoder_fill_kv(self.h, layer, K, V, K.shape[1])

    def step(self, token, pos, want_logits=True):
        lg = np.empty(self.cfg["vocab"], np.float32) if want_logits else None
        t = self.r.lib.ref_decoder_step(self.h, token, pos, None if lg is None else lg.ctypes.data)
        if t < 0:
            raise ValueError("reference decoder step raised")
        return int(t), lg

    def close(self):
        if self.h:
            self.r.lib.ref_decoder_destroy(self.h)
            self.h = None


def load_port():
    path = os.path.join(_HERE, "liborc.so")
    if not os.path.exists(path):
        from . import build
        build.build_port()
    return Port(path)


def load_ref():
    path = os.path.join(_HERE, "_ref", "libtlref.so")
    return Ref(path) if os.path.exists(path) else None
