"""Host-side mirror of the reference's ``tl::cuda::`` operator interface
(include/cuda.h of the reference) over the C-ABI library.

Same names, argument meaning and error behaviour as the reference facade, with
two deliberate differences: operands are torch CUDA tensors (torch owns device
memory and the current stream; nothing else of torch is used), and a call the
kernels cannot serve raises ``TlbError`` instead of returning ``false`` and
letting a CPU path take over -- this backend has no CPU fallback.
"""
import ctypes as C

import torch

from ._lib import TlbError, check, lib

kQ4Group = 32  # include/types.h:28


def _s():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _f32c(t, name):
    if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
        raise ValueError(f"{name}: expected a contiguous float32 CUDA tensor")
    return t


def available():
    """cuda::available (include/cuda.h:493)."""
    return lib().tlb_device_count() > 0


def flush():
    """cuda::flush (include/cuda.h:501-506): block until the stream is idle."""
    check(lib().tlb_sync(_s()))


def q4_bytes(N, K):
    """include/types.h:29-31."""
    return N * K // 2 + N * (K // kQ4Group) * 4


class Q4Weight:
    """The reference's q4 array (include/types.h:15-31): logical shape [K, N], one
    byte buffer = packed nibbles [N][K/2] then f32 scales [N][K/32]."""

    def __init__(self, buf, K, N):
        assert buf.dtype == torch.uint8 and buf.numel() == q4_bytes(N, K)
        self.buf, self.K, self.N = buf, K, N

    @property
    def shape(self):
        return (self.K, self.N)

    @property
    def qw_ptr(self):
        return C.c_void_p(self.buf.data_ptr())

    @property
    def scales_ptr(self):
        # include/array.h:1621-1622: scales sit at native + N*K/2 bytes
        return C.c_void_p(self.buf.data_ptr() + self.N * self.K // 2)

    def to_f32(self):
        """array::to_f32 (include/array.h:666-684): dequantised logical [K, N]."""
        out = torch.empty((self.K, self.N), dtype=torch.float32, device=self.buf.device)
        check(lib().tlb_q4_to_f32(self.qw_ptr, self.K, self.N, _p(out), _s()))
        return out

    @staticmethod
    def from_bytes(host_bytes, K, N, device="cuda"):
        t = torch.from_numpy(host_bytes).to(device)
        return Q4Weight(t, K, N)


def to_q4(w):
    """array::to_q4 (include/array.h:703-742) on the device. w: f32 [K, N]."""
    _f32c(w, "to_q4")
    if w.dim() != 2:
        raise ValueError("tl::to_q4: expect [K,N]")
    K, N = w.shape
    if K % kQ4Group:
        raise ValueError("tl::to_q4: K must be a multiple of kQ4Group (32)")
    buf = torch.empty(q4_bytes(N, K), dtype=torch.uint8, device=w.device)
    check(lib().tlb_to_q4(_p(w), K, N, _p(buf), _s()))
    return Q4Weight(buf, K, N)


def gemv_q4(a, wq, y=None):
    """cuda::gemv_q4 (include/cuda.h:886-905): y[N] = a[K] . dequant(Wq)."""
    _f32c(a, "gemv_q4")
    if a.numel() != wq.K:
        raise ValueError("gemv_q4: a must hold K elements")
    if y is None:
        y = torch.empty(wq.N, dtype=torch.float32, device=a.device)
    check(lib().tlb_gemv_q4(_p(a), wq.qw_ptr, wq.scales_ptr, _p(y), wq.N, wq.K, kQ4Group, _s()))
    return y


def gemv_bf16_row(a, W, y=None):
    """cuda::gemv_bf16_row (include/cuda.h:770-785): y[N] = W[N, K] (bf16, row-major) . a[K]."""
    _f32c(a, "gemv_bf16_row a")
    if W.dtype != torch.bfloat16 or W.dim() != 2 or not W.is_contiguous() or not W.is_cuda:
        raise ValueError("gemv_bf16_row: W must be a contiguous bf16 CUDA matrix [N, K]")
    N, K = W.shape
    if a.numel() != K:
        raise ValueError("gemv_bf16_row: a must hold K elements")
    if y is None:
        y = torch.empty(N, dtype=torch.float32, device=a.device)
    check(lib().tlb_gemv_bf16_row(_p(a), _p(W), _p(y), N, K, _s()))
    return y


class Q4Packed:
    """A q4 matrix in the library's tile-packed layout (2560-byte units of 16 rows x
    256 k: nibble words in MMA-fragment order, then the unit's scales).  Made once from
    a Q4Weight; no counterpart in the reference."""

    def __init__(self, wq):
        nbytes = lib().tlb_q4p_bytes(wq.N, wq.K)
        if nbytes < 0:
            raise ValueError("Q4Packed: bad shape")
        self.K, self.N = wq.K, wq.N
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=wq.buf.device)
        check(lib().tlb_q4_pack(wq.qw_ptr, wq.N, wq.K, _p(self.buf), _s()))


def gemv_q4p(a, wp, alpha=1.0, beta=0.0, y=None):
    """The decode GEMV on packed weights: y[N] = (a[K] . dequant(W)) * alpha + beta."""
    _f32c(a, "gemv_q4p")
    if a.numel() != wp.K:
        raise ValueError("gemv_q4p: a must hold K elements")
    if y is None:
        y = torch.empty(wp.N, dtype=torch.float32, device=a.device)
    check(lib().tlb_gemv_q4p(_p(a), _p(wp.buf), _p(y), wp.N, wp.K, alpha, beta, _s()))
    return y


def gemm_q4(x, wq, alpha=1.0, beta=0.0, y=None, simt=False):
    """The dot node with its fused affine epilogue (include/array.h:1305-1311,
    2109-2141): y[M,N] = (x[M,K] . dequant(Wq)) * alpha + beta, any M."""
    _f32c(x, "gemm_q4")
    x2 = x.reshape(-1, x.shape[-1])
    M, K = x2.shape
    if K != wq.K:
        raise ValueError("tl::dot: inner dimensions differ")
    if y is None:
        y = torch.empty((M, wq.N), dtype=torch.float32, device=x.device)
    fn = lib().tlb_gemm_q4_simt if simt else lib().tlb_gemm_q4
    check(fn(_p(x2), M, K, wq.qw_ptr, wq.scales_ptr, _p(y), wq.N, wq.N, K, alpha, beta, _s()))
    return y


def attn_decode(q, K, V, scale, ctx=None, out=None):
    """cuda::attn_decode (include/cuda.h:966-1009). q [n_q, D]; K, V [n_kv, kv_max, D]
    read over the prefix [0, ctx) (ctx defaults to kv_max, the array path of
    include/array.h:1632-1651)."""
    _f32c(q, "attn_decode q")
    bf = K.dtype == torch.bfloat16           # bf16 cache (kv_cache with dtype bf16)
    if not bf:
        _f32c(K, "attn_decode K"), _f32c(V, "attn_decode V")
    elif V.dtype != torch.bfloat16 or not (K.is_contiguous() and V.is_contiguous()):
        raise ValueError("tl::attn_decode: a bf16 cache needs contiguous bf16 K and V")
    if q.dim() != 2 or K.dim() != 3 or V.shape != K.shape:
        raise ValueError("tl::attn_decode: q must be [H,D], K/V [H,ctx,D] and equal")
    n_q, D = q.shape
    n_kv, kv_max, _ = K.shape
    ctx = kv_max if ctx is None else ctx
    if out is None:
        out = torch.empty_like(q)
    fn = lib().tlb_attn_decode_bf16 if bf else lib().tlb_attn_decode
    check(fn(_p(q), _p(K), _p(V), _p(out), n_q, n_kv, ctx, kv_max, D, scale, _s()))
    return out


def attn_decode_noalloc(q, K, V, scale, ctx=None, out=None):
    """attn_decode for callers that may not allocate device memory at call time (no
    counterpart in the reference): split partials live in a fixed 4 MiB array inside
    the library.  Shapes beyond that array raise TlbError.  The output tensor is the
    caller's; pass `out` to keep torch from allocating one here."""
    _f32c(q, "attn_decode_noalloc q"), _f32c(K, "attn_decode_noalloc K"), _f32c(V, "attn_decode_noalloc V")
    n_q, D = q.shape
    n_kv, kv_max, _ = K.shape
    ctx = kv_max if ctx is None else ctx
    if out is None:
        out = torch.empty_like(q)
    check(lib().tlb_attn_decode_noalloc(_p(q), _p(K), _p(V), _p(out), n_q, n_kv, ctx, kv_max, D,
                                        scale, _s()))
    return out


def rope(x, pos, base=10000.0, bias=None, out=None):
    """cuda::rope (include/cuda.h:1205-1222). x [H, D] or [H, T, D]."""
    _f32c(x, "rope")
    D = x.shape[-1]
    T = x.shape[1] if x.dim() == 3 else 1
    rows = x.numel() // D
    if out is None:
        out = torch.empty_like(x)
    check(lib().tlb_rope(_p(x), _p(out), rows, T, D, pos, base, _p(bias), _s()))
    return out


def rope_dpos(x, d_pos, base=10000.0, bias=None, out=None):
    """cuda::rope_dpos (include/cuda.h:1018-1035): position read from a device u32."""
    _f32c(x, "rope_dpos")
    D = x.shape[-1]
    T = x.shape[1] if x.dim() == 3 else 1
    if out is None:
        out = torch.empty_like(x)
    check(lib().tlb_rope_dpos(_p(x), _p(out), x.numel() // D, T, D, _p(d_pos), base, _p(bias), _s()))
    return out


def rmsnorm(x, w, eps, out=None):
    """cuda::rmsnorm (include/cuda.h:1287-1302); rows = all leading dims."""
    _f32c(x, "rmsnorm")
    n = x.shape[-1]
    if out is None:
        out = torch.empty_like(x)
    check(lib().tlb_rmsnorm(_p(x), _p(w), _p(out), n, eps, x.numel() // n, _s()))
    return out


def rmsnorm_res(x, delta, w, eps, xout=None, hout=None):
    """cuda::rmsnorm_res (include/cuda.h:1233-1252): xout = x + delta; hout = rmsnorm(xout)*w."""
    _f32c(x, "rmsnorm_res")
    n = x.shape[-1]
    xout = torch.empty_like(x) if xout is None else xout
    hout = torch.empty_like(x) if hout is None else hout
    check(lib().tlb_rmsnorm_res(_p(x), _p(delta), _p(w), _p(xout), _p(hout), n, eps,
                                x.numel() // n, _s()))
    return xout, hout


def swiglu(gu, ff, out=None):
    """cuda::swiglu (include/cuda.h:1306-1319) on the fused [rows, 2*ff] buffer."""
    _f32c(gu, "swiglu")
    rows = gu.numel() // (2 * ff)
    if out is None:
        out = torch.empty((rows, ff), dtype=torch.float32, device=gu.device)
    check(lib().tlb_swiglu(_p(gu), _p(out), ff, rows, _s()))
    return out


def split_heads(src, bias, T, ld, off, H, D, out=None):
    """cuda::split_heads (include/cuda.h:848-864): [T, ld] token-major -> [H, T, D] (+ bias[H*D])."""
    if out is None:
        out = torch.empty((H, T, D), dtype=torch.float32, device=src.device)
    check(lib().tlb_split_heads(_p(src), _p(bias), _p(out), T, ld, off, H, D, _s()))
    return out


def merge_heads(src, out=None):
    """cuda::merge_heads (include/cuda.h:867-879): [H, T, D] -> [T, H*D]."""
    H, T, D = src.shape
    if out is None:
        out = torch.empty((T, H * D), dtype=torch.float32, device=src.device)
    check(lib().tlb_merge_heads(_p(src), _p(out), T, H, D, _s()))
    return out


def attn_prefill(q, K, V, scale, pos0=0, out=None):
    """cuda::attn_prefill (include/cuda.h:1171-1201): causal attention of a prompt chunk.
    q [n_q, T, D]; K, V caches [n_kv, kv_max, D] already holding rows [0, pos0 + T)."""
    _f32c(q, "attn_prefill q")
    bf = K.dtype == torch.bfloat16
    if not bf:
        _f32c(K, "attn_prefill K"), _f32c(V, "attn_prefill V")
    elif V.dtype != torch.bfloat16 or not (K.is_contiguous() and V.is_contiguous()):
        raise ValueError("attn_prefill: a bf16 cache needs contiguous bf16 K and V")
    n_q, T, D = q.shape
    n_kv, kv_max, _ = K.shape
    if out is None:
        out = torch.empty_like(q)
    fn = lib().tlb_attn_prefill_bf16 if bf else lib().tlb_attn_prefill
    check(fn(_p(q), _p(K), _p(V), _p(out), n_q, n_kv, T, kv_max, D, scale, pos0, _s()))
    return out


def argmax(v):
    """cuda::argmax (include/cuda.h:1261-1282): smallest index among the maxima."""
    _f32c(v, "argmax")
    idx = C.c_int64(0)
    check(lib().tlb_argmax(_p(v), v.numel(), C.byref(idx), _s()))
    return int(idx.value)


def incr_u32(d_pos):
    check(lib().tlb_incr_u32(_p(d_pos), _s()))


class kv_cache:
    """cuda::kv_cache (include/cuda.h:1326-1405): K, V [n_kv_heads, max_ctx, D] in f32 or
    bf16 (kv_cache::init's dtype argument) plus a running position."""

    def __init__(self, n_kv_heads, max_ctx, D, device="cuda", dtype=torch.float32):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("kv_cache: dtype must be float32 or bfloat16")
        self.n_kv_heads, self.max_ctx, self.D, self.pos = n_kv_heads, max_ctx, D, 0
        self.bf16 = dtype == torch.bfloat16
        self.K = torch.zeros((n_kv_heads, max_ctx, D), dtype=dtype, device=device)
        self.V = torch.zeros_like(self.K)
        self.dpos_partials = None

    def _fn(self, name):
        return getattr(lib(), name + ("_bf16" if self.bf16 else ""))

    def append(self, k_new, v_new):
        if self.pos >= self.max_ctx:
            raise IndexError("kv_cache.append: cache is full")
        check(self._fn("tlb_kv_append")(_p(self.K), _p(self.V), _p(k_new), _p(v_new), self.pos,
                                        self.max_ctx, self.n_kv_heads, self.D, _s()))
        self.pos += 1

    def attn(self, q, scale, out=None):
        return attn_decode(q, self.K, self.V, scale, ctx=self.pos, out=out)

    def prefill(self, q, k_src, v_src, scale, out=None):
        """kv_cache::prefill (include/cuda.h:1383-1398): append a block of k, v
        ([n_kv, T, D]) at the current position and run causal attention for q [n_q, T, D]."""
        T = k_src.shape[1]
        if T <= 0 or self.pos + T > self.max_ctx:
            raise IndexError("kv_cache.prefill: block does not fit the cache")
        check(self._fn("tlb_kv_fill")(_p(self.K), _p(self.V), _p(k_src), _p(v_src), T, self.max_ctx,
                                      self.n_kv_heads, self.D, self.pos, _s()))
        p0 = self.pos
        self.pos += T
        return attn_prefill(q, self.K, self.V, scale, pos0=p0, out=out)

    def fill(self, k_src, v_src):
        """cuda::kv_fill (include/cuda.h:1143-1164): a block of k, v [n_kv, T, D] into the
        rows from the current position on (narrowed to bf16 when the cache is bf16)."""
        T = k_src.shape[1]
        if T <= 0 or self.pos + T > self.max_ctx:
            raise IndexError("kv_cache.fill: block does not fit the cache")
        check(self._fn("tlb_kv_fill")(_p(self.K), _p(self.V), _p(k_src), _p(v_src), T, self.max_ctx,
                                      self.n_kv_heads, self.D, self.pos, _s()))
        self.pos += T

    def append_dpos(self, k_new, v_new, d_pos):
        check(self._fn("tlb_kv_append_dpos")(_p(self.K), _p(self.V), _p(k_new), _p(v_new), _p(d_pos),
                                             self.max_ctx, self.n_kv_heads, self.D, _s()))

    def attn_dpos(self, q, d_pos, scale, out=None):
        n_q = q.shape[0]
        if self.dpos_partials is None:
            nb = lib().tlb_attn_partials_bytes(n_q, self.n_kv_heads, self.max_ctx, self.D)
            self.dpos_partials = torch.zeros(nb, dtype=torch.uint8, device=q.device)
        if out is None:
            out = torch.empty_like(q)
        check(self._fn("tlb_attn_decode_dpos")(_p(q), _p(self.K), _p(self.V), _p(out), n_q,
                                               self.n_kv_heads, _p(d_pos), self.max_ctx, self.D, scale,
                                               _p(self.dpos_partials), _s()))
        return out
