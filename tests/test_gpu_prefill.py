"""Batched-prefill ops through the C-ABI against the oracle.  Causal prefill of a
chunk equals, row by row, a decode step over the cache prefix that row may see
(reference include/cuda.h:1166-1201; bench/cuda/check/check_attn64.cpp checks it the
same way), so the checker is the oracle's attn_decode called once per query.
Head moves and the cache fill are pure copies: bit-exact."""
import numpy as np
import pytest
import torch

import synth

pytestmark = pytest.mark.gpu


def relerr(a, b):
    return float(np.max(np.abs(np.asarray(a, np.float64) - b) / (1.0 + np.abs(b))))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def tl():
    from cpp_tensorlib_b200 import cuda as tlc
    assert tlc.available(), "no CUDA device: the GPU tests have no fallback"
    yield tlc
    from cpp_tensorlib_b200 import check, lib
    import ctypes
    st = (ctypes.c_int * 2)()
    check(lib().tlb_device_status(st, 0))


def causal_reference(port, q, K, V, scale, pos0):
    n_q, T, D = q.shape
    out = np.empty_like(q)
    for p in range(T):
        out[:, p] = port.attn_decode(q[:, p], K, V, scale, ctx=pos0 + p + 1)
    return out


@pytest.mark.parametrize("T,H,D,with_bias", [(1, 2, 64, False), (7, 14, 64, True), (33, 28, 128, True)])
def test_split_and_merge_heads_exact(tl, T, H, D, with_bias):
    ld, off = 3 * H * D + 16, H * D + 16        # a column block inside a wider row
    src = synth.normal(31, T, (T, ld))
    bias = synth.normal(31, 1000 + T, (H * D,)) if with_bias else None
    got = tl.split_heads(dev(src), None if bias is None else dev(bias), T, ld, off, H, D)
    want = src[:, off:off + H * D].reshape(T, H, D).transpose(1, 0, 2)
    if bias is not None:
        want = want + bias.reshape(H, 1, D)
    assert np.array_equal(got.cpu().numpy(), want.astype(np.float32))
    back = tl.merge_heads(got).cpu().numpy()
    assert np.array_equal(back, want.transpose(1, 0, 2).reshape(T, H * D))


@pytest.mark.parametrize("n_q,n_kv,D,T,pos0,kv_max", [
    (2, 2, 64, 1, 0, 8),          # a single token is a decode step
    (14, 2, 64, 37, 0, 64),       # ragged chunk, grouped heads (0.5B geometry)
    (14, 2, 64, 32, 21, 96),      # a second chunk that starts mid-tile
    (8, 2, 128, 70, 5, 128),      # D = 128, three query tiles
    (28, 4, 128, 129, 0, 160),    # 7B geometry, one row past a tile edge
])
def test_attn_prefill_vs_oracle(tl, port, n_q, n_kv, D, T, pos0, kv_max):
    seed = 40 + T
    K = synth.normal(seed, 1, (n_kv, kv_max, D))
    V = synth.normal(seed, 2, (n_kv, kv_max, D))
    q = synth.normal(seed, 3, (n_q, T, D))
    scale = 1.0 / np.sqrt(D)
    got = tl.attn_prefill(dev(q), dev(K), dev(V), scale, pos0=pos0).cpu().numpy()
    want = causal_reference(port, q, K, V, scale, pos0)
    assert relerr(got, want) < 1e-4


def test_kv_cache_prefill_then_decode(tl, port):
    """kv_cache::prefill in two chunks, then one decode step on the same cache."""
    n_q, n_kv, D, maxc = 14, 2, 64, 70
    cache = tl.kv_cache(n_kv, maxc, D)
    Kh, Vh = np.zeros((n_kv, maxc, D), np.float32), np.zeros((n_kv, maxc, D), np.float32)
    scale = 0.125
    pos = 0
    for i, T in enumerate((40, 19)):
        k, v = synth.normal(50, 10 + i, (n_kv, T, D)), synth.normal(50, 20 + i, (n_kv, T, D))
        q = synth.normal(50, 30 + i, (n_q, T, D))
        got = cache.prefill(dev(q), dev(k), dev(v), scale).cpu().numpy()
        Kh[:, pos:pos + T], Vh[:, pos:pos + T] = k, v
        assert relerr(got, causal_reference(port, q, Kh, Vh, scale, pos)) < 1e-4
        pos += T
    assert cache.pos == pos
    assert np.array_equal(cache.K.cpu().numpy(), Kh) and np.array_equal(cache.V.cpu().numpy(), Vh)
    k1, v1 = synth.normal(50, 90, (n_kv, D)), synth.normal(50, 91, (n_kv, D))
    cache.append(dev(k1), dev(v1))
    Kh[:, pos], Vh[:, pos] = k1, v1
    q1 = synth.normal(50, 92, (n_q, D))
    got = cache.attn(dev(q1), scale).cpu().numpy()
    assert relerr(got, port.attn_decode(q1, Kh, Vh, scale, ctx=pos + 1)) < 1e-4
    with pytest.raises(IndexError):
        cache.prefill(dev(q), dev(k), dev(v), scale)      # 60 rows held, 19 more do not fit 70


def test_attn_prefill_full_size_property(tl, port):
    """7B geometry, 2048-token prompt: the last row equals a decode step over the whole
    prompt and row 0 equals V[:, 0] (a softmax over one key)."""
    n_q, n_kv, D, T = 28, 4, 128, 2048
    g = torch.Generator(device="cuda").manual_seed(7)
    K = torch.randn((n_kv, T, D), generator=g, device="cuda")
    V = torch.randn((n_kv, T, D), generator=g, device="cuda")
    q = torch.randn((n_q, T, D), generator=g, device="cuda")
    scale = 1.0 / np.sqrt(D)
    out = tl.attn_prefill(q, K, V, scale)
    last = tl.attn_decode(q[:, -1].contiguous(), K, V, scale, ctx=T)
    assert relerr(out[:, -1].cpu().numpy(), last.cpu().numpy().astype(np.float64)) < 1e-4
    first = V[:, 0].repeat_interleave(n_q // n_kv, dim=0)
    assert relerr(out[:, 0].cpu().numpy(), first.cpu().numpy().astype(np.float64)) < 1e-6
    mid = 1000
    want = port.attn_decode(q[:, mid].cpu().numpy(), K.cpu().numpy(), V.cpu().numpy(), scale, ctx=mid + 1)
    assert relerr(out[:, mid].cpu().numpy(), want) < 1e-4


def test_prefill_bad_arguments(tl):
    from cpp_tensorlib_b200 import TlbError
    q = torch.zeros((4, 8, 64), device="cuda")
    K = torch.zeros((2, 8, 64), device="cuda")
    with pytest.raises(TlbError):
        tl.attn_prefill(q, K, K, 0.125, pos0=1)         # chunk runs past kv_max
    q3 = torch.zeros((3, 8, 64), device="cuda")
    with pytest.raises(TlbError):
        tl.attn_prefill(q3, K, K, 0.125)                # 3 % 2 != 0
    q96 = torch.zeros((4, 8, 96), device="cuda")
    K96 = torch.zeros((2, 8, 96), device="cuda")
    with pytest.raises(TlbError):
        tl.attn_prefill(q96, K96, K96, 0.125)           # D outside {64, 128}


def bf16_round(a):
    x = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    x = (x + 0x7fff + ((x >> 16) & 1)) >> 16
    return (x.astype(np.uint32) << 16).view(np.float32).reshape(np.shape(a))


@pytest.mark.parametrize("n_q,n_kv,D,T,pos0,kv_max", [(14, 2, 64, 37, 0, 64), (8, 2, 128, 70, 5, 128)])
def test_attn_prefill_bf16_cache(tl, port, n_q, n_kv, D, T, pos0, kv_max):
    """Tiled prefill on a bf16 cache: the f32 oracle on the bf16-rounded cache, 1e-4."""
    K, V = synth.normal(80, 1, (n_kv, kv_max, D)), synth.normal(80, 2, (n_kv, kv_max, D))
    q = synth.normal(80, 3, (n_q, T, D))
    scale = 1.0 / np.sqrt(D)
    got = tl.attn_prefill(dev(q), dev(K).to(torch.bfloat16), dev(V).to(torch.bfloat16), scale,
                          pos0=pos0).cpu().numpy()
    assert relerr(got, causal_reference(port, q, bf16_round(K), bf16_round(V), scale, pos0)) < 1e-4


def test_kv_cache_bf16_prefill(tl, port):
    n_q, n_kv, D, maxc, T = 14, 2, 64, 48, 33
    cache = tl.kv_cache(n_kv, maxc, D, dtype=torch.bfloat16)
    k, v = synth.normal(81, 1, (n_kv, T, D)), synth.normal(81, 2, (n_kv, T, D))
    q = synth.normal(81, 3, (n_q, T, D))
    got = cache.prefill(dev(q), dev(k), dev(v), 0.125).cpu().numpy()
    Kh, Vh = np.zeros((n_kv, maxc, D), np.float32), np.zeros((n_kv, maxc, D), np.float32)
    Kh[:, :T], Vh[:, :T] = bf16_round(k), bf16_round(v)
    assert cache.pos == T
    assert relerr(got, causal_reference(port, q, Kh, Vh, 0.125, 0)) < 1e-4
