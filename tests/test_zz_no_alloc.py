"""The allocation-free attention entry point (tlb_attn_decode_noalloc).

It exists for embedders that cannot allocate device memory at call time -- a server
whose own arena owns the whole device heap, code running where cudaMalloc's implicit
device-wide synchronisation is not acceptable, a process held to a memory budget fixed
at start-up.  Its scratch is a 4 MiB array inside the library image instead of a
buffer the library allocates.  Called through the C-ABI, twice in a row on different
shapes, it must reproduce the regular entry point (same kernel, same split plan, so
the comparison is exact; the 1e-4 relative bound the attention tests use is checked as
well) and, on its own, the oracle; and it must refuse a shape whose partials do not fit
the array.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn, q, K, V, out, ctx, scale):
    from cpp_tensorlib_b200 import lib
    n_q, D = q.shape
    n_kv, kv_max, _ = K.shape
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())
    return getattr(lib(), fn)(p(q), p(K), p(V), p(out), n_q, n_kv, ctx, kv_max, D, scale, stream)


def test_noalloc_attention_matches_regular_entry_point_twice(port):
    from cpp_tensorlib_b200 import check, lib
    g = torch.Generator(device="cuda").manual_seed(77)
    cases = [(28, 4, 128, 4224, 4100), (14, 2, 64, 700, 650)]   # second call reuses the array
    for n_q, n_kv, D, kv_max, ctx in cases:
        q = torch.randn((n_q, D), generator=g, device="cuda")
        K = torch.randn((n_kv, kv_max, D), generator=g, device="cuda")
        V = torch.randn((n_kv, kv_max, D), generator=g, device="cuda")
        want, got = torch.empty_like(q), torch.full_like(q, float("nan"))
        scale = float(D) ** -0.5
        check(_call("tlb_attn_decode", q, K, V, want, ctx, scale))
        check(_call("tlb_attn_decode_noalloc", q, K, V, got, ctx, scale))
        torch.cuda.synchronize()
        w, o = want.cpu().numpy().astype(np.float64), got.cpu().numpy()
        assert np.max(np.abs(o - w) / (1.0 + np.abs(w))) < 1e-4
        assert torch.equal(got, want)
        # and against the oracle directly, so this test stands without the regular entry point
        ref = port.attn_decode(q.cpu().numpy(), K.cpu().numpy(), V.cpu().numpy(), scale, ctx=ctx)
        assert np.max(np.abs(o - ref.astype(np.float64)) / (1.0 + np.abs(ref))) < 1e-4


def test_noalloc_attention_back_to_back_without_sync(port):
    """Stream-ordered reuse of the one array: three calls on different shapes queued on one
    stream with no synchronisation in between (a split case, the single-split case ctx = 1,
    and a wide case), each into its own output, all checked afterwards against the oracle."""
    from cpp_tensorlib_b200 import check
    g = torch.Generator(device="cuda").manual_seed(78)
    shapes = [(28, 4, 128, 2048, 2048), (14, 2, 64, 64, 1), (32, 8, 128, 600, 511)]
    runs = []
    for n_q, n_kv, D, kv_max, ctx in shapes:
        q = torch.randn((n_q, D), generator=g, device="cuda")
        K = torch.randn((n_kv, kv_max, D), generator=g, device="cuda")
        V = torch.randn((n_kv, kv_max, D), generator=g, device="cuda")
        runs.append((q, K, V, torch.full_like(q, float("nan")), ctx, float(D) ** -0.5))
    for q, K, V, out, ctx, scale in runs:
        check(_call("tlb_attn_decode_noalloc", q, K, V, out, ctx, scale))
    torch.cuda.synchronize()
    for q, K, V, out, ctx, scale in runs:
        ref = port.attn_decode(q.cpu().numpy(), K.cpu().numpy(), V.cpu().numpy(), scale, ctx=ctx)
        assert np.max(np.abs(out.cpu().numpy() - ref.astype(np.float64)) / (1.0 + np.abs(ref))) < 1e-4


def test_noalloc_attention_second_device():
    """The array's address and the kernels' shared-memory attribute are per device: the second
    GPU of a process must work after the first."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from cpp_tensorlib_b200 import check
    outs = []
    for devi in (0, 1):
        with torch.cuda.device(devi):
            g = torch.Generator(device=f"cuda:{devi}").manual_seed(79)
            q = torch.randn((28, 128), generator=g, device=f"cuda:{devi}")
            K = torch.randn((4, 1024, 128), generator=g, device=f"cuda:{devi}")
            V = torch.randn((4, 1024, 128), generator=g, device=f"cuda:{devi}")
            a, b = torch.empty_like(q), torch.empty_like(q)
            check(_call("tlb_attn_decode", q, K, V, a, 1000, 0.0884))
            check(_call("tlb_attn_decode_noalloc", q, K, V, b, 1000, 0.0884))
            torch.cuda.synchronize()
            assert torch.equal(a, b)
            outs.append(a.cpu())
    assert torch.equal(outs[0], outs[1])


def test_noalloc_attention_rejects_oversized_partials():
    from cpp_tensorlib_b200 import lib
    n_q, n_kv, D, kv_max = 4096, 64, 128, 12288      # 4096 heads x 2 splits x 528 B > 4 MiB
    q = torch.zeros((n_q, D), device="cuda")
    K = torch.zeros((n_kv, kv_max, D), device="cuda")
    out = torch.empty_like(q)
    rc = _call("tlb_attn_decode_noalloc", q, K, K, out, kv_max, 1.0)
    assert rc == 3                                     # TLB_ERR_UNSUPPORTED
    assert b"built-in scratch" in lib().tlb_last_error()
