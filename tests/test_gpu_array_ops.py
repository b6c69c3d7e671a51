"""The rest of the evaluator's GPU surface through the C-ABI (csrc/array_ops.cu): elementwise
binaries and unaries with the fused affine epilogue, rank-2 broadcast, row reductions and
softmax, the f32 GEMM in its four layouts, the [K,N]-layout GEMVs on f32 / bf16 weights and the
bf16 prefill GEMM.  Each is a floating-point kernel whose expression is the reference's
(kernels/tensorlib_cuda.cu:25-82, 222-276, 611-682; include/array.h ref:: loops on the CPU),
so the check is a float64 numpy evaluation of that expression: 1e-6 relative for the
elementwise ops (one rounding each, libm vs device intrinsics 2 ulp), 1e-5 for reductions
and contractions (summation order differs), 1e-4 where a single f32 accumulator runs over
thousands of terms (rows of 151936 columns, K = 4864): the bound follows sqrt(terms) * 2^-24."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _s():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return C.c_void_p(t.data_ptr())


def relerr(got, want):
    want = np.asarray(want, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - want) / (1.0 + np.abs(want))))


@pytest.fixture(scope="module")
def L():
    from cpp_tensorlib_b200 import check, lib
    check(lib().tlb_init(0))
    return lib()


def rnd(shape, seed, lo=-2.0, hi=2.0):
    g = np.random.Generator(np.random.Philox(seed))
    return (g.random(shape, dtype=np.float32) * (hi - lo) + lo).astype(np.float32)


BIN = {0: np.add, 1: np.subtract, 2: np.multiply, 3: np.divide, 4: np.power}


@pytest.mark.parametrize("op", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("n,off", [(1, 0), (7, 0), (4096, 0), (100003, 0), (4099, 1)])
def test_binary_with_epilogue(L, op, n, off):
    from cpp_tensorlib_b200 import check
    a, b = rnd(n + off, 1, 0.5, 3.0), rnd(n + off, 2, 0.5, 3.0)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    out = torch.empty(n + off, device="cuda")
    # `off` shifts the operands off the 16-byte boundary: the scalar path
    check(L.tlb_binary(op, C.c_void_p(da.data_ptr() + 4 * off), C.c_void_p(db.data_ptr() + 4 * off),
                       C.c_void_p(out.data_ptr() + 4 * off), n, 0.5, 1.25, _s()))
    want = BIN[op](a[off:].astype(np.float64), b[off:].astype(np.float64)) * 0.5 + 1.25
    assert relerr(out[off:].cpu().numpy(), want) < 2e-6


@pytest.mark.parametrize("op", [0, 2, 3, 4])
def test_binary_broadcast_rank2(L, op):
    """Row vector, column vector and scalar operands (strides 0 on the broadcast axis), as
    include/array.h:1487-1506 hands them over."""
    from cpp_tensorlib_b200 import check
    rows, cols = 37, 129
    a = rnd((rows, cols), 3, 0.5, 3.0)
    for bshape, brs, bcs in (((1, cols), 0, 1), ((rows, 1), 1, 0), ((1, 1), 0, 0)):
        b = rnd(bshape, 4, 0.5, 3.0)
        da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        out = torch.empty((rows, cols), device="cuda")
        check(L.tlb_binary_bcast(op, _p(da), cols, 1, _p(db), brs, bcs, _p(out), rows, cols, 2.0, -0.5, _s()))
        want = BIN[op](a.astype(np.float64), b.astype(np.float64)) * 2.0 - 0.5
        assert relerr(out.cpu().numpy(), want) < 2e-6, bshape
        # and with the broadcast operand on the left
        check(L.tlb_binary_bcast(op, _p(db), brs, bcs, _p(da), cols, 1, _p(out), rows, cols, 1.0, 0.0, _s()))
        assert relerr(out.cpu().numpy(), BIN[op](b.astype(np.float64), a.astype(np.float64))) < 2e-6, bshape


UNA = {0: np.exp, 1: np.log, 2: np.sqrt, 3: lambda x: 1.0 / (1.0 + np.exp(-x)), 4: lambda x: np.maximum(x, 0.0),
       5: lambda x: x}


@pytest.mark.parametrize("op", [0, 1, 2, 3, 4, 5])
@pytest.mark.parametrize("n", [1, 5, 4096, 70001])
def test_unary_with_epilogue(L, op, n):
    from cpp_tensorlib_b200 import check
    a = rnd(n, 5, 0.1, 4.0) if op in (1, 2) else rnd(n, 5, -4.0, 4.0)
    da = torch.from_numpy(a).cuda()
    out = torch.empty(n, device="cuda")
    check(L.tlb_unary(op, _p(da), _p(out), n, 1.5, -2.0, _s()))
    assert relerr(out.cpu().numpy(), UNA[op](a.astype(np.float64)) * 1.5 - 2.0) < 2e-6


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 7), (28, 4096), (5, 151936), (300, 33)])
def test_row_ops(L, rows, cols):
    from cpp_tensorlib_b200 import check
    x = rnd((rows, cols), 6, -3.0, 3.0)
    dx = torch.from_numpy(x).cuda()
    x64 = x.astype(np.float64)
    out = torch.empty((rows, cols), device="cuda")
    check(L.tlb_row_op(0, _p(dx), _p(out), rows, cols, 9.0, 9.0, _s()))      # softmax ignores the epilogue
    e = np.exp(x64 - x64.max(1, keepdims=True))
    assert relerr(out.cpu().numpy(), e / e.sum(1, keepdims=True)) < 1e-6
    red = torch.empty(rows, device="cuda")
    check(L.tlb_row_op(1, _p(dx), _p(red), rows, cols, 0.5, 1.0, _s()))
    assert relerr(red.cpu().numpy(), x64.sum(1) * 0.5 + 1.0) < (1e-4 if cols > 10000 else 1e-5)
    check(L.tlb_row_op(2, _p(dx), _p(red), rows, cols, 2.0, -1.0, _s()))
    assert relerr(red.cpu().numpy(), x64.max(1) * 2.0 - 1.0) < 1e-6


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (5, 7, 3), (64, 64, 16), (65, 130, 33), (128, 896, 4864), (300, 257, 129)])
@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (0, 1), (1, 1)])
def test_gemm_f32_layouts(L, m, n, k, ta, tb):
    """include/cuda.h:1409-1483 contract: A(i,k) = ta ? A[k*lda+i] : A[i*lda+k], likewise B."""
    from cpp_tensorlib_b200 import check
    A, B = rnd((m, k), 7, -1.0, 1.0), rnd((k, n), 8, -1.0, 1.0)
    As = np.ascontiguousarray(A.T) if ta else A
    Bs = np.ascontiguousarray(B.T) if tb else B
    dA, dB = torch.from_numpy(As).cuda(), torch.from_numpy(Bs).cuda()
    out = torch.empty((m, n), device="cuda")
    check(L.tlb_gemm_f32(_p(dA), As.shape[1], ta, _p(dB), Bs.shape[1], tb, _p(out), m, n, k, 0.5, 1.0, _s()))
    want = A.astype(np.float64) @ B.astype(np.float64) * 0.5 + 1.0
    assert relerr(out.cpu().numpy(), want) < (1e-4 if k > 1024 else 1e-5)


@pytest.mark.parametrize("K,N", [(8, 1), (896, 4864), (3584, 1000), (129, 131), (4864, 896)])
def test_gemv_kn_f32_and_bf16(L, K, N):
    from cpp_tensorlib_b200 import check
    a, B = rnd(K, 9, -1.0, 1.0), rnd((K, N), 10, -0.1, 0.1)
    da, dB = torch.from_numpy(a).cuda(), torch.from_numpy(B).cuda()
    y = torch.empty(N, device="cuda")
    check(L.tlb_gemv_f32(_p(da), _p(dB), _p(y), N, K, _s()))
    assert relerr(y.cpu().numpy(), a.astype(np.float64) @ B.astype(np.float64)) < 1e-5
    Bb = dB.to(torch.bfloat16)
    check(L.tlb_gemv_bf16(_p(da), _p(Bb), _p(y), N, K, _s()))
    want = a.astype(np.float64) @ Bb.float().cpu().numpy().astype(np.float64)
    assert relerr(y.cpu().numpy(), want) < 1e-5


@pytest.mark.parametrize("M,N,K", [(1, 8, 8), (5, 100, 264), (256, 1152, 896), (77, 3584, 512)])
def test_gemm_bf16_nt(L, M, N, K):
    """include/cuda.h:790-841: C = A . W^T with W bf16 row-major [N, K] (exact widening)."""
    from cpp_tensorlib_b200 import check
    A, W = rnd((M, K), 11, -1.0, 1.0), rnd((N, K), 12, -0.1, 0.1)
    dA, dW = torch.from_numpy(A).cuda(), torch.from_numpy(W).cuda().to(torch.bfloat16)
    out = torch.empty((M, N), device="cuda")
    check(L.tlb_gemm_bf16_nt(_p(dA), _p(dW), _p(out), M, N, K, _s()))
    want = A.astype(np.float64) @ dW.float().cpu().numpy().astype(np.float64).T
    assert relerr(out.cpu().numpy(), want) < 1e-5
