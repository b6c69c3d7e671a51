// The rest of the array surface the lazy-graph evaluator offers to a GPU backend: elementwise
// binary / unary ops with the fused affine epilogue, rank-2 broadcast binaries, row reductions
// and softmax over the last axis, the f32 GEMM, and the [K,N]-layout decode GEMVs on f32 / bf16
// weights plus the weight-native bf16 prefill GEMM.  Replaces tl_add..tl_affine, tl_row_sum /
// tl_row_max / tl_softmax, tl_sgemm / tl_sgemm_rb, tl_gemv_f32 / tl_gemv_bf16 and
// gemm_bf16_nt_core of the reference (kernels/tensorlib_cuda.cu:25-82, 222-421, 474-682) behind
// the facade functions of include/cuda.h:640-742, 790-841, 1409-1503.  None of this is on the
// decode token's path; the kernels are plain, coalesced, HBM-bound CUDA-core code with exact
// f32 arithmetic (every expression is the reference's: out = expr * scale + offset).
#include <cuda_bf16.h>

#include "common.cuh"

namespace tlb {

namespace {

enum : int { OP_ADD = 0, OP_SUB = 1, OP_MUL = 2, OP_DIV = 3, OP_POW = 4 };
enum : int { U_EXP = 0, U_LOG = 1, U_SQRT = 2, U_SIGMOID = 3, U_RELU = 4, U_AFFINE = 5 };
enum : int { R_SOFTMAX = 0, R_SUM = 1, R_MAX = 2 };

template <int OP>
__device__ __forceinline__ float bin(float a, float b) {
  if (OP == OP_ADD) return a + b;
  if (OP == OP_SUB) return a - b;
  if (OP == OP_MUL) return a * b;
  if (OP == OP_DIV) return a / b;
  return powf(a, b);
}
template <int OP>
__device__ __forceinline__ float una(float a) {
  if (OP == U_EXP) return expf(a);
  if (OP == U_LOG) return logf(a);
  if (OP == U_SQRT) return sqrtf(a);
  if (OP == U_SIGMOID) return 1.0f / (1.0f + expf(-a));
  if (OP == U_RELU) return a > 0.0f ? a : 0.0f;
  return a;
}

// out = (a OP b) * scale + offset; VEC: all three pointers 16-byte aligned, 4 elements per thread
template <int OP, bool VEC>
__global__ void ew_binary_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                 long long n, float scale, float offset) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * (VEC ? 4 : 1);
  if (VEC) {
    if (i + 3 < n) {
      const float4 x = *(const float4*)(a + i), y = *(const float4*)(b + i);
      *(float4*)(out + i) = make_float4(bin<OP>(x.x, y.x) * scale + offset, bin<OP>(x.y, y.y) * scale + offset,
                                        bin<OP>(x.z, y.z) * scale + offset, bin<OP>(x.w, y.w) * scale + offset);
    } else {
      for (long long j = i; j < n; j++) out[j] = bin<OP>(a[j], b[j]) * scale + offset;
    }
  } else if (i < n) {
    out[i] = bin<OP>(a[i], b[i]) * scale + offset;
  }
}

// rank-2 broadcast: out[r, c] = (a[r * ars + c * acs] OP b[r * brs + c * bcs]) * scale + offset
template <int OP>
__global__ void ew_bcast_kernel(const float* __restrict__ a, long long ars, long long acs,
                                const float* __restrict__ b, long long brs, long long bcs,
                                float* __restrict__ out, long long rows, long long cols, float scale,
                                float offset) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * cols) return;
  const long long r = i / cols, c = i - r * cols;
  out[i] = bin<OP>(a[r * ars + c * acs], b[r * brs + c * bcs]) * scale + offset;
}

template <int OP, bool VEC>
__global__ void ew_unary_kernel(const float* __restrict__ a, float* __restrict__ out, long long n, float scale,
                                float offset) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * (VEC ? 4 : 1);
  if (VEC) {
    if (i + 3 < n) {
      const float4 x = *(const float4*)(a + i);
      *(float4*)(out + i) = make_float4(una<OP>(x.x) * scale + offset, una<OP>(x.y) * scale + offset,
                                        una<OP>(x.z) * scale + offset, una<OP>(x.w) * scale + offset);
    } else {
      for (long long j = i; j < n; j++) out[j] = una<OP>(a[j]) * scale + offset;
    }
  } else if (i < n) {
    out[i] = una<OP>(a[i]) * scale + offset;
  }
}

__device__ __forceinline__ float block_reduce(float v, float* sm, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  if (lane == 0) sm[warp] = v;
  __syncthreads();
  float r = sm[0];
  for (int w = 1; w < nw; w++) r = is_max ? fmaxf(r, sm[w]) : r + sm[w];   // fixed order
  __syncthreads();
  return r;
}

// one block per row over the last axis: softmax writes the row (scale / offset ignored, as in
// the reference), row_sum / row_max write one value with the affine epilogue
template <int OP>
__global__ void row_op_kernel(const float* __restrict__ in, float* __restrict__ out, long long cols, float scale,
                              float offset) {
  __shared__ float sm[32];
  const float* src = in + (size_t)blockIdx.x * cols;
  if (OP == R_SUM) {
    float acc = 0.f;
    for (long long c = threadIdx.x; c < cols; c += blockDim.x) acc += src[c];
    acc = block_reduce(acc, sm, false);
    if (threadIdx.x == 0) out[blockIdx.x] = acc * scale + offset;
    return;
  }
  float m = -3.402823466e+38f;
  for (long long c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, src[c]);
  m = block_reduce(m, sm, true);
  if (OP == R_MAX) {
    if (threadIdx.x == 0) out[blockIdx.x] = m * scale + offset;
    return;
  }
  float s = 0.f;
  for (long long c = threadIdx.x; c < cols; c += blockDim.x) s += expf(src[c] - m);
  s = block_reduce(s, sm, false);
  const float inv = 1.0f / s;
  float* dst = out + (size_t)blockIdx.x * cols;
  for (long long c = threadIdx.x; c < cols; c += blockDim.x) dst[c] = expf(src[c] - m) * inv;
}

// ---- f32 GEMM: C[m,n] = (A . B) * scale + offset -----------------------------------------
// A(i,k) = ta ? A[k*lda + i] : A[i*lda + k];  B(k,j) = tb ? B[j*ldb + k] : B[k*ldb + j]
// (the layout contract of tl_sgemm, kernels/tensorlib_cuda.cu:262-276).  BT = float, or
// __nv_bfloat16 for the weight-native prefill GEMM on bf16 [N,K] weights (tb = true).
// 64 x 64 output tile per block, k-tiles of 16, 4 x 4 outputs per thread, operands staged in
// shared memory k-major; global loads are coalesced along whichever index is contiguous.
constexpr int GM_BM = 64, GM_BN = 64, GM_BK = 16;

__device__ __forceinline__ float ldb_elem(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float ldb_elem(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }

template <typename BT>
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ A, long long lda, int ta,
                                                       const BT* __restrict__ B, long long ldb, int tb,
                                                       float* __restrict__ C, int m, int n, int k, float scale,
                                                       float offset) {
  __shared__ float As[GM_BK][GM_BM + 4];
  __shared__ float Bs[GM_BK][GM_BN + 4];
  const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
  const int i0 = blockIdx.y * GM_BM, j0 = blockIdx.x * GM_BN;
  float acc[4][4];
#pragma unroll
  for (int r = 0; r < 4; r++)
#pragma unroll
    for (int c = 0; c < 4; c++) acc[r][c] = 0.f;
  for (int k0 = 0; k0 < k; k0 += GM_BK) {
#pragma unroll
    for (int r = 0; r < 4; r++) {
      int ii, kk;
      if (ta) { ii = t & 63; kk = (t >> 6) + 4 * r; } else { kk = t & 15; ii = (t >> 4) + 16 * r; }
      const int gi = i0 + ii, gk = k0 + kk;
      float v = 0.f;
      if (gi < m && gk < k) v = ta ? A[(size_t)gk * lda + gi] : A[(size_t)gi * lda + gk];
      As[kk][ii] = v;
      int jj, kb;
      if (tb) { kb = t & 15; jj = (t >> 4) + 16 * r; } else { jj = t & 63; kb = (t >> 6) + 4 * r; }
      const int gj = j0 + jj, gkb = k0 + kb;
      float w = 0.f;
      if (gj < n && gkb < k) w = tb ? ldb_elem(B, (size_t)gj * ldb + gkb) : ldb_elem(B, (size_t)gkb * ldb + gj);
      Bs[kb][jj] = w;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GM_BK; kk++) {
      const float4 a4 = *(const float4*)&As[kk][ty * 4];
      const float4 b4 = *(const float4*)&Bs[kk][tx * 4];
      const float av[4] = {a4.x, a4.y, a4.z, a4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int r = 0; r < 4; r++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[r][c] = fmaf(av[r], bv[c], acc[r][c]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; r++) {
    const int gi = i0 + ty * 4 + r;
    if (gi >= m) continue;
#pragma unroll
    for (int c = 0; c < 4; c++) {
      const int gj = j0 + tx * 4 + c;
      if (gj < n) C[(size_t)gi * n + gj] = acc[r][c] * scale + offset;
    }
  }
}

// ---- decode GEMV on [K,N] weights: y[n] = sum_k a[k] * B[k*N + n] ---------------------------
// (tl_gemv_f32 / tl_gemv_bf16, kernels/tensorlib_cuda.cu:611-682.)  A block covers 128 columns;
// its 8 warps take every 8th k, a lane owns 4 adjacent columns (one 16-byte f32 load or one
// 8-byte bf16 load per k), the warps' partial sums meet in shared memory in warp order.
template <typename BT>
__global__ void __launch_bounds__(256) gemv_kn_kernel(const float* __restrict__ a, const BT* __restrict__ B,
                                                      float* __restrict__ y, int N, int K) {
  __shared__ float part[8][128];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = blockIdx.x * 128 + lane * 4;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const bool full = n0 + 3 < N && (N % 4) == 0;
  for (int kk = warp; kk < K; kk += 8) {
    const float av = a[kk];
    if (full) {
      if (sizeof(BT) == 4) {
        const float4 w = *(const float4*)((const float*)B + (size_t)kk * N + n0);
        acc[0] = fmaf(av, w.x, acc[0]); acc[1] = fmaf(av, w.y, acc[1]);
        acc[2] = fmaf(av, w.z, acc[2]); acc[3] = fmaf(av, w.w, acc[3]);
      } else {
        const uint2 w = *(const uint2*)((const __nv_bfloat16*)B + (size_t)kk * N + n0);
        acc[0] = fmaf(av, __uint_as_float(w.x << 16), acc[0]);
        acc[1] = fmaf(av, __uint_as_float(w.x & 0xffff0000u), acc[1]);
        acc[2] = fmaf(av, __uint_as_float(w.y << 16), acc[2]);
        acc[3] = fmaf(av, __uint_as_float(w.y & 0xffff0000u), acc[3]);
      }
    } else {
#pragma unroll
      for (int c = 0; c < 4; c++)
        if (n0 + c < N) acc[c] = fmaf(av, ldb_elem(B, (size_t)kk * N + n0 + c), acc[c]);
    }
  }
#pragma unroll
  for (int c = 0; c < 4; c++) part[warp][lane * 4 + c] = acc[c];
  __syncthreads();
  if (threadIdx.x < 128) {
    const int n = blockIdx.x * 128 + threadIdx.x;
    if (n < N) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; w++) s += part[w][threadIdx.x];
      y[n] = s;
    }
  }
}

}  // namespace

template <int OP>
static int launch_binary_t(const float* a, const float* b, float* out, long long n, float scale, float offset,
                           cudaStream_t s) {
  const bool vec = ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) == 0);
  const long long per = vec ? 4 : 1, threads = (n + per - 1) / per;
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  if (vec) ew_binary_kernel<OP, true><<<blocks, 256, 0, s>>>(a, b, out, n, scale, offset);
  else ew_binary_kernel<OP, false><<<blocks, 256, 0, s>>>(a, b, out, n, scale, offset);
  TLB_CUDA(cudaGetLastError());
  return TLB_OK;
}
template <int OP>
static int launch_unary_t(const float* a, float* out, long long n, float scale, float offset, cudaStream_t s) {
  const bool vec = ((((uintptr_t)a | (uintptr_t)out) & 15) == 0);
  const long long per = vec ? 4 : 1, threads = (n + per - 1) / per;
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  if (vec) ew_unary_kernel<OP, true><<<blocks, 256, 0, s>>>(a, out, n, scale, offset);
  else ew_unary_kernel<OP, false><<<blocks, 256, 0, s>>>(a, out, n, scale, offset);
  TLB_CUDA(cudaGetLastError());
  return TLB_OK;
}
template <int OP>
static int launch_bcast_t(const float* a, long long ars, long long acs, const float* b, long long brs,
                          long long bcs, float* out, long long rows, long long cols, float scale, float offset,
                          cudaStream_t s) {
  const unsigned blocks = (unsigned)((rows * cols + 255) / 256);
  ew_bcast_kernel<OP><<<blocks, 256, 0, s>>>(a, ars, acs, b, brs, bcs, out, rows, cols, scale, offset);
  TLB_CUDA(cudaGetLastError());
  return TLB_OK;
}

}  // namespace tlb

using namespace tlb;
static inline cudaStream_t S_(void* s) { return reinterpret_cast<cudaStream_t>(s); }

extern "C" {

int tlb_binary(int op, const float* a, const float* b, float* out, int64_t n, float scale, float offset,
               void* stream) {
  TLB_REQUIRE(a && b && out && n >= 0 && n < (1ll << 40), "tlb_binary: bad arguments");
  if (n == 0) return TLB_OK;
  switch (op) {
    case OP_ADD: return launch_binary_t<OP_ADD>(a, b, out, n, scale, offset, S_(stream));
    case OP_SUB: return launch_binary_t<OP_SUB>(a, b, out, n, scale, offset, S_(stream));
    case OP_MUL: return launch_binary_t<OP_MUL>(a, b, out, n, scale, offset, S_(stream));
    case OP_DIV: return launch_binary_t<OP_DIV>(a, b, out, n, scale, offset, S_(stream));
    case OP_POW: return launch_binary_t<OP_POW>(a, b, out, n, scale, offset, S_(stream));
  }
  return set_error(TLB_ERR_ARG, "tlb_binary: unknown op");
}

int tlb_binary_bcast(int op, const float* a, int64_t a_rs, int64_t a_cs, const float* b, int64_t b_rs,
                     int64_t b_cs, float* out, int64_t rows, int64_t cols, float scale, float offset,
                     void* stream) {
  TLB_REQUIRE(a && b && out && rows >= 0 && cols >= 0 && rows * cols < (1ll << 40), "tlb_binary_bcast: bad arguments");
  if (rows * cols == 0) return TLB_OK;
  cudaStream_t s = S_(stream);
  switch (op) {
    case OP_ADD: return launch_bcast_t<OP_ADD>(a, a_rs, a_cs, b, b_rs, b_cs, out, rows, cols, scale, offset, s);
    case OP_SUB: return launch_bcast_t<OP_SUB>(a, a_rs, a_cs, b, b_rs, b_cs, out, rows, cols, scale, offset, s);
    case OP_MUL: return launch_bcast_t<OP_MUL>(a, a_rs, a_cs, b, b_rs, b_cs, out, rows, cols, scale, offset, s);
    case OP_DIV: return launch_bcast_t<OP_DIV>(a, a_rs, a_cs, b, b_rs, b_cs, out, rows, cols, scale, offset, s);
    case OP_POW: return launch_bcast_t<OP_POW>(a, a_rs, a_cs, b, b_rs, b_cs, out, rows, cols, scale, offset, s);
  }
  return set_error(TLB_ERR_ARG, "tlb_binary_bcast: unknown op");
}

int tlb_unary(int op, const float* a, float* out, int64_t n, float scale, float offset, void* stream) {
  TLB_REQUIRE(a && out && n >= 0 && n < (1ll << 40), "tlb_unary: bad arguments");
  if (n == 0) return TLB_OK;
  switch (op) {
    case U_EXP: return launch_unary_t<U_EXP>(a, out, n, scale, offset, S_(stream));
    case U_LOG: return launch_unary_t<U_LOG>(a, out, n, scale, offset, S_(stream));
    case U_SQRT: return launch_unary_t<U_SQRT>(a, out, n, scale, offset, S_(stream));
    case U_SIGMOID: return launch_unary_t<U_SIGMOID>(a, out, n, scale, offset, S_(stream));
    case U_RELU: return launch_unary_t<U_RELU>(a, out, n, scale, offset, S_(stream));
    case U_AFFINE: return launch_unary_t<U_AFFINE>(a, out, n, scale, offset, S_(stream));
  }
  return set_error(TLB_ERR_ARG, "tlb_unary: unknown op");
}

int tlb_row_op(int op, const float* in, float* out, int64_t rows, int64_t cols, float scale, float offset,
               void* stream) {
  TLB_REQUIRE(in && out && rows >= 0 && cols > 0 && rows < (1ll << 31), "tlb_row_op: bad arguments");
  if (rows == 0) return TLB_OK;
  const unsigned g = (unsigned)rows;
  switch (op) {
    case R_SOFTMAX: row_op_kernel<R_SOFTMAX><<<g, 256, 0, S_(stream)>>>(in, out, cols, scale, offset); break;
    case R_SUM: row_op_kernel<R_SUM><<<g, 256, 0, S_(stream)>>>(in, out, cols, scale, offset); break;
    case R_MAX: row_op_kernel<R_MAX><<<g, 256, 0, S_(stream)>>>(in, out, cols, scale, offset); break;
    default: return set_error(TLB_ERR_ARG, "tlb_row_op: unknown op");
  }
  TLB_CUDA(cudaGetLastError());
  return TLB_OK;
}

int tlb_gemm_f32(const float* a, int64_t lda, int ta, const float* b, int64_t ldb, int tb, float* out,
                 int64_t m, int64_t n, int64_t k, float scale, float offset, void* stream) {
  TLB_REQUIRE(a && b && out && m >= 0 && n >= 0 && k >= 0 && m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31),
              "tlb_gemm_f32: bad arguments");
  if (m == 0 || n == 0) return TLB_OK;
  dim3 grid((unsigned)((n + GM_BN - 1) / GM_BN), (unsigned)((m + GM_BM - 1) / GM_BM));
  TLB_REQUIRE(grid.y <= 65535, "tlb_gemm_f32: too many rows");
  gemm_f32_kernel<float><<<grid, 256, 0, S_(stream)>>>(a, lda, ta, b, ldb, tb, out, (int)m, (int)n, (int)k, scale,
                                                        offset);
  TLB_CUDA(cudaGetLastError());
  return TLB_OK;
}

int tlb_gemm_bf16_nt(const float* a, const void* w, float* c, int64_t M, int64_t N, int64_t K, void* stream) {
  TLB_REQUIRE(a && w && c && M > 0 && N > 0 && K > 0 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31),
              "tlb_gemm_bf16_nt: bad arguments");
  dim3 grid((unsigned)((N + GM_BN - 1) / GM_BN), (unsigned)((M + GM_BM - 1) / GM_BM));
  TLB_REQUIRE(grid.y <= 65535, "tlb_gemm_bf16_nt: too many rows");
  gemm_f32_kernel<__nv_bfloat16><<<grid, 256, 0, S_(stream)>>>(a, K, 0, (const __nv_bfloat16*)w, K, 1, c, (int)M,
                                                                (int)N, (int)K, 1.0f, 0.0f);
  TLB_CUDA(cudaGetLastError());
  return TLB_OK;
}

int tlb_gemv_f32(const float* a, const float* B, float* y, int64_t n, int64_t k, void* stream) {
  TLB_REQUIRE(a && B && y && n > 0 && k > 0 && n < (1ll << 31) && k < (1ll << 31), "tlb_gemv_f32: bad arguments");
  TLB_REQUIRE(((uintptr_t)B & 15) == 0, "tlb_gemv_f32: B must be 16-byte aligned");
  gemv_kn_kernel<float><<<(unsigned)((n + 127) / 128), 256, 0, S_(stream)>>>(a, B, y, (int)n, (int)k);
  TLB_CUDA(cudaGetLastError());
  return TLB_OK;
}

int tlb_gemv_bf16(const float* a, const void* B, float* y, int64_t n, int64_t k, void* stream) {
  TLB_REQUIRE(a && B && y && n > 0 && k > 0 && n < (1ll << 31) && k < (1ll << 31), "tlb_gemv_bf16: bad arguments");
  TLB_REQUIRE(((uintptr_t)B & 7) == 0, "tlb_gemv_bf16: B must be 8-byte aligned");
  gemv_kn_kernel<__nv_bfloat16><<<(unsigned)((n + 127) / 128), 256, 0, S_(stream)>>>(
      a, (const __nv_bfloat16*)B, y, (int)n, (int)k);
  TLB_CUDA(cudaGetLastError());
  return TLB_OK;
}

}  // extern "C"
