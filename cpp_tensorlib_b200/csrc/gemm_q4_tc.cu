// int4 dequant-matmul for many activation rows (prefill / batched rows, M > 8):
// Y[M,N] = alpha * X[M,K] . dequant(Wq) + beta on the 5th-generation tensor cores
// (tcgen05.mma, accumulator in TMEM).  The reference has no weight-native int4
// GEMM: it dequantises the whole matrix on the host on every call, uploads the f32
// copy and runs tl_sgemm_rb (include/array.h:1980-1984, 1546-1569,
// kernels/tensorlib_cuda.cu:310-421).
//
// Tiling: one CTA per 128 weight rows (N = 18944 = 148 x 128: one wave of the 148
// SMs).  The WEIGHT tile is the UMMA "A" operand (M = 128), the activation rows are
// the "B" operand (UMMA N = up to 256 rows of X per pass), so the accumulator in
// TMEM is Y^T[128 n][Mt m] and every weight is dequantised exactly once per pass.
//
// Precision: the 1e-4 bar against the dequantised-f32 oracle forbids plain
// bf16/tf32 operands, so both operands are split exactly into tf32 hi + lo parts
// (hi = f32 with the low 13 mantissa bits cleared, lo = x - hi) and three MMAs per
// k-step accumulate Wh.Xh + Wh.Xl + Wl.Xh in f32 (kind::tf32; dropped term 2^-22).
//
// Warp roles (192 threads): warp 0 = TMA producer (packed nibbles + scales in raw
// 128-k stages; X hi/lo tiles per 32-k block), warp 1 = TMEM allocator and the one
// MMA-issuing thread, warps 2-5 = dequantisers (thread r owns weight row r: 32
// nibbles + 1 scale -> 32 tf32 hi/lo pairs written in the 128-byte-swizzled K-major
// UMMA layout) and, at the end, the epilogue (tcgen05.ld, affine, coalesced stores).
// All waits are bounded; a timeout sets the status word, the kernel still frees
// its TMEM and returns.
#include "common.cuh"

namespace tlb {

constexpr int TC_THREADS = 192;
constexpr int TC_ROWS = 128;       // weight rows per CTA (UMMA M)
constexpr int TC_KB = 32;          // k per block (one 128-byte swizzle atom of tf32)
constexpr int TC_RAW_KB = 4;       // k-blocks per raw stage (128 k)
constexpr int TC_STAGES = 2;
constexpr int TC_MT_MAX = 256;     // activation rows per pass (UMMA N)

struct TcParams {
  float* y;
  long long ldy;
  int M, N, K;
  int m0, Mt;        // rows [m0, m0 + Mt) of X in this pass; Mt % 16 == 0
  float alpha, beta;
  int* status;
};

struct TcSmem {
  size_t raw_w, raw_s, a_hi, a_lo, b_hi, b_lo, bars, tmem_slot, total;
};
__host__ __device__ inline TcSmem tc_smem_layout(int Mt) {
  TcSmem L;
  size_t o = 0;
  L.raw_w = o; o += (size_t)TC_STAGES * TC_ROWS * 64;        // 128 rows x 64 B (128 k)
  L.raw_s = o; o += (size_t)TC_STAGES * TC_ROWS * 16;        // 128 rows x 4 f32
  o = (o + 1023) & ~(size_t)1023;
  L.a_hi = o; o += (size_t)TC_STAGES * TC_ROWS * 128;
  L.a_lo = o; o += (size_t)TC_STAGES * TC_ROWS * 128;
  L.b_hi = o; o += (size_t)TC_STAGES * Mt * 128;
  L.b_lo = o; o += (size_t)TC_STAGES * Mt * 128;
  L.bars = o; o += 16 * 8;
  L.tmem_slot = o; o += 16;
  L.total = o + 1024;
  return L;
}

// ---- tcgen05 wrappers -------------------------------------------------------
__device__ __forceinline__ void tc_alloc(uint32_t* slot_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(slot_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// K-major, 128-byte swizzle shared-memory matrix descriptor: rows of 128 bytes,
// 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t tc_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);         // start address
  d |= (uint64_t)1 << 16;                               // leading byte offset (unused here)
  d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset: 8 rows x 128 B
  d |= (uint64_t)1 << 46;                               // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
  return d;
}
// kind::tf32, f32 accumulate, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t tc_idesc_tf32(int n) {
  uint32_t d = 0;
  d |= 1u << 4;                    // D format f32
  d |= 2u << 7;                    // A format tf32
  d |= 2u << 10;                   // B format tf32
  d |= (uint32_t)(n >> 3) << 17;   // N / 8
  d |= (uint32_t)(TC_ROWS >> 4) << 24;  // M / 16
  return d;
}

enum { B_RAW_FULL = 0, B_RAW_EMPTY = 2, B_B_FULL = 4, B_A_READY = 6, B_AB_EMPTY = 8, B_ACC = 10 };

__global__ void __launch_bounds__(TC_THREADS, 1)
    gemm_q4_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
                      const __grid_constant__ CUtensorMap tmXh, const __grid_constant__ CUtensorMap tmXl,
                      TcParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const TcSmem L = tc_smem_layout(p.Mt);
  uint64_t* bars = (uint64_t*)(base + L.bars);
  uint32_t* tmem_slot = (uint32_t*)(base + L.tmem_slot);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * TC_ROWS;
  const int nkb = (p.K + TC_KB - 1) / TC_KB;
  uint32_t ncols = 32;
  while ((int)ncols < p.Mt) ncols <<= 1;

  if (tid == 0) {
    for (int s = 0; s < TC_STAGES; s++) {
      mbar_init(&bars[B_RAW_FULL + s], 1);
      mbar_init(&bars[B_RAW_EMPTY + s], 4);
      mbar_init(&bars[B_B_FULL + s], 1);
      mbar_init(&bars[B_A_READY + s], 4);
      mbar_init(&bars[B_AB_EMPTY + s], 1);
    }
    mbar_init(&bars[B_ACC], 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tc_alloc(tmem_slot, ncols);
    tc_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  bool failed = false;

  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      for (int kb = 0; kb < nkb && !failed; kb++) {
        if (kb % TC_RAW_KB == 0) {
          const int ri = kb / TC_RAW_KB, rs = ri % TC_STAGES;
          if (!mbar_wait_bounded(&bars[B_RAW_EMPTY + rs], ((ri / TC_STAGES) & 1) ^ 1, p.status, 500)) { failed = true; break; }
          mbar_expect_tx(&bars[B_RAW_FULL + rs], TC_ROWS * 64 + TC_ROWS * 16);
          tma_load_2d(base + L.raw_w + (size_t)rs * TC_ROWS * 64, &tmW, ri * 16, n0, &bars[B_RAW_FULL + rs]);
          tma_load_2d(base + L.raw_s + (size_t)rs * TC_ROWS * 16, &tmS, ri * 4, n0, &bars[B_RAW_FULL + rs]);
        }
        const int s = kb % TC_STAGES;
        if (!mbar_wait_bounded(&bars[B_AB_EMPTY + s], ((kb / TC_STAGES) & 1) ^ 1, p.status, 501)) { failed = true; break; }
        mbar_expect_tx(&bars[B_B_FULL + s], 2u * p.Mt * 128u);
        tma_load_2d(base + L.b_hi + (size_t)s * p.Mt * 128, &tmXh, kb * TC_KB, p.m0, &bars[B_B_FULL + s]);
        tma_load_2d(base + L.b_lo + (size_t)s * p.Mt * 128, &tmXl, kb * TC_KB, p.m0, &bars[B_B_FULL + s]);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = tc_idesc_tf32(p.Mt);
      for (int kb = 0; kb < nkb && !failed; kb++) {
        const int s = kb % TC_STAGES;
        const uint32_t ph = (kb / TC_STAGES) & 1;
        if (!mbar_wait_bounded(&bars[B_B_FULL + s], ph, p.status, 510)) { failed = true; break; }
        if (!mbar_wait_bounded(&bars[B_A_READY + s], ph, p.status, 511)) { failed = true; break; }
        tc_fence_after();
        const uint64_t ah = tc_desc_sw128(smem_u32(base + L.a_hi + (size_t)s * TC_ROWS * 128));
        const uint64_t al = tc_desc_sw128(smem_u32(base + L.a_lo + (size_t)s * TC_ROWS * 128));
        const uint64_t bh = tc_desc_sw128(smem_u32(base + L.b_hi + (size_t)s * p.Mt * 128));
        const uint64_t bl = tc_desc_sw128(smem_u32(base + L.b_lo + (size_t)s * p.Mt * 128));
#pragma unroll
        for (int ks = 0; ks < TC_KB / 8; ks++) {
          const uint64_t adv = (uint64_t)(ks * 32 >> 4);  // 8 tf32 = 32 bytes along K
          tc_mma_tf32(tmem, ah + adv, bh + adv, idesc, (kb | ks) ? 1u : 0u);
          tc_mma_tf32(tmem, ah + adv, bl + adv, idesc, 1u);
          tc_mma_tf32(tmem, al + adv, bh + adv, idesc, 1u);
        }
        tc_commit(&bars[B_AB_EMPTY + s]);  // frees this stage's A and B when the MMAs retire
      }
      tc_commit(&bars[B_ACC]);
    }
  } else {
    // ---------------- dequantisers (thread r = weight row r) ----------------
    const int r = tid - 64;
    for (int kb = 0; kb < nkb && !failed; kb++) {
      const int ri = kb / TC_RAW_KB, rs = ri % TC_STAGES, c = kb % TC_RAW_KB;
      const int s = kb % TC_STAGES;
      if (c == 0 && !mbar_wait_bounded(&bars[B_RAW_FULL + rs], (ri / TC_STAGES) & 1, p.status, 520)) { failed = true; break; }
      if (!mbar_wait_bounded(&bars[B_AB_EMPTY + s], ((kb / TC_STAGES) & 1) ^ 1, p.status, 521)) { failed = true; break; }
      // raw tile: 64-byte rows, 64-byte swizzle (chunk ^ ((row >> 1) & 3))
      const unsigned char* rw = base + L.raw_w + (size_t)rs * TC_ROWS * 64;
      const uint4 q = *(const uint4*)(rw + r * 64 + ((c ^ ((r >> 1) & 3)) << 4));
      const float sc = *(const float*)(base + L.raw_s + (size_t)rs * TC_ROWS * 16 + r * 16 + c * 4);
      const unsigned w4[4] = {q.x, q.y, q.z, q.w};
      unsigned char* ahi = base + L.a_hi + (size_t)s * TC_ROWS * 128 + r * 128;
      unsigned char* alo = base + L.a_lo + (size_t)s * TC_ROWS * 128 + r * 128;
#pragma unroll
      for (int j = 0; j < 8; j++) {  // chunk j = 4 consecutive k
        const unsigned word = w4[j >> 1] >> ((j & 1) * 16);
        float hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float wv = sc * (float)((int)((word >> (4 * e)) & 0xFu) - 8);
          hi[e] = __uint_as_float(__float_as_uint(wv) & 0xFFFFE000u);
          lo[e] = wv - hi[e];
        }
        const int pc = (j ^ (r & 7)) << 4;
        *(float4*)(ahi + pc) = make_float4(hi[0], hi[1], hi[2], hi[3]);
        *(float4*)(alo + pc) = make_float4(lo[0], lo[1], lo[2], lo[3]);
      }
      fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars[B_A_READY + s]);
        if (c == TC_RAW_KB - 1 || kb == nkb - 1) mbar_arrive(&bars[B_RAW_EMPTY + rs]);
      }
    }
    // ---------------- epilogue: TMEM -> registers -> Y ----------------
    if (!failed && mbar_wait_bounded(&bars[B_ACC], 0, p.status, 530)) {
      tc_fence_after();
      const int quarter = warp & 3;                 // TMEM lanes this warp may read
      const int n = n0 + quarter * 32 + lane;
      const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16);
      for (int c0 = 0; c0 < p.Mt; c0 += 16) {
        float v[16];
        tc_ld16(tbase + (uint32_t)c0, v);
        if (n < p.N) {
#pragma unroll
          for (int i = 0; i < 16; i++) {
            const int m = p.m0 + c0 + i;
            if (m < p.M) p.y[(long long)m * p.ldy + n] = v[i] * p.alpha + p.beta;
          }
        }
      }
      tc_fence_before();
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tc_dealloc(tmem, ncols);
  }
}

// X -> tf32 hi / lo planes ([M][K] f32 each, contiguous)
__global__ void split_tf32_kernel(const float* __restrict__ x, long long ldx, int M, int K,
                                  float* __restrict__ xh, float* __restrict__ xl) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)M * K) return;
  const int m = (int)(i / K), k = (int)(i % K);
  const float v = x[(long long)m * ldx + k];
  const float h = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
  xh[i] = h;
  xl[i] = v - h;
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
bool gemm_q4_tc_eligible(const void* qw, const void* scales, int N, int K, int M) {
  if (M <= 8 || N <= 0) return false;
  if (K % 128 != 0) return false;
  return (((uintptr_t)qw & 15) == 0) && (((uintptr_t)scales & 15) == 0);
}

int gemm_q4_tc_launch(DeviceCtx* c, const float* x, long long ldx, int M, const void* qw,
                      const float* scales, float* y, long long ldy, int N, int K, float alpha,
                      float beta, float* xsplit, cudaStream_t stream) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return set_error(TLB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  float* xh = xsplit;
  float* xl = xsplit + (size_t)M * K;
  {
    const size_t tot = (size_t)M * K;
    LaunchCfg lc(dim3((unsigned)((tot + 255) / 256)), dim3(256), 0, stream, pdl_enabled());
    TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, split_tf32_kernel, x, ldx, M, K, xh, xl));
  }
  CUtensorMap tmW, tmS, tmXh, tmXl;
  cuuint32_t es[2] = {1, 1};
  {
    cuuint64_t dim[2] = {(cuuint64_t)(K / 8), (cuuint64_t)N};
    cuuint64_t str[1] = {(cuuint64_t)(K / 2)};
    cuuint32_t box[2] = {16, TC_ROWS};
    if (enc(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(qw), dim, str, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return set_error(TLB_ERR_CUDA, "gemm_q4_tc: tensor map (weights) encode failed");
  }
  {
    cuuint64_t dim[2] = {(cuuint64_t)(K / 32), (cuuint64_t)N};
    cuuint64_t str[1] = {(cuuint64_t)(K / 8)};
    cuuint32_t box[2] = {4, TC_ROWS};
    if (enc(&tmS, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(scales), dim, str, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return set_error(TLB_ERR_CUDA, "gemm_q4_tc: tensor map (scales) encode failed");
  }
  static std::atomic<unsigned long long> attr_done{0};
  {
    const int rc_attr = ensure_dynamic_smem(gemm_q4_tc_kernel, 227 * 1024, attr_done);
    if (rc_attr) return rc_attr;
  }
  for (int m0 = 0; m0 < M; m0 += TC_MT_MAX) {
    int Mt = M - m0 < TC_MT_MAX ? M - m0 : TC_MT_MAX;
    Mt = (Mt + 15) / 16 * 16;
    cuuint64_t dim[2] = {(cuuint64_t)K, (cuuint64_t)M};
    cuuint64_t str[1] = {(cuuint64_t)K * 4};
    cuuint32_t box[2] = {TC_KB, (cuuint32_t)Mt};
    if (enc(&tmXh, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, xh, dim, str, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
        enc(&tmXl, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, xl, dim, str, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return set_error(TLB_ERR_CUDA, "gemm_q4_tc: tensor map (activations) encode failed");
    TcParams p;
    p.y = y; p.ldy = ldy; p.M = M; p.N = N; p.K = K; p.m0 = m0; p.Mt = Mt;
    p.alpha = alpha; p.beta = beta; p.status = c->status;
    LaunchCfg lc(dim3((N + TC_ROWS - 1) / TC_ROWS), dim3(TC_THREADS), tc_smem_layout(Mt).total, stream,
                 pdl_enabled());
    TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, gemm_q4_tc_kernel, tmW, tmS, tmXh, tmXl, p));
  }
  return TLB_OK;
}

}  // namespace tlb
