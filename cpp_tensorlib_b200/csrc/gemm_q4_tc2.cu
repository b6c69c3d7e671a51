// int4 dequant-matmul for many activation rows (prefill / batched rows, M > 8), second
// formulation: Y[M,N] = alpha * X[M,K] . dequant(Wq) + beta on the 5th-generation tensor cores
// with the GROUP SCALES KEPT OUT of the tensor-core operands.
//
//   y[m,n] = sum_g sc[n,g] * ( sum_{k in group g} (nib[n,k] - 8) * x[m,k] )
//
// The inner sum is an exact-operand contraction: nib - 8 is an integer in [-8, 7], exact in
// fp16, and x is carried as TWO fp16 planes (hi + lo of x * 2^-e_m, e_m a per-row power of two
// that keeps the row inside the fp16 range; 22 mantissa bits, the precision the tf32 hi/lo
// split gave).  So a group of 32 k costs 2 k-steps x 2 planes = 4 tcgen05.mma.kind::f16
// (K = 16 each) instead of 12 kind::tf32 MMAs at half the rate: a sixth of the tensor time of
// the formulation that folds the f32 scale into the weight operand (gemm_q4_tc.cu), which is
// tensor bound at a third of the tf32 peak.  Each group's product lands in one of four TMEM
// accumulators used in rotation; accumulate warps read it back with tcgen05.ld, multiply by
// the row's f32 group scale and add into registers -- the same order of operations as the
// reference's dequantise-then-multiply in f32 (include/array.h:666-684, 1980-1984).
//
// One CTA = 128 weight rows (UMMA M) x MT activation rows (UMMA N, 32 / 64 / 128), grid =
// (N / 128, M / MT).  Warp roles (512 threads): warp 0 TMA producer of the X planes (64-k
// stages, 128-byte swizzle), warp 1 TMEM allocator, warps 1 and 15 the MMA issuers (first / second group of a stage), warps 2-5
// nibble -> fp16 converters (thread r owns weight row r; the k order inside every group of 8
// is the one the nibble extraction produces -- 0,4,1,5,2,6,3,7 -- and the X planes are stored
// in the same order, so no byte permute is needed), warps 6-13 accumulate + epilogue (two per
// TMEM lane quarter, each half of the MT columns), warp 14 TMA producer of the PACKED weights:
// 128 rows x 128 bytes (256 k) per box into a ring of four, 64 KB in flight per SM.  (Register
// loads by the converters, 32 bytes per row and stage with four stages in flight, kept only
// 16 KB per SM in flight and paced the whole kernel at ~1 TB/s of weight bytes.)  All waits
// are bounded; a timeout sets the status word, the kernel still frees its TMEM and returns.
// No cluster launch, no multicast.
#include <cuda_fp16.h>

#include "common.cuh"

namespace tlb {

namespace {

constexpr int T2_THREADS = 512;
constexpr int T2_ROWS = 128;     // weight rows per CTA (UMMA M)
constexpr int T2_KS = 64;        // k per stage = two groups = one 128-byte swizzle row of fp16
constexpr int T2_RAW_STAGES = 4;              // ring of packed-weight boxes
constexpr int T2_RAW_BYTES = T2_ROWS * 128;   // one box: 128 rows x 128 bytes = 256 k per row
constexpr int T2_SUB = 4;                     // 64-k stages per packed box

struct T2Params {
  const unsigned* qw;        // packed nibbles, u32 [N][K/8]
  const float* scales;       // [N][K/32]
  const float* rowscale;     // [M] 2^e_m
  float* y;
  long long ldy;
  int M, N, K;
  float alpha, beta;
  int* status;
};

template <int MT>
struct T2Smem {
  static constexpr int STAGES = MT == 128 ? 3 : 4;                            // what fits beside the weight ring
  static constexpr size_t A = 0;                                              // [stages][128][128 B]
  static constexpr size_t B = A + (size_t)STAGES * T2_ROWS * 128;             // [stages][2 planes][MT][128 B]
  static constexpr size_t RAW = B + (size_t)STAGES * 2 * MT * 128;            // [raw stages][128][128 B]
  static constexpr size_t BARS = RAW + (size_t)T2_RAW_STAGES * T2_RAW_BYTES;
  static constexpr size_t SLOT = BARS + 32 * 8;
  static constexpr size_t TOTAL = SLOT + 16 + 1024;
};

__device__ __forceinline__ void t2_alloc(uint32_t* slot_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void t2_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void t2_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void t2_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void t2_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void t2_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void t2_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 16 consecutive columns of this warp's TMEM lane quarter (issue only; see t2_wait_ld)
__device__ __forceinline__ void t2_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ bool t2_elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
// the whole warp waits and agrees on the outcome, so a timeout cannot split it
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, int* status, int where) {
  return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity, status, where));
}
__device__ __forceinline__ void t2_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte swizzle shared-memory matrix descriptor: rows of 128 bytes, 8-row groups
// 1024 bytes apart (the layout TMA's SWIZZLE_128B box produces and the converters write).
__device__ __forceinline__ uint64_t t2_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16 with fp16 operands (format code 0), f32 accumulate, both K-major, M = 128, N = n
__device__ __forceinline__ uint32_t t2_idesc_f16(int n) {
  uint32_t d = 0;
  d |= 1u << 4;                          // D format f32
  d |= (uint32_t)(n >> 3) << 17;         // N / 8
  d |= (uint32_t)(T2_ROWS >> 4) << 24;   // M / 16
  return d;
}

// barrier indices
enum { T2_X_FULL = 0, T2_A_READY = 4, T2_ST_EMPTY = 8, T2_D_FULL = 12, T2_D_EMPTY = 16, T2_RAW_FULL = 20,
       T2_RAW_EMPTY = 24 };
// TMEM accumulators in rotation: the MMA thread runs up to T2_NBUF groups ahead of the
// accumulate warps, whose tcgen05.ld round trip (not the MMAs) is the latency of a group
constexpr int T2_NBUF = 4;

template <int MT>
__global__ void __launch_bounds__(T2_THREADS, 1)
    gemm_q4_tc2_kernel(const __grid_constant__ CUtensorMap tmX1, const __grid_constant__ CUtensorMap tmX2,
                       const __grid_constant__ CUtensorMap tmW, T2Params p) {
  using S = T2Smem<MT>;
  constexpr int T2_STAGES = S::STAGES;
  constexpr uint32_t NCOLS = T2_NBUF * MT;   // accumulators of MT columns each: 128 / 256 / 512
  constexpr int HC = MT / 2;              // columns per accumulate warp
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = (uint64_t*)(base + S::BARS);
  uint32_t* tmem_slot = (uint32_t*)(base + S::SLOT);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * T2_ROWS, m0 = blockIdx.y * MT;
  const int nst = p.K / T2_KS, ngr = p.K / 32, nraw = (nst + T2_SUB - 1) / T2_SUB;

  if (tid == 0) {
    for (int s = 0; s < T2_STAGES; s++) {
      mbar_init(&bars[T2_X_FULL + s], 1);
      mbar_init(&bars[T2_A_READY + s], 4);
      mbar_init(&bars[T2_ST_EMPTY + s], 2);   // one commit per issuer warp
    }
    for (int b = 0; b < T2_NBUF; b++) {
      mbar_init(&bars[T2_D_FULL + b], 1);
      mbar_init(&bars[T2_D_EMPTY + b], 8);
    }
    for (int q = 0; q < T2_RAW_STAGES; q++) {
      mbar_init(&bars[T2_RAW_FULL + q], 1);
      mbar_init(&bars[T2_RAW_EMPTY + q], 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    t2_alloc(tmem_slot, NCOLS);
    t2_relinquish();
  }
  t2_fence_before();
  __syncthreads();
  t2_fence_after();
  const uint32_t tmem = *tmem_slot;

  // the packed weights are not written by the kernel before this one: their producer starts
  // at once; every other role touches activations, the status block or y and waits
  if (warp != 14) pdl_wait();
  pdl_launch_dependents();

  if (warp == 14) {
    // ---------------- TMA producer: packed weights, 128 rows x 256 k per box ----------------
    if (lane == 0) {
      for (int q = 0; q < nraw; q++) {
        const int rs = q % T2_RAW_STAGES;
        if (!mbar_wait_bounded(&bars[T2_RAW_EMPTY + rs], ((q / T2_RAW_STAGES) & 1) ^ 1, p.status, 640)) break;
        mbar_expect_tx(&bars[T2_RAW_FULL + rs], (uint32_t)T2_RAW_BYTES);
        tma_load_2d(base + S::RAW + (size_t)rs * T2_RAW_BYTES, &tmW, q * 128, n0, &bars[T2_RAW_FULL + rs]);
      }
    }
  } else if (warp == 0) {
    // ---------------- TMA producer: the two fp16 planes of X, one 64-k stage at a time ----------------
    if (lane == 0) {
      for (int it = 0; it < nst; it++) {
        const int s = it % T2_STAGES;
        if (!mbar_wait_bounded(&bars[T2_ST_EMPTY + s], ((it / T2_STAGES) & 1) ^ 1, p.status, 600)) break;
        mbar_expect_tx(&bars[T2_X_FULL + s], 2u * MT * 128u);
        const int kx = it * T2_KS;
        tma_load_2d(base + S::B + (size_t)(s * 2 + 0) * MT * 128, &tmX1, kx, m0, &bars[T2_X_FULL + s]);
        tma_load_2d(base + S::B + (size_t)(s * 2 + 1) * MT * 128, &tmX2, kx, m0, &bars[T2_X_FULL + s]);
      }
    }
  } else if (warp == 1 || warp == 15) {
    // ---------------- MMA issuers: warp 1 the first group of every stage, warp 15 the second ----------------
    // The whole warp runs the loop (waits included) so that descriptors and addresses stay
    // warp-uniform values, and one elected lane issues; two issuers because the issue cost of
    // a tcgen05.mma (not its execution) bounds a single thread at this instruction size.
    const int grp = warp == 1 ? 0 : 1;
    const uint32_t idesc = t2_idesc_f16(MT);
    const bool leader = t2_elect_one();
    for (int it = 0; it < nst; it++) {
      const int s = it % T2_STAGES;
      const uint32_t ph = (it / T2_STAGES) & 1;
      const int gi = 2 * it + grp, buf = gi % T2_NBUF;
      if (!mbar_wait_warp(&bars[T2_D_EMPTY + buf], ((gi / T2_NBUF) & 1) ^ 1, p.status, 612)) break;
      if (!mbar_wait_warp(&bars[T2_X_FULL + s], ph, p.status, 610)) break;
      if (!mbar_wait_warp(&bars[T2_A_READY + s], ph, p.status, 611)) break;
      t2_fence_after();
      const uint64_t a = t2_desc_sw128(smem_u32(base + S::A + (size_t)s * T2_ROWS * 128));
      const uint64_t b1 = t2_desc_sw128(smem_u32(base + S::B + (size_t)(s * 2 + 0) * MT * 128));
      const uint64_t b2 = t2_desc_sw128(smem_u32(base + S::B + (size_t)(s * 2 + 1) * MT * 128));
      const uint32_t d = tmem + (uint32_t)(buf * MT);
      if (leader) {
#pragma unroll
        for (int ks = 0; ks < 2; ks++) {
          const uint64_t adv = (uint64_t)(((2 * grp + ks) * 32) >> 4);   // 16 fp16 = 32 bytes along K
          t2_mma_f16(d, a + adv, b1 + adv, idesc, ks ? 1u : 0u);
          t2_mma_f16(d, a + adv, b2 + adv, idesc, 1u);
        }
        t2_commit(&bars[T2_D_FULL + buf]);     // the group's product is complete when these retire
        t2_commit(&bars[T2_ST_EMPTY + s]);     // ... and (with the other issuer's) the stage can be overwritten
      }
      __syncwarp();
    }
  } else if (warp < 6) {
    // ---------------- nibble -> fp16 converters (thread r = weight row r) ----------------
    const int r = tid - 64;
    const __half2 off = __floats2half2_rn(1032.0f, 1032.0f);
    bool conv_ok = true;
    for (int q = 0; q < nraw && conv_ok; q++) {
      const int rs = q % T2_RAW_STAGES;
      if (!mbar_wait_bounded(&bars[T2_RAW_FULL + rs], (q / T2_RAW_STAGES) & 1, p.status, 621)) break;
      // the row's 128 packed bytes of this box: chunk c (16 bytes = 32 k) sits at c ^ (r & 7)
      const unsigned char* rrow = base + S::RAW + (size_t)rs * T2_RAW_BYTES + r * 128;
      uint4 wq[2 * T2_SUB];
#pragma unroll
      for (int c = 0; c < 2 * T2_SUB; c++) wq[c] = *(const uint4*)(rrow + ((c ^ (r & 7)) << 4));
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[T2_RAW_EMPTY + rs]);   // the box is in registers: refill it
#pragma unroll
      for (int u = 0; u < T2_SUB; u++) {
        const int it = q * T2_SUB + u;
        if (it >= nst) break;
        const int s = it % T2_STAGES;
        const uint4 c0 = wq[2 * u], c1 = wq[2 * u + 1];
        if (!mbar_wait_bounded(&bars[T2_ST_EMPTY + s], ((it / T2_STAGES) & 1) ^ 1, p.status, 620)) {
          conv_ok = false;
          break;
        }
        unsigned char* arow = base + S::A + (size_t)s * T2_ROWS * 128 + r * 128;
        const unsigned words[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
        for (int j = 0; j < 8; j++) {
          // slot e of the chunk holds (k = e, k = e + 4) of this word: fp16(1024 + nib) has the
          // bit pattern 0x6400 | nib, and 1024 + nib - 1032 = nib - 8 exactly
          unsigned qv[4];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const unsigned t = ((words[j] >> (4 * e)) & 0x000F000Fu) | 0x64006400u;
            const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&t), off);
            qv[e] = *reinterpret_cast<const unsigned*>(&v);
          }
          *(uint4*)(arow + ((j ^ (r & 7)) << 4)) = make_uint4(qv[0], qv[1], qv[2], qv[3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor core reads
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[T2_A_READY + s]);
      }
    }
  } else if (warp < 14) {
    // ---------------- accumulate (sc * group product) + epilogue ----------------
    const int quarter = warp & 3, half = (warp - 6) >> 2;
    const int r = quarter * 32 + lane, n = n0 + r;
    const int c_lo = half * HC;
    const float* sc_row = p.scales + (size_t)(n < p.N ? n : p.N - 1) * (p.K / 32);
    float acc[HC];
#pragma unroll
    for (int i = 0; i < HC; i++) acc[i] = 0.f;
    // the row's group scales, four at a time (K % 128 == 0), fetched two blocks ahead: one L2
    // round trip is longer than a group takes
    const float4* sc4 = (const float4*)sc_row;
    const int nblk = ngr / 4;
    float4 sc_blk = __ldg(sc4), sc_n1 = nblk > 1 ? __ldg(sc4 + 1) : sc_blk, sc_n2 = sc_blk;
    bool ok = true;
    for (int gi = 0; gi < ngr; gi++) {
      const int buf = gi % T2_NBUF;
      if ((gi & 3) == 0) {
        if (gi) { sc_blk = sc_n1; sc_n1 = sc_n2; }
        if ((gi >> 2) + 2 < nblk) sc_n2 = __ldg(sc4 + (gi >> 2) + 2);
      }
      const float sc = (gi & 3) == 0 ? sc_blk.x : ((gi & 3) == 1 ? sc_blk.y : ((gi & 3) == 2 ? sc_blk.z : sc_blk.w));
      if (!mbar_wait_bounded(&bars[T2_D_FULL + buf], (gi / T2_NBUF) & 1, p.status, 630)) { ok = false; break; }
      t2_fence_after();
      const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * MT + c_lo);
      // 32 columns per read; the accumulator goes back to the issuers as soon as the last
      // read has landed, before its FMAs.  (Measured and dropped: fma.rn.f32x2 pairs -- the
      // register pairing costs more than the halved FMA count saves, 200 vs 170 us at M = 512 --
      // and 16-column reads in flight under the previous 16 columns' FMAs.)
      constexpr int BATCH = HC < 32 ? HC : 32;
#pragma unroll
      for (int c0 = 0; c0 < HC; c0 += BATCH) {
        uint32_t v[BATCH / 16][16];
#pragma unroll
        for (int b = 0; b < BATCH / 16; b++) t2_ld16_issue(taddr + (uint32_t)(c0 + 16 * b), v[b]);
        t2_wait_ld();
        if (c0 + BATCH >= HC) {
          t2_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[T2_D_EMPTY + buf]);
        }
#pragma unroll
        for (int b = 0; b < BATCH / 16; b++)
#pragma unroll
          for (int i = 0; i < 16; i++) acc[c0 + 16 * b + i] = fmaf(sc, __uint_as_float(v[b][i]), acc[c0 + 16 * b + i]);
      }
    }
    if (ok && n < p.N) {
#pragma unroll
      for (int i = 0; i < HC; i++) {
        const int m = m0 + c_lo + i;
        if (m < p.M) p.y[(long long)m * p.ldy + n] = (acc[i] * __ldg(p.rowscale + m)) * p.alpha + p.beta;
      }
    }
  }
  t2_fence_before();
  __syncthreads();
  if (warp == 1) {
    t2_fence_after();
    t2_dealloc(tmem, NCOLS);
  }
}

// X -> two fp16 planes of x * 2^-e_m (hi, lo) + the row's 2^e_m.  One block per row.  Inside every
// group of 8 k the planes are stored in the order 0,4,1,5,2,6,3,7 -- the order in which the
// converters' nibble extraction lays out the weights.
__global__ void split_f16_kernel(const float* __restrict__ x, long long ldx, int K, __half* __restrict__ x1,
                                 __half* __restrict__ x2, float* __restrict__ rowscale) {
  __shared__ float sm[32];
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x;
  const float* row = x + (long long)m * ldx;
  const bool vec = ((uintptr_t)row & 15) == 0;   // K % 8 == 0 always; 16-byte rows take the float4 path
  float mx = 0.f;
  if (vec) {
    const float4* row4 = (const float4*)row;
    for (int i = threadIdx.x; i < K / 4; i += blockDim.x) {
      const float4 a = __ldg(row4 + i);
      mx = fmaxf(fmaxf(mx, fmaxf(fabsf(a.x), fabsf(a.y))), fmaxf(fabsf(a.z), fabsf(a.w)));
    }
  } else {
    for (int k = threadIdx.x; k < K; k += blockDim.x) mx = fmaxf(mx, fabsf(row[k]));
  }
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); w++) mx = fmaxf(mx, sm[w]);
  int e = 0;
  if (mx > 0.f && mx < 3.0e38f) {
    int ex;
    frexpf(mx, &ex);            // mx = f * 2^ex, f in [0.5, 1)
    e = ex - 14;                // the scaled row stays below 2^14
    e = e < -100 ? -100 : (e > 100 ? 100 : e);
  }
  const float s = ldexpf(1.0f, -e);
  if (threadIdx.x == 0) rowscale[m] = ldexpf(1.0f, e);
  if (vec) {
    const float4* row4 = (const float4*)row;
    uint4* o1 = (uint4*)(x1 + (size_t)m * K);
    uint4* o2 = (uint4*)(x2 + (size_t)m * K);
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
      const float4 a = __ldg(row4 + 2 * i), b = __ldg(row4 + 2 * i + 1);
      const float f[8] = {a.x * s, b.x * s, a.y * s, b.y * s, a.z * s, b.z * s, a.w * s, b.w * s};   // k 0,4,1,5,2,6,3,7
      unsigned w1[4], w2[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const __half ha = __float2half_rn(f[2 * j]), hb = __float2half_rn(f[2 * j + 1]);
        const __half la = __float2half_rn(f[2 * j] - __half2float(ha)), lb = __float2half_rn(f[2 * j + 1] - __half2float(hb));
        w1[j] = (unsigned)__half_as_ushort(ha) | ((unsigned)__half_as_ushort(hb) << 16);
        w2[j] = (unsigned)__half_as_ushort(la) | ((unsigned)__half_as_ushort(lb) << 16);
      }
      o1[i] = make_uint4(w1[0], w1[1], w1[2], w1[3]);
      o2[i] = make_uint4(w2[0], w2[1], w2[2], w2[3]);
    }
    return;
  }
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    const float v = row[k] * s;
    const __half h1 = __float2half_rn(v);
    const __half h2 = __float2half_rn(v - __half2float(h1));
    const int k8 = k & 7;
    const size_t pos = (size_t)m * K + (k & ~7) + (k8 < 4 ? 2 * k8 : 2 * (k8 - 4) + 1);
    x1[pos] = h1;
    x2[pos] = h2;
  }
}

template <int MT>
int t2_launch(const CUtensorMap& tm1, const CUtensorMap& tm2, const CUtensorMap& tmw, const T2Params& p,
              cudaStream_t stream) {
  static std::atomic<unsigned long long> attr_done{0};
  {
    const int rc_attr = ensure_dynamic_smem(gemm_q4_tc2_kernel<MT>, (int)T2Smem<MT>::TOTAL, attr_done);
    if (rc_attr) return rc_attr;
  }
  LaunchCfg lc(dim3((p.N + T2_ROWS - 1) / T2_ROWS, (p.M + MT - 1) / MT), dim3(T2_THREADS), T2Smem<MT>::TOTAL, stream,
               pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, gemm_q4_tc2_kernel<MT>, tm1, tm2, tmw, p));
  return TLB_OK;
}

}  // namespace

// bytes of the activation scratch: two fp16 planes + the row scales
size_t gemm_q4_tc2_scratch_bytes(int M, int K) { return (size_t)M * K * 4 + (size_t)((M + 3) & ~3) * 4 + 256; }

bool gemm_q4_tc2_eligible(const void* qw, const void* scales, int N, int K, int M) {
  if (M <= 8 || N <= 0 || M > 65535 * 32) return false;
  if (K % 128 != 0) return false;
  return (((uintptr_t)qw & 15) == 0) && (((uintptr_t)scales & 15) == 0);
}

int gemm_q4_tc2_launch(DeviceCtx* c, const float* x, long long ldx, int M, const void* qw, const float* scales,
                       float* y, long long ldy, int N, int K, float alpha, float beta, void* scratch,
                       cudaStream_t stream) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return set_error(TLB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  __half* x1 = (__half*)scratch;
  __half* x2 = x1 + (size_t)M * K;
  float* rowscale = (float*)(((uintptr_t)(x2 + (size_t)M * K) + 255) & ~(uintptr_t)255);
  {
    LaunchCfg lc(dim3((unsigned)M), dim3(256), 0, stream, pdl_enabled());
    TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, split_f16_kernel, x, ldx, K, x1, x2, rowscale));
  }
  const int MT = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  CUtensorMap tm1, tm2;
  cuuint64_t dim[2] = {(cuuint64_t)K, (cuuint64_t)M};
  cuuint64_t str[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {(cuuint32_t)T2_KS, (cuuint32_t)MT};
  cuuint32_t es[2] = {1, 1};
  if (enc(&tm1, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x1, dim, str, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) !=
          CUDA_SUCCESS ||
      enc(&tm2, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x2, dim, str, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) !=
          CUDA_SUCCESS)
    return set_error(TLB_ERR_CUDA, "gemm_q4_tc2: tensor map (activation planes) encode failed");
  // packed weights as bytes [N][K/2]; boxes past K/2 or N read as zeros and are never converted / stored
  CUtensorMap tmw;
  cuuint64_t wdim[2] = {(cuuint64_t)K / 2, (cuuint64_t)N};
  cuuint64_t wstr[1] = {(cuuint64_t)K / 2};
  cuuint32_t wbox[2] = {128, (cuuint32_t)T2_ROWS};
  if (enc(&tmw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(qw), wdim, wstr, wbox, es,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return set_error(TLB_ERR_CUDA, "gemm_q4_tc2: tensor map (packed weights) encode failed");
  T2Params p;
  p.qw = (const unsigned*)qw; p.scales = scales; p.rowscale = rowscale; p.y = y; p.ldy = ldy;
  p.M = M; p.N = N; p.K = K; p.alpha = alpha; p.beta = beta; p.status = c->status;
  if (MT == 32) return t2_launch<32>(tm1, tm2, tmw, p, stream);
  if (MT == 64) return t2_launch<64>(tm1, tm2, tmw, p, stream);
  return t2_launch<128>(tm1, tm2, tmw, p, stream);
}

}  // namespace tlb
