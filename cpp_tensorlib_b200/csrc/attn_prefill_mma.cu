// Causal attention over a prompt chunk on the tensor pipe (f32 cache, D = 64 or 128): the
// contract of cuda::attn_prefill / tl_attn_prefill_tiled_* of the reference
// (include/cuda.h:1171-1201, kernels/tensorlib_cuda.cu:1211-1350) -- q, out [n_q, T, D]; K, V a
// [n_kv, kv_max, D] cache; query p sits at absolute position pos0 + p and attends keys
// 0..pos0+p -- as a dense contraction instead of per-row CUDA-core dot products.
//
//  * grid = (query tiles of 64, q heads).  Four compute warps own 16 query rows each; a producer
//    warp streams K/V tiles of 32 keys by TMA (boxes of 32 rows x 32 floats, 128-byte swizzle,
//    no multicast) through a 4-slot mbarrier ring that every compute warp consumes in order.
//  * S[16 q x 32 keys] = Q . K^T and out[16 q x D] += P . V as mma.sync.m16n8k8 tf32 with both
//    operands split exactly into tf32 hi + lo (three MMAs per step, dropped term 2^-22), so the
//    result keeps the 1e-4 bound of the CUDA-core form.  Q is split once into fragment order
//    in shared memory; P goes through a per-warp buffer to change from the accumulator layout
//    to the A-operand layout; the output columns of an MMA tile are a permutation of D chosen
//    so that the V fragments are read without a bank conflict.
//  * Online softmax per query row in the accumulator layout (exp2, log2(e) folded into Q),
//    causal mask by select; rows of the last tile that lie past the chunk are cleared in
//    shared memory before use (their P is zero, but 0 * NaN is NaN).
#include "attn_common.cuh"

namespace tlb {

namespace {

constexpr int PM_QT = 64;            // queries per CTA
constexpr int PM_WARPS = 4;          // compute warps (16 query rows each) + 1 producer warp
constexpr int PM_TK = 32;            // keys per tile
constexpr int PM_STAGES = 4;
constexpr int PM_BOX = 32 * 128;     // one TMA box: 32 rows x 32 floats
constexpr int PM_PSTRIDE = 36;       // floats per row of the per-warp P buffer (conflict-free A reads)

template <int D>
struct PmCfg {
  static constexpr int SEGS = D / 32;
  static constexpr int KSTEPS = D / 8;
  static constexpr int NT = D / 8;                      // output column tiles of 8
  static constexpr int TILE_BYTES = 2 * SEGS * PM_BOX;  // K part then V part
  static constexpr size_t RING = (size_t)PM_STAGES * TILE_BYTES;
  static constexpr size_t QF = (size_t)PM_WARPS * KSTEPS * 32 * 32;   // two uint4 per (warp, step, lane)
  static constexpr size_t PS = (size_t)PM_WARPS * 16 * PM_PSTRIDE * 4;
  static constexpr size_t BARS = 2 * PM_STAGES * 8;
  static constexpr size_t TOTAL = 1024 + RING + QF + PS + BARS + 64;
};

__device__ __forceinline__ void pm_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                       unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pm_split(float x, unsigned& hi, unsigned& lo) {
  hi = __float_as_uint(x) & 0xffffe000u;
  lo = __float_as_uint(x - __uint_as_float(hi));
}
__device__ __forceinline__ float pm_lds(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 pm_lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ float pm_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct PmParams {
  const float* q;
  float* out;
  int T, n_kv, group, kv_rows, pos0;
  float scale;
  int* status;
};

template <int D>
__global__ void __launch_bounds__(32 * (PM_WARPS + 1), 1)
    attn_prefill_mma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                            PmParams p) {
  using C = PmCfg<D>;
  constexpr int SEGS = C::SEGS, KSTEPS = C::KSTEPS, NT = C::NT;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* ring = base;
  uint4* Qf = (uint4*)(base + C::RING);
  float* Ps = (float*)(base + C::RING + C::QF);
  uint64_t* full = (uint64_t*)(base + C::RING + C::QF + C::PS);
  uint64_t* empty = full + PM_STAGES;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int h = blockIdx.y, kh = h / p.group;
  const int q0 = blockIdx.x * PM_QT;

  if (tid == 0) {
    for (int s = 0; s < PM_STAGES; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], PM_WARPS);
    }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_wait();
  pdl_launch_dependents();

  int cta_last_q = q0 + PM_QT - 1;
  if (cta_last_q > p.T - 1) cta_last_q = p.T - 1;
  const int n_keys = p.pos0 + cta_last_q + 1;            // keys this CTA may attend: [0, n_keys)
  const int n_tiles = (n_keys + PM_TK - 1) / PM_TK;
  const int row0 = kh * p.kv_rows;

  if (warp == PM_WARPS) {
    // ---------------- producer ----------------
    if (lane == 0) {
      for (int i = 0; i < n_tiles; i++) {
        const int st = i % PM_STAGES;
        if (i >= PM_STAGES && !mbar_wait_bounded(&empty[st], ((i / PM_STAGES) - 1) & 1, p.status, 710 + st)) break;
        unsigned char* dst = ring + (size_t)st * C::TILE_BYTES;
        mbar_expect_tx(&full[st], C::TILE_BYTES);
#pragma unroll
        for (int sg = 0; sg < SEGS; sg++) {
          tma_load_2d(dst + sg * PM_BOX, &tmK, sg * 32, row0 + i * PM_TK, &full[st]);
          tma_load_2d(dst + (SEGS + sg) * PM_BOX, &tmV, sg * 32, row0 + i * PM_TK, &full[st]);
        }
      }
    }
    return;
  }

  // ---------------- compute warps ----------------
  const int qrow = q0 + 16 * warp;                 // first query row of this warp
  // Q fragments of this warp, scaled by scale * log2(e) and split into tf32 hi / lo:
  // step ks, lane (g, t): a0 = Q[g][8ks+t], a1 = Q[g+8][8ks+t], a2 = Q[g][8ks+t+4], a3 = Q[g+8][8ks+t+4]
  {
    const float qs = p.scale * 1.4426950408889634f;
    const bool r0ok = qrow + g < p.T, r1ok = qrow + g + 8 < p.T;
    const float* qa = p.q + ((size_t)h * p.T + (r0ok ? qrow + g : 0)) * D;
    const float* qb = p.q + ((size_t)h * p.T + (r1ok ? qrow + g + 8 : 0)) * D;
    uint4* mine = Qf + (size_t)warp * KSTEPS * 64 + lane * 2;
#pragma unroll 4
    for (int ks = 0; ks < KSTEPS; ks++) {
      const float a0 = r0ok ? qa[8 * ks + t] * qs : 0.f, a1 = r1ok ? qb[8 * ks + t] * qs : 0.f;
      const float a2 = r0ok ? qa[8 * ks + t + 4] * qs : 0.f, a3 = r1ok ? qb[8 * ks + t + 4] * qs : 0.f;
      uint4 hi, lo;
      pm_split(a0, hi.x, lo.x);
      pm_split(a1, hi.y, lo.y);
      pm_split(a2, hi.z, lo.z);
      pm_split(a3, hi.w, lo.w);
      mine[ks * 64] = hi;
      mine[ks * 64 + 1] = lo;
    }
    __syncwarp();
  }
  const uint32_t ring32 = smem_u32(ring);
  const uint32_t qf32 = smem_u32(Qf) + (uint32_t)((warp * KSTEPS * 64 + lane * 2) * 16);
  float* myP = Ps + warp * 16 * PM_PSTRIDE;
  const uint32_t myP32 = smem_u32(myP);
  // K fragment (B operand of S): key row 8j + g of the tile, word t of chunk c, chunk XOR (row & 7) = g
  const uint32_t kbase = (uint32_t)(g * 128 + t * 4) | ((uint32_t)g << 4);
  // V fragment (B operand of P.V): key row t (+4), column g of output tile (seg, c) = dimension
  // 32 seg + 16 (g >> 2) + 4 c + (g & 3): chunk ((g >> 2) * 4 + c) XOR (row & 7)
  const uint32_t vbase = (uint32_t)(t * 128 + (g & 3) * 4) | ((uint32_t)((((g >> 2) * 4) ^ t) & 7) << 4);

  const int qpos0 = p.pos0 + qrow + g, qpos1 = qpos0 + 8;        // absolute positions of rows g, g + 8
  int warp_last_key = p.pos0 + qrow + 15;
  if (warp_last_key > n_keys - 1) warp_last_key = n_keys - 1;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  bool dead = false;   // a bounded wait gave up: stop computing, but keep every rendezvous below
  for (int it = 0; it < n_tiles; it++) {
    const int st = it % PM_STAGES;
    const int k0 = it * PM_TK;
    if (!dead && !mbar_wait_bounded(&full[st], (it / PM_STAGES) & 1, p.status, 700 + st)) dead = true;
    const uint32_t kt = ring32 + (uint32_t)st * C::TILE_BYTES;
    const uint32_t vt = kt + SEGS * PM_BOX;
    if (it == n_tiles - 1 && n_keys - k0 < PM_TK) {
      // rows past the chunk hold whatever the cache holds: clear their V (warp 0), then all
      // four warps meet before anyone reads the tile
      if (warp == 0) {
        const int first = n_keys - k0;
        for (int i = lane; i < (PM_TK - first) * (D / 4); i += 32) {
          const int r = first + i / (D / 4), c4 = i % (D / 4);
          const int sg = c4 >> 3, ch = c4 & 7;
          *(float4*)(ring + (size_t)st * C::TILE_BYTES + (size_t)(SEGS + sg) * PM_BOX + r * 128 +
                     ((ch ^ (r & 7)) << 4)) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      asm volatile("bar.sync 1, %0;" ::"r"(32 * PM_WARPS) : "memory");
    }
    if (!dead && k0 <= warp_last_key) {
      // ---- S = Q . K^T over the tile's 32 keys: four column tiles of 8 keys ----
      float s[4][4], sx[4][4];
#pragma unroll
      for (int j = 0; j < 4; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) s[j][i] = sx[j][i] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ks++) {
        const uint4 qh = pm_lds128(qf32 + (uint32_t)ks * 64u * 16u);
        const uint4 ql = pm_lds128(qf32 + (uint32_t)ks * 64u * 16u + 16u);
        const uint32_t c0 = (uint32_t)((ks & 3) * 2) << 4;
        const uint32_t ka = kt + (uint32_t)(ks >> 2) * PM_BOX + (kbase ^ c0);
        const uint32_t kb = kt + (uint32_t)(ks >> 2) * PM_BOX + (kbase ^ (c0 | 16u));
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const float b0 = pm_lds(ka + (uint32_t)j * 1024u), b1 = pm_lds(kb + (uint32_t)j * 1024u);
          unsigned h0, h1, e0, e1;
          pm_split(b0, h0, e0);
          pm_split(b1, h1, e1);
          pm_mma(s[j], qh.x, qh.y, qh.z, qh.w, h0, h1);
          pm_mma(sx[j], qh.x, qh.y, qh.z, qh.w, e0, e1);
          pm_mma(sx[j], ql.x, ql.y, ql.z, ql.w, h0, h1);
        }
      }
      // causal mask + row maxima (rows g and g + 8; a lane holds keys 8j + 2t, 8j + 2t + 1)
      float bm0 = -INFINITY, bm1 = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int key = k0 + 8 * j + 2 * t;
        s[j][0] = key <= qpos0 ? s[j][0] + sx[j][0] : -INFINITY;
        s[j][1] = key + 1 <= qpos0 ? s[j][1] + sx[j][1] : -INFINITY;
        s[j][2] = key <= qpos1 ? s[j][2] + sx[j][2] : -INFINITY;
        s[j][3] = key + 1 <= qpos1 ? s[j][3] + sx[j][3] : -INFINITY;
        bm0 = fmaxf(bm0, fmaxf(s[j][0], s[j][1]));
        bm1 = fmaxf(bm1, fmaxf(s[j][2], s[j][3]));
      }
      bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 1));
      bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 2));
      bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 1));
      bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 2));
      const float n0 = fmaxf(m0, bm0), n1 = fmaxf(m1, bm1);
      // a row with no visible key yet keeps m = -inf: use 0 as the reference point so that
      // exp2(-inf - 0) = 0 and nothing becomes NaN
      const float r0 = n0 == -INFINITY ? 0.f : n0, r1 = n1 == -INFINITY ? 0.f : n1;
      const float f0 = pm_ex2(m0 - r0), f1 = pm_ex2(m1 - r1);
      l0 *= f0;
      l1 *= f1;
#pragma unroll
      for (int j = 0; j < NT; j++) {
        acc[j][0] *= f0; acc[j][1] *= f0;
        acc[j][2] *= f1; acc[j][3] *= f1;
      }
      m0 = n0;
      m1 = n1;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float p00 = pm_ex2(s[j][0] - r0), p01 = pm_ex2(s[j][1] - r0);
        const float p10 = pm_ex2(s[j][2] - r1), p11 = pm_ex2(s[j][3] - r1);
        l0 += p00 + p01;
        l1 += p10 + p11;
        *(float2*)(myP + g * PM_PSTRIDE + 8 * j + 2 * t) = make_float2(p00, p01);
        *(float2*)(myP + (g + 8) * PM_PSTRIDE + 8 * j + 2 * t) = make_float2(p10, p11);
      }
      __syncwarp();
      // ---- out += P . V: four k-steps of 8 keys, D / 8 column tiles ----
#pragma unroll
      for (int kk = 0; kk < 4; kk++) {
        const float a0 = pm_lds(myP32 + (uint32_t)(g * PM_PSTRIDE + 8 * kk + t) * 4u);
        const float a1 = pm_lds(myP32 + (uint32_t)((g + 8) * PM_PSTRIDE + 8 * kk + t) * 4u);
        const float a2 = pm_lds(myP32 + (uint32_t)(g * PM_PSTRIDE + 8 * kk + t + 4) * 4u);
        const float a3 = pm_lds(myP32 + (uint32_t)((g + 8) * PM_PSTRIDE + 8 * kk + t + 4) * 4u);
        unsigned ah0, ah1, ah2, ah3, al0, al1, al2, al3;
        pm_split(a0, ah0, al0);
        pm_split(a1, ah1, al1);
        pm_split(a2, ah2, al2);
        pm_split(a3, ah3, al3);
        const uint32_t vrow = vt + (uint32_t)(8 * kk) * 128u;
#pragma unroll
        for (int j = 0; j < NT; j++) {
          // output tile j = (seg j >> 2, c = j & 3)
          const uint32_t a = vrow + (uint32_t)(j >> 2) * PM_BOX + (vbase ^ ((uint32_t)(j & 3) << 4));
          const float b0 = pm_lds(a), b1 = pm_lds((a ^ 64u) + 512u);
          unsigned h0, h1, e0, e1;
          pm_split(b0, h0, e0);
          pm_split(b1, h1, e1);
          pm_mma(acc[j], ah0, ah1, ah2, ah3, h0, h1);
          pm_mma(acc[j], ah0, ah1, ah2, ah3, e0, e1);
          pm_mma(acc[j], al0, al1, al2, al3, h0, h1);
        }
      }
      __syncwarp();
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[st]);
  }

  // ---- row sums across the quad, normalise, store ----
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = 1.0f / l0, i1 = 1.0f / l1;
  const int ra = qrow + g, rb = qrow + g + 8;
#pragma unroll
  for (int j = 0; j < NT; j++) {
    // accumulator columns 2t, 2t + 1 of tile (seg, c): dimensions d, d + 1 with
    // d = 32 seg + 16 ((2t) >> 2) + 4 c + ((2t) & 3)
    const int d = 32 * (j >> 2) + 16 * ((2 * t) >> 2) + 4 * (j & 3) + ((2 * t) & 3);
    if (ra < p.T) *(float2*)(p.out + ((size_t)h * p.T + ra) * D + d) = make_float2(acc[j][0] * i0, acc[j][1] * i0);
    if (rb < p.T) *(float2*)(p.out + ((size_t)h * p.T + rb) * D + d) = make_float2(acc[j][2] * i1, acc[j][3] * i1);
  }
}

template <int D>
int pm_launch(const PmParams& p, const void* K, const void* V, int n_q, cudaStream_t stream) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return set_error(TLB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  CUtensorMap tmK, tmV;
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)p.n_kv * (cuuint64_t)p.kv_rows};
  cuuint64_t strides[1] = {(cuuint64_t)D * 4};
  cuuint32_t box[2] = {32, (cuuint32_t)PM_TK};
  cuuint32_t es[2] = {1, 1};
  for (int which = 0; which < 2; which++) {
    CUresult r = enc(which ? &tmV : &tmK, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(which ? V : K), dims,
                     strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(TLB_ERR_CUDA, "attn_prefill: tensor map encode failed");
  }
  static std::atomic<unsigned long long> attr_done{0};
  {
    const int rc_attr = ensure_dynamic_smem(attn_prefill_mma_kernel<D>, (int)PmCfg<D>::TOTAL, attr_done);
    if (rc_attr) return rc_attr;
  }
  LaunchCfg lc(dim3((p.T + PM_QT - 1) / PM_QT, n_q), dim3(32 * (PM_WARPS + 1)), PmCfg<D>::TOTAL, stream,
               pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, attn_prefill_mma_kernel<D>, tmK, tmV, p));
  return TLB_OK;
}

}  // namespace

bool attn_prefill_mma_eligible(int D, int n_kv, long long kv_max, int bf) {
  return !bf && (D == 64 || D == 128) && (long long)n_kv * kv_max < (1ll << 31);
}

int attn_prefill_mma_launch(DeviceCtx* c, const float* q, const void* K, const void* V, float* out, int n_q,
                            int n_kv, int T, long long kv_max, int D, float scale, int pos0, cudaStream_t s) {
  PmParams p;
  p.q = q; p.out = out; p.T = T; p.n_kv = n_kv; p.group = n_q / n_kv; p.kv_rows = (int)kv_max; p.pos0 = pos0;
  p.scale = scale; p.status = c->status;
  if (D == 128) return pm_launch<128>(p, K, V, n_q, s);
  return pm_launch<64>(p, K, V, n_q, s);
}

}  // namespace tlb
