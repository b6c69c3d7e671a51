// Decode attention for GQA groups on the tensor pipe (f32 cache, 3..8 query heads per KV
// head, D = 64 or 128): the same contract as attn_decode.cu -- out[h,:] =
// softmax(scale * q[h] . K[kv(h)]^T) . V[kv(h)] over the cache prefix [0, ctx), cuda::attn_decode
// / attn_decode_dpos of the reference (include/cuda.h:966-1114, kernels
// tl_attn_decode_split* + tl_attn_combine, kernels/tensorlib_cuda.cu:842-1061) -- for the shape
// where the CUDA-core form is bound by instruction issue: with 7 heads sharing every KV row
// the two products are a contraction with a head dimension of 7, and as scalar FMAs +
// shuffles they cost more than the row's bytes.
//
//  * grid = (context splits, KV heads), the split plan of attn_split.cuh.  A CTA serves ALL
//    query heads of its KV head (they are the N = 8 columns of the MMAs, zero padded), so a
//    KV byte is read once.
//  * K/V tiles of 32 keys arrive by TMA (cp.async.bulk.tensor.2d, no multicast) as boxes of
//    32 rows x 32 floats with the 128-byte swizzle, one mbarrier per ring slot, issued by a
//    producer warp; with it every operand fragment below is read without a bank conflict.
//  * A warp owns blocks of 16 keys.  S^T[16 keys x 8 heads] = K_blk . Q^T as
//    mma.sync.m16n8k8 tf32 with BOTH operands split exactly into tf32 hi + lo and three
//    MMAs per step (hi.hi + hi.lo + lo.hi, dropped term 2^-22): f32-grade scores, so the
//    kernel meets the same 1e-4 bound as the CUDA-core form.  Online softmax in the
//    accumulator layout (a lane holds heads 2t, 2t+1 of keys g, g+8), exp2 with log2(e)
//    folded into the query.  P goes through 512 bytes of per-warp shared memory to become the
//    B operand of out^T[D x 8 heads] += V_blk^T . P, again three tf32 MMAs per step.
//  * The warps' (acc, m, l) meet in shared memory, the CTA's partial goes to scratch, an
//    acq_rel ticket per KV head elects the last CTA, which folds the splits in split order
//    with every load of the fold in flight at once (one L2 round trip).  One launch,
//    deterministic; the device-position variant derives its ranges from ctx by the same
//    functions, so it is bit-identical to the host-position variant at every position
//    (bench/cuda/check/check_attn64.cpp:91-102).
#include <string>

#include "attn_split.cuh"

namespace tlb {

namespace {

constexpr int MM_TK = AT_TK;          // keys per TMA tile
constexpr int MM_BOX_BYTES = 32 * 128;  // one box: 32 rows x 32 floats

template <int D>
struct MmaCfg {
  static constexpr int WARPS = D / 16;              // compute warps; + 1 producer warp
  static constexpr int THREADS = 32 * (WARPS + 1);
  static constexpr int SEGS = D / 32;               // boxes per K (or V) tile
  static constexpr int TILE_BYTES = 2 * SEGS * MM_BOX_BYTES;   // K part then V part
  // Ring slots: a multiple of the number of warp pairs (WARPS / 2), so that slot s is always
  // consumed by the same pair.  A pair then never waits for phase k of a slot before it has
  // itself seen phase k - 1 complete, which is what makes a parity wait unambiguous (with a
  // slot shared between pairs, a pair arriving early would read the previous phase's parity
  // as "done").
  static constexpr int STAGES = D == 128 ? 4 : 6;
  static_assert(STAGES % (WARPS / 2) == 0, "a ring slot must belong to one warp pair");
  static constexpr int KSTEPS = D / 8;
  // shared memory: ring | Q fragments | per-warp P | per-warp merge entries | barriers
  static constexpr size_t RING = (size_t)STAGES * TILE_BYTES;
  static constexpr size_t QF = (size_t)KSTEPS * 32 * 16;
  static constexpr size_t PS = (size_t)WARPS * 16 * 8 * 4;
  static constexpr size_t ENT = (size_t)WARPS * (D * 8 + 16) * 4;
  static constexpr size_t BARS = 2 * STAGES * 8;
  static constexpr size_t TOTAL = 1024 + RING + QF + PS + ENT + BARS + 64;
};

__device__ __forceinline__ void mma_tf32(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// exact split x = hi + lo with hi representable in tf32 (the low 13 mantissa bits cleared);
// lo is then used as a tf32 operand, which keeps its leading 11 bits
__device__ __forceinline__ void split_tf32(float x, unsigned& hi, unsigned& lo) {
  hi = __float_as_uint(x) & 0xffffe000u;
  lo = __float_as_uint(x - __uint_as_float(hi));
}
__device__ __forceinline__ float lds_f32(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 lds_u128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(MmaCfg<D>::THREADS, 1)
    attn_decode_mma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                           AttnParams p) {
  using C = MmaCfg<D>;
  constexpr int W = C::WARPS, SEGS = C::SEGS, STAGES = C::STAGES, KSTEPS = C::KSTEPS;
  extern __shared__ unsigned char smem_raw[];
  // the swizzle of a TMA box follows the SHARED-space address: align that one to 1024 bytes
  unsigned char* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* ring = base;
  uint4* Qf = (uint4*)(base + C::RING);
  float* Ps = (float*)(base + C::RING + C::QF);
  float* ent = (float*)(base + C::RING + C::QF + C::PS);
  uint64_t* full = (uint64_t*)(base + C::RING + C::QF + C::PS + C::ENT);
  uint64_t* empty = full + STAGES;
  __shared__ int is_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kh = blockIdx.y, sp = blockIdx.x;

  // the position is an L2 round trip away and everything below depends on it: ask for it
  // before the barrier setup, not after
  const int ctx = p.d_pos ? (int)(*(const volatile unsigned*)p.d_pos) + 1 : p.ctx;
  if (tid == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 2);   // the two warps that share a tile
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (p.d_pos && (ctx > p.kv_rows || ctx < 1)) {
    // position beyond the cache: read nothing, leave the tickets alone, tell the host
    pdl_wait();
    pdl_launch_dependents();
    if (p.status && tid == 0) atomicExch(&p.status[ST_KV_OVERFLOW], 1);
    return;
  }
  const int chunk = attn_chunk(p.n_kv, ctx, p.sm2);
  const int s_live = (ctx + chunk - 1) / chunk;
  const bool dead = sp >= s_live;
  const int k_begin = sp * chunk;
  const int k_end = k_begin + chunk < ctx ? k_begin + chunk : ctx;
  const int n_tiles = dead ? 0 : (k_end - k_begin + MM_TK - 1) / MM_TK;
  const int row0 = kh * p.kv_rows + k_begin;   // first cache row of this CTA in the [n_kv * kv_max, D] view

  // ======================= producer: first tiles =======================
  const bool producer = (warp == W && lane == 0);
  // A long context is read once per token and is far larger than the L2 over the layers of a
  // model: mark it evict-first, so that the small things every launch re-reads (biases, norm
  // weights, activations, scratch) stay.  A short one may survive to the next token: leave it.
  const uint64_t pol = (size_t)p.n_kv * ctx * D * 8 >= ((size_t)8 << 20) ? l2_evict_first_policy()
                                                                          : l2_evict_normal_policy();
  auto issue = [&](int i) {
    const int st = i % STAGES;
    unsigned char* dst = ring + (size_t)st * C::TILE_BYTES;
    mbar_expect_tx(&full[st], C::TILE_BYTES);
#pragma unroll
    for (int sg = 0; sg < SEGS; sg++) {
      tma_load_2d_hint(dst + sg * MM_BOX_BYTES, &tmK, sg * 32, row0 + i * MM_TK, &full[st], pol);
      tma_load_2d_hint(dst + (SEGS + sg) * MM_BOX_BYTES, &tmV, sg * 32, row0 + i * MM_TK, &full[st], pol);
    }
  };
  const int first = n_tiles < STAGES ? n_tiles : STAGES;
  int issued = 0;
  // Tiles that end below the newest row do not depend on the preceding kernel (it only
  // appends row ctx-1): with early_kv they are requested while that kernel drains.
  if (producer && p.early_kv)
    while (issued < first && k_begin + (issued + 1) * MM_TK <= ctx - 1) issue(issued++);
  pdl_wait();
  pdl_launch_dependents();
  if (dead) return;
  if (producer)
    while (issued < first) issue(issued++);

  // ======================= Q fragments =======================
  // B operand of S^T = K . Q^T, step ks: b0 = q[head g][8 ks + t], b1 = q[head g][8 ks + t + 4],
  // scaled by scale * log2(e), split into tf32 hi / lo: one uint4 per (step, lane).
  {
    const float qs = p.scale * 1.4426950408889634f;
    for (int i = tid; i < KSTEPS * 32; i += C::THREADS) {
      const int ks = i >> 5, ln = i & 31, hg = ln >> 2, ht = ln & 3;
      float b0 = 0.f, b1 = 0.f;
      if (hg < p.grp) {
        const float* qp = p.q + (size_t)(kh * p.grp + hg) * D + 8 * ks + ht;
        b0 = qp[0] * qs;
        b1 = qp[4] * qs;
      }
      uint4 f;
      split_tf32(b0, f.x, f.z);
      split_tf32(b1, f.y, f.w);
      Qf[i] = f;
    }
  }
  __syncthreads();

  // ======================= producer: refill the ring =======================
  if (producer) {
    for (int i = STAGES; i < n_tiles; i++) {
      const int st = i % STAGES;
      if (!mbar_wait_bounded(&empty[st], ((i / STAGES) - 1) & 1, p.status, 210 + st)) break;
      issue(i);
    }
  }
  // every tile of this CTA is requested: ask the L2 for the head of the next kernel's weights
  if (warp == W && p.pf.wp) {
    __syncwarp();
    const unsigned me = blockIdx.y * gridDim.x + blockIdx.x, step = gridDim.x * gridDim.y;
    for (unsigned nc = me; nc < (unsigned)p.pf.grid; nc += step) gv_prefetch_head(p.pf, nc, lane);
  }

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // heads 2t, 2t+1
  float acc[2 * SEGS][4];
#pragma unroll
  for (int j = 0; j < 2 * SEGS; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  if (warp < W) {
    const uint32_t ring32 = smem_u32(ring);
    const uint32_t qf32 = smem_u32(Qf) + (uint32_t)lane * 16u;
    float* myP = Ps + warp * 128;
    const uint32_t myP32 = smem_u32(myP);
    const int half = warp & 1;                      // which 16 keys of a tile
    // K fragment addressing: row (16 half + g) of a box, word t, chunk XOR (row & 7) = g
    const uint32_t kbase = (uint32_t)((16 * half + g) * 128 + t * 4) | ((uint32_t)g << 4);
    // V fragment addressing (see the file comment): row = key t (+4), word g & 3,
    // chunk ((g >> 2) * 4 + 2 p (+1)) XOR (row & 7)
    const uint32_t vbase = (uint32_t)(t * 128 + (g & 3) * 4) | ((uint32_t)((((g >> 2) * 4) ^ t) & 7) << 4);

    for (int it = warp >> 1; it < n_tiles; it += W / 2) {
      const int st = it % STAGES;
      const int blk0 = k_begin + it * MM_TK + 16 * half;     // first key of this warp's block
      if (!mbar_wait_bounded(&full[st], (it / STAGES) & 1, p.status, 200 + st)) break;
      const int valid = k_end - blk0;                         // keys of the block inside the range
      if (valid > 0) {
        const uint32_t kt = ring32 + (uint32_t)st * C::TILE_BYTES;
        const uint32_t vt = kt + SEGS * MM_BOX_BYTES;
        if (valid < 16) {
          // ragged end: rows past the context hold whatever the cache holds there; P is zero
          // for them, but 0 * NaN is NaN, so their V rows are cleared (this warp is the only
          // reader of these 16 rows)
          for (int i = lane; i < (16 - valid) * (D / 4); i += 32) {
            const int r = 16 * half + valid + i / (D / 4), c4 = i % (D / 4);
            const int sg = c4 >> 3, ch = c4 & 7;
            *(float4*)(ring + (size_t)st * C::TILE_BYTES + (size_t)(SEGS + sg) * MM_BOX_BYTES + r * 128 +
                       ((ch ^ (r & 7)) << 4)) = make_float4(0.f, 0.f, 0.f, 0.f);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // a later TMA refills this slot
          __syncwarp();
        }
        // ---- S^T = K_blk . Q^T ----
        // three accumulators, one per term of the split product: three independent MMA chains
        // of KSTEPS instead of one of 3 KSTEPS (the chain's latency is what a block costs)
        float s[4] = {0.f, 0.f, 0.f, 0.f}, s_hl[4] = {0.f, 0.f, 0.f, 0.f}, s_lh[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
          const uint32_t c0 = (uint32_t)((ks & 3) * 2) << 4;
          const uint32_t a = kt + (uint32_t)(ks >> 2) * MM_BOX_BYTES + (kbase ^ c0);
          const uint32_t a2 = kt + (uint32_t)(ks >> 2) * MM_BOX_BYTES + (kbase ^ (c0 | 16u));
          const float k0 = lds_f32(a), k1 = lds_f32(a + 1024), k2 = lds_f32(a2), k3 = lds_f32(a2 + 1024);
          const uint4 qf = lds_u128(qf32 + (uint32_t)ks * 512u);
          unsigned h0, h1, h2, h3, e0, e1, e2, e3;
          split_tf32(k0, h0, e0);
          split_tf32(k1, h1, e1);
          split_tf32(k2, h2, e2);
          split_tf32(k3, h3, e3);
          mma_tf32(s, h0, h1, h2, h3, qf.x, qf.y);
          mma_tf32(s_hl, h0, h1, h2, h3, qf.z, qf.w);
          mma_tf32(s_lh, e0, e1, e2, e3, qf.x, qf.y);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) s[i] += s_hl[i] + s_lh[i];
        // s[0], s[1]: key g, heads 2t, 2t+1;  s[2], s[3]: key g + 8
        if (g >= valid) s[0] = s[1] = -INFINITY;
        if (g + 8 >= valid) s[2] = s[3] = -INFINITY;
        float bm0 = fmaxf(s[0], s[2]), bm1 = fmaxf(s[1], s[3]);
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, o));
          bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, o));
        }
        const float n0 = fmaxf(m0, bm0), n1 = fmaxf(m1, bm1);   // finite: the block has a valid key
        if (n0 != m0 || n1 != m1) {        // warp-uniform per quad column; cheap either way
          const float f0 = ex2(m0 - n0), f1 = ex2(m1 - n1);     // exp2(-inf) = 0 at the start
          l0 *= f0;
          l1 *= f1;
#pragma unroll
          for (int j = 0; j < 2 * SEGS; j++) {
            acc[j][0] *= f0; acc[j][2] *= f0;
            acc[j][1] *= f1; acc[j][3] *= f1;
          }
          m0 = n0;
          m1 = n1;
        }
        const float p00 = ex2(s[0] - m0), p01 = ex2(s[1] - m1), p10 = ex2(s[2] - m0), p11 = ex2(s[3] - m1);
        l0 += p00 + p10;
        l1 += p01 + p11;
        // P[16 keys][8 heads] through the warp's own shared memory into the B layout
        *(float2*)(myP + g * 8 + 2 * t) = make_float2(p00, p01);
        *(float2*)(myP + (g + 8) * 8 + 2 * t) = make_float2(p10, p11);
        __syncwarp();
        // ---- out^T[d][head] += V_blk^T . P ----
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
          const float pb0 = lds_f32(myP32 + (uint32_t)((8 * kk + t) * 8 + g) * 4u);
          const float pb1 = lds_f32(myP32 + (uint32_t)((8 * kk + t + 4) * 8 + g) * 4u);
          unsigned ph0, ph1, pl0, pl1;
          split_tf32(pb0, ph0, pl0);
          split_tf32(pb1, ph1, pl1);
          const uint32_t vrow = vt + (uint32_t)(16 * half + 8 * kk) * 128u;
#pragma unroll
          for (int j = 0; j < 2 * SEGS; j++) {
            const uint32_t a = vrow + (uint32_t)(j >> 1) * MM_BOX_BYTES + (vbase ^ ((uint32_t)(j & 1) << 5));
            const float v0 = lds_f32(a), v1 = lds_f32(a ^ 16u), v2 = lds_f32((a ^ 64u) + 512u),
                        v3 = lds_f32((a ^ 80u) + 512u);
            unsigned h0, h1, h2, h3, e0, e1, e2, e3;
            split_tf32(v0, h0, e0);
            split_tf32(v1, h1, e1);
            split_tf32(v2, h2, e2);
            split_tf32(v3, h3, e3);
            mma_tf32(acc[j], h0, h1, h2, h3, ph0, ph1);
            mma_tf32(acc[j], h0, h1, h2, h3, pl0, pl1);
            mma_tf32(acc[j], e0, e1, e2, e3, ph0, ph1);
          }
        }
        __syncwarp();   // the warp's P is rewritten by its next block
      }
      // this warp is done with the slot
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);
    }

    // ---- the warp's (acc, m, l) into its merge entry: acc^T[d][8 heads], then m[8], l[8] ----
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, o);
      l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    }
    float* e = ent + (size_t)warp * (D * 8 + 16);
#pragma unroll
    for (int j = 0; j < 2 * SEGS; j++) {
      // rows of m-tile j: d(g, hf) = 32 (j >> 1) + 16 (g >> 2) + 4 (2 (j & 1) + hf) + (g & 3)
      const int d0 = 32 * (j >> 1) + 16 * (g >> 2) + 8 * (j & 1) + (g & 3);
      *(float2*)(e + d0 * 8 + 2 * t) = make_float2(acc[j][0], acc[j][1]);
      *(float2*)(e + (d0 + 4) * 8 + 2 * t) = make_float2(acc[j][2], acc[j][3]);
    }
    if (g == 0) {
      e[D * 8 + 2 * t] = m0;
      e[D * 8 + 2 * t + 1] = m1;
      e[D * 8 + 8 + 2 * t] = l0;
      e[D * 8 + 8 + 2 * t + 1] = l1;
    }
  }
  __syncthreads();

  // ======================= CTA merge over the warps =======================
  const bool single = (s_live == 1);
  for (int idx = tid; idx < D * 8; idx += C::THREADS) {
    const int d = idx >> 3, h = idx & 7;
    if (h >= p.grp) continue;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < W; w++) M = fmaxf(M, ent[(size_t)w * (D * 8 + 16) + D * 8 + h]);
    float a = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < W; w++) {
      const float* e = ent + (size_t)w * (D * 8 + 16);
      const float mw = e[D * 8 + h];
      const float c = (mw == -INFINITY) ? 0.f : ex2(mw - M);
      a = fmaf(e[d * 8 + h], c, a);
      ll = fmaf(e[D * 8 + 8 + h], c, ll);
    }
    const int qh = kh * p.grp + h;
    if (single) {
      p.out[(size_t)qh * D + d] = a / ll;
    } else {
      float* dst = p.partials + ((size_t)qh * p.s_cap + sp) * (D + 4);
      __stcg(&dst[d], a);
      if (d == 0) __stcg((float2*)&dst[D], make_float2(M, ll));
    }
  }
  if (single) return;

  // ======================= split merge by the last CTA of this KV head =======================
  // The barrier orders every thread's partial stores before thread 0's acq_rel ticket, the
  // ticket's acquire side plus the second barrier orders the other CTAs' partials before this
  // CTA's loads.
  __syncthreads();
  if (tid == 0) {
    int old;
    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], %2;" : "=r"(old) : "l"(&p.counters[kh]), "r"(1) : "memory");
    is_last = (old == s_live - 1);
  }
  __syncthreads();
  if (!is_last) return;
  // IPH = D/4 lanes serve one head, lane li of them owns 4 dims.  The same lanes fetch the
  // (m, l) pairs of the head's splits (split li, li + IPH, ...: one L2 round trip), agree on
  // the maximum by shuffles and keep the rescale coefficients c_s = exp2(m_s - M) in
  // registers; the accumulators are folded in split order, 16 splits per batch, two batches
  // in flight, each coefficient fetched from the lane that owns it.
  {
    constexpr int IPH = D / 4, NML = 96 / IPH;
    const int items = p.grp * IPH;
    if (warp * 32 < items) {
      const int item = warp * 32 + lane;
      const bool has = item < items;
      const int h = has ? item / IPH : p.grp - 1, li = lane & (IPH - 1), lbase = lane & ~(IPH - 1);
      const float* src = p.partials + (size_t)(kh * p.grp + h) * p.s_cap * (D + 4);
      const float* vsrc = src + li * 4;
      float4 va[16], vb[16];
      auto load16 = [&](float4 (&v)[16], int s0) {
#pragma unroll
        for (int k = 0; k < 16; k++)
          v[k] = (s0 + k < s_live) ? __ldcg((const float4*)(vsrc + (size_t)(s0 + k) * (D + 4)))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
      };
      float2 ml[NML];
#pragma unroll
      for (int k = 0; k < NML; k++) {
        const int s2 = li + IPH * k;
        ml[k] = s2 < s_live ? __ldcg((const float2*)(src + (size_t)s2 * (D + 4) + D)) : make_float2(-INFINITY, 0.f);
      }
      load16(va, 0);
      load16(vb, 16);
      float M = -INFINITY;
#pragma unroll
      for (int k = 0; k < NML; k++) M = fmaxf(M, ml[k].x);
#pragma unroll
      for (int o = IPH / 2; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
      float cf[NML], lsum = 0.f;
#pragma unroll
      for (int k = 0; k < NML; k++) {
        cf[k] = (ml[k].x == -INFINITY) ? 0.f : ex2(ml[k].x - M);
        lsum = fmaf(ml[k].y, cf[k], lsum);
      }
#pragma unroll
      for (int o = IPH / 2; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      auto fold16 = [&](const float4 (&v)[16], int chunk_c) {
        // splits 16 c .. 16 c + 15 live in coefficient slot (16 c) / IPH of lanes (16 c) % IPH + k
#pragma unroll
        for (int k = 0; k < 16; k++) {
          float c = 0.f;
#pragma unroll
          for (int sl = 0; sl < NML; sl++)
            if (sl == (16 * chunk_c) / IPH) c = __shfl_sync(0xffffffffu, cf[sl], lbase + (16 * chunk_c) % IPH + k);
          a.x = fmaf(v[k].x, c, a.x); a.y = fmaf(v[k].y, c, a.y);
          a.z = fmaf(v[k].z, c, a.z); a.w = fmaf(v[k].w, c, a.w);
        }
      };
      // 96 splits at most (attn_splits_wanted): six batches, every branch warp-uniform
#define TLB_FOLD(CA, CB)                                  \
  if (16 * (CA) < s_live) {                               \
    fold16(va, (CA));                                     \
    if (16 * ((CA) + 2) < s_live) load16(va, 16 * ((CA) + 2)); \
  }                                                       \
  if (16 * (CB) < s_live) {                               \
    fold16(vb, (CB));                                     \
    if (16 * ((CB) + 2) < s_live) load16(vb, 16 * ((CB) + 2)); \
  }
      TLB_FOLD(0, 1)
      TLB_FOLD(2, 3)
      TLB_FOLD(4, 5)
#undef TLB_FOLD
      if (has) {
        const float inv = 1.0f / lsum;
        *(float4*)(p.out + (size_t)(kh * p.grp + h) * D + li * 4) =
            make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
      }
    }
  }
  __syncthreads();
  if (tid == 0) p.counters[kh] = 0;   // clean for the next launch
}

template <int D>
int launch_mma_t(const AttnParams& p, int splits, cudaStream_t stream) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return set_error(TLB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  CUtensorMap tmK, tmV;
  const cuuint64_t rows = (cuuint64_t)p.n_kv * (cuuint64_t)p.kv_rows;
  cuuint64_t dims[2] = {(cuuint64_t)D, rows};
  cuuint64_t strides[1] = {(cuuint64_t)D * 4};
  cuuint32_t box[2] = {32, (cuuint32_t)MM_TK};
  cuuint32_t es[2] = {1, 1};
  for (int which = 0; which < 2; which++) {
    CUresult r = enc(which ? &tmV : &tmK, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                     const_cast<void*>(which ? p.V : p.K), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(TLB_ERR_CUDA, "attn_decode: tensor map encode failed");
  }
  static std::atomic<unsigned long long> attr_done{0};
  {
    const int rc_attr = ensure_dynamic_smem(attn_decode_mma_kernel<D>, (int)MmaCfg<D>::TOTAL, attr_done);
    if (rc_attr) return rc_attr;
  }
  LaunchCfg lc(dim3(splits, p.n_kv), dim3(MmaCfg<D>::THREADS), MmaCfg<D>::TOTAL, stream, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, attn_decode_mma_kernel<D>, tmK, tmV, p));
  return TLB_OK;
}

}  // namespace

// f32 cache, 3..8 query heads per KV head, 16-byte aligned operands (checked by the caller),
// row count of the [n_kv * kv_max, D] view within the TMA coordinate range
bool attn_decode_mma_eligible(int grp, int D, int n_kv, long long kv_max, int kv_bf16) {
  return !kv_bf16 && grp >= 3 && grp <= 8 && (D == 64 || D == 128) && (long long)n_kv * kv_max < (1ll << 31);
}

int attn_decode_mma_launch(const AttnParams& p, int D, int splits, cudaStream_t stream) {
  if (D == 128) return launch_mma_t<128>(p, splits, stream);
  return launch_mma_t<64>(p, splits, stream);
}

}  // namespace tlb
