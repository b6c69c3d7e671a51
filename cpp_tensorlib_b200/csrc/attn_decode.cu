// Decode attention: out[h,:] = softmax(scale * q[h] . K[kv(h)]^T) . V[kv(h)] for
// one query row per head over the valid prefix [0,ctx) of a [n_kv, kv_max, D]
// f32 cache.  Replaces cuda::attn_decode / attn_decode_dpos and the kernels
// tl_attn_decode_*, tl_attn_decode_split*, tl_attn_combine
// (include/cuda.h:966-1114, kernels/tensorlib_cuda.cu:842-1061).
//
// Design (HBM-bound: every K and V byte is read once):
//  * grid = (splits, kv heads).  A CTA owns one KV head and one contiguous chunk
//    of the context and serves ALL q heads of that KV head's group from the same
//    shared-memory tiles, so GQA costs no extra HBM or L2 traffic (the reference
//    launches one block per q head and re-reads the cache group-size times).
//  * K/V tiles of 32 keys are contiguous in the cache, so each is one 1-D bulk
//    async copy (cp.async.bulk) into a 3-4 stage mbarrier ring.
//  * 8 lanes share a key (each owns D/8 dims as 16-byte chunks -> conflict-free
//    shared loads); a warp covers 4 keys per step and up to 4 q heads, with a
//    per-lane online softmax that only rescales when the running max moves.
//  * Split-K over the context with an ON-CHIP merge: each CTA writes its
//    (m, l, acc) partial, takes a ticket on a per-KV-head counter, and the last
//    CTA to arrive folds the partials in split order.  One launch, no second
//    kernel, deterministic.
//  * The device-position variant reads ctx = *d_pos + 1 and launches the
//    capacity's split count; split boundaries are derived from ctx by the same
//    device function in both variants, so the two are bit-identical at every
//    position (the property check_attn64.cpp:91-102 of the reference guards).
#include <cstdlib>
#include <mutex>
#include <string>

#include "attn_split.cuh"

namespace tlb {

unsigned long long* g_attn_dbg = nullptr;

// Warps across heads: ceil(grp / HW) rounded up to a divisor of the warp count.
__host__ __device__ inline int attn_hs(int grp, int HW, int warps) {
  int hs = (grp + HW - 1) / HW;
  while (warps % hs) hs++;
  return hs;
}

// LPK = lanes that share a key: 8 (8 warps, 4 keys per warp step) or 16 (16 warps, 2 keys
// per step, half the per-lane state; an experiment for wide groups, not the default).
// BF: the cache holds bf16 (kv_ld / kv_st of the reference, kernels/tensorlib_cuda.cu:828-831:
// widened to f32 for the dot and the accumulate, q / out / partials stay f32).  A lane then
// owns 16-byte chunks of 8 dims instead of 4.
template <int D, int HW, int LPK, bool BF>
struct AttnCfg {
  static constexpr int STAGES = HW >= 4 ? 4 : 3;
  static constexpr int ELT = BF ? 2 : 4;
  static constexpr int TILE_BYTES = AT_TK * D * ELT;
  static constexpr int CH = D / (4 * LPK);  // 16-byte chunks per lane
  static constexpr int WARPS = LPK;
  static constexpr int THREADS = 32 * LPK;
  static constexpr int KPS = 32 / LPK;       // keys per warp step
};

// the ring; the CTA merge reuses it and needs WARPS * KPS * HW entries of D+4 floats
template <int D, int HW, int LPK, bool BF>
__host__ __device__ constexpr size_t attn_ring_bytes() {
  using C = AttnCfg<D, HW, LPK, BF>;
  const size_t ring = (size_t)C::STAGES * 2 * C::TILE_BYTES;
  const size_t ent = (size_t)C::WARPS * C::KPS * HW * (D + 4) * sizeof(float);
  return ring < ent ? ent : ring;
}
template <int D, int HW, int LPK, bool BF>
size_t attn_smem_bytes(int) {
  return 128 + attn_ring_bytes<D, HW, LPK, BF>() + 64;  // alignment slack, ring, barriers
}

template <int D, int HW, int LPK, bool BF>
__global__ void __launch_bounds__(32 * LPK, ((HW >= 4 || LPK > 8) ? 1 : 2))
    attn_decode_kernel(AttnParams p) {
  using C = AttnCfg<D, HW, LPK, BF>;
  static_assert(!BF || C::CH % 2 == 0, "bf16 rows are read in 16-byte chunks of 8 dims");
  constexpr int AT_THREADS = C::THREADS, AT_WARPS = C::WARPS, KPS = C::KPS;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  float* Kt = (float*)base;
  float* Vt = (float*)(base + (size_t)C::STAGES * C::TILE_BYTES);
  uint64_t* bars = (uint64_t*)(base + attn_ring_bytes<D, HW, LPK, BF>());

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kslot = lane / LPK, sub = lane % LPK;
  const int kh = blockIdx.y, sp = blockIdx.x;
  auto stamp = [&](int i) {
    if (p.dbg && tid == 0) {
      unsigned long long tt;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(tt));
      p.dbg[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 8 + i] = tt;
    }
  };
  stamp(0);
  const int hs = attn_hs(p.grp, HW, AT_WARPS);  // warps across heads
  const int ks = AT_WARPS / hs;          // warps across keys
  const int hslot = warp % hs, kslice = warp / hs;

  if (tid == 0) {
    for (int s = 0; s < C::STAGES; s++) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  const int ctx = p.d_pos ? (int)(*p.d_pos) + 1 : p.ctx;
  if (p.d_pos && (ctx > p.kv_rows || ctx < 1)) {
    // The position ran past the cache (the host checks this before it launches; this is the
    // second line of defence for graphs replayed without the host's bookkeeping): read
    // nothing, leave the tickets untouched, tell the host through the status block.
    pdl_wait();
    pdl_launch_dependents();
    if (p.status && tid == 0) atomicExch(&p.status[ST_KV_OVERFLOW], 1);
    return;
  }
  const int chunk = attn_chunk(p.n_kv, ctx, p.sm2);
  const int s_live = (ctx + chunk - 1) / chunk;
  const bool dead = sp >= s_live;  // capacity-sized grid: splits past the live count do nothing
  const int k_begin = sp * chunk;
  const int k_end = k_begin + chunk < ctx ? k_begin + chunk : ctx;
  const int n_tiles = dead ? 0 : (k_end - k_begin + AT_TK - 1) / AT_TK;

  const unsigned char* Kh = (const unsigned char*)p.K + (size_t)kh * p.kv_stride * C::ELT;
  const unsigned char* Vh = (const unsigned char*)p.V + (size_t)kh * p.kv_stride * C::ELT;

  auto issue = [&](int i) {
    const int st = i % C::STAGES;
    const int r0 = k_begin + i * AT_TK;
    const int rows = (k_end - r0) < AT_TK ? (k_end - r0) : AT_TK;
    const uint32_t bytes = (uint32_t)rows * D * C::ELT;
    mbar_expect_tx(&bars[st], 2 * bytes);
    bulk_load_1d((unsigned char*)Kt + (size_t)st * C::TILE_BYTES, Kh + (size_t)r0 * D * C::ELT, bytes,
                 &bars[st]);
    bulk_load_1d((unsigned char*)Vt + (size_t)st * C::TILE_BYTES, Vh + (size_t)r0 * D * C::ELT, bytes,
                 &bars[st]);
  };
  // Tiles that end below the newest row do not depend on the preceding kernel (it only
  // appends row ctx-1): with early_kv they stream while that kernel drains.
  const int pre = n_tiles < C::STAGES ? n_tiles : C::STAGES;
  int early = 0;
  if (p.early_kv && tid == 0) {
    while (early < pre && k_begin + (early + 1) * AT_TK <= ctx - 1) issue(early++);
  }

  pdl_wait();
  pdl_launch_dependents();
  stamp(1);
  if (dead) return;
  if (tid == 0) {
    for (int i = early; i < pre; i++) issue(i);
  }

  // q fragments: lane owns chunks {sub + LPK*i}
  float4 qf[HW][C::CH];
#pragma unroll
  for (int h = 0; h < HW; h++) {
    const int hh = hslot * HW + h;
    const bool live = hh < p.grp;
    const float* qp = p.q + (size_t)(kh * p.grp + (live ? hh : 0)) * D;
#pragma unroll
    for (int i = 0; i < C::CH; i++)
      qf[h][i] = live ? *(const float4*)(qp + attn_dim0<LPK, BF>(sub, i)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float m[HW], l[HW];
  float4 acc[HW][C::CH];
#pragma unroll
  for (int h = 0; h < HW; h++) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < C::CH; i++) acc[h][i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }

  for (int it = 0; it < n_tiles; it++) {
    const int st = it % C::STAGES;
    if (!mbar_wait_bounded(&bars[st], (it / C::STAGES) & 1, p.status, 200 + st)) return;
    if (it == 0) stamp(2);
    if (it == n_tiles - 1) stamp(7);
    const int r0 = k_begin + it * AT_TK;
    const int rows = (k_end - r0) < AT_TK ? (k_end - r0) : AT_TK;
    const unsigned char* Ks = (const unsigned char*)Kt + (size_t)st * C::TILE_BYTES;
    const unsigned char* Vs = (const unsigned char*)Vt + (size_t)st * C::TILE_BYTES;
    for (int step = kslice; step < AT_TK / KPS; step += ks) {
      const int row = step * KPS + kslot;
      if (step * KPS >= rows) break;
      const bool valid = row < rows;
      const int rr = valid ? row : 0;
      float4 kv[C::CH];
      attn_load_row<D, LPK, C::CH, BF>(Ks + (size_t)rr * D * C::ELT, sub, kv);
      float s[HW];
#pragma unroll
      for (int h = 0; h < HW; h++) {
        // four independent partial sums keep the FMA chain short
        float dx = 0.f, dy = 0.f, dz = 0.f, dw = 0.f;
#pragma unroll
        for (int i = 0; i < C::CH; i++) {
          dx = fmaf(qf[h][i].x, kv[i].x, dx);
          dy = fmaf(qf[h][i].y, kv[i].y, dy);
          dz = fmaf(qf[h][i].z, kv[i].z, dz);
          dw = fmaf(qf[h][i].w, kv[i].w, dw);
        }
        float d = (dx + dy) + (dz + dw);
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        d += __shfl_xor_sync(0xffffffffu, d, 4);
        if (LPK > 8) d += __shfl_xor_sync(0xffffffffu, d, 8);
        s[h] = valid ? d * p.scale : -INFINITY;
      }
      attn_load_row<D, LPK, C::CH, BF>(Vs + (size_t)rr * D * C::ELT, sub, kv);
      // The four key slots of the warp share one running max per head, so the rescale
      // branch is warp-uniform and the slots' sums can later be added without exps.
      float sm[HW];
      bool grow = false;
#pragma unroll
      for (int h = 0; h < HW; h++) {
        sm[h] = fmaxf(s[h], __shfl_xor_sync(0xffffffffu, s[h], 16));
        if (LPK == 8) sm[h] = fmaxf(sm[h], __shfl_xor_sync(0xffffffffu, sm[h], 8));
        grow = grow || (sm[h] > m[h]);
      }
      if (grow) {  // one warp-uniform branch per step, rare after the first keys
#pragma unroll
        for (int h = 0; h < HW; h++) {
          const float mn = fmaxf(m[h], sm[h]);
          const float corr = (mn == m[h]) ? 1.0f : __expf(m[h] - mn);  // exp(-inf) = 0 at the start
          l[h] *= corr;
#pragma unroll
          for (int i = 0; i < C::CH; i++) {
            acc[h][i].x *= corr; acc[h][i].y *= corr;
            acc[h][i].z *= corr; acc[h][i].w *= corr;
          }
          m[h] = mn;
        }
      }
#pragma unroll
      for (int h = 0; h < HW; h++) {
        const float pr = __expf(s[h] - m[h]);    // 0 for an invalid row (s = -inf)
        l[h] += pr;
#pragma unroll
        for (int i = 0; i < C::CH; i++) {
          acc[h][i].x = fmaf(pr, kv[i].x, acc[h][i].x);
          acc[h][i].y = fmaf(pr, kv[i].y, acc[h][i].y);
          acc[h][i].z = fmaf(pr, kv[i].z, acc[h][i].z);
          acc[h][i].w = fmaf(pr, kv[i].w, acc[h][i].w);
        }
      }
    }
    __syncthreads();  // every warp is done with this stage
    if (tid == 0 && it + C::STAGES < n_tiles) issue(it + C::STAGES);
  }

  stamp(3);
  // ---- every key slot of every warp leaves (acc, m, l) in shared memory (the tile
  // ring is free now): entry [(kslice*4 + kslot)][head][D+4] = acc[D], m, l, pad, pad.
  // Slots of one warp share m, so the CTA merge needs one exp per (warp, head).
  const int nheads_pad = hs * HW;
  float* ent = (float*)base;
  {
#pragma unroll
    for (int h = 0; h < HW; h++) {
      float* dst = ent + ((size_t)(kslice * KPS + kslot) * nheads_pad + hslot * HW + h) * (D + 4);
      if (sub == 0) { dst[D] = m[h]; dst[D + 1] = l[h]; }
#pragma unroll
      for (int i = 0; i < C::CH; i++) *(float4*)(dst + attn_dim0<LPK, BF>(sub, i)) = acc[h][i];
    }
  }
  __syncthreads();

  // ---- CTA merge over warps and key slots, then either the output or a split partial
  const bool single = (s_live == 1);
  for (int idx = tid; idx < p.grp * (D / 4); idx += AT_THREADS) {
    const int hh = idx / (D / 4), d4 = idx - hh * (D / 4);
    float mm = -INFINITY;
    for (int k2 = 0; k2 < ks; k2++)
      mm = fmaxf(mm, ent[((size_t)(k2 * KPS) * nheads_pad + hh) * (D + 4) + D]);
    float ll = 0.f;
    float4 aa = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k2 = 0; k2 < ks; k2++) {
      const float mk = ent[((size_t)(k2 * KPS) * nheads_pad + hh) * (D + 4) + D];
      const float c = (mk == -INFINITY) ? 0.f : __expf(mk - mm);
#pragma unroll
      for (int j = 0; j < KPS; j++) {
        const float* src = ent + ((size_t)(k2 * KPS + j) * nheads_pad + hh) * (D + 4);
        const float4 a = *(const float4*)(src + d4 * 4);
        ll = fmaf(src[D + 1], c, ll);
        aa.x = fmaf(a.x, c, aa.x); aa.y = fmaf(a.y, c, aa.y);
        aa.z = fmaf(a.z, c, aa.z); aa.w = fmaf(a.w, c, aa.w);
      }
    }
    const int qh = kh * p.grp + hh;
    if (single) {
      const float inv = 1.0f / ll;
      *(float4*)(p.out + (size_t)qh * D + d4 * 4) = make_float4(aa.x * inv, aa.y * inv, aa.z * inv, aa.w * inv);
    } else {
      // global partial entry: acc[D], m, l, pad, pad  (stride D+4 floats, 16-byte aligned)
      float* dst = p.partials + ((size_t)qh * p.s_cap + sp) * (D + 4);
      if (d4 == 0) __stcg((float2*)&dst[D], make_float2(mm, ll));
      __stcg((float4*)&dst[d4 * 4], aa);
    }
  }
  stamp(4);
  if (single) return;

  // ---- on-chip split merge: last CTA of this KV head folds the partials ------
  // The barrier orders every thread's partial stores before thread 0's acq_rel ticket
  // (release is cumulative), and the ticket's acquire side plus the second barrier
  // orders the other CTAs' partials before this CTA's loads: no membar needed.
  __shared__ int is_last;
  __syncthreads();
  if (tid == 0) {
    int old;
    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], %2;" : "=r"(old) : "l"(&p.counters[kh]), "r"(1) : "memory");
    is_last = (old == s_live - 1);
  }
  __syncthreads();
  stamp(5);
  if (!is_last) return;
  // One thread per (head, 4 dims).  The first 16 splits' accumulators are requested
  // before the coefficient phase, so its round trip overlaps theirs.
  const int my = tid;
  const bool has = my < p.grp * (D / 4);
  const int mh = has ? my / (D / 4) : 0, md4 = has ? my - mh * (D / 4) : 0;
  const float* msrc = p.partials + (size_t)(kh * p.grp + mh) * p.s_cap * (D + 4) + md4 * 4;
  float4 v0[16];
#pragma unroll
  for (int k2 = 0; k2 < 16; k2++)
    v0[k2] = (has && k2 < s_live) ? __ldcg((const float4*)(msrc + (size_t)k2 * (D + 4)))
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
  // Phase 1 (one warp per head): rescale coefficients c_s = exp(m_s - max m) and the
  // denominator, splits spread over the lanes.  The tile ring is free by now and
  // holds the coefficients (behind the CTA-merge entries nobody reads any more).
  float* cw = Kt;                       // [grp][s_live]
  float* lden = Kt + p.grp * s_live;    // [grp]
  for (int hh = warp; hh < p.grp; hh += AT_WARPS) {
    const int qh = kh * p.grp + hh;
    const float* src0 = p.partials + (size_t)qh * p.s_cap * (D + 4) + D;
    // one round trip: every lane fetches (m, l) of its splits (up to 3 per lane)
    float2 ml[3];
#pragma unroll
    for (int k2 = 0; k2 < 3; k2++) {
      const int s2 = lane + 32 * k2;
      ml[k2] = s2 < s_live ? __ldcg((const float2*)(src0 + (size_t)s2 * (D + 4)))
                           : make_float2(-INFINITY, 0.f);
    }
    float mm = warp_max(fmaxf(ml[0].x, fmaxf(ml[1].x, ml[2].x)));
    float ll = 0.f;
#pragma unroll
    for (int k2 = 0; k2 < 3; k2++) {
      const int s2 = lane + 32 * k2;
      if (s2 < s_live) {
        const float c = __expf(ml[k2].x - mm);
        cw[hh * s_live + s2] = c;
        ll += ml[k2].y * c;
      }
    }
    ll = warp_sum(ll);
    if (lane == 0) lden[hh] = ll;
  }
  __syncthreads();
  // Phase 2: fold, 16 independent 16-byte loads in flight per thread.
  if (has) {
    const float* cwh = cw + mh * s_live;
    float4 aa = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k2 = 0; k2 < 16; k2++)
      if (k2 < s_live) {
        const float c = cwh[k2];
        aa.x = fmaf(v0[k2].x, c, aa.x); aa.y = fmaf(v0[k2].y, c, aa.y);
        aa.z = fmaf(v0[k2].z, c, aa.z); aa.w = fmaf(v0[k2].w, c, aa.w);
      }
    for (int s0 = 16; s0 < s_live; s0 += 16) {
      float4 v[16];
#pragma unroll
      for (int k2 = 0; k2 < 16; k2++)
        v[k2] = (s0 + k2 < s_live) ? __ldcg((const float4*)(msrc + (size_t)(s0 + k2) * (D + 4)))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int k2 = 0; k2 < 16; k2++)
        if (s0 + k2 < s_live) {
          const float c = cwh[s0 + k2];
          aa.x = fmaf(v[k2].x, c, aa.x); aa.y = fmaf(v[k2].y, c, aa.y);
          aa.z = fmaf(v[k2].z, c, aa.z); aa.w = fmaf(v[k2].w, c, aa.w);
        }
    }
    const float inv = 1.0f / lden[mh];
    *(float4*)(p.out + (size_t)(kh * p.grp + mh) * D + md4 * 4) =
        make_float4(aa.x * inv, aa.y * inv, aa.z * inv, aa.w * inv);
  }
  // groups wider than 256 / (D/4) heads: the remaining (head, 4 dims) items
  for (int idx = tid + AT_THREADS; idx < p.grp * (D / 4); idx += AT_THREADS) {
    const int hh = idx / (D / 4), d4 = idx - hh * (D / 4);
    const float* src0 = p.partials + (size_t)(kh * p.grp + hh) * p.s_cap * (D + 4) + d4 * 4;
    const float* cwh = cw + hh * s_live;
    float4 aa = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < s_live; s0 += 16) {
      float4 v[16];
#pragma unroll
      for (int k2 = 0; k2 < 16; k2++)
        v[k2] = (s0 + k2 < s_live) ? __ldcg((const float4*)(src0 + (size_t)(s0 + k2) * (D + 4)))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int k2 = 0; k2 < 16; k2++)
        if (s0 + k2 < s_live) {
          const float c = cwh[s0 + k2];
          aa.x = fmaf(v[k2].x, c, aa.x); aa.y = fmaf(v[k2].y, c, aa.y);
          aa.z = fmaf(v[k2].z, c, aa.z); aa.w = fmaf(v[k2].w, c, aa.w);
        }
    }
    const float inv = 1.0f / lden[hh];
    *(float4*)(p.out + (size_t)(kh * p.grp + hh) * D + d4 * 4) =
        make_float4(aa.x * inv, aa.y * inv, aa.z * inv, aa.w * inv);
  }
  stamp(6);
  if (tid == 0) p.counters[kh] = 0;
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
size_t attn_partials_bytes(int n_q, int n_kv, long long kv_max, int D, int sm_count) {
  int s = attn_splits_wanted(n_kv, (int)kv_max, attn_target(n_kv > 0 ? n_q / n_kv : 1, sm_count));
  return (size_t)n_q * s * (D + 4) * sizeof(float);
}

template <int D, int HW, int LPK, bool BF>
static int launch_b(const AttnParams& p, int splits, cudaStream_t stream) {
  size_t smem = attn_smem_bytes<D, HW, LPK, BF>(p.grp);
  static std::atomic<unsigned long long> attr_done{0};
  {
    const int rc_attr = ensure_dynamic_smem(attn_decode_kernel<D, HW, LPK, BF>, 200 * 1024, attr_done);
    if (rc_attr) return rc_attr;
  }
  LaunchCfg lc(dim3(splits, p.n_kv), dim3(32 * LPK), smem, stream, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, attn_decode_kernel<D, HW, LPK, BF>, p));
  return TLB_OK;
}
template <int D, int HW, int LPK>
static int launch_t(const AttnParams& p, int splits, cudaStream_t stream, bool bf) {
  if (bf) return launch_b<D, HW, LPK, true>(p, splits, stream);
  return launch_b<D, HW, LPK, false>(p, splits, stream);
}

bool attn_decode_mma_eligible(int grp, int D, int n_kv, long long kv_max, int kv_bf16);
int attn_decode_mma_launch(const AttnParams& p, int D, int splits, cudaStream_t stream);

// ctx >= 1 and d_pos == nullptr: host-position variant.  d_pos != nullptr: the
// context is *d_pos + 1 and the grid is sized from kv_max.
int attn_decode_launch(DeviceCtx* c, const float* q, const void* K, const void* V, float* out,
                       int n_q, int n_kv, int ctx, long long kv_max, int D, float scale,
                       const unsigned* d_pos, float* partials, int* counters,
                       cudaStream_t stream, int early_kv, int kv_bf16, const GvStream* prefetch) {
  if (D != 64 && D != 128) return set_error(TLB_ERR_UNSUPPORTED, "attn_decode: D must be 64 or 128");
  if (n_kv <= 0 || n_q <= 0 || n_q % n_kv != 0)
    return set_error(TLB_ERR_ARG, "attn_decode: need n_q > 0, n_kv > 0 and n_q % n_kv == 0");
  if (kv_max <= 0 || kv_max > (1ll << 30) || kv_max * D > (1ll << 40))
    return set_error(TLB_ERR_ARG, "attn_decode: kv_max out of range");
  const int grp = n_q / n_kv;
  if (grp > 32) return set_error(TLB_ERR_UNSUPPORTED, "attn_decode: GQA group > 32");
  if (((uintptr_t)K & 15) || ((uintptr_t)V & 15) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15))
    return set_error(TLB_ERR_ARG, "attn_decode: q/K/V/out must be 16-byte aligned");
  AttnParams p;
  p.q = q; p.K = K; p.V = V; p.out = out; p.partials = partials; p.counters = counters;
  p.d_pos = d_pos; p.ctx = ctx; p.n_q = n_q; p.n_kv = n_kv; p.grp = grp;
  p.kv_stride = kv_max * D; p.kv_rows = (int)kv_max; p.scale = scale; p.sm2 = attn_target(grp, c->sm_count); p.status = c->status; p.dbg = g_attn_dbg; p.early_kv = early_kv;
  const int basis = d_pos ? (int)kv_max : ctx;
  const int splits = d_pos ? attn_splits_wanted(n_kv, basis, p.sm2)
                           : (ctx + attn_chunk(n_kv, ctx, p.sm2) - 1) / attn_chunk(n_kv, ctx, p.sm2);
  p.s_cap = d_pos ? splits : attn_splits_wanted(n_kv, basis, p.sm2);
  // GQA groups of 3..8 heads on an f32 cache: the tensor-core form (attn_decode_mma.cu).
  // TLB_ATTN_MMA=0 keeps the CUDA-core form (a diagnostic switch for A/B timing).
  static const bool mma_on = !(getenv("TLB_ATTN_MMA") && atoi(getenv("TLB_ATTN_MMA")) == 0);
  if (mma_on && attn_decode_mma_eligible(grp, D, n_kv, kv_max, kv_bf16))
    return attn_decode_mma_launch(p, D, splits, stream);
  // heads per warp: the smallest of {1,2,4} such that ceil(grp/HW) divides 8
  int HW = grp == 1 ? 1 : (grp == 2 ? 2 : 4);
  if (D == 128) {
    if (HW == 1) return launch_t<128, 1, 8>(p, splits, stream, kv_bf16 != 0);
    if (HW == 2) return launch_t<128, 2, 8>(p, splits, stream, kv_bf16 != 0);
    // TLB_ATTN_LPK=16 selects the 16-warp form (16 lanes per key); measured 6 % slower than
    // the 8-warp form on the 7B layer shape (14.4 vs 13.6 us), so it is not the default
    static const int lpk = getenv("TLB_ATTN_LPK") ? atoi(getenv("TLB_ATTN_LPK")) : 8;
    if (lpk == 16) return launch_t<128, 4, 16>(p, splits, stream, kv_bf16 != 0);
    return launch_t<128, 4, 8>(p, splits, stream, kv_bf16 != 0);
  }
  if (HW == 1) return launch_t<64, 1, 8>(p, splits, stream, kv_bf16 != 0);
  if (HW == 2) return launch_t<64, 2, 8>(p, splits, stream, kv_bf16 != 0);
  return launch_t<64, 4, 8>(p, splits, stream, kv_bf16 != 0);
}

}  // namespace tlb

namespace tlb {

// ---------------------------------------------------------------------------
// Allocation-free entry point.
//
// Some hosts that embed this library may not allocate device memory at the moment
// they need attention: a serving loop that has handed the whole device heap to
// its own arena, a plugin called from inside a region where the embedder forbids
// cudaMalloc (it synchronises the device and can fail late), or a process that
// runs under a fixed memory budget agreed at start-up.  For them this variant
// keeps the split-KV partials and the merge counters in a fixed array that is
// part of the library image, so every GPU that loads the library holds it (4 MiB)
// until the process exits, and the call itself allocates nothing.
// ---------------------------------------------------------------------------
constexpr size_t NOALLOC_COUNTER_BYTES = 256;                  // merge counters, n_kv <= 64
constexpr size_t NOALLOC_BYTES = 4u << 20;                     // whole array: 4 MiB
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_BYTES];

namespace {
struct NoallocDev {
  void* ptr = nullptr;  // device address of g_noalloc_scratch on that device
  int sm_count = 0;
};
NoallocDev g_noalloc_dev[64];
std::mutex g_noalloc_mu;

// Once per device, with that device current: the array's name is only a host-side
// handle, the kernel needs the address the runtime reports for this device.
int noalloc_setup(int dev, NoallocDev** out) {
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  NoallocDev& d = g_noalloc_dev[dev];
  if (!d.ptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_noalloc_scratch)");
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute(MultiProcessorCount)");
    d.sm_count = sms;
    d.ptr = p;
  }
  *out = &d;
  return TLB_OK;
}
}  // namespace

}  // namespace tlb

extern "C" int tlb_attn_decode_noalloc(const float* q, const float* K, const float* V, float* out,
                                       int64_t n_q, int64_t n_kv, int64_t ctx, int64_t kv_max,
                                       int64_t D, float scale, void* stream) {
  using namespace tlb;
  TLB_REQUIRE(q && K && V && out, "tlb_attn_decode_noalloc: null pointer");
  TLB_REQUIRE(ctx >= 1 && ctx <= kv_max, "tlb_attn_decode_noalloc: need 1 <= ctx <= kv_max");
  TLB_REQUIRE(n_kv > 0 && n_kv <= 64, "tlb_attn_decode_noalloc: n_kv must be 1..64");
  TLB_REQUIRE(n_q > 0 && n_q <= (1 << 24) && n_q % n_kv == 0,
              "tlb_attn_decode_noalloc: need 0 < n_q <= 2^24 and n_q % n_kv == 0");
  TLB_REQUIRE(kv_max <= (1ll << 30), "tlb_attn_decode_noalloc: kv_max out of range");
  TLB_REQUIRE(D == 64 || D == 128, "tlb_attn_decode_noalloc: D must be 64 or 128");
  int dev = 0;
  TLB_CUDA(cudaGetDevice(&dev));
  TLB_REQUIRE(dev >= 0 && dev < 64, "tlb_attn_decode_noalloc: device index out of range");
  NoallocDev* nd = nullptr;
  int rc = noalloc_setup(dev, &nd);
  if (rc) return rc;
  const size_t need = attn_partials_bytes((int)n_q, (int)n_kv, ctx, (int)D, nd->sm_count);
  if (need > NOALLOC_BYTES - NOALLOC_COUNTER_BYTES)
    return set_error(TLB_ERR_UNSUPPORTED,
                     "tlb_attn_decode_noalloc: the split partials need " + std::to_string(need) +
                         " bytes, the built-in scratch holds " +
                         std::to_string(NOALLOC_BYTES - NOALLOC_COUNTER_BYTES) +
                         "; use tlb_attn_decode or fewer heads");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left: the counters must start at zero.
  TLB_CUDA(cudaMemsetAsync(nd->ptr, 0, NOALLOC_COUNTER_BYTES, s));
  // Only the SM count and the status block are read.  The status block is the library's
  // per-device one when some other call created it already (then an expired wait shows up
  // in tlb_device_status); this call never creates it, because that would allocate.
  DeviceCtx local;
  local.sm_count = nd->sm_count;
  const DeviceCtx* existing = find_ctx();
  local.status = existing ? existing->status : nullptr;
  return attn_decode_launch(&local, q, K, V, out, (int)n_q, (int)n_kv, (int)ctx, kv_max, (int)D,
                            scale, nullptr, (float*)((unsigned char*)nd->ptr + NOALLOC_COUNTER_BYTES),
                            (int*)nd->ptr, s, 0, 0, nullptr);
}
