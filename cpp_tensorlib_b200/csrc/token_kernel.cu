// Persistent per-token decoder kernel (single GPU): every op of one decode token
// -- the 113 int4 GEMVs with their fused residual-add + RMSNorm / SwiGLU prologues,
// RoPE + bias + KV append + split-KV attention, the argmax -- runs inside ONE
// cooperative launch of one CTA per SM, phases separated by a grid barrier.
//
// Why: with one kernel per op the token is bound by per-kernel latency chains
// (launch, barrier init, first TMA round trip, drain), not by HBM.  Here each warp
// sees its whole token as ONE stream of weight units: its TMA producer cursor runs
// up to a ring ahead of its consumer cursor and crosses phase boundaries freely
// (weights are static), so the weights of the next projection are already in
// shared memory when the barrier opens.
//
// The arithmetic is that of gemv_q4_mma_kernel / attn_decode_kernel / the row ops
// (same fragments, same split-K fix-up order, same softmax merge), so results match
// the multi-kernel path to rounding; it replaces the launch sequence of the
// reference's run_layers_ (bench/cuda/qwen_model.h:673-740) + captured_decoder.
// Every wait (mbarrier, grid barrier) is bounded and reports through the status word.
#include "q4_mma.cuh"
#include "token_kernel.cuh"

namespace tlb {

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Grid-wide barrier for a cooperative launch (all CTAs co-resident).  Bounded:
// after ~1 s, or as soon as any wait has already failed, it stops waiting.
__device__ __forceinline__ void tk_grid_barrier(unsigned* bar, unsigned& gen, int* status) {
  __syncthreads();
  if (threadIdx.x == 0) {
    // release-arrive: the CTA's writes (ordered before this by the block barrier) become
    // visible to whoever acquires the new generation
    unsigned old;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(&bar[0]) : "memory");
    if (old == gridDim.x - 1) {
      asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(&bar[0]), "r"(0u) : "memory");
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(&bar[1]), "r"(gen + 1u) : "memory");
    } else {
      const long long t0 = clock64();
      while (ld_acquire_gpu(&bar[1]) == gen) {
        if (clock64() - t0 > 200000ll) {   // only look at the slow-path conditions now and then
          if (*(volatile int*)&status[ST_WAIT_TIMEOUT]) break;
          if (clock64() - t0 > 2000000000ll) {
            atomicExch(&status[ST_WAIT_TIMEOUT], 1);
            atomicExch(&status[ST_WAIT_WHERE], 600);
            break;
          }
        }
      }
    }
  }
  gen++;
  __syncthreads();
}

__device__ __forceinline__ unsigned long long tk_argmax_key(float v, unsigned idx) {
  unsigned b = __float_as_uint(v);
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return ((unsigned long long)b << 32) | (unsigned long long)(0xFFFFFFFFu - idx);
}

template <int D>
__global__ void __launch_bounds__(TK_THREADS, 1) token_kernel(TkParams P) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int grp = P.n_q / P.n_kv;
  // k_max is implied by the layout the host computed: the offsets below only depend
  // on it through the GEMV view, which the host sized for the largest K.
  __shared__ TkSmem L;
  __shared__ int is_last_s;
  if (tid == 0) {
    int kmax = 0, kin = 0;
    for (int i = 0; i < P.n_phases; i++) {
      if (P.phases[i].type == 0 && P.phases[i].K > kmax) kmax = P.phases[i].K;
      if (P.phases[i].type == 1 && i > 0 && P.phases[i - 1].type == 0 && P.phases[i - 1].K > kin)
        kin = P.phases[i - 1].K;
    }
    L = tk_smem_layout(kmax, kin, P.hd, grp);
  }
  __syncthreads();

  uint64_t* bars = (uint64_t*)(base + L.bars);
  unsigned char* myW = base + L.w_ring + (size_t)warp * TK_STAGES * GVU_W_BYTES;
  unsigned char* myS = base + L.s_ring + (size_t)warp * TK_STAGES * GVU_S_BYTES;
  uint64_t* mybar = bars + warp * TK_STAGES;
  uint64_t* at_bars = (uint64_t*)(base + L.at_bars);
  const unsigned wid = blockIdx.x * TK_WARPS + warp;

  if (lane == 0)
    for (int s = 0; s < TK_STAGES; s++) mbar_init(&mybar[s], 1);
  if (tid == 0)
    for (int s = 0; s < TK_ATT_STAGES; s++) mbar_init(&at_bars[s], 1);
  mbar_fence_init();
  __syncthreads();

  unsigned gen = *(volatile unsigned*)&P.bar[1];
  const int tok = *P.d_tok;
  const unsigned pos = *P.d_pos;
  // cos/sin of this token's position for every rotary pair, once per token (double
  // angle as in rope_kernel; every attention phase reads the table)
  float* rope_cs = (float*)(base + L.rope);
  if (tid < D / 2) {
    const double theta = exp2(-2.0 * (double)tid / (double)D * log2((double)P.rope_base));
    double sd, cd;
    sincos((double)pos * theta, &sd, &cd);
    rope_cs[tid] = (float)cd;
    rope_cs[D / 2 + tid] = (float)sd;
  }
  __syncthreads();

  // ---------------- producer cursor of this warp's weight stream ----------------
  int prod_ph = -1, prod_SL = 1, prod_map = 0, prod_rt = 0, prod_s = 0, prod_stage = 0;
  unsigned prod_u = 0, prod_u1 = 0;
  int inflight = 0;
  // Two ways to deal a projection's units to the warps (TkPhase::cta_tiles):
  //  0  every warp of the grid owns a contiguous unit range (row-tile-major); used
  //     when there are at least as many row tiles as warps -- no tile is shared;
  //  1  every CTA owns whole row tiles (tile = blockIdx.x, += gridDim.x) and its 16
  //     warps split the tile's K slabs (slab = warp, += 16); the partial sums meet
  //     in shared memory.  Used for the small-N projections, where sharing a tile
  //     across CTAs would need a round trip through global memory.
  int prod_mode = 0, prod_RT = 0;
  auto prod_open = [&](int ph) -> bool {
    const TkPhase& H = P.phases[ph];
    if (H.type != 0) return false;
    prod_SL = H.SL;
    prod_map = H.map;
    prod_mode = H.cta_tiles;
    if (prod_mode == 1) {
      prod_RT = H.RT;
      prod_rt = (int)blockIdx.x;
      prod_s = warp;
      prod_u = 0;
      prod_u1 = (prod_rt < prod_RT && prod_s < prod_SL) ? 1u : 0u;  // "has a next unit"
      return prod_u1 != 0;
    }
    if (wid >= H.Wtot) return false;
    const GvSplit sp = {H.q, H.r};
    prod_u = gv_start(wid, sp);
    prod_u1 = gv_start(wid + 1, sp);
    prod_rt = (int)(prod_u / (unsigned)prod_SL);
    prod_s = (int)(prod_u - (unsigned)prod_rt * prod_SL);
    return prod_u1 > prod_u;
  };
  auto issue_more = [&]() {
    while (inflight < TK_STAGES) {
      if (prod_u >= prod_u1) {
        bool found = false;
        while (prod_ph + 1 < P.n_phases) {
          prod_ph++;
          if (prod_open(prod_ph)) { found = true; break; }
        }
        if (!found) { prod_ph = P.n_phases; break; }
      }
      if (lane == 0) {
        mbar_expect_tx(&mybar[prod_stage], GVU_W_BYTES + GVU_S_BYTES);
        tma_load_2d(myW + prod_stage * GVU_W_BYTES, &P.maps[2 * prod_map], prod_s * 32, prod_rt * 16,
                    &mybar[prod_stage]);
        tma_load_2d(myS + prod_stage * GVU_S_BYTES, &P.maps[2 * prod_map + 1], prod_s * 8,
                    prod_rt * 16, &mybar[prod_stage]);
      }
      if (prod_mode == 1) {
        prod_s += TK_WARPS;
        if (prod_s >= prod_SL) { prod_s = warp; prod_rt += (int)gridDim.x; }
        if (prod_rt >= prod_RT) prod_u = prod_u1;  // exhausted
      } else {
        if (++prod_s == prod_SL) { prod_s = 0; prod_rt++; }
        prod_u++;
      }
      if (++prod_stage == TK_STAGES) prod_stage = 0;
      inflight++;
    }
  };
  issue_more();  // weights of the first projection start streaming at once

  int cons_stage = 0;
  unsigned cons_parity = 0;
  bool dead = false;    // a bounded wait expired: stop computing, keep the barriers going
  unsigned long long best_key = 0ull;

  unsigned at_ctr = 0;  // attention tiles consumed so far by this CTA (ring position)
  // ---- attention work plan (depends only on pos): splits, chunk, this CTA's items ----
  const int at_ctx = (int)pos + 1;
  int at_swant = (int)gridDim.x / P.n_kv;
  if (at_swant > at_ctx / 128) at_swant = at_ctx / 128;
  if (at_swant > P.attn_s_cap) at_swant = P.attn_s_cap;
  if (at_swant > 96) at_swant = 96;
  if (at_swant < 1) at_swant = 1;
  int at_chunk = (at_ctx + at_swant - 1) / at_swant;
  at_chunk = (at_chunk + TK_ATT_TK - 1) / TK_ATT_TK * TK_ATT_TK;
  const int at_slive = (at_ctx + at_chunk - 1) / at_chunk;
  constexpr int AT_TILE_BYTES = TK_ATT_TK * D * 4;
  // Issue tile i of an item (rows of one KV head's cache) into the attention ring.
  auto at_issue = [&](const float* Kc, const float* Vc, int item, int i) {
    const int kh = item / at_slive, sp = item - kh * at_slive;
    const int k_begin = sp * at_chunk;
    const int k_end = k_begin + at_chunk < at_ctx ? k_begin + at_chunk : at_ctx;
    const int k_stop = sp == at_slive - 1 ? k_end - 1 : k_end;
    const unsigned c = at_ctr + (unsigned)i;
    const int st = (int)(c % TK_ATT_STAGES);
    const int r0 = k_begin + i * TK_ATT_TK;
    const int rows = (k_stop - r0) < TK_ATT_TK ? (k_stop - r0) : TK_ATT_TK;
    const uint32_t bytes = (uint32_t)rows * D * 4;
    const size_t off = ((size_t)kh * P.max_ctx + r0) * D;
    mbar_expect_tx(&at_bars[st], 2 * bytes);
    bulk_load_1d(base + L.at_k + (size_t)st * AT_TILE_BYTES, Kc + off, bytes, &at_bars[st]);
    bulk_load_1d(base + L.at_v + (size_t)st * AT_TILE_BYTES, Vc + off, bytes, &at_bars[st]);
  };
  auto at_tiles_of = [&](int item) {
    const int sp = item % at_slive;
    const int k_begin = sp * at_chunk;
    const int k_end = k_begin + at_chunk < at_ctx ? k_begin + at_chunk : at_ctx;
    const int k_stop = sp == at_slive - 1 ? k_end - 1 : k_end;
    return (k_stop - k_begin + TK_ATT_TK - 1) / TK_ATT_TK;
  };
  int at_prefetched = 0;  // tiles of this CTA's first item already in flight (issued before the barrier)

  auto stamp = [&](int ph, int i) {
    if (P.dbg && blockIdx.x == 0 && tid == 0) {
      unsigned long long tt;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(tt));
      P.dbg[(size_t)ph * 4 + i] = tt;
    }
  };
  for (int ph = 0; ph < P.n_phases; ph++) {
    const TkPhase& H = P.phases[ph];
    stamp(ph, 0);
    if (H.type == 0) {
      // =========================== GEMV phase ===========================
      const int SL = H.SL, G = SL * 8, K = H.K;
      float* Pslab = (float*)(base + L.pslab);
      float* Qg = (float*)(base + L.q);
      uint4* Bfrag = (uint4*)(base + L.bfrag);
      float* red = (float*)(base + L.red);
      const float* xsrc = H.x_from_embed ? P.embed + (size_t)tok * K : H.x;
      float nrm_inv = 1.f;
      constexpr int PB = 4;
      for (int job0 = warp; job0 < SL || job0 == warp; job0 += TK_WARPS * PB) {
        float vv[PB][8], uu[PB][8];
#pragma unroll
        for (int b = 0; b < PB; b++) {
          const int sl = job0 + b * TK_WARPS;
          const int k0 = sl * 256 + lane * 8;
          const bool on = sl < SL && k0 + 8 <= K;   // K % 32 == 0 and lane*8 steps: whole or nothing
          if (on) {
            const float4 a0 = *(const float4*)(xsrc + k0), a1 = *(const float4*)(xsrc + k0 + 4);
            vv[b][0] = a0.x; vv[b][1] = a0.y; vv[b][2] = a0.z; vv[b][3] = a0.w;
            vv[b][4] = a1.x; vv[b][5] = a1.y; vv[b][6] = a1.z; vv[b][7] = a1.w;
            if (H.act != 0) {
              const float* o = H.act == 1 ? xsrc + K + k0 : H.delta + k0;
              const float4 b0 = *(const float4*)o, b1 = *(const float4*)(o + 4);
              uu[b][0] = b0.x; uu[b][1] = b0.y; uu[b][2] = b0.z; uu[b][3] = b0.w;
              uu[b][4] = b1.x; uu[b][5] = b1.y; uu[b][6] = b1.z; uu[b][7] = b1.w;
            } else {
#pragma unroll
              for (int i = 0; i < 8; i++) uu[b][i] = 0.f;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; i++) vv[b][i] = uu[b][i] = 0.f;
          }
        }
        if (job0 == warp && H.act == 2) {
          float sq = 0.f;
#pragma unroll
          for (int b = 0; b < PB; b++)
#pragma unroll
            for (int i = 0; i < 8; i++) {
              const float sv = vv[b][i] + uu[b][i];
              sq = fmaf(sv, sv, sq);
            }
          sq = warp_sum(sq);
          if (lane == 0) red[warp] = sq;
          __syncthreads();
          float tot = 0.f;
          for (int w = 0; w < TK_WARPS; w++) tot += red[w];
          nrm_inv = 1.0f / sqrtf(tot / (float)K + P.eps);
        }
#pragma unroll
        for (int b = 0; b < PB; b++) {
          const int sl = job0 + b * TK_WARPS;
          if (sl >= SL) break;
          const int k0 = sl * 256 + lane * 8;
          const bool in = k0 + 8 <= K;
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; i++) v[i] = vv[b][i];
          if (H.act == 1) {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = (v[i] / (1.0f + expf(-v[i]))) * uu[b][i];
          } else if (H.act == 2) {
            if (in) {
              const float4 w0 = *(const float4*)(H.nw + k0), w1 = *(const float4*)(H.nw + k0 + 4);
              const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
              float sv[8];
#pragma unroll
              for (int i = 0; i < 8; i++) sv[i] = v[i] + uu[b][i];
              if (blockIdx.x == 0) {
                *(float4*)(H.xout + k0) = make_float4(sv[0], sv[1], sv[2], sv[3]);
                *(float4*)(H.xout + k0 + 4) = make_float4(sv[4], sv[5], sv[6], sv[7]);
              }
#pragma unroll
              for (int i = 0; i < 8; i++) v[i] = sv[i] * nrm_inv * wv[i];
            }
          }
          float mx = 0.f;
#pragma unroll
          for (int i = 0; i < 8; i++) mx = fmaxf(mx, fabsf(v[i]));
          mx = warp_max(mx);
          int e = (int)((__float_as_uint(mx) >> 23) & 0xff) - 126;
          e = mx > 0.f ? (e < -100 ? -100 : (e > 100 ? 100 : e)) : 0;
          const float s12 = __uint_as_float((unsigned)(127 + 12 - e) << 23);
          const float s8 = __uint_as_float((unsigned)(127 + 8 - e) << 23);
          float sum = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          __half hi[8], lo[8];
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const float f = v[i] * ((i & 1) ? s8 : s12);
            hi[i] = __float2half_rn(f);
            lo[i] = __float2half_rn(f - __half2float(hi[i]));
          }
          uint4 fh, fl;
          fh.x = pack_h2(hi[0], hi[4]); fh.y = pack_h2(hi[1], hi[5]);
          fh.z = pack_h2(hi[2], hi[6]); fh.w = pack_h2(hi[3], hi[7]);
          fl.x = pack_h2(lo[0], lo[4]); fl.y = pack_h2(lo[1], lo[5]);
          fl.z = pack_h2(lo[2], lo[6]); fl.w = pack_h2(lo[3], lo[7]);
          const int j = sl * 8 + (lane >> 2), tt = lane & 3;
          Bfrag[((size_t)j * 2 + 0) * 4 + tt] = fh;
          Bfrag[((size_t)j * 2 + 1) * 4 + tt] = fl;
          if (tt == 0) Qg[j] = 8.0f * sum;
          if (lane == 0) Pslab[sl] = __uint_as_float((unsigned)(127 + 12 + e) << 23);
        }
      }
      __syncthreads();
      stamp(ph, 1);

      // ---- streaming loop over this warp's units of the phase ----
      float acc0 = 0.f, acc1 = 0.f, corr0 = 0.f, corr1 = 0.f;
      const bool use_b = g < 2;
      const unsigned g7x4 = (unsigned)(g & 7) * 4u;
      const unsigned wbase = (unsigned)g * 32u + (unsigned)t;
      auto emit = [&](int n, float v) {
        H.y[n] = v;
        if (H.argmax) {
          const unsigned long long k = tk_argmax_key(v, (unsigned)n);
          best_key = k > best_key ? k : best_key;
        }
      };
      // one unit (16 rows x 256 k, slab s) out of the ring into acc/corr
      auto compute_unit = [&](int s) -> bool {
        if (!mbar_wait_bounded(&mybar[cons_stage], cons_parity, P.status, 100 + cons_stage)) return false;
        const unsigned* Wst = (const unsigned*)(myW + cons_stage * GVU_W_BYTES);
        const float* Sst = (const float*)(myS + cons_stage * GVU_S_BYTES);
        const uint4* Bu = Bfrag + (size_t)(s * 8) * 2 * 4;
        const float4 sa0 = *(const float4*)(Sst + g * 8), sa1 = *(const float4*)(Sst + g * 8 + 4);
        const float4 sb0 = *(const float4*)(Sst + (g + 8) * 8), sb1 = *(const float4*)(Sst + (g + 8) * 8 + 4);
        const float sc0[8] = {sa0.x, sa0.y, sa0.z, sa0.w, sa1.x, sa1.y, sa1.z, sa1.w};
        const float sc1[8] = {sb0.x, sb0.y, sb0.z, sb0.w, sb1.x, sb1.y, sb1.z, sb1.w};
        float ua0 = 0.f, ua1 = 0.f;
#pragma unroll
        for (int jj = 0; jj < 8; jj++) {
          const unsigned wo = wbase + (((unsigned)jj * 4u) ^ g7x4);
          unsigned w0 = Wst[wo], w1 = Wst[wo + 256];
          const unsigned a0 = w0 & 0x000f000fu, a2 = w0 & 0x00f000f0u;
          const unsigned a1 = w1 & 0x000f000fu, a3 = w1 & 0x00f000f0u;
          w0 >>= 8;
          w1 >>= 8;
          const unsigned a4 = w0 & 0x000f000fu, a6 = w0 & 0x00f000f0u;
          const unsigned a5 = w1 & 0x000f000fu, a7 = w1 & 0x00f000f0u;
          uint4 b = make_uint4(0u, 0u, 0u, 0u);
          if (use_b) b = Bu[((size_t)jj * 2 + g) * 4 + t];
          float c[4];
          mma16816_z(c, a0, a1, a2, a3, b.x, b.y);
          mma16816(c, a4, a5, a6, a7, b.z, b.w);
          ua0 = fmaf(sc0[jj], c[0] + c[1], ua0);
          ua1 = fmaf(sc1[jj], c[2] + c[3], ua1);
        }
        {
          const float2 q = *(const float2*)(Qg + s * 8 + 2 * t);
          const float2 c0 = *(const float2*)(Sst + g * 8 + 2 * t);
          const float2 c1 = *(const float2*)(Sst + (g + 8) * 8 + 2 * t);
          corr0 = fmaf(c0.x, q.x, fmaf(c0.y, q.y, corr0));
          corr1 = fmaf(c1.x, q.x, fmaf(c1.y, q.y, corr1));
        }
        const float Pw = Pslab[s];
        acc0 = fmaf(Pw, ua0, acc0);
        acc1 = fmaf(Pw, ua1, acc1);
        __syncwarp();
        inflight--;
        if (++cons_stage == TK_STAGES) { cons_stage = 0; cons_parity ^= 1u; }
        issue_more();  // may already reach into the next projection's weights
        return true;
      };
      // value of the finished accumulators (the -8*sum(x) correction folded in)
      auto tile_value = [&](float& v0, float& v1) {
        float c0 = corr0, c1 = corr1;
        c0 += __shfl_xor_sync(0xffffffffu, c0, 1);
        c0 += __shfl_xor_sync(0xffffffffu, c0, 2);
        c1 += __shfl_xor_sync(0xffffffffu, c1, 1);
        c1 += __shfl_xor_sync(0xffffffffu, c1, 2);
        v0 = acc0 - c0;
        v1 = acc1 - c1;
        acc0 = acc1 = corr0 = corr1 = 0.f;
      };

      if (H.cta_tiles == 1) {
        // CTA-owned row tiles; the warps' K-slab partials meet in shared memory
        float* part = red;  // [TK_WARPS][16]
        for (int rt = (int)blockIdx.x; rt < H.RT; rt += (int)gridDim.x) {
          if (rt == (int)blockIdx.x) stamp(P.n_phases + ph, 0);
          if (!dead)
            for (int sl = warp; sl < SL; sl += TK_WARPS)
              if (!compute_unit(sl)) { dead = true; break; }
          if (rt == (int)blockIdx.x) stamp(P.n_phases + ph, 1);
          float v0, v1;
          tile_value(v0, v1);
          if (t == 0) { part[warp * 16 + g] = v0; part[warp * 16 + g + 8] = v1; }
          __syncthreads();
          if (rt == (int)blockIdx.x) stamp(P.n_phases + ph, 2);
          if (warp == 0 && lane < 16) {
            float sum = 0.f;
            const int nw = SL < TK_WARPS ? SL : TK_WARPS;   // warps that had a slab
            for (int w = 0; w < nw; w++) sum += part[w * 16 + lane];
            const int n = rt * 16 + lane;
            if (n < H.N) emit(n, sum);
          }
          __syncthreads();
          if (rt == (int)blockIdx.x) stamp(P.n_phases + ph, 3);
        }
      } else if (wid < H.Wtot && !dead) {
        const GvSplit sp = {H.q, H.r};
        const unsigned u0 = gv_start(wid, sp), u1 = gv_start(wid + 1, sp);
        const int n_units = (int)(u1 - u0);
        auto flush = [&](int rt) {
          float v0, v1;
          tile_value(v0, v1);
          const unsigned t0 = (unsigned)rt * SL, t1 = t0 + SL;
          const bool complete = (u0 <= t0) && (u1 >= t1);
          const int r0 = rt * 16;
          if (complete) {
            if (t == 0) {
              if (r0 + g < H.N) emit(r0 + g, v0);
              if (r0 + g + 8 < H.N) emit(r0 + g + 8, v1);
            }
            return;
          }
          const int slot = (u0 >= t0) ? 0 : 1;
          float* mine = P.gemv_partials + ((size_t)wid * 2 + slot) * 128;
          if (t == 0) {
            __stcg(&mine[g], v0);
            __stcg(&mine[g + 8], v1);
          }
          __syncwarp();
          const unsigned wf = gv_owner(t0, sp), wl = gv_owner(t1 - 1, sp);
          int old = 0;
          if (lane == 0) old = (int)atom_add_acq_rel(&P.gemv_counters[rt], 1);
          old = __shfl_sync(0xffffffffu, old, 0);
          if (old != (int)(wl - wf)) return;
          float s0 = 0.f, s1 = 0.f;
          for (unsigned w = wf; w <= wl; w += 4) {
            float a[4], b[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
              const unsigned ww = w + k;
              const bool on = ww <= wl;
              const unsigned wc = on ? ww : wl;
              const int sl2 = (gv_start(wc, sp) >= t0) ? 0 : 1;
              const float* src = P.gemv_partials + ((size_t)wc * 2 + sl2) * 128;
              a[k] = on ? __ldcg(&src[g]) : 0.f;
              b[k] = on ? __ldcg(&src[g + 8]) : 0.f;
            }
#pragma unroll
            for (int k = 0; k < 4; k++) { s0 += a[k]; s1 += b[k]; }
          }
          if (t == 0) {
            if (r0 + g < H.N) emit(r0 + g, s0);
            if (r0 + g + 8 < H.N) emit(r0 + g + 8, s1);
          }
          if (lane == 0) P.gemv_counters[rt] = 0;
        };
        int rt = (int)(u0 / (unsigned)SL), s = (int)(u0 - (unsigned)rt * SL);
        for (int i = 0; i < n_units; i++) {
          if (!compute_unit(s)) { dead = true; break; }
          if (++s == SL) {
            flush(rt);
            s = 0;
            rt++;
          }
        }
        if (!dead && n_units > 0 && s != 0) flush(rt);
      }
      // The cached K/V rows are as static as the weights: start the next attention
      // phase's first tiles now, so they cross HBM while the grid barrier is pending.
      if (ph + 1 < P.n_phases && P.phases[ph + 1].type == 1 && (int)blockIdx.x < P.n_kv * at_slive) {
        const int nt = at_tiles_of((int)blockIdx.x);
        at_prefetched = nt < TK_ATT_STAGES ? nt : TK_ATT_STAGES;
        if (tid == 0)
          for (int i = 0; i < at_prefetched; i++)
            at_issue(P.phases[ph + 1].Kc, P.phases[ph + 1].Vc, (int)blockIdx.x, i);
      }
      if (H.argmax) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const unsigned long long other = __shfl_xor_sync(0xffffffffu, best_key, o);
          best_key = other > best_key ? other : best_key;
        }
        if (lane == 0 && best_key) atomicMax(P.argmax_cell, best_key);
      }
    } else if (H.type == 1) {
      // =========================== attention phase ===========================
      // qkv holds the fused projection of this token.  Per (kv head, context split)
      // item: rope+bias the group's q heads into shared memory, the split that owns
      // the new position also ropes k, biases v, appends both to the cache and scores
      // them from shared memory; the cached prefix streams through bulk-copy tiles.
      constexpr int CH = D / 32;
      const int ctx = at_ctx, chunk = at_chunk, s_live = at_slive;
      const long long kv_stride = (long long)P.max_ctx * D;
      int hs = (grp + TK_HW - 1) / TK_HW;
      while (TK_WARPS % hs) hs++;
      const int ks = TK_WARPS / hs, hslot = warp % hs, kslice = warp / hs;
      const int nheads_pad = hs * TK_HW;
      const int kslot = lane >> 3, sub = lane & 7;
      float* Kt = (float*)(base + L.at_k);
      float* Vt = (float*)(base + L.at_v);
      float* qs = (float*)(base + L.at_q);
      float* newkv = (float*)(base + L.at_new);
      float* mrg = (float*)(base + L.at_mrg);
      constexpr int TILE_BYTES = AT_TILE_BYTES;

      for (int item = blockIdx.x; item < P.n_kv * s_live; item += gridDim.x) {
        const int kh = item / s_live, sp = item - kh * s_live;
        const int k_begin = sp * chunk;
        const int k_end = k_begin + chunk < ctx ? k_begin + chunk : ctx;
        const bool last = sp == s_live - 1;           // owns row `pos`
        const int k_stop = last ? k_end - 1 : k_end;  // rows streamed from the cache
        const int n_tiles = (k_stop - k_begin + TK_ATT_TK - 1) / TK_ATT_TK;
        const float* Kh = H.Kc + (size_t)kh * kv_stride;
        const float* Vh = H.Vc + (size_t)kh * kv_stride;
        auto issue_tile = [&](int i) { at_issue(H.Kc, H.Vc, item, i); };
        if (tid == 0) {
          const int pre = n_tiles < TK_ATT_STAGES ? n_tiles : TK_ATT_STAGES;
          for (int i = (item == (int)blockIdx.x ? at_prefetched : 0); i < pre; i++) issue_tile(i);
        }
        if (item == (int)blockIdx.x) at_prefetched = 0;
        // rope(q + bq) for the group's heads (double angle, as rope_kernel)
        constexpr int half = D / 2;
        for (int idx = tid; idx < grp * half; idx += TK_THREADS) {
          const int hh = idx / half, j = idx - hh * half;
          const int qh = kh * grp + hh;
          const float c = rope_cs[j], sn = rope_cs[half + j];
          float x0 = H.qkv[(size_t)qh * D + j], x1 = H.qkv[(size_t)qh * D + j + half];
          if (H.bq) { x0 += H.bq[qh * D + j]; x1 += H.bq[qh * D + j + half]; }
          qs[hh * D + j] = x0 * c - x1 * sn;
          qs[hh * D + j + half] = x0 * sn + x1 * c;
        }
        if (last) {
          const float* ksrc = H.qkv + (size_t)(P.n_q + kh) * D;
          const float* vsrc = H.qkv + (size_t)(P.n_q + P.n_kv + kh) * D;
          float* kdst = H.Kc + (size_t)kh * kv_stride + (size_t)pos * D;
          float* vdst = H.Vc + (size_t)kh * kv_stride + (size_t)pos * D;
          for (int j = tid; j < half; j += TK_THREADS) {
            const float c = rope_cs[j], sn = rope_cs[half + j];
            float x0 = ksrc[j], x1 = ksrc[j + half];
            if (H.bk) { x0 += H.bk[kh * D + j]; x1 += H.bk[kh * D + j + half]; }
            const float r0 = x0 * c - x1 * sn, r1 = x0 * sn + x1 * c;
            newkv[j] = r0; newkv[j + half] = r1;
            kdst[j] = r0; kdst[j + half] = r1;
          }
          for (int j = tid; j < D; j += TK_THREADS) {
            float v = vsrc[j];
            if (H.bv) v += H.bv[kh * D + j];
            newkv[D + j] = v;
            vdst[j] = v;
          }
        }
        __syncthreads();
        stamp(P.n_phases + ph, 0);

        float4 qf[TK_HW][CH];
#pragma unroll
        for (int h = 0; h < TK_HW; h++) {
          const int hh = hslot * TK_HW + h;
          const float4* qp = (const float4*)(qs + (hh < grp ? hh : 0) * D);
#pragma unroll
          for (int i = 0; i < CH; i++)
            qf[h][i] = hh < grp ? qp[sub + 8 * i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float m[TK_HW], l[TK_HW];
        float4 acc[TK_HW][CH];
#pragma unroll
        for (int h = 0; h < TK_HW; h++) {
          m[h] = -INFINITY;
          l[h] = 0.f;
#pragma unroll
          for (int i = 0; i < CH; i++) acc[h][i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        // one key row for this lane group: scores for the warp's heads, online softmax
        auto row_step = [&](const float4* Krow, const float4* Vrow, bool valid) {
          float4 kv[CH];
#pragma unroll
          for (int i = 0; i < CH; i++) kv[i] = Krow[sub + 8 * i];
          float sc[TK_HW];
#pragma unroll
          for (int h = 0; h < TK_HW; h++) {
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < CH; i++) {
              d = fmaf(qf[h][i].x, kv[i].x, d);
              d = fmaf(qf[h][i].y, kv[i].y, d);
              d = fmaf(qf[h][i].z, kv[i].z, d);
              d = fmaf(qf[h][i].w, kv[i].w, d);
            }
            d += __shfl_xor_sync(0xffffffffu, d, 1);
            d += __shfl_xor_sync(0xffffffffu, d, 2);
            d += __shfl_xor_sync(0xffffffffu, d, 4);
            sc[h] = d * P.scale;
          }
#pragma unroll
          for (int i = 0; i < CH; i++) kv[i] = Vrow[sub + 8 * i];
          if (valid) {
#pragma unroll
            for (int h = 0; h < TK_HW; h++) {
              if (sc[h] > m[h]) {
                const float corr = __expf(m[h] - sc[h]);
                l[h] *= corr;
#pragma unroll
                for (int i = 0; i < CH; i++) {
                  acc[h][i].x *= corr; acc[h][i].y *= corr;
                  acc[h][i].z *= corr; acc[h][i].w *= corr;
                }
                m[h] = sc[h];
              }
              const float pr = __expf(sc[h] - m[h]);
              l[h] += pr;
#pragma unroll
              for (int i = 0; i < CH; i++) {
                acc[h][i].x = fmaf(pr, kv[i].x, acc[h][i].x);
                acc[h][i].y = fmaf(pr, kv[i].y, acc[h][i].y);
                acc[h][i].z = fmaf(pr, kv[i].z, acc[h][i].z);
                acc[h][i].w = fmaf(pr, kv[i].w, acc[h][i].w);
              }
            }
          }
        };
        for (int it = 0; it < n_tiles; it++) {
          const unsigned c = at_ctr + (unsigned)it;
          const int st = (int)(c % TK_ATT_STAGES);
          if (!dead && !mbar_wait_bounded(&at_bars[st], (c / TK_ATT_STAGES) & 1u, P.status, 200 + st)) dead = true;
          const int r0 = k_begin + it * TK_ATT_TK;
          const int rows = (k_stop - r0) < TK_ATT_TK ? (k_stop - r0) : TK_ATT_TK;
          const float4* Ks = (const float4*)((unsigned char*)Kt + (size_t)st * TILE_BYTES);
          const float4* Vs = (const float4*)((unsigned char*)Vt + (size_t)st * TILE_BYTES);
          if (!dead) {
            for (int step = kslice; step < TK_ATT_TK / 4; step += ks) {
              if (step * 4 >= rows) break;
              const int row = step * 4 + kslot;
              const bool valid = row < rows;
              const int rr = valid ? row : 0;
              row_step(Ks + rr * (D / 4), Vs + rr * (D / 4), valid);
            }
          }
          __syncthreads();
          if (tid == 0 && it + TK_ATT_STAGES < n_tiles) issue_tile(it + TK_ATT_STAGES);
        }
        at_ctr += (unsigned)n_tiles;
        stamp(P.n_phases + ph, 1);
        if (last && kslice == 0)  // the new token's own key/value, from shared memory
          row_step((const float4*)newkv, (const float4*)(newkv + D), kslot == 0);

        // ---- merge the 4 key slots of the warp (lanes xor 8, 16), fixed order ----
#pragma unroll
        for (int h = 0; h < TK_HW; h++) {
#pragma unroll
          for (int o = 8; o <= 16; o <<= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[h], o);
            const float lo = __shfl_xor_sync(0xffffffffu, l[h], o);
            const float mn = fmaxf(m[h], mo);
            const bool low = (lane & o) == 0;
            const float ma = low ? m[h] : mo, mb = low ? mo : m[h];
            const float la = low ? l[h] : lo, lb = low ? lo : l[h];
            const float ca = (ma == -INFINITY) ? 0.f : __expf(ma - mn);
            const float cb = (mb == -INFINITY) ? 0.f : __expf(mb - mn);
            l[h] = la * ca + lb * cb;
#pragma unroll
            for (int i = 0; i < CH; i++) {
              float4 ao;
              ao.x = __shfl_xor_sync(0xffffffffu, acc[h][i].x, o);
              ao.y = __shfl_xor_sync(0xffffffffu, acc[h][i].y, o);
              ao.z = __shfl_xor_sync(0xffffffffu, acc[h][i].z, o);
              ao.w = __shfl_xor_sync(0xffffffffu, acc[h][i].w, o);
              const float4 a = low ? acc[h][i] : ao, b = low ? ao : acc[h][i];
              acc[h][i].x = a.x * ca + b.x * cb;
              acc[h][i].y = a.y * ca + b.y * cb;
              acc[h][i].z = a.z * ca + b.z * cb;
              acc[h][i].w = a.w * ca + b.w * cb;
            }
            m[h] = mn;
          }
        }
        if (kslot == 0) {
#pragma unroll
          for (int h = 0; h < TK_HW; h++) {
            float* dst = mrg + ((size_t)kslice * nheads_pad + hslot * TK_HW + h) * (D + 4);
            if (sub == 0) { dst[D] = m[h]; dst[D + 1] = l[h]; }
#pragma unroll
            for (int i = 0; i < CH; i++) *(float4*)(dst + (sub + 8 * i) * 4) = acc[h][i];
          }
        }
        __syncthreads();
        // ---- CTA merge over key slices -> output (one split) or a split partial ----
        const bool single = s_live == 1;
        for (int idx = tid; idx < grp * D; idx += TK_THREADS) {
          const int hh = idx / D, d = idx - hh * D;
          float mm = -INFINITY;
          for (int k2 = 0; k2 < ks; k2++) mm = fmaxf(mm, mrg[((size_t)k2 * nheads_pad + hh) * (D + 4) + D]);
          float ll = 0.f, aa = 0.f;
          for (int k2 = 0; k2 < ks; k2++) {
            const float* src = mrg + ((size_t)k2 * nheads_pad + hh) * (D + 4);
            const float c = (src[D] == -INFINITY) ? 0.f : __expf(src[D] - mm);
            ll += src[D + 1] * c;
            aa += src[d] * c;
          }
          const int qh = kh * grp + hh;
          if (single) {
            H.att[(size_t)qh * D + d] = aa / ll;
          } else {
            float* dst = P.attn_partials + ((size_t)qh * P.attn_s_cap + sp) * (D + 4);
            if (d == 0) { __stcg(&dst[D], mm); __stcg(&dst[D + 1], ll); }
            __stcg(&dst[d], aa);
          }
        }
        stamp(P.n_phases + ph, 2);
        if (!single) {
          __threadfence();
          __syncthreads();
          if (tid == 0) is_last_s = atomicAdd(&P.attn_counters[kh], 1) == s_live - 1;
          __syncthreads();
          if (is_last_s) {
            __threadfence();
            float* cw = Kt;
            float* lden = Kt + grp * s_live;
            for (int hh = warp; hh < grp; hh += TK_WARPS) {
              const int qh = kh * grp + hh;
              const float* src0 = P.attn_partials + (size_t)qh * P.attn_s_cap * (D + 4) + D;
              float2 ml[3];
#pragma unroll
              for (int k2 = 0; k2 < 3; k2++) {
                const int s2 = lane + 32 * k2;
                ml[k2] = s2 < s_live ? __ldcg((const float2*)(src0 + (size_t)s2 * (D + 4)))
                                     : make_float2(-INFINITY, 0.f);
              }
              const float mm = warp_max(fmaxf(ml[0].x, fmaxf(ml[1].x, ml[2].x)));
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
            for (int idx = tid; idx < grp * (D / 4); idx += TK_THREADS) {
              const int hh = idx / (D / 4), d4 = idx - hh * (D / 4);
              const int qh = kh * grp + hh;
              const float* src0 = P.attn_partials + (size_t)qh * P.attn_s_cap * (D + 4) + d4 * 4;
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
              const float den = lden[hh];
              *(float4*)(H.att + (size_t)qh * D + d4 * 4) =
                  make_float4(aa.x / den, aa.y / den, aa.z / den, aa.w / den);
            }
            if (tid == 0) P.attn_counters[kh] = 0;
          }
        }
        __syncthreads();  // shared memory of this item is free again
        stamp(P.n_phases + ph, 3);
      }
    }
    stamp(ph, 2);
    tk_grid_barrier(P.bar, gen, P.status);
    stamp(ph, 3);
  }

  // ---- the token: argmax of the last projection, position + 1 ----
  if (blockIdx.x == 0 && tid == 0) {
    const unsigned long long k = atomicExch(P.argmax_cell, 0ull);
    const int idx = (int)(0xFFFFFFFFu - (unsigned)(k & 0xFFFFFFFFull));
    *P.d_tok = idx;
    *P.d_tok_out = idx;
    *P.d_pos = pos + 1u;
  }
}

// ---------------------------------------------------------------------------
// host side: one cooperative launch of one CTA per SM
// ---------------------------------------------------------------------------
int token_kernel_launch(const TkParams& P, int D, int k_max, int k_attn_in, int sm_count,
                        cudaStream_t stream) {
  const int grp = P.n_q / P.n_kv;
  const size_t smem = tk_smem_layout(k_max, k_attn_in, D, grp).total;
  if (smem > 227 * 1024 - 512)  // the kernel also has a few static shared words
    return set_error(TLB_ERR_UNSUPPORTED, "token kernel: shared memory need exceeds 227 KB");
  void* fn = D == 128 ? (void*)token_kernel<128> : (void*)token_kernel<64>;
  static size_t attr[2] = {0, 0};
  if (attr[D == 128] < smem) {
    TLB_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr[D == 128] = smem;
  }
  TkParams p = P;
  void* args[] = {&p};
  TLB_CUDA(cudaLaunchCooperativeKernel(fn, dim3(sm_count), dim3(TK_THREADS), args, smem, stream));
  return TLB_OK;
}

}  // namespace tlb
