// int4 dequant-matmul for skinny activations (M = 1 .. 8 rows): the decode GEMV
// and the small batched-rows GEMM.  y[m,n] = alpha * sum_k x[m,k] * sc[n,k/32] *
// (nib[n,k]-8) + beta, on the q4 storage layout of the reference
// (include/types.h:15-31: packed nibbles [N][K/2] then f32 scales [N][K/32]).
// Replaces tl_gemv_q4 (kernels/tensorlib_cuda.cu:772-796) and, for M > 1, the
// host-dequant + tl_sgemm_rb route (include/array.h:1980-1984, 1546-1569).
//
// Design (HBM-bound, 0.625 byte per weight):
//  * Work unit = 16 weight rows x 256 k (2 KB of nibbles + 512 B of scales).
//    Units are numbered row-tile-major and dealt out in equal contiguous ranges
//    to every warp of a persistent grid, so the load balance does not depend on
//    the matrix shape.  Each warp owns a private ring of TMA stages
//    (cp.async.bulk.tensor, 128-byte swizzle) with one mbarrier per stage: no
//    block-wide barrier sits in the streaming loop and ~100 KB per SM stay in
//    flight.
//  * The nibbles never become f32 on the CUDA cores (that costs > 4 lane
//    instructions per weight; the budget at full HBM speed is ~3.3).  A masked
//    32-bit word is read directly as two fp16 SUBNORMALS (value nib * 2^-24, or
//    nib * 2^-20 for the odd nibble of a byte) and fed to mma.sync m16n8k16 as
//    the A operand; the activation row is the B operand, split exactly into
//    fp16 hi + lo parts (two columns) after a power-of-two normalisation, with
//    the 2^12 / 2^8 factors that cancel the nibble scalings folded in.  fp32
//    accumulation, so the result carries ~22 bits of the activation and all
//    bits of the weights.  Per group of 32 k the -8 offset and the f32 group
//    scale are applied to the accumulator: acc += sc * (P * c - 8 * sum(x_g)).
//  * Split-K falls out of the unit ranges; partial row tiles are combined by the
//    last-arriving warp in a fixed order (deterministic, no float atomics, no
//    spin-wait on another CTA).
#include <cstdlib>
#include <cstring>

#include "comm.cuh"
#include "q4_mma.cuh"

namespace tlb {

constexpr int GV_W_BYTES = 2048;  // 16 rows x 128 B
constexpr int GV_S_BYTES = 512;   // 16 rows x 8 f32
constexpr int GV_MAXM = 8;

struct GemvParams {
  const float* x;
  long long ldx;
  float* y;
  long long ldy;
  int M, N, K;
  float alpha, beta;
  float* partials;  // [workers][2][16*8]
  int* counters;    // [row tiles]
  int* status;
  int RT, SL;       // row tiles (16 rows), k slabs (256 k)
  unsigned U;       // RT * SL
  int x_vec_ok;     // x rows are 16-byte aligned
  int act;          // 0: x as given; 1: x row = [gate(K) | up(K)], activation silu(gate)*up;
                    // 2: x = rmsnorm(x + delta) * nw (M == 1), the sum also written to xout
  const float* delta;
  const float* nw;
  float* xout;
  float eps;
  unsigned long long* dbg;  // optional phase timestamps (diagnostics), [grid][8]
  int push;         // tensor-parallel: store y (M == 1) into every rank's staging slot
  CommDev comm;
};

// Shared-memory carve-up (host and device agree through this one function).
struct GemvSmem {
  size_t w_ring, s_ring, bars, red, pslab, q, bfrag, total;
};
__host__ __device__ inline GemvSmem gemv_smem_layout(int warps, int stages, int M, int K) {
  const int SL = (K + 255) / 256, G = SL * 8;
  GemvSmem L;
  size_t o = 0;
  L.w_ring = o; o += (size_t)warps * stages * GV_W_BYTES;
  L.s_ring = o; o += (size_t)warps * stages * GV_S_BYTES;
  L.bars = o;   o += (size_t)warps * stages * 8;
  o = (o + 15) & ~(size_t)15;
  L.red = o;    o += 64 * sizeof(float);
  L.pslab = o;  o += (size_t)GV_MAXM * SL * sizeof(float);
  o = (o + 15) & ~(size_t)15;
  L.q = o;      o += (size_t)GV_MAXM * G * sizeof(float);
  o = (o + 15) & ~(size_t)15;
  L.bfrag = o;  o += (size_t)G * (2 * M) * 4 * sizeof(uint4);
  L.total = o + 1024;  // slack for the 1 KB alignment of the dynamic base
  return L;
}

// WARPS x STAGES: 8 x 4 (two CTAs per SM, for K up to ~6K) or 16 x 3 (one CTA per
// SM, large K whose activation fragments need more shared memory).  Either way
// 16 warps per SM hide the fixed latencies of the LDS -> LOP -> MMA -> FMA chain.
template <int NT, int WARPS, int STAGES, bool M1>
__global__ void __launch_bounds__(WARPS * 32, (WARPS == 8 ? 2 : 1))
    gemv_q4_mma_kernel(const __grid_constant__ CUtensorMap tmW,
                       const __grid_constant__ CUtensorMap tmS, GemvParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base =
      (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int SL = p.SL, G = SL * 8;
  const int NCU = 2 * p.M;
  const GemvSmem L = gemv_smem_layout(WARPS, STAGES, p.M, p.K);
  auto stamp = [&](int i) {
    if (p.dbg && tid == 0) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
      p.dbg[(size_t)blockIdx.x * 8 + i] = t;
    }
  };
  stamp(0);

  uint64_t* bars = (uint64_t*)(base + L.bars);
  float* Pslab = (float*)(base + L.pslab);   // [m][SL]   2^(12+e) of the slab
  float* Qg = (float*)(base + L.q);          // [m][G]    8 * sum of the group's activations
  uint4* Bfrag = (uint4*)(base + L.bfrag);   // [G][2M][4]

  unsigned char* myW = base + L.w_ring + (size_t)warp * STAGES * GV_W_BYTES;
  unsigned char* myS = base + L.s_ring + (size_t)warp * STAGES * GV_S_BYTES;
  uint64_t* mybar = bars + warp * STAGES;

  // Never more workers than units, so every worker's range is non-empty and the
  // contributors of a row tile are exactly the owners of its first..last unit.
  const unsigned Wall = gridDim.x * WARPS;
  const unsigned Wtot = Wall < p.U ? Wall : p.U;
  const unsigned wid = blockIdx.x * WARPS + warp;
  const bool idle = wid >= Wtot;
  const GvSplit sp = {p.U / Wtot, p.U % Wtot};
  const unsigned u0 = idle ? 0u : gv_start(wid, sp);
  const unsigned u1 = idle ? 0u : gv_start(wid + 1, sp);
  const int n_units = (int)(u1 - u0);

  if (lane == 0) {
    for (int s = 0; s < STAGES; s++) mbar_init(&mybar[s], 1);
    mbar_fence_init();
  }
  __syncwarp();

  // producer cursor (lane 0 issues; every lane tracks it, no divisions in the loop)
  int irt = (int)(u0 / (unsigned)SL), is = (int)(u0 - (unsigned)irt * SL), istage = 0;
  auto issue_next = [&]() {
    if (lane == 0) {
      mbar_expect_tx(&mybar[istage], GV_W_BYTES + GV_S_BYTES);
      tma_load_2d(myW + istage * GV_W_BYTES, &tmW, is * 32, irt * 16, &mybar[istage]);
      tma_load_2d(myS + istage * GV_S_BYTES, &tmS, is * 8, irt * 16, &mybar[istage]);
    }
    if (++is == SL) { is = 0; irt++; }
    if (++istage == STAGES) istage = 0;
  };
  // Weights do not depend on the previous kernel: the first stage streams before the
  // wait.  The other stages are issued right AFTER the activation loads below, so
  // those small loads are not queued behind ~100 KB of weight traffic per SM.
  const int pre_total = n_units < STAGES ? n_units : STAGES;
  if (pre_total > 0) issue_next();

  pdl_wait();  // activations and the fix-up scratch are valid from here
  stamp(1);

  // ---- activation prep.  One warp per (row m, slab of 256 k): power-of-two
  // normalisation by the slab's max (no block-wide reduction), exact fp16 hi/lo
  // split, B-fragment order.  Lane l covers x[m][256*slab + 8*l .. +8) = group
  // jj = l/4, quad slot tt = l%4.
  float nrm_inv = 1.f;
  // Jobs are taken four at a time: all global loads of a batch are issued before any
  // of it is processed, so a warp pays the load latency once per batch, not per job.
  constexpr int PB = 4;
  const int n_jobs = p.M * SL;
  // (the first pass runs in every warp, also one without jobs: it issues the rest of
  // the warp's weight ring and takes part in the block reduction of the fused norm)
  for (int job0 = warp; job0 < n_jobs || job0 == warp; job0 += WARPS * PB) {
    float vv[PB][8], uu[PB][8];
#pragma unroll
    for (int b = 0; b < PB; b++) {
      const int job = job0 + b * WARPS;
      const bool on = job < n_jobs;
      const int m = on ? job / SL : 0, sl = on ? job - m * SL : 0;
      const int k0 = sl * 256 + lane * 8;
      const float* xr = p.x + (long long)m * p.ldx + k0;
      auto load8 = [&](const float* src, float (&o)[8]) {
        if (on && k0 + 8 <= p.K) {
          if (p.x_vec_ok) {
            const float4 q0 = *(const float4*)src, q1 = *(const float4*)(src + 4);
            o[0] = q0.x; o[1] = q0.y; o[2] = q0.z; o[3] = q0.w;
            o[4] = q1.x; o[5] = q1.y; o[6] = q1.z; o[7] = q1.w;
          } else {
#pragma unroll
            for (int i = 0; i < 8; i++) o[i] = src[i];
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; i++) o[i] = (on && k0 + i < p.K) ? src[i] : 0.f;
        }
      };
      load8(xr, vv[b]);
      if (p.act == 1) load8(xr + p.K, uu[b]);
      if (p.act == 2) load8(p.delta + k0, uu[b]);
    }
    if (job0 == warp) {
      // first batch: its loads are in flight, now queue the rest of the weight ring
      for (int i = 1; i < pre_total; i++) issue_next();
      stamp(6);
      if (p.act == 2) {
        // fused residual add + RMSNorm (tl_add_rmsnorm, kernels/tensorlib_cuda.cu:155-179):
        // every CTA reduces sum((x+delta)^2) itself from the values it just loaded, in
        // the same order everywhere, so all CTAs agree on the scale.  (The host only
        // selects this mode when one batch covers the row.)
        float* red = (float*)(base + L.red);
        float sq = 0.f;
#pragma unroll
        for (int b = 0; b < PB; b++)
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const float sv = vv[b][i] + uu[b][i];   // zero where the job or k is out of range
            sq = fmaf(sv, sv, sq);
          }
        sq = warp_sum(sq);
        if (lane == 0) red[warp] = sq;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < WARPS; w++) tot += red[w];
        nrm_inv = 1.0f / sqrtf(tot / (float)p.K + p.eps);
      }
    }
#pragma unroll
    for (int b = 0; b < PB; b++) {
      const int job = job0 + b * WARPS;
      if (job >= n_jobs) break;  // warp-uniform
      const int m = job / SL, sl = job - m * SL;
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] = vv[b][i];
      if (p.act == 1) {
        // fused SwiGLU (kernels/tensorlib_cuda.cu:185-192 of the reference): the row
        // holds gate then up; same expression g / (1 + exp(-g)) * u
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = (v[i] / (1.0f + expf(-v[i]))) * uu[b][i];
      }
      if (p.act == 2) {
        const int k0 = sl * 256 + lane * 8;
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float sv = v[i] + uu[b][i];
          const bool in = k0 + i < p.K;
          if (in && blockIdx.x == 0) p.xout[k0 + i] = sv;
          v[i] = in ? sv * nrm_inv * p.nw[k0 + i] : 0.f;
        }
      }
      float mx = 0.f;
#pragma unroll
      for (int i = 0; i < 8; i++) mx = fmaxf(mx, fabsf(v[i]));
      mx = warp_max(mx);
      int e = (int)((__float_as_uint(mx) >> 23) & 0xff) - 126;  // mx < 2^e
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
      Bfrag[((size_t)j * NCU + 2 * m) * 4 + tt] = fh;
      Bfrag[((size_t)j * NCU + 2 * m + 1) * 4 + tt] = fl;
      if (tt == 0) Qg[(size_t)m * G + j] = 8.0f * sum;
      if (lane == 0) Pslab[m * SL + sl] = __uint_as_float((unsigned)(127 + 12 + e) << 23);
    }
  }
  stamp(7);
  __syncthreads();
  pdl_launch_dependents();
  stamp(2);

  // ---- streaming loop ------------------------------------------------------
  float acc[NT][2], corr[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = corr[nt][0] = corr[nt][1] = 0.f;
  bool use_b[NT];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) use_b[nt] = (8 * nt + g) < NCU;
  const unsigned g7x4 = (unsigned)(g & 7) * 4u;
  const unsigned wbase = (unsigned)g * 32u + (unsigned)t;

  unsigned ar_seq = 0;
  if (p.push) ar_seq = comm_seq(p.comm);
  const size_t ar_off =
      ((size_t)(ar_seq & 1u) * p.comm.size + p.comm.rank) * (size_t)p.comm.slot_floats;
  auto emit = [&](int m, int n, float v) {
    v = v * p.alpha + p.beta;
    if (p.push) {
      for (int r = 0; r < p.comm.size; r++) st_packet_sys(&p.comm.stage[r][ar_off + n], v, ar_seq + 1u);
    } else {
      p.y[(long long)m * p.ldy + n] = v;
    }
  };
  auto flush = [&](int rt) {
    // fold the -8*sum(x_g) correction in; on the M == 1 path it is spread over the
    // four lanes of a quad and summed here
    float val[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
#pragma unroll
      for (int r = 0; r < 2; r++) {
        float cr = corr[nt][r];
        if (M1) {
          cr += __shfl_xor_sync(0xffffffffu, cr, 1);
          cr += __shfl_xor_sync(0xffffffffu, cr, 2);
        }
        val[nt][r] = acc[nt][r] - cr;
      }
    }
    const unsigned t0 = (unsigned)rt * SL, t1 = t0 + SL;
    const bool complete = (u0 <= t0) && (u1 >= t1);
    const int r0 = rt * 16;
    if (complete) {
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        const int m = 4 * nt + t;
        if (m < p.M) {
          if (r0 + g < p.N) emit(m, r0 + g, val[nt][0]);
          if (r0 + g + 8 < p.N) emit(m, r0 + g + 8, val[nt][1]);
        }
      }
      return;
    }
    // partial: slot 0 when this tile holds the worker's first unit, else slot 1
    const int slot = (u0 >= t0) ? 0 : 1;
    float* mine = p.partials + ((size_t)wid * 2 + slot) * 128;
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      const int m = 4 * nt + t;
      __stcg(&mine[m * 16 + g], val[nt][0]);
      __stcg(&mine[m * 16 + g + 8], val[nt][1]);
    }
    __syncwarp();
    const unsigned wf = gv_owner(t0, sp), wl = gv_owner(t1 - 1, sp);
    int old = 0;
    if (lane == 0) old = (int)atom_add_acq_rel(&p.counters[rt], 1);  // releases the warp's stores
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old != (int)(wl - wf)) return;  // not the last contributor
    // Last contributor: fold the partials in worker order.  Loads are issued four
    // workers at a time before any add so their latencies overlap.
    float sum[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) sum[nt][0] = sum[nt][1] = 0.f;
    for (unsigned w = wf; w <= wl; w += 4) {
      float v[4][NT][2];
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const unsigned ww = w + k;
        const bool on = ww <= wl;
        const int sl = (gv_start(on ? ww : wl, sp) >= t0) ? 0 : 1;  // started inside this tile
        const float* src = p.partials + ((size_t)(on ? ww : wl) * 2 + sl) * 128;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          const int m = 4 * nt + t;
          v[k][nt][0] = on ? __ldcg(&src[m * 16 + g]) : 0.f;
          v[k][nt][1] = on ? __ldcg(&src[m * 16 + g + 8]) : 0.f;
        }
      }
#pragma unroll
      for (int k = 0; k < 4; k++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          sum[nt][0] += v[k][nt][0];
          sum[nt][1] += v[k][nt][1];
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      const int m = 4 * nt + t;
      if (m < p.M) {
        if (r0 + g < p.N) emit(m, r0 + g, sum[nt][0]);
        if (r0 + g + 8 < p.N) emit(m, r0 + g + 8, sum[nt][1]);
      }
    }
    if (lane == 0) p.counters[rt] = 0;  // leave the counter clean for the next launch
  };

  int rt = (int)(u0 / (unsigned)SL), s = (int)(u0 - (unsigned)rt * SL);
  int st = 0;
  unsigned phase = 0;
  for (int i = 0; i < n_units; i++) {
    if (!mbar_wait_bounded(&mybar[st], phase, p.status, 100 + st)) return;
    if (i == 0) stamp(3);
    const unsigned* Wst = (const unsigned*)(myW + st * GV_W_BYTES);
    const float* Sst = (const float*)(myS + st * GV_S_BYTES);
    const uint4* Bu = Bfrag + (size_t)(s * 8) * NCU * 4;
    // the 8 group scales of rows g and g+8
    const float4 sa0 = *(const float4*)(Sst + g * 8), sa1 = *(const float4*)(Sst + g * 8 + 4);
    const float4 sb0 = *(const float4*)(Sst + (g + 8) * 8), sb1 = *(const float4*)(Sst + (g + 8) * 8 + 4);
    const float sc0[8] = {sa0.x, sa0.y, sa0.z, sa0.w, sa1.x, sa1.y, sa1.z, sa1.w};
    const float sc1[8] = {sb0.x, sb0.y, sb0.z, sb0.w, sb1.x, sb1.y, sb1.z, sb1.w};
    float ua[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) ua[nt][0] = ua[nt][1] = 0.f;
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
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        uint4 b = make_uint4(0u, 0u, 0u, 0u);
        if (use_b[nt]) b = Bu[((size_t)jj * NCU + 8 * nt + g) * 4 + t];
        float c[4];
        mma16816_z(c, a0, a1, a2, a3, b.x, b.y);
        mma16816(c, a4, a5, a6, a7, b.z, b.w);
        ua[nt][0] = fmaf(sc0[jj], c[0] + c[1], ua[nt][0]);
        ua[nt][1] = fmaf(sc1[jj], c[2] + c[3], ua[nt][1]);
        if (!M1) {
          const float q = Qg[(size_t)(4 * nt + t) * G + s * 8 + jj];
          corr[nt][0] = fmaf(sc0[jj], q, corr[nt][0]);
          corr[nt][1] = fmaf(sc1[jj], q, corr[nt][1]);
        }
      }
    }
    if (M1) {
      // lane t of the quad handles groups 2t, 2t+1 of the correction term
      const float2 q = *(const float2*)(Qg + s * 8 + 2 * t);
      const float2 c0 = *(const float2*)(Sst + g * 8 + 2 * t);
      const float2 c1 = *(const float2*)(Sst + (g + 8) * 8 + 2 * t);
      corr[0][0] = fmaf(c0.x, q.x, fmaf(c0.y, q.y, corr[0][0]));
      corr[0][1] = fmaf(c1.x, q.x, fmaf(c1.y, q.y, corr[0][1]));
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      const int m = M1 ? 0 : 4 * nt + t;
      const float P = Pslab[m * SL + s];
      acc[nt][0] = fmaf(P, ua[nt][0], acc[nt][0]);
      acc[nt][1] = fmaf(P, ua[nt][1], acc[nt][1]);
    }
    __syncwarp();
    if (i + STAGES < n_units) issue_next();
    if (++st == STAGES) { st = 0; phase ^= 1u; }
    if (++s == SL) {
      flush(rt);
#pragma unroll
      for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = corr[nt][0] = corr[nt][1] = 0.f;
      s = 0;
      rt++;
    }
  }
  stamp(4);
  if (n_units > 0 && s != 0) flush(rt);
  stamp(5);

}

// ---------------------------------------------------------------------------
// General-shape kernel (any K % 32 == 0, any alignment of the pointers beyond
// 4 bytes): one warp per weight row, exact f32 arithmetic in the order
// a[k] * (sc * (float)q) of the reference kernel.  Used when the TMA path's
// alignment rules (K % 128 == 0, 16-byte aligned base) do not hold, and as an
// independent cross-check in the tests.
// ---------------------------------------------------------------------------
__global__ void gemv_q4_simt_kernel(const float* __restrict__ x, long long ldx, int M,
                                    const unsigned char* __restrict__ qw,
                                    const float* __restrict__ scales, float* __restrict__ y,
                                    long long ldy, int N, int K, float alpha, float beta) {
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= N) return;
  const unsigned char* qrow = qw + (size_t)warp * (K / 2);
  const float* srow = scales + (size_t)warp * (K / 32);
  for (int m = 0; m < M; m++) {
    const float* xr = x + (long long)m * ldx;
    float acc = 0.f;
    for (int k0 = lane * 8; k0 < K; k0 += 256) {
      const float sc = srow[k0 >> 5];
#pragma unroll
      for (int b = 0; b < 4; b++) {
        unsigned byte = qrow[(k0 >> 1) + b];
        acc += xr[k0 + 2 * b] * (sc * (float)((int)(byte & 0xF) - 8));
        acc += xr[k0 + 2 * b + 1] * (sc * (float)((int)(byte >> 4) - 8));
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) y[(long long)m * ldy + warp] = acc * alpha + beta;
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
int make_q4_tensor_maps(const void* qw, const void* scales, int N, int K, CUtensorMap* tmW,
                        CUtensorMap* tmS) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return set_error(TLB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  cuuint64_t dimW[2] = {(cuuint64_t)(K / 8), (cuuint64_t)N};
  cuuint64_t strW[1] = {(cuuint64_t)(K / 2)};
  cuuint32_t boxW[2] = {32, 16};
  cuuint32_t es[2] = {1, 1};
  CUresult r = enc(tmW, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(qw), dimW, strW, boxW,
                   es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(TLB_ERR_CUDA, "tensor map (weights) encode failed");
  cuuint64_t dimS[2] = {(cuuint64_t)(K / 32), (cuuint64_t)N};
  cuuint64_t strS[1] = {(cuuint64_t)(K / 8)};
  cuuint32_t boxS[2] = {8, 16};
  r = enc(tmS, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(scales), dimS, strS, boxS, es,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(TLB_ERR_CUDA, "tensor map (scales) encode failed");
  return TLB_OK;
}

// Kernel shape for a problem: 8 warps x 4 stages when two CTAs fit on an SM,
// else 16 warps x 3 stages.
static void gemv_pick(int M, int K, int* warps, int* stages) {
  if (const char* e = getenv("TLB_GEMV_CFG")) {  // diagnostics: "16x3" / "16x4"
    if (!strcmp(e, "16x3")) { *warps = 16; *stages = 3; return; }
    if (!strcmp(e, "16x4")) { *warps = 16; *stages = 4; return; }
  }
  const size_t small = gemv_smem_layout(8, 4, M, K).total;
  if (small <= 113 * 1024) { *warps = 8; *stages = 4; }
  else { *warps = 16; *stages = 3; }
}

bool gemv_q4_tma_eligible(const void* qw, const void* scales, int N, int K, int M) {
  if (K % 128 != 0 || M < 1 || M > GV_MAXM) return false;
  if (((uintptr_t)qw & 15) || ((uintptr_t)scales & 15)) return false;
  int w, st;
  gemv_pick(M, K, &w, &st);
  if (gemv_smem_layout(w, st, M, K).total > 227 * 1024) return false;
  return N > 0;
}

template <int NT, int WARPS, int STAGES, bool M1>
static int gemv_launch_t(const CUtensorMap& tmW, const CUtensorMap& tmS, const GemvParams& p,
                         int ctas, size_t smem, cudaStream_t stream) {
  static std::atomic<unsigned long long> attr_done{0};
  {
    const int rc_attr = ensure_dynamic_smem(gemv_q4_mma_kernel<NT, WARPS, STAGES, M1>, 227 * 1024, attr_done);
    if (rc_attr) return rc_attr;
  }
  LaunchCfg lc(dim3(ctas), dim3(WARPS * 32), smem, stream, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, gemv_q4_mma_kernel<NT, WARPS, STAGES, M1>, tmW, tmS, p));
  return TLB_OK;
}

// Diagnostics: when set, every launch records per-CTA phase timestamps there.
unsigned long long* g_gemv_dbg = nullptr;

// Launch with ready tensor maps (the decoder caches them per weight).
int gemv_q4_launch(DeviceCtx* c, const CUtensorMap& tmW, const CUtensorMap& tmS, const float* x,
                   long long ldx, int M, float* y, long long ldy, int N, int K, float alpha,
                   float beta, cudaStream_t stream, int max_ctas, const CommDev* push_comm,
                   int act, const float* delta, const float* nw, float* xout, float eps) {
  GemvParams p;
  p.act = act;
  p.delta = delta; p.nw = nw; p.xout = xout; p.eps = eps;
  p.dbg = g_gemv_dbg;
  if (act == 2 && (M != 1 || !delta || !nw || !xout))
    return set_error(TLB_ERR_ARG, "gemv_q4: fused add+rmsnorm needs M == 1 and its three buffers");
  if (act == 2 && (K + 255) / 256 > 8 * 4)
    return set_error(TLB_ERR_UNSUPPORTED, "gemv_q4: fused add+rmsnorm needs K <= 8192");
  p.push = push_comm ? 1 : 0;
  if (push_comm) {
    if (M != 1) return set_error(TLB_ERR_ARG, "gemv_q4: the tensor-parallel push needs M == 1");
    p.comm = *push_comm;
  }
  p.x = x; p.ldx = ldx; p.y = y; p.ldy = ldy; p.M = M; p.N = N; p.K = K;
  p.alpha = alpha; p.beta = beta;
  p.partials = c->gemv_partials; p.counters = c->gemv_counters; p.status = c->status;
  p.RT = (N + 15) / 16; p.SL = (K + 255) / 256;
  p.U = (unsigned)p.RT * (unsigned)p.SL;
  p.x_vec_ok = (((uintptr_t)x & 15) == 0 && (ldx % 4) == 0 && (K % 4) == 0) ? 1 : 0;
  if (p.RT > c->gemv_max_tiles)
    return set_error(TLB_ERR_UNSUPPORTED, "gemv_q4: N exceeds the fix-up counter capacity");
  int warps, stages;
  gemv_pick(M, K, &warps, &stages);
  int ctas = max_ctas > 0 ? max_ctas : c->sm_count * (warps == 8 ? 2 : 1);
  const int need = (int)((p.U + warps - 1) / warps);
  if (ctas > need) ctas = need;
  if (ctas * warps > c->gemv_max_workers) ctas = c->gemv_max_workers / warps;
  const size_t smem = gemv_smem_layout(warps, stages, M, K).total;
  if (warps == 8) {
    if (M == 1) return gemv_launch_t<1, 8, 4, true>(tmW, tmS, p, ctas, smem, stream);
    if (M <= 4) return gemv_launch_t<1, 8, 4, false>(tmW, tmS, p, ctas, smem, stream);
    return gemv_launch_t<2, 8, 4, false>(tmW, tmS, p, ctas, smem, stream);
  }
  if (M == 1 && stages == 4) return gemv_launch_t<1, 16, 4, true>(tmW, tmS, p, ctas, smem, stream);
  if (M == 1) return gemv_launch_t<1, 16, 3, true>(tmW, tmS, p, ctas, smem, stream);
  if (M <= 4) return gemv_launch_t<1, 16, 3, false>(tmW, tmS, p, ctas, smem, stream);
  return gemv_launch_t<2, 16, 3, false>(tmW, tmS, p, ctas, smem, stream);
}

int gemv_q4_simt_launch(const float* x, long long ldx, int M, const void* qw, const void* scales,
                        float* y, long long ldy, int N, int K, float alpha, float beta,
                        cudaStream_t stream) {
  int threads = 256, rows_per_block = threads / 32;
  LaunchCfg lc(dim3((N + rows_per_block - 1) / rows_per_block), dim3(threads), 0, stream,
               pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, gemv_q4_simt_kernel, x, ldx, M, (const unsigned char*)qw,
                              (const float*)scales, y, ldy, N, K, alpha, beta));
  return TLB_OK;
}

}  // namespace tlb
