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
#include "comm.cuh"

namespace tlb {

constexpr int GV_WARPS = 8;
constexpr int GV_STAGES = 6;
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
  int push;         // tensor-parallel: store y (M == 1) into every rank's staging slot
  CommDev comm;
};

__device__ __forceinline__ unsigned gv_start(unsigned w, unsigned U, unsigned W) {
  return (unsigned)(((unsigned long long)w * U) / W);
}
__device__ __forceinline__ unsigned gv_owner(unsigned u, unsigned U, unsigned W) {
  unsigned w = (unsigned)(((unsigned long long)u * W) / U);
  while (w + 1 < W && gv_start(w + 1, U, W) <= u) w++;
  return w;
}

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2,
                                         unsigned a3, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned pack_h2(__half a, __half b) {
  return (unsigned)__half_as_ushort(a) | ((unsigned)__half_as_ushort(b) << 16);
}

size_t gemv_smem_bytes(int M, int K) {
  int SL = (K + 255) / 256, G = SL * 8;
  int NT = M <= 4 ? 1 : 2;
  size_t b = 1024;  // alignment slack
  b += (size_t)GV_WARPS * GV_STAGES * (GV_W_BYTES + GV_S_BYTES);
  b += (size_t)GV_WARPS * GV_STAGES * 8;
  b += 64 * sizeof(float);                     // amax reduce
  b += (size_t)G * (4 * NT) * sizeof(float2);  // PQ
  b += (size_t)G * (2 * M) * 4 * sizeof(uint4);  // Bfrag
  return b;
}

template <int NT>
__global__ void __launch_bounds__(GV_WARPS * 32, 1)
    gemv_q4_mma_kernel(const __grid_constant__ CUtensorMap tmW,
                       const __grid_constant__ CUtensorMap tmS, GemvParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base =
      (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  constexpr int MPAD = 4 * NT;
  const int G = p.SL * 8;
  const int NCU = 2 * p.M;

  unsigned char* Wring = base;
  unsigned char* Sring = Wring + GV_WARPS * GV_STAGES * GV_W_BYTES;
  uint64_t* bars = (uint64_t*)(Sring + GV_WARPS * GV_STAGES * GV_S_BYTES);
  float* red = (float*)(bars + GV_WARPS * GV_STAGES);
  float2* PQ = (float2*)(red + 64);
  uint4* Bfrag = (uint4*)(PQ + (size_t)G * MPAD);

  unsigned char* myW = Wring + warp * GV_STAGES * GV_W_BYTES;
  unsigned char* myS = Sring + warp * GV_STAGES * GV_S_BYTES;
  uint64_t* mybar = bars + warp * GV_STAGES;

  // Never more workers than units, so every worker's range is non-empty and the
  // contributors of a row tile are exactly the owners of its first..last unit.
  const unsigned Wall = gridDim.x * GV_WARPS;
  const unsigned Wtot = Wall < p.U ? Wall : p.U;
  const unsigned wid = blockIdx.x * GV_WARPS + warp;
  const bool idle = wid >= Wtot;
  const unsigned u0 = idle ? 0u : gv_start(wid, p.U, Wtot);
  const unsigned u1 = idle ? 0u : gv_start(wid + 1, p.U, Wtot);
  const int n_units = (int)(u1 - u0);

  if (lane == 0) {
    for (int s = 0; s < GV_STAGES; s++) mbar_init(&mybar[s], 1);
    mbar_fence_init();
  }
  __syncwarp();

  auto issue = [&](int i) {
    unsigned u = u0 + i;
    int rt = u / p.SL, s = u - rt * p.SL;
    int st = i % GV_STAGES;
    mbar_expect_tx(&mybar[st], GV_W_BYTES + GV_S_BYTES);
    tma_load_2d(myW + st * GV_W_BYTES, &tmW, s * 32, rt * 16, &mybar[st]);
    tma_load_2d(myS + st * GV_S_BYTES, &tmS, s * 8, rt * 16, &mybar[st]);
  };
  // Weights do not depend on the previous kernel: start streaming them before
  // waiting for it.
  if (lane == 0) {
    int pre = n_units < GV_STAGES ? n_units : GV_STAGES;
    for (int i = 0; i < pre; i++) issue(i);
  }

  pdl_wait();  // activations and the fix-up scratch are valid from here

  // ---- activation prep: per-row power-of-two normalisation, fp16 hi/lo split,
  // B-fragment order.  Slot (m, j, t) covers x[m][32j+8t .. +8).
  {
    for (int m = 0; m < p.M; m++) {
      float mx = 0.f;
      const float* xr = p.x + (long long)m * p.ldx;
      for (int k = tid; k < p.K; k += blockDim.x) mx = fmaxf(mx, fabsf(xr[k]));
      mx = warp_max(mx);
      if (lane == 0) red[m * GV_WARPS + warp] = mx;
    }
    __syncthreads();
    const int slots = p.M * G * 4;
    for (int slot = tid; slot < ((slots + 3) & ~3); slot += blockDim.x) {
      const bool live = slot < slots;
      int m = live ? slot / (G * 4) : 0;
      int rem = slot - m * (G * 4);
      int j = rem >> 2, tt = rem & 3;
      float mx = 0.f;
#pragma unroll
      for (int w = 0; w < GV_WARPS; w++) mx = fmaxf(mx, red[m * GV_WARPS + w]);
      int e = (int)((__float_as_uint(mx) >> 23) & 0xff) - 126;  // mx < 2^e
      e = mx > 0.f ? (e < -100 ? -100 : (e > 100 ? 100 : e)) : 0;
      const float s12 = __uint_as_float((unsigned)(127 + 12 - e) << 23);
      const float s8 = __uint_as_float((unsigned)(127 + 8 - e) << 23);
      const float P = __uint_as_float((unsigned)(127 + 12 + e) << 23);
      float v[8];
      const int k0 = j * 32 + tt * 8;
      const float* xr = p.x + (long long)m * p.ldx + k0;
      if (live && k0 + 8 <= p.K) {
        if (p.x_vec_ok) {
          float4 a = *(const float4*)xr, b = *(const float4*)(xr + 4);
          v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
          v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
          for (int i = 0; i < 8; i++) v[i] = xr[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = (live && k0 + i < p.K) ? xr[i] : 0.f;
      }
      float sum = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if (live) {
        __half hi[8], lo[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
          float f = v[i] * ((i & 1) ? s8 : s12);
          hi[i] = __float2half_rn(f);
          lo[i] = __float2half_rn(f - __half2float(hi[i]));
        }
        uint4 fh, fl;
        fh.x = pack_h2(hi[0], hi[4]); fh.y = pack_h2(hi[1], hi[5]);
        fh.z = pack_h2(hi[2], hi[6]); fh.w = pack_h2(hi[3], hi[7]);
        fl.x = pack_h2(lo[0], lo[4]); fl.y = pack_h2(lo[1], lo[5]);
        fl.z = pack_h2(lo[2], lo[6]); fl.w = pack_h2(lo[3], lo[7]);
        Bfrag[((size_t)j * NCU + 2 * m) * 4 + tt] = fh;
        Bfrag[((size_t)j * NCU + 2 * m + 1) * 4 + tt] = fl;
        if (tt == 0) PQ[(size_t)j * MPAD + m] = make_float2(P, 8.0f * sum);
      }
    }
    for (int i = tid; i < G * MPAD; i += blockDim.x) {
      int m = i % MPAD;
      if (m >= p.M) PQ[i] = make_float2(0.f, 0.f);
    }
    __syncthreads();
  }
  pdl_launch_dependents();

  // ---- streaming loop ------------------------------------------------------
  float acc[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = 0.f;
  bool use_b[NT];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) use_b[nt] = (8 * nt + g) < NCU;
  const unsigned g7x4 = (unsigned)(g & 7) * 4u;

  unsigned ar_seq = 0;
  if (p.push) ar_seq = *(volatile unsigned*)p.comm.seq;
  const size_t ar_off =
      ((size_t)(ar_seq & 1u) * p.comm.size + p.comm.rank) * (size_t)p.comm.slot_floats;
  auto emit = [&](int m, int n, float v) {
    v = v * p.alpha + p.beta;
    if (p.push) {
      for (int r = 0; r < p.comm.size; r++) p.comm.stage[r][ar_off + n] = v;
    } else {
      p.y[(long long)m * p.ldy + n] = v;
    }
  };
  auto flush = [&](int rt) {
    const unsigned t0 = (unsigned)rt * p.SL, t1 = t0 + p.SL;
    const bool complete = (u0 <= t0) && (u1 >= t1);
    const int r0 = rt * 16;
    if (complete) {
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        int m = 4 * nt + t;
        if (m < p.M) {
          if (r0 + g < p.N) emit(m, r0 + g, acc[nt][0]);
          if (r0 + g + 8 < p.N) emit(m, r0 + g + 8, acc[nt][1]);
        }
      }
      return;
    }
    // partial: slot 0 when this tile holds the worker's first unit, else slot 1
    const int slot = ((int)(u0 / p.SL) == rt) ? 0 : 1;
    float* mine = p.partials + ((size_t)wid * 2 + slot) * 128;
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      int m = 4 * nt + t;
      __stcg(&mine[m * 16 + g], acc[nt][0]);
      __stcg(&mine[m * 16 + g + 8], acc[nt][1]);
    }
    __threadfence();
    __syncwarp();
    const unsigned wf = gv_owner(t0, p.U, Wtot), wl = gv_owner(t1 - 1, p.U, Wtot);
    int old = 0;
    if (lane == 0) old = atomicAdd(&p.counters[rt], 1);
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old != (int)(wl - wf)) return;  // not the last contributor
    __threadfence();
    float sum[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) sum[nt][0] = sum[nt][1] = 0.f;
    for (unsigned w = wf; w <= wl; w++) {
      const int sl = ((int)(gv_start(w, p.U, Wtot) / p.SL) == rt) ? 0 : 1;
      const float* src = p.partials + ((size_t)w * 2 + sl) * 128;
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        int m = 4 * nt + t;
        sum[nt][0] += __ldcg(&src[m * 16 + g]);
        sum[nt][1] += __ldcg(&src[m * 16 + g + 8]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      int m = 4 * nt + t;
      if (m < p.M) {
        if (r0 + g < p.N) emit(m, r0 + g, sum[nt][0]);
        if (r0 + g + 8 < p.N) emit(m, r0 + g + 8, sum[nt][1]);
      }
    }
    if (lane == 0) p.counters[rt] = 0;  // leave the counter clean for the next launch
  };

  int cur_rt = n_units > 0 ? (int)(u0 / p.SL) : -1;
  for (int i = 0; i < n_units; i++) {
    const unsigned u = u0 + i;
    const int rt = u / p.SL, s = u - rt * p.SL;
    if (rt != cur_rt) {
      flush(cur_rt);
#pragma unroll
      for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = 0.f;
      cur_rt = rt;
    }
    const int st = i % GV_STAGES;
    if (!mbar_wait_bounded(&mybar[st], (i / GV_STAGES) & 1, p.status, 100 + st)) return;
    const unsigned* Wst = (const unsigned*)(myW + st * GV_W_BYTES);
    const float* Sst = (const float*)(myS + st * GV_S_BYTES);
    const uint4* Bu = Bfrag + (size_t)(s * 8) * NCU * 4;
    const float2* PQu = PQ + (size_t)(s * 8) * MPAD;
#pragma unroll
    for (int jj = 0; jj < 8; jj++) {
      const unsigned wo = (unsigned)g * 32u + (((unsigned)jj * 4u) ^ g7x4) + (unsigned)t;
      unsigned w0 = Wst[wo], w1 = Wst[wo + 256];
      const float sc0 = Sst[g * 8 + jj], sc1 = Sst[(g + 8) * 8 + jj];
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
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        mma16816(c, a0, a1, a2, a3, b.x, b.y);
        mma16816(c, a4, a5, a6, a7, b.z, b.w);
        const float2 pq = PQu[jj * MPAD + 4 * nt + t];
        acc[nt][0] = fmaf(sc0, fmaf(pq.x, c[0] + c[1], -pq.y), acc[nt][0]);
        acc[nt][1] = fmaf(sc1, fmaf(pq.x, c[2] + c[3], -pq.y), acc[nt][1]);
      }
    }
    __syncwarp();
    if (lane == 0 && i + GV_STAGES < n_units) issue(i + GV_STAGES);
  }
  if (cur_rt >= 0) flush(cur_rt);

  // Tensor-parallel push: when the last worker of this rank has stored its tiles,
  // publish the sequence number in every rank's flag word.
  if (p.push && !idle) {
    __threadfence_system();
    __syncwarp();
    if (lane == 0) {
      const unsigned old = atomicAdd(p.comm.done, 1u);
      if (old == Wtot - 1) {
        *p.comm.done = 0u;
        __threadfence_system();
        for (int r = 0; r < p.comm.size; r++)
          st_release_sys(&p.comm.flags[r][(ar_seq & 1u) * p.comm.size + p.comm.rank], ar_seq + 1u);
      }
    }
  }
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

bool gemv_q4_tma_eligible(const void* qw, const void* scales, int N, int K, int M) {
  if (K % 128 != 0 || M < 1 || M > GV_MAXM) return false;
  if (((uintptr_t)qw & 15) || ((uintptr_t)scales & 15)) return false;
  if (gemv_smem_bytes(M, K) > 227 * 1024) return false;
  return N > 0;
}

// Launch with ready tensor maps (the decoder caches them per weight).
int gemv_q4_launch(DeviceCtx* c, const CUtensorMap& tmW, const CUtensorMap& tmS, const float* x,
                   long long ldx, int M, float* y, long long ldy, int N, int K, float alpha,
                   float beta, cudaStream_t stream, int max_ctas, const CommDev* push_comm) {
  GemvParams p;
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
  p.x_vec_ok = (((uintptr_t)x & 15) == 0 && (ldx % 4) == 0) ? 1 : 0;
  if (p.RT > c->gemv_max_tiles)
    return set_error(TLB_ERR_UNSUPPORTED, "gemv_q4: N exceeds the fix-up counter capacity");
  int ctas = max_ctas > 0 ? max_ctas : c->sm_count;
  int need = (int)((p.U + GV_WARPS - 1) / GV_WARPS);
  if (ctas > need) ctas = need;
  if (ctas * GV_WARPS > c->gemv_max_workers) ctas = c->gemv_max_workers / GV_WARPS;
  size_t smem = gemv_smem_bytes(M, K);
  LaunchCfg lc(dim3(ctas), dim3(GV_WARPS * 32), smem, stream, pdl_enabled());
  if (M <= 4) {
    static bool attr1 = false;
    if (!attr1) {
      TLB_CUDA(cudaFuncSetAttribute(gemv_q4_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    227 * 1024));
      attr1 = true;
    }
    TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, gemv_q4_mma_kernel<1>, tmW, tmS, p));
  } else {
    static bool attr2 = false;
    if (!attr2) {
      TLB_CUDA(cudaFuncSetAttribute(gemv_q4_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    227 * 1024));
      attr2 = true;
    }
    TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, gemv_q4_mma_kernel<2>, tmW, tmS, p));
  }
  return TLB_OK;
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
