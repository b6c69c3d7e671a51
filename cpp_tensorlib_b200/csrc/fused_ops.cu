// Small fused row ops of the decode path: rmsnorm, residual-add + rmsnorm,
// swiglu, rope (+bias), KV append, argmax, the q4 converters and the embedding
// row gather.  Each is HBM/latency bound and a few KB per launch; all are
// programmatic-dependent-launch aware (griddepcontrol.wait first) so they can be
// chained in a CUDA graph without full kernel-boundary drains.
#include <cuda_bf16.h>

#include "comm.cuh"

namespace tlb {

// ---------------------------------------------------------------------------
// block reduction helper (sum), blockDim.x <= 1024
// ---------------------------------------------------------------------------
__device__ __forceinline__ float block_sum(float v, float* sm) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) sm[warp] = v;
  __syncthreads();
  float r = 0.f;
  for (int w = 0; w < nw; w++) r += sm[w];  // fixed order: same value in every thread
  __syncthreads();
  return r;
}

// out = x * (1/sqrtf(mean(x^2)+eps)) * w   -- kernels/tensorlib_cuda.cu:131-149
// (exact 1/sqrtf, not rsqrtf, like the reference).  out may alias x.
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               float* out, int n, float eps) {
  __shared__ float sm[32];
  pdl_wait();
  pdl_launch_dependents();
  const size_t base = (size_t)blockIdx.x * n;
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = x[base + i];
    acc += v * v;
  }
  const float tot = block_sum(acc, sm);
  const float inv = 1.0f / sqrtf(tot / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) out[base + i] = x[base + i] * inv * w[i];
}

// xout = a + b; hout = rmsnorm(xout) * w   -- kernels/tensorlib_cuda.cu:155-179.
// xout may alias a.
__global__ void add_rmsnorm_kernel(const float* a, const float* __restrict__ b,
                                   const float* __restrict__ w, float* xout, float* hout, int n,
                                   float eps) {
  __shared__ float sm[32];
  pdl_wait();
  pdl_launch_dependents();
  const size_t base = (size_t)blockIdx.x * n;
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = a[base + i] + b[base + i];
    xout[base + i] = v;
    acc += v * v;
  }
  const float tot = block_sum(acc, sm);
  const float inv = 1.0f / sqrtf(tot / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    hout[base + i] = xout[base + i] * inv * w[i];
}

// out[r,f] = silu(g[r,f]) * u[r,f]   -- kernels/tensorlib_cuda.cu:185-192; gate and up rows
// each with their own row stride (the fused [rows, 2 ff] buffer is g = gu, u = gu + ff,
// both strides 2 ff)
__global__ void swiglu_kernel(const float* __restrict__ gate, long long ldg,
                              const float* __restrict__ up, long long ldu, float* __restrict__ out,
                              int ff) {
  pdl_wait();
  pdl_launch_dependents();
  const int f = blockIdx.x * blockDim.x + threadIdx.x;
  if (f >= ff) return;
  const float g = gate[(size_t)blockIdx.y * ldg + f];
  out[(size_t)blockIdx.y * ff + f] = (g / (1.0f + expf(-g))) * up[(size_t)blockIdx.y * ldu + f];
}

// Half-split RoPE with an optional fused bias -- kernels/tensorlib_cuda.cu:1360-1395
// for the layout (pairs (j, j+D/2), row r at position pos + r%T, bias added
// before the rotation).  The angle is formed in double like the reference's CPU
// path (include/array.h:1719-1727): with base 1e6 and positions beyond 4096 the
// f32 fast intrinsics of the reference kernel drift by more than the 1e-3
// tolerance allows on the low-j pairs.
__device__ __forceinline__ void rope_pair(const float* x, const float* bias, float* out,
                                          size_t bi, int j, int half, int D, unsigned position,
                                          float base) {
  const double theta = exp2(-2.0 * (double)j / (double)D * log2((double)base));
  const double ang = (double)position * theta;
  double sd, cd;
  sincos(ang, &sd, &cd);
  const float c = (float)cd, s = (float)sd;
  float x0 = x[bi + j], x1 = x[bi + j + half];
  if (bias) {
    x0 += bias[bi + j];
    x1 += bias[bi + j + half];
  }
  out[bi + j] = x0 * c - x1 * s;
  out[bi + j + half] = x0 * s + x1 * c;
}

__global__ void rope_kernel(const float* x, const float* __restrict__ bias, float* out, int T,
                            int D, unsigned pos, const unsigned* __restrict__ d_pos, float base) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x, j = threadIdx.x, half = D >> 1;
  if (j >= half) return;
  const unsigned p0 = d_pos ? *d_pos : pos;
  const unsigned t = T ? (unsigned)(r % T) : 0u;
  rope_pair(x, bias, out, (size_t)r * D, j, half, D, p0 + t, base);
}

// Scatter one token's k,v ([n_kv, D]) into the cache ([n_kv, kv_max, D]) at
// row pos (or *d_pos) -- kernels/tensorlib_cuda.cu:1068-1102.
// bf: the cache stores bf16 (kv_st of the reference, kernels/tensorlib_cuda.cu:831:
// round to nearest even).
__global__ void kv_append_kernel(void* __restrict__ Kc, void* __restrict__ Vc,
                                 const float* __restrict__ k, const float* __restrict__ v,
                                 unsigned pos, const unsigned* __restrict__ d_pos,
                                 long long kv_stride, int D, int bf, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const unsigned p0 = d_pos ? *d_pos : pos;
  const int h = blockIdx.x, d = threadIdx.x;
  if (d >= D) return;
  if ((long long)p0 * D >= kv_stride) {   // row beyond the cache: refuse, tell the host
    if (status && d == 0) atomicExch(&status[ST_KV_OVERFLOW], 1);
    return;
  }
  const size_t dst = (size_t)h * kv_stride + (size_t)p0 * D + d;
  if (bf) {
    ((__nv_bfloat16*)Kc)[dst] = __float2bfloat16_rn(k[h * D + d]);
    ((__nv_bfloat16*)Vc)[dst] = __float2bfloat16_rn(v[h * D + d]);
  } else {
    ((float*)Kc)[dst] = k[h * D + d];
    ((float*)Vc)[dst] = v[h * D + d];
  }
}

// kernels/tensorlib_cuda.cu:1399
__global__ void incr_u32_kernel(unsigned* p) {
  pdl_wait();
  pdl_launch_dependents();
  ++*p;
}

// Decoder seam after the fused QKV projection: q <- rope(q + bq) in place,
// rope(k + bk) and v + bv written straight into the cache row *d_pos.  One block
// per head (q heads, then k heads, then v heads), D/2 threads.  Same arithmetic as
// rope_kernel + the v bias add + kv_append_kernel of the unfused sequence
// (bench/cuda/qwen_model.h:700-716).
__global__ void qkv_post_kernel(float* qkv, const float* __restrict__ bq,
                                const float* __restrict__ bk, const float* __restrict__ bv,
                                float* __restrict__ Kc, float* __restrict__ Vc, int n_q, int n_kv,
                                int D, const unsigned* __restrict__ d_pos, long long kv_stride,
                                float base, int kv_bf16, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, j = threadIdx.x, half = D >> 1;
  if (j >= half) return;
  const unsigned pos = *d_pos;
  if ((long long)pos * D >= kv_stride) {   // the cache is full: refuse, tell the host
    if (status && j == 0) atomicExch(&status[ST_KV_OVERFLOW], 1);
    return;
  }
  if (b < n_q) {
    rope_pair(qkv, bq, qkv, (size_t)b * D, j, half, D, pos, base);
  } else if (b < n_q + n_kv) {
    const int kh = b - n_q;
    // rotate into the cache row: out pointer offset so that index bi+j lands there
    const size_t row = (size_t)kh * kv_stride + (size_t)pos * D;
    const float* src = qkv + (size_t)b * D;
    const double theta = exp2(-2.0 * (double)j / (double)D * log2((double)base));
    double sd, cd;
    sincos((double)pos * theta, &sd, &cd);
    const float c = (float)cd, s = (float)sd;
    float x0 = src[j], x1 = src[j + half];
    if (bk) {
      x0 += bk[kh * D + j];
      x1 += bk[kh * D + j + half];
    }
    if (kv_bf16) {
      __nv_bfloat16* dst = (__nv_bfloat16*)Kc + row;
      dst[j] = __float2bfloat16_rn(x0 * c - x1 * s);
      dst[j + half] = __float2bfloat16_rn(x0 * s + x1 * c);
    } else {
      Kc[row + j] = x0 * c - x1 * s;
      Kc[row + j + half] = x0 * s + x1 * c;
    }
  } else {
    const int kh = b - n_q - n_kv;
    const size_t row = (size_t)kh * kv_stride + (size_t)pos * D;
    const float* src = qkv + (size_t)b * D;
    float v0 = src[j], v1 = src[j + half];
    if (bv) {
      v0 += bv[kh * D + j];
      v1 += bv[kh * D + j + half];
    }
    if (kv_bf16) {
      __nv_bfloat16* dst = (__nv_bfloat16*)Vc + row;
      dst[j] = __float2bfloat16_rn(v0);
      dst[j + half] = __float2bfloat16_rn(v1);
    } else {
      Vc[row + j] = v0;
      Vc[row + j + half] = v1;
    }
  }
}

// x0 <- embed[*d_tok]  (one block).  The reference gathers the row on the host
// and uploads it (bench/cuda/qwen_model.h:530-535, 768-772); here the table is
// resident in HBM and only the 4-byte token id crosses PCIe.
// With rope_cs != NULL the block also fills the token's rotary table: (cos, sin) of
// (*d_pos) * base^(-2j/D) for j < D/2, the double-precision expression of rope_pair,
// so that the 28 layers' projections read 64 pairs instead of each evaluating sincos.
// With nw != NULL it also leaves rmsnorm(x) * nw in hout (the first layer's attention norm,
// same arithmetic as rmsnorm_kernel), so the token needs no separate norm launch.
__global__ void embed_gather_kernel(const float* __restrict__ embed,
                                    const int* __restrict__ d_tok, float* __restrict__ x, int n,
                                    float2* __restrict__ rope_cs, const unsigned* __restrict__ d_pos,
                                    int D, float rope_base, const float* __restrict__ nw,
                                    float* __restrict__ hout, float eps) {
  __shared__ float sm[32];
  pdl_wait();
  pdl_launch_dependents();
  const size_t base = (size_t)(*d_tok) * n;
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = embed[base + i];
    x[i] = v;
    acc += v * v;
  }
  if (nw) {
    const float tot = block_sum(acc, sm);
    const float inv = 1.0f / sqrtf(tot / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) hout[i] = x[i] * inv * nw[i];
  }
  if (rope_cs && (int)threadIdx.x < D / 2) {
    const int j = threadIdx.x;
    const double theta = exp2(-2.0 * (double)j / (double)D * log2((double)rope_base));
    double sd, cd;
    sincos((double)(*d_pos) * theta, &sd, &cd);
    rope_cs[j] = make_float2((float)cd, (float)sd);
  }
}

// Batched form for the prompt pass: row t <- embed[ids[t]] (one block per row).
__global__ void embed_rows_kernel(const float* __restrict__ embed, const int* __restrict__ ids,
                                  float* __restrict__ x, int n) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t src = (size_t)ids[blockIdx.x] * n, dst = (size_t)blockIdx.x * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) x[dst + i] = embed[src + i];
}

// ---------------------------------------------------------------------------
// argmax: smallest index among the maxima (kernels/tensorlib_cuda.cu:90-119).
// Multi-block: each thread keeps (value, index) with strict '>', a packed
// 64-bit key (ordered float bits << 32 | ~index) is max-reduced through
// shuffles, shared memory and one atomicMax per block; the last block to finish
// publishes the index and clears the cell and the ticket (self-cleaning).
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long argmax_key(float v, unsigned idx) {
  unsigned b = __float_as_uint(v);
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return ((unsigned long long)b << 32) | (unsigned long long)(0xFFFFFFFFu - idx);
}

__global__ void argmax_kernel(const float* __restrict__ in, int n, unsigned long long* cell,
                              int* out_idx, int* out_idx2) {
  __shared__ unsigned long long sm[32];
  pdl_wait();
  pdl_launch_dependents();
  float best = -3.402823466e+38f;
  unsigned besti = 0;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < (unsigned)n;
       i += gridDim.x * blockDim.x) {
    float v = in[i];
    if (v > best) { best = v; besti = i; }
  }
  unsigned long long key = argmax_key(best, besti);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
    key = other > key ? other : key;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sm[warp] = key;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); w++) key = sm[w] > key ? sm[w] : key;
    atomicMax(&cell[0], key);
    __threadfence();
    unsigned ticket = atomicAdd((unsigned*)&cell[1], 1u);
    if (ticket == gridDim.x - 1) {
      __threadfence();
      unsigned long long k = atomicExch(&cell[0], 0ull);
      int idx = (int)(0xFFFFFFFFu - (unsigned)(k & 0xFFFFFFFFull));
      *out_idx = idx;
      if (out_idx2) *out_idx2 = idx;
      *(unsigned*)&cell[1] = 0u;
    }
  }
}

// ---------------------------------------------------------------------------
// q4 converters (include/array.h:703-742 to_q4, 666-684 to_f32) on the device,
// bit-exact with the host loops: scale = max(1e-8, maxabs)/7, q =
// clamp(round-half-away(w/scale), -8, 7), nibble q+8, low nibble = even k.
// One 32x32 thread block handles one k-group (32 k) of 32 output rows.
// ---------------------------------------------------------------------------
__global__ void to_q4_kernel(const float* __restrict__ w, int K, int N, unsigned char* q4) {
  __shared__ float tile[32][33];
  const int g = blockIdx.y, n0 = blockIdx.x * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
  {
    int n = n0 + tx, k = g * 32 + ty;
    tile[ty][tx] = n < N ? w[(size_t)k * N + n] : 0.f;
  }
  __syncthreads();
  const int n = n0 + ty;  // warp ty owns output row n, lane tx owns k = g*32+tx
  const float v = tile[tx][ty];
  float mx = warp_max(fmaxf(1e-8f, fabsf(v)));
  const float scale = mx / 7.0f;
  int q = (int)roundf(v / scale);
  q = q < -8 ? -8 : (q > 7 ? 7 : q);
  unsigned nib = (unsigned)(q + 8);
  unsigned hi = __shfl_down_sync(0xffffffffu, nib, 1);
  if (n < N) {
    if ((tx & 1) == 0)
      q4[(size_t)n * (K / 2) + (g * 32 + tx) / 2] = (unsigned char)(nib | (hi << 4));
    if (tx == 0) {
      float* sc = (float*)(q4 + (size_t)N * K / 2);
      sc[(size_t)n * (K / 32) + g] = scale;
    }
  }
}

__global__ void q4_to_f32_kernel(const unsigned char* __restrict__ q4, int K, int N,
                                 float* __restrict__ out) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)K * N) return;
  const int k = (int)(idx / N), n = (int)(idx % N);
  const float* sc = (const float*)(q4 + (size_t)N * K / 2);
  const unsigned char b = q4[(size_t)n * (K / 2) + k / 2];
  const int nib = (k & 1) ? (b >> 4) : (b & 0xF);
  out[idx] = sc[(size_t)n * (K / 32) + k / 32] * (float)(nib - 8);
}

// ---------------------------------------------------------------------------
// Tensor-parallel consumers of the one-shot exchange (see comm.cuh).
// ---------------------------------------------------------------------------

// xout = a + sum_r partial_r ; hout = rmsnorm(xout) * w, for one row.  The
// partials are the row-parallel GEMV outputs every rank pushed into this rank's
// staging buffer; they are summed in rank order so all ranks compute identical
// bits.  Fuses the all-reduce's reduction, the residual add and the norm
// (the tl_add_rmsnorm seam of the single-GPU path).
__global__ void add_rmsnorm_ar_kernel(const float* a, const float* __restrict__ w, float* xout,
                                      float* hout, int n, float eps, CommDev comm, int* status) {
  __shared__ float sm[32];
  pdl_wait();
  pdl_launch_dependents();
  const unsigned seq = comm_seq(comm);
  const uint2* st = comm.stage[comm.rank] + (size_t)(seq & 1u) * comm.size * comm.slot_floats;
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    uint2 pk[TP_MAX];
#pragma unroll
    for (int r = 0; r < TP_MAX; r++)          // all polls in flight before the first check
      if (r < comm.size) pk[r] = ld_packet_sys(&st[(size_t)r * comm.slot_floats + i]);
    float d = 0.f;
#pragma unroll
    for (int r = 0; r < TP_MAX; r++)
      if (r < comm.size) {
        if (pk[r].y != seq + 1u)
          pk[r] = wait_packet_bounded(&st[(size_t)r * comm.slot_floats + i], seq + 1u, status, 300 + r);
        d += __uint_as_float(pk[r].x);
      }
    const float v = a[i] + d;
    xout[i] = v;
    acc += v * v;
  }
  const float tot = block_sum(acc, sm);
  const float inv = 1.0f / sqrtf(tot / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) hout[i] = xout[i] * inv * w[i];
}

// out[i] = sum_r partial_r[i]: only the reduction of an exchange, spread over many CTAs so that
// every poll of every rank's packet is in flight at once (one thread per element, tp loads
// each).  The sum lands in this GPU's own memory; the residual add and the norm are then the
// ordinary fused prologue of the next projection, which reads a plain local vector instead of
// polling system-scope packets from every SM.  Partials are added in rank order, so all ranks
// compute identical bits.
//
// With two ranks the kernel does NOT wait for the pushing projection in front of it before it
// polls: packets validate themselves by their tag, so polling may begin as soon as CTAs of that
// projection exit, and the dependency wait comes LAST (this kernel's completion must still imply
// the projection's, whose fix-up counters the next projection reuses; `out` was last read a whole
// attention block / MLP ago).  Measured: 789 -> 805 tokens/s on 2 GPUs, no change on 4, and on 8
// GPUs -- where the projection's grid leaves SMs free and the pollers really run beside it and
// beside the peers' incoming stores -- 1035 -> 996, so from three ranks on the wait comes first.
// The sequence number (a device-resident counter, stable within a token) is read before the wait
// either way.
__global__ void ar_sum_kernel(float* __restrict__ out, int n, CommDev comm, int* status) {
  pdl_launch_dependents();
  const unsigned seq = comm_seq(comm);
  const bool early = comm.size <= 2;
  if (!early) pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const uint2* st = comm.stage[comm.rank] + (size_t)(seq & 1u) * comm.size * comm.slot_floats + i;
    uint2 pk[TP_MAX];
#pragma unroll
    for (int r = 0; r < TP_MAX; r++)
      if (r < comm.size) pk[r] = ld_packet_sys(st + (size_t)r * comm.slot_floats);
    float d = 0.f;
#pragma unroll
    for (int r = 0; r < TP_MAX; r++)
      if (r < comm.size) {
        if (pk[r].y != seq + 1u)
          pk[r] = wait_packet_bounded(st + (size_t)r * comm.slot_floats, seq + 1u, status, 300 + r);
        d += __uint_as_float(pk[r].x);
      }
    out[i] = d;
  }
  if (early) pdl_wait();
}

// Vocabulary-parallel argmax: each rank reduces its logits shard to a packed key
// (ordered float bits, inverted GLOBAL index), the last block pushes the key to
// every rank as two tagged packets, and argmax_finish_kernel takes the maximum.
__global__ void argmax_push_kernel(const float* __restrict__ in, int n, unsigned vocab_offset,
                                   unsigned long long* cell, CommDev comm) {
  __shared__ unsigned long long sm[32];
  pdl_wait();
  pdl_launch_dependents();
  float best = -3.402823466e+38f;
  unsigned besti = 0;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < (unsigned)n;
       i += gridDim.x * blockDim.x) {
    float v = in[i];
    if (v > best) { best = v; besti = i; }
  }
  unsigned long long key = argmax_key(best, besti + vocab_offset);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
    key = other > key ? other : key;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sm[warp] = key;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); w++) key = sm[w] > key ? sm[w] : key;
    atomicMax(&cell[0], key);
    __threadfence();
    unsigned ticket = atomicAdd((unsigned*)&cell[1], 1u);
    if (ticket == gridDim.x - 1) {
      __threadfence();
      unsigned long long k = atomicExch(&cell[0], 0ull);
      *(unsigned*)&cell[1] = 0u;
      const unsigned seq = comm_seq(comm);
      const size_t off = ((size_t)(seq & 1u) * comm.size + comm.rank) * (size_t)comm.slot_floats;
      for (int r = 0; r < comm.size; r++) {
        st_packet_sys(&comm.stage[r][off], __uint_as_float((unsigned)(k & 0xFFFFFFFFull)), seq + 1u);
        st_packet_sys(&comm.stage[r][off + 1], __uint_as_float((unsigned)(k >> 32)), seq + 1u);
      }
    }
  }
}

__global__ void argmax_finish_kernel(CommDev comm, int* out_idx, int* out_idx2, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    const unsigned seq = comm_seq(comm);
    const uint2* st = comm.stage[comm.rank] + (size_t)(seq & 1u) * comm.size * comm.slot_floats;
    unsigned long long best = 0ull;
    for (int r = 0; r < comm.size; r++) {
      const uint2 lo = wait_packet_bounded(&st[(size_t)r * comm.slot_floats], seq + 1u, status, 400 + r);
      const uint2 hi = wait_packet_bounded(&st[(size_t)r * comm.slot_floats + 1], seq + 1u, status, 400 + r);
      const unsigned long long k = ((unsigned long long)hi.x << 32) | lo.x;
      best = k > best ? k : best;
    }
    const int idx = (int)(0xFFFFFFFFu - (unsigned)(best & 0xFFFFFFFFull));
    *out_idx = idx;
    if (out_idx2) *out_idx2 = idx;
    *comm.seq = *(volatile unsigned*)comm.seq + 1u;   // the token's last exchange: advance the token counter
  }
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
static int row_threads(int n) {
  int t = ((n + 3) / 4 + 31) / 32 * 32;
  return t < 64 ? 64 : (t > 1024 ? 1024 : t);
}

int launch_rmsnorm(const float* x, const float* w, float* out, int n, float eps, int rows,
                   cudaStream_t s) {
  LaunchCfg lc(dim3(rows), dim3(row_threads(n)), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, rmsnorm_kernel, x, w, out, n, eps));
  return TLB_OK;
}
int launch_add_rmsnorm(const float* a, const float* b, const float* w, float* xout, float* hout,
                       int n, float eps, int rows, cudaStream_t s) {
  LaunchCfg lc(dim3(rows), dim3(row_threads(n)), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, add_rmsnorm_kernel, a, b, w, xout, hout, n, eps));
  return TLB_OK;
}
int launch_swiglu_split(const float* g, long long ldg, const float* u, long long ldu, float* out, int ff,
                        int rows, cudaStream_t s) {
  LaunchCfg lc(dim3((ff + 255) / 256, rows), dim3(256), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, swiglu_kernel, g, ldg, u, ldu, out, ff));
  return TLB_OK;
}
int launch_swiglu(const float* gu, float* out, int ff, int rows, cudaStream_t s) {
  return launch_swiglu_split(gu, 2ll * ff, gu + ff, 2ll * ff, out, ff, rows, s);
}
int launch_rope(const float* x, const float* bias, float* out, int rows, int T, int D,
                unsigned pos, const unsigned* d_pos, float base, cudaStream_t s) {
  LaunchCfg lc(dim3(rows), dim3(D / 2), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, rope_kernel, x, bias, out, T, D, pos, d_pos, base));
  return TLB_OK;
}
int launch_kv_append(void* Kc, void* Vc, const float* k, const float* v, unsigned pos,
                     const unsigned* d_pos, long long kv_max, int n_kv, int D, int bf, int* status,
                     cudaStream_t s) {
  LaunchCfg lc(dim3(n_kv), dim3(D), 0, s, pdl_enabled());
  long long kv_stride = kv_max * D;
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, kv_append_kernel, Kc, Vc, k, v, pos, d_pos, kv_stride, D, bf, status));
  return TLB_OK;
}
int launch_incr_u32(unsigned* p, cudaStream_t s) {
  LaunchCfg lc(dim3(1), dim3(1), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, incr_u32_kernel, p));
  return TLB_OK;
}
int launch_qkv_post(float* qkv, const float* bq, const float* bk, const float* bv, float* Kc,
                    float* Vc, int n_q, int n_kv, int D, const unsigned* d_pos, long long kv_max,
                    float base, int kv_bf16, int* status, cudaStream_t s) {
  LaunchCfg lc(dim3(n_q + 2 * n_kv), dim3(D / 2), 0, s, pdl_enabled());
  long long kv_stride = kv_max * D;
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, qkv_post_kernel, qkv, bq, bk, bv, Kc, Vc, n_q, n_kv, D,
                              d_pos, kv_stride, base, kv_bf16, status));
  return TLB_OK;
}
int launch_embed_gather(const float* embed, const int* d_tok, float* x, int n, float2* rope_cs,
                        const unsigned* d_pos, int D, float rope_base, const float* nw, float* hout,
                        float eps, cudaStream_t s) {
  int threads = row_threads(n);
  if (threads < D / 2) threads = D / 2;
  LaunchCfg lc(dim3(1), dim3(threads), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, embed_gather_kernel, embed, d_tok, x, n, rope_cs, d_pos, D, rope_base, nw, hout, eps));
  return TLB_OK;
}
int launch_embed_rows(const float* embed, const int* ids, float* x, int n, int rows, cudaStream_t s) {
  LaunchCfg lc(dim3(rows), dim3(row_threads(n)), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, embed_rows_kernel, embed, ids, x, n));
  return TLB_OK;
}
int launch_argmax(DeviceCtx* c, const float* in, int n, int* out_idx, int* out_idx2,
                  cudaStream_t s) {
  int blocks = (n + 1023) / 1024;
  if (blocks > c->sm_count) blocks = c->sm_count;
  if (blocks < 1) blocks = 1;
  LaunchCfg lc(dim3(blocks), dim3(256), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, argmax_kernel, in, n, c->argmax_cell, out_idx, out_idx2));
  return TLB_OK;
}
int launch_to_q4(const float* w, int K, int N, unsigned char* q4, cudaStream_t s) {
  dim3 grid((N + 31) / 32, K / 32), block(32, 32);
  to_q4_kernel<<<grid, block, 0, s>>>(w, K, N, q4);
  TLB_CUDA(cudaGetLastError());
  return TLB_OK;
}
int launch_q4_to_f32(const unsigned char* q4, int K, int N, float* out, cudaStream_t s) {
  size_t tot = (size_t)K * N;
  q4_to_f32_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, s>>>(q4, K, N, out);
  TLB_CUDA(cudaGetLastError());
  return TLB_OK;
}

int launch_add_rmsnorm_ar(const float* a, const float* w, float* xout, float* hout, int n,
                          float eps, const CommDev& comm, int* status, cudaStream_t s) {
  LaunchCfg lc(dim3(1), dim3(row_threads(n)), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, add_rmsnorm_ar_kernel, a, w, xout, hout, n, eps, comm, status));
  return TLB_OK;
}
int launch_ar_sum(float* out, int n, const CommDev& comm, int* status, cudaStream_t s) {
  // 128 threads: a CTA of this size does NOT fit into the registers an SM has left beside a
  // 512-thread GEMV CTA, so the polling starts where that grid leaves SMs free or as its CTAs
  // exit.  (64-thread CTAs, which fit beside it, were measured: 790 against 805 tokens/s on 2
  // GPUs -- pollers sharing an SM with the stream cost it more than they save.)
  const int threads = 128;
  LaunchCfg lc(dim3((n + threads - 1) / threads), dim3(threads), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, ar_sum_kernel, out, n, comm, status));
  return TLB_OK;
}
int launch_argmax_tp(DeviceCtx* c, const float* in, int n, unsigned vocab_offset,
                     const CommDev& comm, int* out_idx, int* out_idx2, cudaStream_t s) {
  int blocks = (n + 1023) / 1024;
  if (blocks > c->sm_count) blocks = c->sm_count;
  if (blocks < 1) blocks = 1;
  LaunchCfg lc(dim3(blocks), dim3(256), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, argmax_push_kernel, in, n, vocab_offset, c->argmax_cell, comm));
  LaunchCfg lf(dim3(1), dim3(32), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lf.cfg, argmax_finish_kernel, comm, out_idx, out_idx2, c->status));
  return TLB_OK;
}

}  // namespace tlb
