// Batched-prefill pieces of the attention path: token-major <-> head-major moves,
// bulk KV fill, and causal attention over a prompt chunk.  Replaces
// tl_split_heads / tl_merge_heads (kernels/tensorlib_cuda.cu:200-218), tl_kv_fill
// (:1109-1130) and tl_attn_prefill_tiled_* (:1211-1350) of the reference
// (launchers include/cuda.h:848-879, 1143-1201).
//
// attn_prefill: q, out [n_q, T, D]; K, V a [n_kv, kv_max, D] cache read over
// [0, pos0 + T); query p sits at absolute position pos0 + p and attends keys
// 0..pos0+p.  One CTA per (q head, 32-query tile); a group of 8 lanes owns one query
// row (q fragment, running max / sum / accumulator in registers), the four row
// groups of a warp share each key row, K/V tiles of 32 keys arrive by bulk copy into
// a two-stage ring.  f32 throughout (the parity bar is 1e-4 against a double CPU
// reference).  This CUDA-core form serves bf16 caches; f32 caches take the tensor-core form in
// attn_prefill_mma.cu.
#include <cuda_bf16.h>

#include <cstdlib>

#include "attn_common.cuh"

namespace tlb {

__global__ void split_heads_kernel(const float* __restrict__ src, const float* __restrict__ bias,
                                   float* __restrict__ dst, int T, long long ld, long long off, int D) {
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, t = blockIdx.y, d = threadIdx.x;
  if (d >= D) return;
  float v = src[(long long)t * ld + off + (long long)h * D + d];
  if (bias) v += bias[h * D + d];
  dst[((size_t)h * T + t) * D + d] = v;
}

__global__ void merge_heads_kernel(const float* __restrict__ src, float* __restrict__ dst, int T,
                                   int H, int D) {
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, t = blockIdx.y, d = threadIdx.x;
  if (d >= D) return;
  dst[(size_t)t * H * D + (size_t)h * D + d] = src[((size_t)h * T + t) * D + d];
}

__global__ void kv_fill_kernel(void* __restrict__ Kc, void* __restrict__ Vc,
                               const float* __restrict__ K, const float* __restrict__ V, int T,
                               long long kv_stride, int pos0, int D, int bf) {
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, t = blockIdx.y, d = threadIdx.x;
  if (d >= D) return;
  const size_t dst = (size_t)h * kv_stride + (size_t)(pos0 + t) * D + d;
  const size_t src = ((size_t)h * T + t) * D + d;
  if (bf) {   // bf16 cache: round to nearest even, like kv_st of the reference
    ((__nv_bfloat16*)Kc)[dst] = __float2bfloat16_rn(K[src]);
    ((__nv_bfloat16*)Vc)[dst] = __float2bfloat16_rn(V[src]);
  } else {
    ((float*)Kc)[dst] = K[src];
    ((float*)Vc)[dst] = V[src];
  }
}

constexpr int PF_THREADS = 256;
constexpr int PF_QT = 32;   // queries per CTA (8 warps x 4 row groups)
constexpr int PF_KT = 32;   // keys per tile

// BF: bf16 cache (widened to f32 on load; q, out stay f32), same lane mapping as the decode kernel.
template <int D, bool BF>
__global__ void __launch_bounds__(PF_THREADS, 2)
    attn_prefill_kernel(const float* __restrict__ q, const void* __restrict__ K,
                        const void* __restrict__ V, float* __restrict__ out, int T,
                        long long kv_stride, int group, float scale, int pos0, int* status) {
  constexpr int CH = D / 32;
  constexpr int ELT = BF ? 2 : 4;
  constexpr int TILE_BYTES = PF_KT * D * ELT;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  float* Kt = (float*)base;
  float* Vt = (float*)(base + 2 * TILE_BYTES);
  uint64_t* bars = (uint64_t*)(base + 4 * TILE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = lane >> 3, sub = lane & 7;
  const int qt = blockIdx.x, h = blockIdx.y, kh = h / group;
  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_fence_init();
  }
  __syncthreads();
  pdl_wait();
  pdl_launch_dependents();

  const int row = qt * PF_QT + warp * 4 + rg;
  const bool row_ok = row < T;
  const int row_last_key = pos0 + row;                 // inclusive
  int warp_last_key = pos0 + qt * PF_QT + warp * 4 + 3;
  if (warp_last_key > pos0 + T - 1) warp_last_key = pos0 + T - 1;
  int cta_last_key = pos0 + qt * PF_QT + PF_QT - 1;
  if (cta_last_key > pos0 + T - 1) cta_last_key = pos0 + T - 1;
  const int n_tiles = cta_last_key / PF_KT + 1;
  const unsigned char* Kh = (const unsigned char*)K + (size_t)kh * kv_stride * ELT;
  const unsigned char* Vh = (const unsigned char*)V + (size_t)kh * kv_stride * ELT;

  auto issue = [&](int i) {
    const int st = i & 1;
    const int r0 = i * PF_KT;
    const int rows = (cta_last_key + 1 - r0) < PF_KT ? (cta_last_key + 1 - r0) : PF_KT;
    const uint32_t bytes = (uint32_t)rows * D * ELT;
    mbar_expect_tx(&bars[st], 2 * bytes);
    bulk_load_1d((unsigned char*)Kt + (size_t)st * TILE_BYTES, Kh + (size_t)r0 * D * ELT, bytes, &bars[st]);
    bulk_load_1d((unsigned char*)Vt + (size_t)st * TILE_BYTES, Vh + (size_t)r0 * D * ELT, bytes, &bars[st]);
  };
  if (tid == 0) {
    issue(0);
    if (n_tiles > 1) issue(1);
  }

  float4 qf[CH];
  {
    const float* qp = q + ((size_t)h * T + (row_ok ? row : 0)) * D;
#pragma unroll
    for (int i = 0; i < CH; i++)
      qf[i] = row_ok ? *(const float4*)(qp + attn_dim0<8, BF>(sub, i)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float m = -INFINITY, l = 0.f;
  float4 acc[CH];
#pragma unroll
  for (int i = 0; i < CH; i++) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);

  bool dead = false;
  for (int it = 0; it < n_tiles; it++) {
    const int st = it & 1;
    if (!dead && !mbar_wait_bounded(&bars[st], (it >> 1) & 1, status, 700 + st)) dead = true;
    const unsigned char* Ks = (const unsigned char*)Kt + (size_t)st * TILE_BYTES;
    const unsigned char* Vs = (const unsigned char*)Vt + (size_t)st * TILE_BYTES;
    const int k0 = it * PF_KT;
    int jmax = warp_last_key - k0 + 1;          // keys of this tile the warp needs
    if (jmax > PF_KT) jmax = PF_KT;
    if (!dead) {
      for (int j = 0; j < jmax; j++) {
        float4 kv[CH];
        attn_load_row<D, 8, CH, BF>(Ks + (size_t)j * D * ELT, sub, kv);
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < CH; i++) {
          d = fmaf(qf[i].x, kv[i].x, d);
          d = fmaf(qf[i].y, kv[i].y, d);
          d = fmaf(qf[i].z, kv[i].z, d);
          d = fmaf(qf[i].w, kv[i].w, d);
        }
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        d += __shfl_xor_sync(0xffffffffu, d, 4);
        const float s = d * scale;
        attn_load_row<D, 8, CH, BF>(Vs + (size_t)j * D * ELT, sub, kv);
        if (row_ok && k0 + j <= row_last_key) {
          if (s > m) {
            const float corr = __expf(m - s);
            l *= corr;
#pragma unroll
            for (int i = 0; i < CH; i++) {
              acc[i].x *= corr; acc[i].y *= corr; acc[i].z *= corr; acc[i].w *= corr;
            }
            m = s;
          }
          const float pr = __expf(s - m);
          l += pr;
#pragma unroll
          for (int i = 0; i < CH; i++) {
            acc[i].x = fmaf(pr, kv[i].x, acc[i].x);
            acc[i].y = fmaf(pr, kv[i].y, acc[i].y);
            acc[i].z = fmaf(pr, kv[i].z, acc[i].z);
            acc[i].w = fmaf(pr, kv[i].w, acc[i].w);
          }
        }
      }
    }
    __syncthreads();
    if (tid == 0 && it + 2 < n_tiles) issue(it + 2);
  }
  if (row_ok) {
    float* op = out + ((size_t)h * T + row) * D;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < CH; i++)
      *(float4*)(op + attn_dim0<8, BF>(sub, i)) =
          make_float4(acc[i].x * inv, acc[i].y * inv, acc[i].z * inv, acc[i].w * inv);
  }
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
int launch_split_heads(const float* src, const float* bias, float* dst, int T, long long ld,
                       long long off, int H, int D, cudaStream_t s) {
  LaunchCfg lc(dim3(H, T), dim3(D), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, split_heads_kernel, src, bias, dst, T, ld, off, D));
  return TLB_OK;
}
int launch_merge_heads(const float* src, float* dst, int T, int H, int D, cudaStream_t s) {
  LaunchCfg lc(dim3(H, T), dim3(D), 0, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, merge_heads_kernel, src, dst, T, H, D));
  return TLB_OK;
}
int launch_kv_fill(void* Kc, void* Vc, const float* K, const float* V, int T, long long kv_max,
                   int n_kv, int D, int pos0, int bf, cudaStream_t s) {
  LaunchCfg lc(dim3(n_kv, T), dim3(D), 0, s, pdl_enabled());
  long long kv_stride = kv_max * D;
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, kv_fill_kernel, Kc, Vc, K, V, T, kv_stride, pos0, D, bf));
  return TLB_OK;
}
template <int D, bool BF>
static int launch_attn_prefill_t(DeviceCtx* c, const float* q, const void* K, const void* V, float* out,
                                 int n_q, int n_kv, int T, long long kv_max, float scale, int pos0,
                                 cudaStream_t s) {
  const int group = n_q / n_kv;
  long long kv_stride = kv_max * D;
  const size_t smem = 4 * (size_t)PF_KT * D * (BF ? 2 : 4) + 64 + 128;
  LaunchCfg lc(dim3((T + PF_QT - 1) / PF_QT, n_q), dim3(PF_THREADS), smem, s, pdl_enabled());
  static std::atomic<unsigned long long> attr_done{0};
  {
    const int rc_attr = ensure_dynamic_smem(attn_prefill_kernel<D, BF>, 100 * 1024, attr_done);
    if (rc_attr) return rc_attr;
  }
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, attn_prefill_kernel<D, BF>, q, K, V, out, T, kv_stride, group, scale,
                              pos0, c->status));
  return TLB_OK;
}
bool attn_prefill_mma_eligible(int D, int n_kv, long long kv_max, int bf);
int attn_prefill_mma_launch(DeviceCtx* c, const float* q, const void* K, const void* V, float* out, int n_q,
                            int n_kv, int T, long long kv_max, int D, float scale, int pos0, cudaStream_t s);

int launch_attn_prefill(DeviceCtx* c, const float* q, const void* K, const void* V, float* out,
                        int n_q, int n_kv, int T, long long kv_max, int D, float scale, int pos0,
                        int bf, cudaStream_t s) {
  // f32 caches: the tensor-core form (attn_prefill_mma.cu); TLB_PREFILL_MMA=0 keeps the CUDA-core
  // form below (a diagnostic switch for A/B timing), which also serves bf16 caches
  static const bool mma_on = !(getenv("TLB_PREFILL_MMA") && atoi(getenv("TLB_PREFILL_MMA")) == 0);
  if (mma_on && attn_prefill_mma_eligible(D, n_kv, kv_max, bf))
    return attn_prefill_mma_launch(c, q, K, V, out, n_q, n_kv, T, kv_max, D, scale, pos0, s);
  if (D == 128)
    return bf ? launch_attn_prefill_t<128, true>(c, q, K, V, out, n_q, n_kv, T, kv_max, scale, pos0, s)
              : launch_attn_prefill_t<128, false>(c, q, K, V, out, n_q, n_kv, T, kv_max, scale, pos0, s);
  return bf ? launch_attn_prefill_t<64, true>(c, q, K, V, out, n_q, n_kv, T, kv_max, scale, pos0, s)
            : launch_attn_prefill_t<64, false>(c, q, K, V, out, n_q, n_kv, T, kv_max, scale, pos0, s);
}

}  // namespace tlb
