// bf16 row-major weight GEMV: y[n] = sum_k a[k] * W[n][k], W bf16 [N][K], a and y f32.
// Replaces tl_gemv_bf16_row (kernels/tensorlib_cuda.cu:730-752; launcher include/cuda.h:770-785),
// the decode projection of the reference's bf16-weight models.
//
// HBM bound (2 bytes per weight).  The activation vector is staged once per CTA in shared
// memory; a warp owns whole rows (grid-stride over the rows), every lane keeps four 16-byte
// streaming loads in flight (8 bf16 each, L1 no-allocate), widens with one shift or mask per
// element and accumulates in f32; one shuffle tree per row.  No split-K: a row is at least a few
// KB and there are thousands of rows.
#include "common.cuh"

namespace tlb {

constexpr int GB_WARPS = 8;

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ float dot8_bf16(const uint4& w, const float4& x0, const float4& x1, float acc) {
  acc = fmaf(__uint_as_float(w.x << 16), x0.x, acc);
  acc = fmaf(__uint_as_float(w.x & 0xffff0000u), x0.y, acc);
  acc = fmaf(__uint_as_float(w.y << 16), x0.z, acc);
  acc = fmaf(__uint_as_float(w.y & 0xffff0000u), x0.w, acc);
  acc = fmaf(__uint_as_float(w.z << 16), x1.x, acc);
  acc = fmaf(__uint_as_float(w.z & 0xffff0000u), x1.y, acc);
  acc = fmaf(__uint_as_float(w.w << 16), x1.z, acc);
  acc = fmaf(__uint_as_float(w.w & 0xffff0000u), x1.w, acc);
  return acc;
}

__global__ void __launch_bounds__(GB_WARPS * 32, 4)
    gemv_bf16_row_kernel(const float* __restrict__ a, const unsigned short* __restrict__ W,
                         float* __restrict__ y, int N, int K) {
  extern __shared__ float4 xs[];  // K floats, K % 8 == 0
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_wait();
  pdl_launch_dependents();
  for (int i = tid; i < K / 4; i += GB_WARPS * 32) xs[i] = ((const float4*)a)[i];
  __syncthreads();
  const int chunks = K / 8;  // 16-byte chunks per row
  for (int n = blockIdx.x * GB_WARPS + warp; n < N; n += gridDim.x * GB_WARPS) {
    const uint4* row = (const uint4*)(W + (size_t)n * K);
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    int c = lane;
    for (; c + 96 < chunks; c += 128) {
      const uint4 w0 = ldg_stream16(row + c), w1 = ldg_stream16(row + c + 32);
      const uint4 w2 = ldg_stream16(row + c + 64), w3 = ldg_stream16(row + c + 96);
      acc0 = dot8_bf16(w0, xs[2 * c], xs[2 * c + 1], acc0);
      acc1 = dot8_bf16(w1, xs[2 * (c + 32)], xs[2 * (c + 32) + 1], acc1);
      acc2 = dot8_bf16(w2, xs[2 * (c + 64)], xs[2 * (c + 64) + 1], acc2);
      acc3 = dot8_bf16(w3, xs[2 * (c + 96)], xs[2 * (c + 96) + 1], acc3);
    }
    for (; c < chunks; c += 32) acc0 = dot8_bf16(ldg_stream16(row + c), xs[2 * c], xs[2 * c + 1], acc0);
    float acc = (acc0 + acc1) + (acc2 + acc3);
    acc = warp_sum(acc);
    if (lane == 0) y[n] = acc;
  }
}

int launch_gemv_bf16_row(DeviceCtx* c, const float* a, const void* W, float* y, int N, int K,
                         cudaStream_t s) {
  const size_t smem = (size_t)K * sizeof(float);
  if (smem > 200 * 1024) return set_error(TLB_ERR_UNSUPPORTED, "gemv_bf16_row: K too large for the activation stage");
  static std::atomic<unsigned long long> attr_done{0};
  {
    const int rc_attr = ensure_dynamic_smem(gemv_bf16_row_kernel, 200 * 1024, attr_done);
    if (rc_attr) return rc_attr;
  }
  int ctas = c->sm_count * 4;
  const int need = (N + GB_WARPS - 1) / GB_WARPS;
  if (ctas > need) ctas = need;
  LaunchCfg lc(dim3(ctas), dim3(GB_WARPS * 32), smem, s, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, gemv_bf16_row_kernel, a, (const unsigned short*)W, y, N, K));
  return TLB_OK;
}

}  // namespace tlb
