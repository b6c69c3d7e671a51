// Shared device helpers (mbarrier / TMA / PDL inline PTX for sm_100a) and the
// per-device host context of the C-ABI library.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <string>

#include "../../include/tlb200.h"

namespace tlb {

// status codes (TLB_OK, TLB_ERR_*) come from the public C header
// Device status word indices (written by kernels whose bounded waits expire).
// Words 2..3 hold the wait limit in clock64 ticks as one 64-bit value (set by the host,
// read by a kernel only after a first unsuccessful poll); word 4 is set when a kernel
// refused to touch a cache row at or beyond the cache's capacity.
enum : int { ST_WAIT_TIMEOUT = 0, ST_WAIT_WHERE = 1, ST_WAIT_LIMIT = 2, ST_KV_OVERFLOW = 4, ST_WORDS = 8 };
constexpr long long WAIT_LIMIT_DEFAULT = 2000000000ll;  // about one second at ~2 GHz

int set_error(int code, const std::string& msg);
int cuda_fail(cudaError_t e, const char* what);

#define TLB_CUDA(expr)                                   \
  do {                                                   \
    cudaError_t _e = (expr);                             \
    if (_e != cudaSuccess) return tlb::cuda_fail(_e, #expr); \
  } while (0)

#define TLB_REQUIRE(cond, msg)                                         \
  do {                                                                 \
    if (!(cond)) return tlb::set_error(TLB_ERR_ARG, std::string(msg)); \
  } while (0)

// ---------------------------------------------------------------------------
// Per-device context: scratch owned by the library (never by a kernel launch),
// driver entry points resolved through the runtime (nothing is linked against
// libcuda).
// ---------------------------------------------------------------------------
struct DeviceCtx {
  int device = -1;
  int sm_count = 0;
  int l2_bytes = 0;
  // GEMV split-K fix-up scratch (deterministic last-arriver reduction)
  float* gemv_partials = nullptr;  // [max_workers][2][16*8]
  int* gemv_counters = nullptr;    // [max_row_tiles], zero between launches
  int gemv_max_workers = 0, gemv_max_tiles = 0;
  unsigned long long* chain_cell = nullptr;   // arrival counter of the GEMV chains' phase barrier
  // attention split-KV partials for the host-ctx entry point (grown on demand)
  float* attn_scratch = nullptr;
  size_t attn_scratch_bytes = 0;
  int* attn_counters = nullptr;  // [max kv-head*... ] zero between launches
  int attn_max_counters = 0;
  // argmax result cell (packed key) + small status block
  // tf32 hi/lo planes of the activations for the tensor-core GEMM (grown on demand)
  float* xsplit = nullptr;
  size_t xsplit_bytes = 0;
  unsigned long long* argmax_cell = nullptr;
  int* status = nullptr;        // device, ST_WORDS ints
  int* status_host = nullptr;   // pinned mirror for reads
  // CUDA-graph capture state of the reference-style capture_begin/end API
  cudaStream_t cap_stream = nullptr;
  bool capturing = false;
};

int get_ctx(DeviceCtx** out);  // context of the current device (created on first use)
DeviceCtx* find_ctx();         // the same if it exists already, else NULL; allocates nothing
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();

// ---------------------------------------------------------------------------
// device-side PTX wrappers
// ---------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// The limit of every bounded wait, in clock64 ticks: the value the host stored in the
// status block (tlb_set_wait_limit_cycles), about one second when there is no block.
__device__ __forceinline__ long long wait_limit(const int* status) {
  if (!status) return WAIT_LIMIT_DEFAULT;
  const long long v = *(const volatile long long*)&status[ST_WAIT_LIMIT];
  return v > 0 ? v : WAIT_LIMIT_DEFAULT;
}
// Bounded wait: gives up after the limit (about one second by default), records where
// in the status block and returns false; the caller must then skip the work that
// depended on it.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* status,
                                                  int where) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  // the first microseconds poll without touching memory: the limit lives in the status block
  // (a load that goes to L2) and a wait that reads it up front pays that round trip every time
  // it does not succeed at once -- several hundred ns per pipeline hand-off
  while (clock64() - t0 < 8192)
    if (mbar_try_wait(bar, parity)) return true;
  const long long limit = wait_limit(status);
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > limit) break;
  }
  if (status) {
    atomicExch(&status[ST_WAIT_TIMEOUT], 1);
    atomicExch(&status[ST_WAIT_WHERE], where);
  }
  return false;
}

// 2-D tiled TMA load (no multicast): box lands at dst, completion on bar.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* tm, int x, int y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, "
      "%3}], [%4];" ::"r"(smem_u32(dst)),
      "l"(tm), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// L2 policy for data that is read once per pass (weight streams): evict it first, so that what
// is re-read every launch -- the kernels' own instructions above all, then activations and
// scratch -- stays in the L2 instead of being pushed out by gigabytes of weights.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_evict_normal_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void bulk_load_1d_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar,
                                                  uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
// 2-D tiled TMA load with an L2 policy (see l2_evict_first_policy).
__device__ __forceinline__ void tma_load_2d_hint(void* dst, const CUtensorMap* tm, int x, int y, uint64_t* bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, "
      "%3}], [%4], %5;" ::"r"(smem_u32(dst)),
      "l"(tm), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
// 1-D bulk copy global -> shared (16-byte aligned addresses and size).
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes,
                                             uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tm) : "memory");
}

// Programmatic dependent launch: wait for the kernels this one depends on /
// let the dependent kernel's CTAs start launching.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

#endif  // __CUDACC__

// Launch helper: optional programmatic-dependent-launch attribute.
struct LaunchCfg {
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  LaunchCfg(dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl) {
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    if (pdl) {
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.numAttrs = 1;
    }
  }
};

bool pdl_enabled();  // process-wide switch (tlb_set_pdl)

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device attribute of a kernel:
// set it the first time the kernel is launched on each device of the process.  `done`
// is one bit per device ordinal, owned by the caller (one per kernel instantiation).
template <typename Kernel>
int ensure_dynamic_smem(Kernel kernel, int bytes, std::atomic<unsigned long long>& done) {
  int dev = 0;
  TLB_CUDA(cudaGetDevice(&dev));
  const bool tracked = dev >= 0 && dev < 64;
  if (tracked && ((done.load(std::memory_order_acquire) >> dev) & 1ull)) return TLB_OK;
  TLB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (tracked) done.fetch_or(1ull << dev, std::memory_order_release);
  return TLB_OK;
}

}  // namespace tlb
