// extern "C" surface (declared in include/tlb200.h), the per-device context and
// error plumbing.  Host code only; kernels live in the sibling .cu files.
#include <cstdlib>
#include <map>
#include <mutex>
#include <string>

#include "../../include/tlb200.h"
#include "comm.cuh"
#include "gemv_q4p.cuh"

namespace tlb {

// launchers defined in the kernel files
int make_q4_tensor_maps(const void* qw, const void* scales, int N, int K, CUtensorMap* tmW,
                        CUtensorMap* tmS);
bool gemv_q4_tma_eligible(const void* qw, const void* scales, int N, int K, int M);
int gemv_q4_launch(DeviceCtx* c, const CUtensorMap& tmW, const CUtensorMap& tmS, const float* x,
                   long long ldx, int M, float* y, long long ldy, int N, int K, float alpha,
                   float beta, cudaStream_t stream, int max_ctas, const CommDev* push_comm,
                   int act, const float* delta, const float* nw, float* xout, float eps);
int gemv_q4_simt_launch(const float* x, long long ldx, int M, const void* qw, const void* scales,
                        float* y, long long ldy, int N, int K, float alpha, float beta,
                        cudaStream_t stream);
bool gemm_q4_tc_eligible(const void* qw, const void* scales, int N, int K, int M);
int gemm_q4_tc_launch(DeviceCtx* c, const float* x, long long ldx, int M, const void* qw,
                      const float* scales, float* y, long long ldy, int N, int K, float alpha,
                      float beta, float* xsplit, cudaStream_t stream);
bool gemm_q4_tc2_eligible(const void* qw, const void* scales, int N, int K, int M);
size_t gemm_q4_tc2_scratch_bytes(int M, int K);
int gemm_q4_tc2_launch(DeviceCtx* c, const float* x, long long ldx, int M, const void* qw, const float* scales,
                       float* y, long long ldy, int N, int K, float alpha, float beta, void* scratch,
                       cudaStream_t stream);
size_t attn_partials_bytes(int n_q, int n_kv, long long kv_max, int D, int sm_count);
int attn_decode_launch(DeviceCtx* c, const float* q, const void* K, const void* V, float* out,
                       int n_q, int n_kv, int ctx, long long kv_max, int D, float scale,
                       const unsigned* d_pos, float* partials, int* counters, cudaStream_t stream,
                       int early_kv, int kv_bf16, const GvStream* prefetch = nullptr);
int launch_rmsnorm(const float*, const float*, float*, int, float, int, cudaStream_t);
int launch_add_rmsnorm(const float*, const float*, const float*, float*, float*, int, float, int,
                       cudaStream_t);
int launch_swiglu(const float*, float*, int, int, cudaStream_t);
int launch_swiglu_split(const float*, long long, const float*, long long, float*, int, int, cudaStream_t);
int launch_rope(const float*, const float*, float*, int, int, int, unsigned, const unsigned*,
                float, cudaStream_t);
int launch_kv_append(void*, void*, const float*, const float*, unsigned, const unsigned*, long long,
                     int, int, int, int*, cudaStream_t);
int launch_incr_u32(unsigned*, cudaStream_t);
int launch_argmax(DeviceCtx*, const float*, int, int*, int*, cudaStream_t);
int launch_to_q4(const float*, int, int, unsigned char*, cudaStream_t);

int launch_gemv_bf16_row(DeviceCtx*, const float*, const void*, float*, int, int, cudaStream_t);
int launch_split_heads(const float*, const float*, float*, int, long long, long long, int, int, cudaStream_t);
int launch_merge_heads(const float*, float*, int, int, int, cudaStream_t);
int launch_kv_fill(void*, void*, const float*, const float*, int, long long, int, int, int, int,
                   cudaStream_t);
int launch_attn_prefill(DeviceCtx*, const float*, const void*, const void*, float*, int, int, int,
                        long long, int, float, int, int, cudaStream_t);
int launch_q4_to_f32(const unsigned char*, int, int, float*, cudaStream_t);

extern unsigned long long* g_gemv_dbg;
extern unsigned long long* g_attn_dbg;
static thread_local std::string g_err;
static std::mutex g_mu;
static std::map<int, DeviceCtx*> g_ctx;
static bool g_pdl = true;

int set_error(int code, const std::string& msg) {
  g_err = msg;
  return code;
}
int cuda_fail(cudaError_t e, const char* what) {
  g_err = std::string(what) + ": " + cudaGetErrorString(e);
  cudaGetLastError();  // clear the sticky-less error state
  return TLB_ERR_CUDA;
}
bool pdl_enabled() { return g_pdl; }

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) ==
            cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

static int create_ctx(int dev, DeviceCtx** out) {
  auto* c = new DeviceCtx();
  c->device = dev;
  cudaDeviceProp prop;
  TLB_CUDA(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10)
    return set_error(TLB_ERR_UNSUPPORTED,
                     "tlb200 is built for sm_100a only; found compute capability " +
                         std::to_string(prop.major) + "." + std::to_string(prop.minor));
  c->sm_count = prop.multiProcessorCount;
  c->l2_bytes = prop.l2CacheSize;
  c->gemv_max_workers = c->sm_count * 2 * 8;
  c->gemv_max_tiles = 1 << 16;  // N up to 1,048,576 rows
  TLB_CUDA(cudaMalloc(&c->gemv_partials, (size_t)c->gemv_max_workers * 2 * 128 * sizeof(float)));
  TLB_CUDA(cudaMalloc(&c->gemv_counters, (size_t)c->gemv_max_tiles * sizeof(int)));
  TLB_CUDA(cudaMemset(c->gemv_counters, 0, (size_t)c->gemv_max_tiles * sizeof(int)));
  TLB_CUDA(cudaMalloc(&c->chain_cell, 64));
  TLB_CUDA(cudaMemset(c->chain_cell, 0, 64));
  c->attn_max_counters = 1024;
  TLB_CUDA(cudaMalloc(&c->attn_counters, c->attn_max_counters * sizeof(int)));
  TLB_CUDA(cudaMemset(c->attn_counters, 0, c->attn_max_counters * sizeof(int)));
  TLB_CUDA(cudaMalloc(&c->argmax_cell, 4 * sizeof(unsigned long long)));
  TLB_CUDA(cudaMemset(c->argmax_cell, 0, 4 * sizeof(unsigned long long)));
  TLB_CUDA(cudaMalloc(&c->status, ST_WORDS * sizeof(int)));
  TLB_CUDA(cudaMemset(c->status, 0, ST_WORDS * sizeof(int)));
  {
    const long long limit = WAIT_LIMIT_DEFAULT;
    TLB_CUDA(cudaMemcpy(&c->status[ST_WAIT_LIMIT], &limit, sizeof(limit), cudaMemcpyHostToDevice));
  }
  TLB_CUDA(cudaMallocHost(&c->status_host, ST_WORDS * sizeof(int)));
  TLB_CUDA(cudaDeviceSynchronize());
  *out = c;
  return TLB_OK;
}

int get_ctx(DeviceCtx** out) {
  int dev = 0;
  TLB_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_ctx.find(dev);
  if (it != g_ctx.end()) {
    *out = it->second;
    return TLB_OK;
  }
  DeviceCtx* c = nullptr;
  int rc = create_ctx(dev, &c);
  if (rc) return rc;
  g_ctx[dev] = c;
  *out = c;
  return TLB_OK;
}

// The context of the current device if one was created already; never creates (and so
// never allocates).
DeviceCtx* find_ctx() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_ctx.find(dev);
  return it == g_ctx.end() ? nullptr : it->second;
}

static inline cudaStream_t S(void* s) { return reinterpret_cast<cudaStream_t>(s); }

}  // namespace tlb

using namespace tlb;

#define CTX(c)          \
  DeviceCtx* c = nullptr; \
  do {                  \
    int _rc = get_ctx(&c); \
    if (_rc) return _rc; \
  } while (0)

extern "C" {

int tlb_init(int device) {
  TLB_CUDA(cudaSetDevice(device));
  CTX(c);
  return TLB_OK;
}
int tlb_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}
const char* tlb_last_error(void) { return g_err.c_str(); }
int tlb_version(void) { return 100; }
int tlb_set_pdl(int enabled) {
  g_pdl = enabled != 0;
  return TLB_OK;
}
int tlb_device_status(int* out2, int clear) {
  CTX(c);
  TLB_CUDA(cudaMemcpy(c->status_host, c->status, ST_WORDS * sizeof(int), cudaMemcpyDeviceToHost));
  if (out2) {
    out2[0] = c->status_host[ST_WAIT_TIMEOUT];
    out2[1] = c->status_host[ST_WAIT_WHERE];
  }
  const bool timed_out = c->status_host[ST_WAIT_TIMEOUT] != 0;
  const bool overflow = c->status_host[ST_KV_OVERFLOW] != 0;
  if (clear) {
    // the wait limit (words 2..3) survives a clear
    TLB_CUDA(cudaMemset(c->status, 0, 2 * sizeof(int)));
    TLB_CUDA(cudaMemset(&c->status[ST_KV_OVERFLOW], 0, sizeof(int)));
    if (timed_out) {
      // a kernel that gave up may have left its fix-up tickets half counted
      TLB_CUDA(cudaMemset(c->gemv_counters, 0, (size_t)c->gemv_max_tiles * sizeof(int)));
      TLB_CUDA(cudaMemset(c->attn_counters, 0, c->attn_max_counters * sizeof(int)));
      TLB_CUDA(cudaMemset(c->chain_cell, 0, 64));
      TLB_CUDA(cudaMemset(c->argmax_cell, 0, 4 * sizeof(unsigned long long)));
    }
  }
  if (timed_out) return set_error(TLB_ERR_DEVICE_WAIT, "a bounded device-side wait expired (where = " +
                                                           std::to_string(c->status_host[ST_WAIT_WHERE]) + ")");
  if (overflow) return set_error(TLB_ERR_STATE, "a kernel was asked to touch a KV-cache row beyond the cache's capacity and skipped it");
  return TLB_OK;
}
int tlb_set_wait_limit_cycles(int64_t cycles) {
  TLB_REQUIRE(cycles > 0, "tlb_set_wait_limit_cycles: the limit must be positive");
  CTX(c);
  const long long limit = cycles;
  TLB_CUDA(cudaDeviceSynchronize());
  TLB_CUDA(cudaMemcpy(&c->status[ST_WAIT_LIMIT], &limit, sizeof(limit), cudaMemcpyHostToDevice));
  return TLB_OK;
}

// Undocumented diagnostic hook: device buffer of [ctas][8] u64 that the GEMV fills
// with %globaltimer stamps of its phases (NULL switches it off).
int tlb_debug_attn_timing(void* dbuf) {
  g_attn_dbg = (unsigned long long*)dbuf;
  return TLB_OK;
}
int tlb_debug_gemv_timing(void* dbuf) {
  g_gemv_dbg = (unsigned long long*)dbuf;
  return TLB_OK;
}

int tlb_alloc(int64_t bytes, void** dptr) {
  TLB_REQUIRE(dptr && bytes >= 0, "tlb_alloc: bad arguments");
  TLB_CUDA(cudaMalloc(dptr, (size_t)(bytes > 0 ? bytes : 4)));
  return TLB_OK;
}
int tlb_free(void* dptr) {
  if (dptr) TLB_CUDA(cudaFree(dptr));
  return TLB_OK;
}
int tlb_h2d(void* dst, const void* src, int64_t bytes, void* stream) {
  TLB_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, S(stream)));
  return TLB_OK;
}
int tlb_d2h(void* dst, const void* src, int64_t bytes, void* stream) {
  TLB_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToHost, S(stream)));
  TLB_CUDA(cudaStreamSynchronize(S(stream)));
  return TLB_OK;
}
int tlb_memset(void* dst, int value, int64_t bytes, void* stream) {
  TLB_CUDA(cudaMemsetAsync(dst, value, (size_t)bytes, S(stream)));
  return TLB_OK;
}
int tlb_sync(void* stream) {
  TLB_CUDA(cudaStreamSynchronize(S(stream)));
  return TLB_OK;
}

int64_t tlb_q4_bytes(int64_t N, int64_t K) { return N * K / 2 + N * (K / 32) * 4; }

int tlb_to_q4(const float* w_kn, int64_t K, int64_t N, void* q4, void* stream) {
  TLB_REQUIRE(w_kn && q4, "tlb_to_q4: null pointer");
  TLB_REQUIRE(K > 0 && N > 0 && K % 32 == 0, "tlb_to_q4: K must be a positive multiple of 32");
  TLB_REQUIRE(((uintptr_t)q4 & 3) == 0 && ((N * K / 2) & 3) == 0, "tlb_to_q4: q4 buffer must be 4-byte aligned");
  return launch_to_q4(w_kn, (int)K, (int)N, (unsigned char*)q4, S(stream));
}
int tlb_q4_to_f32(const void* q4, int64_t K, int64_t N, float* out_kn, void* stream) {
  TLB_REQUIRE(q4 && out_kn, "tlb_q4_to_f32: null pointer");
  TLB_REQUIRE(K > 0 && N > 0 && K % 32 == 0, "tlb_q4_to_f32: K must be a positive multiple of 32");
  return launch_q4_to_f32((const unsigned char*)q4, (int)K, (int)N, out_kn, S(stream));
}

int tlb_gemm_q4_simt(const float* x, int64_t M, int64_t ldx, const void* qw, const float* scales,
                     float* y, int64_t ldy, int64_t N, int64_t K, float alpha, float beta,
                     void* stream) {
  TLB_REQUIRE(x && qw && scales && y, "tlb_gemm_q4: null pointer");
  TLB_REQUIRE(M >= 0 && N >= 0 && K > 0 && K % 32 == 0, "tlb_gemm_q4: K must be a multiple of 32");
  if (M == 0 || N == 0) return TLB_OK;
  return gemv_q4_simt_launch(x, ldx, (int)M, qw, scales, y, ldy, (int)N, (int)K, alpha, beta,
                             S(stream));
}

int tlb_gemm_q4(const float* x, int64_t M, int64_t ldx, const void* qw, const float* scales,
                float* y, int64_t ldy, int64_t N, int64_t K, float alpha, float beta,
                void* stream) {
  TLB_REQUIRE(x && qw && scales && y, "tlb_gemm_q4: null pointer");
  TLB_REQUIRE(M >= 0 && N >= 0 && K > 0 && K % 32 == 0, "tlb_gemm_q4: K must be a multiple of 32");
  TLB_REQUIRE(ldx >= K && ldy >= N, "tlb_gemm_q4: row strides shorter than the rows");
  if (M == 0 || N == 0) return TLB_OK;
  CTX(c);
  // Many rows: tensor-core path (tcgen05, TMEM accumulators).  Default: integer weights x two
  // fp16 activation planes, group scales applied outside the tensor core (gemm_q4_tc2.cu);
  // TLB_GEMM_TC=1 selects the earlier formulation with scaled tf32 hi/lo operands.
  static const bool tc_old = getenv("TLB_GEMM_TC") && atoi(getenv("TLB_GEMM_TC")) == 1;
  if (!tc_old && gemm_q4_tc2_eligible(qw, scales, (int)N, (int)K, (int)M)) {
    const size_t need = gemm_q4_tc2_scratch_bytes((int)M, (int)K);
    if (need > c->xsplit_bytes) {
      TLB_CUDA(cudaDeviceSynchronize());
      if (c->xsplit) TLB_CUDA(cudaFree(c->xsplit));
      c->xsplit = nullptr;
      c->xsplit_bytes = 0;
      TLB_CUDA(cudaMalloc(&c->xsplit, need));
      c->xsplit_bytes = need;
    }
    return gemm_q4_tc2_launch(c, x, ldx, (int)M, qw, scales, y, ldy, (int)N, (int)K, alpha, beta, c->xsplit,
                              S(stream));
  }
  if (gemm_q4_tc_eligible(qw, scales, (int)N, (int)K, (int)M)) {
    const size_t need = (size_t)2 * M * K * sizeof(float);
    if (need > c->xsplit_bytes) {
      // grown between launches only; not capturable at a size never seen before
      TLB_CUDA(cudaDeviceSynchronize());
      if (c->xsplit) TLB_CUDA(cudaFree(c->xsplit));
      c->xsplit = nullptr;
      c->xsplit_bytes = 0;
      TLB_CUDA(cudaMalloc(&c->xsplit, need));
      c->xsplit_bytes = need;
    }
    return gemm_q4_tc_launch(c, x, ldx, (int)M, qw, scales, y, ldy, (int)N, (int)K, alpha, beta,
                             c->xsplit, S(stream));
  }
  // Skinny activations: stream the weights once per block of up to 8 rows.
  if (gemv_q4_tma_eligible(qw, scales, (int)N, (int)K, 1)) {
    CUtensorMap tmW, tmS;
    int rc = make_q4_tensor_maps(qw, scales, (int)N, (int)K, &tmW, &tmS);
    if (rc) return rc;
    int64_t m0 = 0;
    while (m0 < M) {
      int mb = (int)((M - m0) < 8 ? (M - m0) : 8);
      while (mb > 1 && !gemv_q4_tma_eligible(qw, scales, (int)N, (int)K, mb)) mb = (mb + 1) / 2;
      rc = gemv_q4_launch(c, tmW, tmS, x + m0 * ldx, ldx, mb, y + m0 * ldy, ldy, (int)N, (int)K,
                          alpha, beta, S(stream), 0, nullptr, 0, nullptr, nullptr, nullptr, 0.f);
      if (rc) return rc;
      m0 += mb;
    }
    return TLB_OK;
  }
  return gemv_q4_simt_launch(x, ldx, (int)M, qw, scales, y, ldy, (int)N, (int)K, alpha, beta,
                             S(stream));
}

int tlb_gemv_bf16_row(const float* a, const void* W, float* y, int64_t N, int64_t K, void* stream) {
  TLB_REQUIRE(a && W && y, "tlb_gemv_bf16_row: null pointer");
  TLB_REQUIRE(N > 0 && N < (1ll << 31) && K > 0 && K % 8 == 0, "tlb_gemv_bf16_row: K must be a positive multiple of 8");
  TLB_REQUIRE((((uintptr_t)a | (uintptr_t)W) & 15) == 0, "tlb_gemv_bf16_row: a and W must be 16-byte aligned");
  CTX(c);
  return launch_gemv_bf16_row(c, a, W, y, (int)N, (int)K, S(stream));
}

int64_t tlb_q4p_bytes(int64_t N, int64_t K) {
  if (N <= 0 || K <= 0 || K % 32 != 0) return -1;
  return q4p_bytes(N, K);
}

int tlb_q4_pack(const void* q4, int64_t N, int64_t K, void* packed, void* stream) {
  TLB_REQUIRE(q4 && packed, "tlb_q4_pack: null pointer");
  TLB_REQUIRE(N > 0 && K > 0 && K % 32 == 0, "tlb_q4_pack: K must be a positive multiple of 32");
  TLB_REQUIRE(N < (1ll << 31) && K <= (1ll << 20), "tlb_q4_pack: shape out of range");
  TLB_REQUIRE((((uintptr_t)q4 | (uintptr_t)packed) & 15) == 0, "tlb_q4_pack: pointers must be 16-byte aligned");
  return launch_q4_pack(q4, (int)N, (int)K, packed, 0, S(stream));
}

int tlb_gemv_q4p(const float* x, const void* packed, float* y, int64_t N, int64_t K, float alpha,
                 float beta, void* stream) {
  TLB_REQUIRE(x && packed && y, "tlb_gemv_q4p: null pointer");
  TLB_REQUIRE(N > 0 && K > 0 && K % 32 == 0, "tlb_gemv_q4p: K must be a positive multiple of 32");
  TLB_REQUIRE(gemv_q4p_supported(N, K), "tlb_gemv_q4p: K too large for the activation fragments");
  TLB_REQUIRE(((uintptr_t)packed & 15) == 0, "tlb_gemv_q4p: packed weights must be 16-byte aligned");
  CTX(c);
  return gemv_q4p_launch(c, packed, x, y, (int)N, (int)K, alpha, beta, S(stream), 0, nullptr, 0,
                         nullptr, nullptr, nullptr, 0.f, nullptr, nullptr);
}

int tlb_gemv_q4(const float* a, const void* qw, const float* scales, float* y, int64_t N,
                int64_t K, int64_t group, void* stream) {
  TLB_REQUIRE(group == 32, "tlb_gemv_q4: group must be 32 (kQ4Group)");
  return tlb_gemm_q4(a, 1, K, qw, scales, y, N, N, K, 1.0f, 0.0f, stream);
}

static int attn_decode_any(const float* q, const void* K, const void* V, float* out, int64_t n_q,
                           int64_t n_kv, int64_t ctx, int64_t kv_max, int64_t D, float scale,
                           void* stream, int kv_bf16) {
  TLB_REQUIRE(q && K && V && out, "tlb_attn_decode: null pointer");
  TLB_REQUIRE(ctx >= 1 && ctx <= kv_max, "tlb_attn_decode: need 1 <= ctx <= kv_max");
  TLB_REQUIRE(n_kv > 0 && n_kv <= 1024, "tlb_attn_decode: n_kv out of range");
  TLB_REQUIRE(n_q > 0 && n_q <= (1 << 24) && n_q % n_kv == 0,
              "tlb_attn_decode: need 0 < n_q <= 2^24 and n_q % n_kv == 0");
  TLB_REQUIRE(kv_max <= (1ll << 30) && (D == 64 || D == 128), "tlb_attn_decode: kv_max / D out of range");
  CTX(c);
  size_t need = attn_partials_bytes((int)n_q, (int)n_kv, ctx, (int)D, c->sm_count);
  if (need > c->attn_scratch_bytes) {
    // grown between launches only; the old buffer may still be in use by queued work
    TLB_CUDA(cudaDeviceSynchronize());
    if (c->attn_scratch) TLB_CUDA(cudaFree(c->attn_scratch));
    c->attn_scratch = nullptr;
    c->attn_scratch_bytes = 0;
    TLB_CUDA(cudaMalloc(&c->attn_scratch, need));
    c->attn_scratch_bytes = need;
  }
  return attn_decode_launch(c, q, K, V, out, (int)n_q, (int)n_kv, (int)ctx, kv_max, (int)D, scale,
                            nullptr, c->attn_scratch, c->attn_counters, S(stream), 0, kv_bf16);
}
int tlb_attn_decode(const float* q, const float* K, const float* V, float* out, int64_t n_q,
                    int64_t n_kv, int64_t ctx, int64_t kv_max, int64_t D, float scale,
                    void* stream) {
  return attn_decode_any(q, K, V, out, n_q, n_kv, ctx, kv_max, D, scale, stream, 0);
}
int tlb_attn_decode_bf16(const float* q, const void* K, const void* V, float* out, int64_t n_q,
                         int64_t n_kv, int64_t ctx, int64_t kv_max, int64_t D, float scale,
                         void* stream) {
  return attn_decode_any(q, K, V, out, n_q, n_kv, ctx, kv_max, D, scale, stream, 1);
}

int64_t tlb_attn_partials_bytes(int64_t n_q, int64_t n_kv, int64_t kv_max, int64_t D) {
  DeviceCtx* c = nullptr;
  if (get_ctx(&c)) return -1;
  return 256 + (int64_t)attn_partials_bytes((int)n_q, (int)n_kv, kv_max, (int)D, c->sm_count);
}

static int attn_decode_dpos_any(const float* q, const void* K, const void* V, float* out, int64_t n_q,
                                int64_t n_kv, const void* d_pos, int64_t kv_max, int64_t D, float scale,
                                void* partials, void* stream, int kv_bf16) {
  TLB_REQUIRE(q && K && V && out && d_pos && partials, "tlb_attn_decode_dpos: null pointer");
  TLB_REQUIRE(n_kv > 0 && n_kv <= 64, "tlb_attn_decode_dpos: n_kv must be 1..64");
  TLB_REQUIRE(n_q > 0 && n_q <= (1 << 24) && n_q % n_kv == 0,
              "tlb_attn_decode_dpos: need 0 < n_q <= 2^24 and n_q % n_kv == 0");
  TLB_REQUIRE(kv_max >= 1 && kv_max <= (1ll << 30), "tlb_attn_decode_dpos: kv_max out of range");
  TLB_REQUIRE(((uintptr_t)partials & 15) == 0, "tlb_attn_decode_dpos: partials must be 16-byte aligned");
  CTX(c);
  return attn_decode_launch(c, q, K, V, out, (int)n_q, (int)n_kv, 0, kv_max, (int)D, scale,
                            (const unsigned*)d_pos, (float*)((char*)partials + 256),
                            (int*)partials, S(stream), 0, kv_bf16);
}
int tlb_attn_decode_dpos(const float* q, const float* K, const float* V, float* out, int64_t n_q,
                         int64_t n_kv, const void* d_pos, int64_t kv_max, int64_t D, float scale,
                         void* partials, void* stream) {
  return attn_decode_dpos_any(q, K, V, out, n_q, n_kv, d_pos, kv_max, D, scale, partials, stream, 0);
}
int tlb_attn_decode_dpos_bf16(const float* q, const void* K, const void* V, float* out, int64_t n_q,
                              int64_t n_kv, const void* d_pos, int64_t kv_max, int64_t D, float scale,
                              void* partials, void* stream) {
  return attn_decode_dpos_any(q, K, V, out, n_q, n_kv, d_pos, kv_max, D, scale, partials, stream, 1);
}

int tlb_rmsnorm(const float* x, const float* w, float* out, int64_t n, float eps, int64_t rows,
                void* stream) {
  TLB_REQUIRE(x && w && out && n > 0 && rows > 0, "tlb_rmsnorm: bad arguments");
  return launch_rmsnorm(x, w, out, (int)n, eps, (int)rows, S(stream));
}
int tlb_rmsnorm_res(const float* x, const float* delta, const float* w, float* xout, float* hout,
                    int64_t n, float eps, int64_t rows, void* stream) {
  TLB_REQUIRE(x && delta && w && xout && hout && n > 0 && rows > 0, "tlb_rmsnorm_res: bad arguments");
  return launch_add_rmsnorm(x, delta, w, xout, hout, (int)n, eps, (int)rows, S(stream));
}
int tlb_swiglu(const float* gu, float* out, int64_t ff, int64_t rows, void* stream) {
  TLB_REQUIRE(gu && out && ff > 0 && rows > 0, "tlb_swiglu: bad arguments");
  return launch_swiglu(gu, out, (int)ff, (int)rows, S(stream));
}
int tlb_swiglu_split(const float* gate, int64_t ldg, const float* up, int64_t ldu, float* out, int64_t ff,
                     int64_t rows, void* stream) {
  TLB_REQUIRE(gate && up && out && ff > 0 && rows > 0 && rows <= 65535 && ldg >= ff && ldu >= ff,
              "tlb_swiglu_split: bad arguments");
  return launch_swiglu_split(gate, ldg, up, ldu, out, (int)ff, (int)rows, S(stream));
}
int tlb_rope(const float* x, float* out, int64_t rows, int64_t T, int64_t D, int64_t pos,
             float base, const float* bias, void* stream) {
  TLB_REQUIRE(x && out && D > 0 && (D & 1) == 0 && D <= 2048, "tlb_rope: D must be even, <= 2048");
  if (rows <= 0) return TLB_OK;
  return launch_rope(x, bias, out, (int)rows, (int)T, (int)D, (unsigned)pos, nullptr, base, S(stream));
}
int tlb_rope_dpos(const float* x, float* out, int64_t rows, int64_t T, int64_t D,
                  const void* d_pos, float base, const float* bias, void* stream) {
  TLB_REQUIRE(x && out && d_pos && D > 0 && (D & 1) == 0 && D <= 2048, "tlb_rope_dpos: bad arguments");
  if (rows <= 0) return TLB_OK;
  return launch_rope(x, bias, out, (int)rows, (int)T, (int)D, 0u, (const unsigned*)d_pos, base,
                     S(stream));
}
int tlb_kv_append(float* Kc, float* Vc, const float* k_new, const float* v_new, int64_t pos,
                  int64_t kv_max, int64_t n_kv, int64_t D, void* stream) {
  TLB_REQUIRE(Kc && Vc && k_new && v_new, "tlb_kv_append: null pointer");
  TLB_REQUIRE(pos >= 0 && pos < kv_max, "tlb_kv_append: pos outside the cache");
  TLB_REQUIRE(D > 0 && D <= 1024 && n_kv > 0, "tlb_kv_append: bad shape");
  CTX(c);
  return launch_kv_append(Kc, Vc, k_new, v_new, (unsigned)pos, nullptr, kv_max, (int)n_kv, (int)D, 0, c->status,
                          S(stream));
}
int tlb_kv_append_bf16(void* Kc, void* Vc, const float* k_new, const float* v_new, int64_t pos,
                       int64_t kv_max, int64_t n_kv, int64_t D, void* stream) {
  TLB_REQUIRE(Kc && Vc && k_new && v_new, "tlb_kv_append_bf16: null pointer");
  TLB_REQUIRE(pos >= 0 && pos < kv_max, "tlb_kv_append_bf16: pos outside the cache");
  TLB_REQUIRE(D > 0 && D <= 1024 && n_kv > 0, "tlb_kv_append_bf16: bad shape");
  CTX(c);
  return launch_kv_append(Kc, Vc, k_new, v_new, (unsigned)pos, nullptr, kv_max, (int)n_kv, (int)D, 1, c->status,
                          S(stream));
}
int tlb_kv_append_dpos(float* Kc, float* Vc, const float* k_new, const float* v_new,
                       const void* d_pos, int64_t kv_max, int64_t n_kv, int64_t D, void* stream) {
  TLB_REQUIRE(Kc && Vc && k_new && v_new && d_pos, "tlb_kv_append_dpos: null pointer");
  TLB_REQUIRE(D > 0 && D <= 1024 && n_kv > 0, "tlb_kv_append_dpos: bad shape");
  CTX(c);
  return launch_kv_append(Kc, Vc, k_new, v_new, 0u, (const unsigned*)d_pos, kv_max, (int)n_kv,
                          (int)D, 0, c->status,
                          S(stream));
}
int tlb_kv_append_dpos_bf16(void* Kc, void* Vc, const float* k_new, const float* v_new,
                            const void* d_pos, int64_t kv_max, int64_t n_kv, int64_t D, void* stream) {
  TLB_REQUIRE(Kc && Vc && k_new && v_new && d_pos, "tlb_kv_append_dpos_bf16: null pointer");
  TLB_REQUIRE(D > 0 && D <= 1024 && n_kv > 0, "tlb_kv_append_dpos_bf16: bad shape");
  CTX(c);
  return launch_kv_append(Kc, Vc, k_new, v_new, 0u, (const unsigned*)d_pos, kv_max, (int)n_kv,
                          (int)D, 1, c->status,
                          S(stream));
}
int tlb_incr_u32(void* d_pos, void* stream) {
  TLB_REQUIRE(d_pos, "tlb_incr_u32: null pointer");
  return launch_incr_u32((unsigned*)d_pos, S(stream));
}
int tlb_argmax_dev(const float* in, int64_t n, void* d_out, void* stream) {
  TLB_REQUIRE(in && d_out && n > 0 && n < (1ll << 31), "tlb_argmax: bad arguments");
  CTX(c);
  return launch_argmax(c, in, (int)n, (int*)d_out, nullptr, S(stream));
}
int tlb_argmax(const float* in, int64_t n, int64_t* out_idx, void* stream) {
  TLB_REQUIRE(in && out_idx && n > 0 && n < (1ll << 31), "tlb_argmax: bad arguments");
  CTX(c);
  int* cell = (int*)(c->argmax_cell + 2);
  int rc = launch_argmax(c, in, (int)n, cell, nullptr, S(stream));
  if (rc) return rc;
  int h = 0;
  TLB_CUDA(cudaMemcpyAsync(&h, cell, sizeof(int), cudaMemcpyDeviceToHost, S(stream)));
  TLB_CUDA(cudaStreamSynchronize(S(stream)));
  *out_idx = h;
  return TLB_OK;
}

int tlb_split_heads(const float* src, const float* bias, float* dst, int64_t T, int64_t ld,
                    int64_t off, int64_t H, int64_t D, void* stream) {
  TLB_REQUIRE(src && dst && T > 0 && H > 0 && D > 0 && D <= 1024 && T <= 65535, "tlb_split_heads: bad arguments");
  return launch_split_heads(src, bias, dst, (int)T, ld, off, (int)H, (int)D, S(stream));
}
int tlb_merge_heads(const float* src, float* dst, int64_t T, int64_t H, int64_t D, void* stream) {
  TLB_REQUIRE(src && dst && T > 0 && H > 0 && D > 0 && D <= 1024 && T <= 65535, "tlb_merge_heads: bad arguments");
  return launch_merge_heads(src, dst, (int)T, (int)H, (int)D, S(stream));
}
int tlb_kv_fill(float* Kc, float* Vc, const float* K, const float* V, int64_t T, int64_t kv_max,
                int64_t n_kv, int64_t D, int64_t pos0, void* stream) {
  TLB_REQUIRE(Kc && Vc && K && V, "tlb_kv_fill: null pointer");
  TLB_REQUIRE(T > 0 && T <= 65535 && pos0 >= 0 && pos0 + T <= kv_max, "tlb_kv_fill: rows outside the cache");
  TLB_REQUIRE(D > 0 && D <= 1024 && n_kv > 0, "tlb_kv_fill: bad shape");
  return launch_kv_fill(Kc, Vc, K, V, (int)T, kv_max, (int)n_kv, (int)D, (int)pos0, 0, S(stream));
}
int tlb_kv_fill_bf16(void* Kc, void* Vc, const float* K, const float* V, int64_t T, int64_t kv_max,
                     int64_t n_kv, int64_t D, int64_t pos0, void* stream) {
  TLB_REQUIRE(Kc && Vc && K && V, "tlb_kv_fill_bf16: null pointer");
  TLB_REQUIRE(T > 0 && T <= 65535 && pos0 >= 0 && pos0 + T <= kv_max, "tlb_kv_fill_bf16: rows outside the cache");
  TLB_REQUIRE(D > 0 && D <= 1024 && n_kv > 0, "tlb_kv_fill_bf16: bad shape");
  return launch_kv_fill(Kc, Vc, K, V, (int)T, kv_max, (int)n_kv, (int)D, (int)pos0, 1, S(stream));
}
static int attn_prefill_any(const float* q, const void* K, const void* V, float* out, int64_t n_q,
                            int64_t n_kv, int64_t T, int64_t kv_max, int64_t D, float scale, int64_t pos0,
                            void* stream, int bf) {
  TLB_REQUIRE(q && K && V && out, "tlb_attn_prefill: null pointer");
  TLB_REQUIRE(D == 64 || D == 128, "tlb_attn_prefill: D must be 64 or 128");
  TLB_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "tlb_attn_prefill: n_q % n_kv != 0");
  TLB_REQUIRE(T > 0 && T <= 65535 && pos0 >= 0 && pos0 + T <= kv_max, "tlb_attn_prefill: chunk outside the cache");
  TLB_REQUIRE((((uintptr_t)q | (uintptr_t)K | (uintptr_t)V | (uintptr_t)out) & 15) == 0,
              "tlb_attn_prefill: pointers must be 16-byte aligned");
  CTX(c);
  return launch_attn_prefill(c, q, K, V, out, (int)n_q, (int)n_kv, (int)T, kv_max, (int)D, scale,
                             (int)pos0, bf, S(stream));
}
int tlb_attn_prefill(const float* q, const float* K, const float* V, float* out, int64_t n_q,
                     int64_t n_kv, int64_t T, int64_t kv_max, int64_t D, float scale, int64_t pos0,
                     void* stream) {
  return attn_prefill_any(q, K, V, out, n_q, n_kv, T, kv_max, D, scale, pos0, stream, 0);
}
int tlb_attn_prefill_bf16(const float* q, const void* K, const void* V, float* out, int64_t n_q,
                          int64_t n_kv, int64_t T, int64_t kv_max, int64_t D, float scale, int64_t pos0,
                          void* stream) {
  return attn_prefill_any(q, K, V, out, n_q, n_kv, T, kv_max, D, scale, pos0, stream, 1);
}

int tlb_capture_begin(void** stream_out) {
  TLB_REQUIRE(stream_out, "tlb_capture_begin: null pointer");
  CTX(c);
  if (c->capturing) return set_error(TLB_ERR_STATE, "capture already in progress");
  TLB_CUDA(cudaDeviceSynchronize());
  if (!c->cap_stream) TLB_CUDA(cudaStreamCreateWithFlags(&c->cap_stream, cudaStreamNonBlocking));
  TLB_CUDA(cudaStreamBeginCapture(c->cap_stream, cudaStreamCaptureModeThreadLocal));
  c->capturing = true;
  *stream_out = c->cap_stream;
  return TLB_OK;
}
int tlb_capture_end(void** graph_exec_out) {
  TLB_REQUIRE(graph_exec_out, "tlb_capture_end: null pointer");
  CTX(c);
  if (!c->capturing) return set_error(TLB_ERR_STATE, "capture_end without capture_begin");
  c->capturing = false;
  cudaGraph_t g = nullptr;
  TLB_CUDA(cudaStreamEndCapture(c->cap_stream, &g));
  cudaGraphExec_t e = nullptr;
  cudaError_t err = cudaGraphInstantiate(&e, g, 0);
  cudaGraphDestroy(g);
  if (err != cudaSuccess) return cuda_fail(err, "cudaGraphInstantiate");
  *graph_exec_out = e;
  return TLB_OK;
}
int tlb_graph_launch(void* graph_exec, void* stream) {
  TLB_REQUIRE(graph_exec, "tlb_graph_launch: null graph");
  TLB_CUDA(cudaGraphLaunch((cudaGraphExec_t)graph_exec, S(stream)));
  return TLB_OK;
}
int tlb_graph_destroy(void* graph_exec) {
  if (graph_exec) TLB_CUDA(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec));
  return TLB_OK;
}

}  // extern "C"
