// Host-side interface of the tile-packed int4 GEMV (gemv_q4p.cu) for the other
// translation units of the library.
#pragma once

#include "comm.cuh"
#include "q4_mma.cuh"

namespace tlb {

// How the NEXT weight-streaming kernel on the stream will walk its packed matrix: enough for
// the kernel in front of it to ask the L2 for the bytes that kernel's CTAs request first
// (their first ring fill), at the moment its own stream runs dry.  The weights of a decoder
// depend on nothing, so the HBM would otherwise idle through the next launch's dependency
// wait and activation prep.  wp == NULL: nothing to prefetch.
struct GvStream {
  const unsigned char* wp = nullptr;
  unsigned U = 0;                 // units of 2560 bytes
  int SL = 0, RT = 0;             // slabs per row tile, row tiles
  int KB = 0;                     // 0: warps own unit ranges; >= 1: CTA-owned blocks, KB slab blocks
  int grid = 0, stages = 0;       // CTAs of that launch, ring slots per warp
};

// What happens to a pair (a, b) = (y[r], y[r + pair_h]) of a pair-packed matrix.
struct PairEpi {
  int kind = 0;        // 0: none (rows written as they are); 1: SwiGLU; 2: q/k/v bias + rope + cache row
  int H = 0;           // pair distance in original rows
  float* out = nullptr;          // kind 1: h[pair index]; kind 2: rotated q [n_q * D]
  float* Kc = nullptr;           // kind 2: caches [n_kv, kv_max, D], row *d_pos is written
  float* Vc = nullptr;
  const float* bq = nullptr;
  const float* bk = nullptr;
  const float* bv = nullptr;
  int n_q = 0, n_kv = 0, D = 0;
  int kv_bf16 = 0;               // kind 2: the caches hold bf16 (rows rounded to nearest even)
  const unsigned* d_pos = nullptr;
  long long kv_stride = 0;
  int kv_rows = 0;               // capacity of the caches in rows: a position at or beyond it is refused
  float base = 0.f;
  const float2* rope_cs = nullptr;  // optional [D/2] (cos, sin) of position *d_pos
};

long long q4p_bytes(long long N, long long K);
bool gemv_q4p_supported(long long N, long long K);
// pair_h = 0: rows in their own order; > 0: rows r and r + pair_h share a thread (see gemv_q4p.cu)
int launch_q4_pack(const void* q4, int N, int K, void* out, int pair_h, cudaStream_t s);
int gemv_q4p_launch(DeviceCtx* c, const void* packed, const float* x, float* y, int N, int K,
                    float alpha, float beta, cudaStream_t stream, int max_ctas,
                    const CommDev* push_comm, int act, const float* delta, const float* nw,
                    float* xout, float eps, const PairEpi* epi, const CommDev* pull_comm,
                    const GvStream* prefetch = nullptr);
// One phase of a chain: y = W . prep(x) with the optional fused add+norm prologue (act 2) and
// pair epilogue of gemv_q4p_launch; alpha = 1, beta = 0, single GPU.
struct GvPhase {
  const void* packed = nullptr;
  const float* x = nullptr;
  float* y = nullptr;
  int N = 0, K = 0, act = 0;
  const float* delta = nullptr;
  const float* nw = nullptr;
  float* xout = nullptr;
  float eps = 0.f;
  const PairEpi* epi = nullptr;
};
int gemv_q4p_chain_launch(DeviceCtx* c, const GvPhase* ph, int nph, cudaStream_t stream, bool* fused);
// The walk a launch with these arguments would take (same decisions as gemv_q4p_launch).
int gemv_q4p_stream_of(DeviceCtx* c, const void* packed, int N, int K, int act, bool has_epi, int max_ctas,
                       GvStream* out);

#ifdef __CUDACC__
__device__ __forceinline__ void l2_prefetch(const void* ptr, unsigned bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr), "r"(bytes) : "memory");
}
// Called by ONE warp: lanes 0..15 stand for the 16 warps of CTA `cta` of the launch `n`
// describes and request what that warp (unit-range mode) or that CTA (owned-block mode)
// streams first.  The address arithmetic mirrors gemv_q4p_kernel.
__device__ __forceinline__ void gv_prefetch_head(const GvStream& n, unsigned cta, int lane) {
#ifdef TLB_PK_WARPS
  constexpr unsigned UNIT = 2560, WARPS = TLB_PK_WARPS;
#else
  constexpr unsigned UNIT = 2560, WARPS = 16;
#endif
  if (lane >= (int)WARPS || cta >= (unsigned)n.grid) return;
  if (n.KB == 0) {
    const unsigned Wall = (unsigned)n.grid * WARPS, Wtot = Wall < n.U ? Wall : n.U;
    const unsigned wid = cta * WARPS + (unsigned)lane;
    if (wid >= Wtot) return;
    const GvSplit sp = {n.U / Wtot, n.U % Wtot};
    const unsigned u0 = gv_start(wid, sp), u1 = gv_start(wid + 1, sp);
    unsigned cnt = u1 - u0;
    if (cnt > (unsigned)n.stages) cnt = (unsigned)n.stages;
    if (cnt) l2_prefetch(n.wp + (size_t)u0 * UNIT, cnt * UNIT);
    return;
  }
  // owned blocks: the CTA's first 16 * stages units in (row tile, slab) order are whole runs of
  // ks consecutive units, one run per row tile; lane l requests run l
  const unsigned KB = (unsigned)n.KB, RB = (unsigned)n.grid / KB;
  const unsigned rb = cta / KB, kb = cta - rb * KB;
  const GvSplit ct = {(unsigned)n.RT / RB, (unsigned)n.RT % RB};
  const GvSplit cs = {(unsigned)n.SL / KB, (unsigned)n.SL % KB};
  const unsigned tile_b = gv_start(rb, ct), tiles = gv_start(rb + 1, ct) - tile_b;
  const unsigned s_b = gv_start(kb, cs), ks = gv_start(kb + 1, cs) - s_b;
  if (!ks) return;
  unsigned want = tiles * ks;
  if (want > WARPS * (unsigned)n.stages) want = WARPS * (unsigned)n.stages;
  const unsigned runs = (want + ks - 1) / ks;
  if ((unsigned)lane < runs)
    l2_prefetch(n.wp + ((size_t)(tile_b + (unsigned)lane) * n.SL + s_b) * UNIT, ks * UNIT);
}
#endif

}  // namespace tlb
