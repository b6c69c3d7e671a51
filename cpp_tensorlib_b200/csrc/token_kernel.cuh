// Phase table and parameters of the persistent per-token decoder kernel
// (token_kernel.cu); shared with the decoder driver that builds the table.
#pragma once

#include "q4_mma.cuh"

namespace tlb {

constexpr int TK_WARPS = 16;
constexpr int TK_THREADS = TK_WARPS * 32;
constexpr int TK_STAGES = 3;
constexpr int TK_ATT_TK = 16;      // keys per attention tile
constexpr int TK_ATT_STAGES = 4;
constexpr int TK_HW = 2;           // q heads per warp in the attention phase

struct TkPhase {
  int type;  // 0 = GEMV, 1 = attention
  // ---- GEMV
  int N, K, RT, SL;
  unsigned U, Wtot, q, r;   // unit split over min(grid warps, U) workers
  int act;                  // 0 x as given, 1 swiglu([gate|up]), 2 rmsnorm(x + delta) * nw
  int argmax;               // reduce the outputs to the argmax key as well
  int map;                  // tensor-map pair index (2*map = nibbles, 2*map+1 = scales)
  int x_from_embed;         // x = embed + token * K (layer 0)
  int cta_tiles;            // 1: CTAs own whole row tiles, warps split K (see token_kernel.cu)
  const float* x;
  const float* delta;
  const float* nw;
  float* xout;
  float* y;
  // ---- attention
  float* qkv;
  const float* bq;
  const float* bk;
  const float* bv;
  float* Kc;
  float* Vc;
  float* att;
};

struct TkParams {
  const TkPhase* phases;
  int n_phases;
  const CUtensorMap* maps;
  int n_q, n_kv, hd, max_ctx;
  float eps, rope_base, scale;
  const float* embed;
  unsigned* d_pos;
  int* d_tok;
  int* d_tok_out;
  float* gemv_partials;
  int* gemv_counters;
  float* attn_partials;   // [n_q][s_cap][D+4]
  int* attn_counters;     // [n_kv]
  int attn_s_cap;
  int sm2;
  unsigned long long* argmax_cell;
  unsigned* bar;          // [0] arrivals, [1] generation
  int* status;
  unsigned long long* dbg;  // optional: [n_phases][4] %globaltimer stamps of CTA 0 (diagnostics)
};

struct TkSmem {
  size_t w_ring, s_ring, bars, red, rope, region, total;
  // GEMV view of the region
  size_t pslab, q, bfrag;
  // attention view of the region
  size_t at_k, at_v, at_bars, at_q, at_new, at_mrg;
};
__host__ __device__ inline size_t tk_gemv_view_bytes(int K) {
  const int SL = (K + 255) / 256, G = SL * 8;
  size_t g = (size_t)SL * sizeof(float);
  g = (g + 15) & ~(size_t)15;
  g += (size_t)G * sizeof(float);
  g = (g + 15) & ~(size_t)15;
  g += (size_t)G * 2 * 4 * sizeof(uint4);
  return g;
}
// k_attn_in: K of the projection that runs right before an attention phase (its
// activation fragments must stay clear of the K/V tiles prefetched during it).
__host__ __device__ inline TkSmem tk_smem_layout(int k_max, int k_attn_in, int hd, int grp) {
  TkSmem L;
  size_t o = 0;
  L.w_ring = o; o += (size_t)TK_WARPS * TK_STAGES * GVU_W_BYTES;
  L.s_ring = o; o += (size_t)TK_WARPS * TK_STAGES * GVU_S_BYTES;
  L.bars = o;   o += (size_t)TK_WARPS * TK_STAGES * 8;
  L.at_bars = o; o += 64;  // attention tile barriers (outside the aliased region)
  L.red = o;    o += 512 * sizeof(float);  // block reductions / [16 warps][16 rows] tile partials
  L.rope = o;   o += (size_t)hd * sizeof(float);  // cos[hd/2], sin[hd/2] of this token's position
  o = (o + 127) & ~(size_t)127;
  L.region = o;
  const int SL = (k_max + 255) / 256, G = SL * 8;
  size_t g = o;
  L.pslab = g; g += (size_t)SL * sizeof(float);
  g = (g + 15) & ~(size_t)15;
  L.q = g;     g += (size_t)G * sizeof(float);
  g = (g + 15) & ~(size_t)15;
  L.bfrag = g; g += (size_t)G * 2 * 4 * sizeof(uint4);
  size_t a = o + ((tk_gemv_view_bytes(k_attn_in) + 127) & ~(size_t)127);
  const size_t tile = (size_t)TK_ATT_TK * hd * 4;
  L.at_k = a; a += TK_ATT_STAGES * tile;
  L.at_v = a; a += TK_ATT_STAGES * tile;
  L.at_q = a; a += (size_t)grp * hd * 4;
  L.at_new = a; a += (size_t)2 * hd * 4;
  L.at_mrg = L.at_k;  // merge buffers reuse the K tiles once every tile is consumed
  L.total = (g > a ? g : a) + 1024;
  return L;
}


int token_kernel_launch(const TkParams& P, int D, int k_max, int k_attn_in, int sm_count,
                        cudaStream_t stream);

}  // namespace tlb
