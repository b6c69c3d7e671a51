// Launch parameters and the context-split plan shared by the decode attention kernels
// (attn_decode.cu: CUDA-core form; attn_decode_mma.cu: tensor-core form for GQA groups).
// Both kernels derive a CTA's key range from the context length with the functions below, on
// the host and on the device alike, which is what keeps the device-position variant
// bit-identical to the host-position one.
#pragma once

#include "attn_common.cuh"
#include "gemv_q4p.cuh"

namespace tlb {

// Diagnostics: when set, every launch records per-CTA phase timestamps there.
extern unsigned long long* g_attn_dbg;
constexpr int AT_TK = 32;  // keys per tile

struct AttnParams {
  const float* q;
  const void* K;   // f32 or bf16 cache (template parameter BF of the kernel)
  const void* V;
  float* out;
  float* partials;     // [n_q][S_cap][D+4]  (acc[D], m, l, pad, pad)
  int* counters;       // [n_kv], zero between launches
  const unsigned* d_pos;  // nullptr: use ctx
  int ctx;
  int n_q, n_kv, grp;
  long long kv_stride;  // kv_max * D
  int kv_rows;          // kv_max: a device-resident position at or beyond it is refused
  float scale;
  int s_cap;     // partial slots per head (= launched splits)
  int sm2;       // CTA target of the grid (attn_target): split count = target / kv heads
  int* status;
  int early_kv;  // cache rows below ctx-1 and *d_pos are older than the preceding kernel:
                 // their tiles may be requested before the grid dependency resolves
  unsigned long long* dbg;
  GvStream pf;   // head of the next kernel's weight stream to request from the L2 (wp == NULL: none)
};

// CTAs the grid should have: one per SM for wide groups (4 heads per warp: one CTA fits an
// SM), two per SM otherwise.
__host__ __device__ inline int attn_target(int grp, int sm_count) {
  return grp >= 3 ? sm_count : 2 * sm_count;
}
// Number of splits wanted for a context length (monotone non-decreasing in ctx).
__host__ __device__ inline int attn_splits_wanted(int n_kv, int ctx, int sm2) {
  int s = sm2 / (n_kv > 0 ? n_kv : 1);
  int cap = (ctx + 63) / 64;     // never less than 64 keys (2 tiles) per split
  if (s > cap) s = cap;
  if (s > 96) s = 96;  // the merge keeps (m, l) of at most 3 splits per lane
  return s < 1 ? 1 : s;
}
// Keys per split: ceil(ctx / wanted) rounded up to a whole tile.
__host__ __device__ inline int attn_chunk(int n_kv, int ctx, int sm2) {
  int s = attn_splits_wanted(n_kv, ctx, sm2);
  int chunk = (ctx + s - 1) / s;
  chunk = (chunk + AT_TK - 1) / AT_TK * AT_TK;
  return chunk < AT_TK ? AT_TK : chunk;
}


}  // namespace tlb
