// Host-side interface of the tile-packed int4 GEMV (gemv_q4p.cu) for the other
// translation units of the library.
#pragma once

#include "comm.cuh"

namespace tlb {

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
                    float* xout, float eps, const PairEpi* epi, const CommDev* pull_comm);

}  // namespace tlb
