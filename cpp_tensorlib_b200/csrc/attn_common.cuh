// Lane-to-dims mapping and key-row loads shared by the decode and the prefill attention
// kernels, for f32 and bf16 caches.
#pragma once

#include "common.cuh"

namespace tlb {

// first dim of a lane's j-th float4 of q / acc / a key row
template <int LPK, bool BF>
__device__ __forceinline__ int attn_dim0(int sub, int j) {
  return BF ? 8 * (sub + LPK * (j >> 1)) + 4 * (j & 1) : 4 * (sub + LPK * j);
}
// the lane's CH float4 of one key row held in a tile (f32 as it is, bf16 widened)
template <int D, int LPK, int CH, bool BF>
__device__ __forceinline__ void attn_load_row(const unsigned char* row, int sub, float4 (&kv)[CH]) {
  if (BF) {
#pragma unroll
    for (int jj = 0; jj < CH / 2; jj++) {
      const uint4 w = *(const uint4*)(row + (size_t)(sub + LPK * jj) * 16);
      kv[2 * jj] = make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u),
                               __uint_as_float(w.y << 16), __uint_as_float(w.y & 0xffff0000u));
      kv[2 * jj + 1] = make_float4(__uint_as_float(w.z << 16), __uint_as_float(w.z & 0xffff0000u),
                                   __uint_as_float(w.w << 16), __uint_as_float(w.w & 0xffff0000u));
    }
  } else {
#pragma unroll
    for (int j = 0; j < CH; j++) kv[j] = *(const float4*)(row + (size_t)(sub + LPK * j) * 16);
  }
}

}  // namespace tlb
