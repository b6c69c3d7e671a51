// Device helpers shared by the int4 GEMV kernels:
// the unit-range split, the acq_rel ticket, the mma.sync wrappers.
#pragma once

#include "common.cuh"

namespace tlb {

constexpr int GVU_W_BYTES = 2048;  // one unit of nibbles: 16 rows x 128 B (256 k)
constexpr int GVU_S_BYTES = 512;   // its scales: 16 rows x 8 f32

// Unit ranges: with q = U / W and r = U % W, worker w owns q+1 units when w < r,
// else q, contiguously.  start(w) needs no division; owner(u) needs one 32-bit one.
struct GvSplit {
  unsigned q, r;
};
__device__ __forceinline__ unsigned gv_start(unsigned w, GvSplit sp) {
  return w * sp.q + (w < sp.r ? w : sp.r);
}
__device__ __forceinline__ unsigned gv_owner(unsigned u, GvSplit sp) {
  const unsigned big = sp.r * (sp.q + 1u);
  return u < big ? u / (sp.q + 1u) : sp.r + (u - big) / sp.q;
}
__device__ __forceinline__ unsigned atom_add_acq_rel(int* p, int v) {
  int old;
  asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return (unsigned)old;
}

// D = A*B (first MMA of a group: zero accumulator input)
__device__ __forceinline__ void mma16816_z(float (&c)[4], unsigned a0, unsigned a1, unsigned a2,
                                           unsigned a3, unsigned b0, unsigned b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2,
                                         unsigned a3, unsigned b0, unsigned b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned pack_h2(__half a, __half b) {
  return (unsigned)__half_as_ushort(a) | ((unsigned)__half_as_ushort(b) << 16);
}


}  // namespace tlb
