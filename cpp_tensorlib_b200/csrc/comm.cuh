// Tensor-parallel exchange over NVLink peer memory (plain ld/st to peer-mapped
// buffers; no multicast of any kind).
//
// One-shot all-reduce of a short f32 vector, split across two kernels so that the
// transfer overlaps the producer's compute tile by tile:
//   * the row-parallel GEMV stores every finished output tile straight into the
//     staging buffer of EVERY rank (its own included) and, when the last of its
//     warps is done, publishes a sequence number in every rank's flag word;
//   * the following residual-add + RMSNorm kernel waits (bounded) for the flags
//     of all ranks, sums the partials in rank order -- every rank adds the same
//     numbers in the same order, so the replicated residual streams stay
//     bit-identical -- and continues into the norm.
// Staging is double-buffered by the parity of the sequence number: a rank can
// only be one all-reduce ahead of the slowest peer, because its next push waits
// for its own reduce, which needs every peer's previous push.
#pragma once

#include "common.cuh"

namespace tlb {

constexpr int TP_MAX = 8;

struct CommDev {
  int rank = 0, size = 1;
  int slot_floats = 0;            // floats per (parity, rank) slot
  float* stage[TP_MAX] = {};      // stage[r]: rank r's staging [2][size][slot_floats]
  unsigned* flags[TP_MAX] = {};   // flags[r]: rank r's flag words [2][size]
  unsigned* seq = nullptr;        // local: number of completed exchanges
  unsigned* done = nullptr;       // local: arrival counter of the pushing kernel
};

#ifdef __CUDACC__
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Wait until *p == want, at most ~1 s; false (and the status block set) on timeout.
__device__ __forceinline__ bool wait_flag_bounded(const unsigned* p, unsigned want, int* status,
                                                  int where) {
  const long long t0 = clock64();
  while (ld_acquire_sys(p) != want) {
    // once any wait has expired, later ones give up at once so a broken exchange
    // costs one timeout, not one per all-reduce
    if (status && *(volatile int*)&status[ST_WAIT_TIMEOUT]) return false;
    if (clock64() - t0 > 2000000000ll) {
      if (status) {
        atomicExch(&status[ST_WAIT_TIMEOUT], 1);
        atomicExch(&status[ST_WAIT_WHERE], where);
      }
      return false;
    }
    __nanosleep(20);
  }
  return true;
}
#endif

}  // namespace tlb
