// Tensor-parallel exchange over NVLink peer memory (plain ld/st to peer-mapped
// buffers; no multicast of any kind).
//
// One-shot all-reduce of a short f32 vector, fused into its producer and its
// consumer so the transfer overlaps the producer's compute tile by tile:
//   * the row-parallel GEMV stores every finished output element straight into the
//     staging buffer of EVERY rank (its own included) as an 8-byte packet
//     {value bits, sequence number + 1}, written and read as ONE 64-bit access
//     (st / ld .relaxed.sys.b64): a naturally aligned 64-bit scalar access is
//     single-copy atomic in the PTX memory model (a two-element vector access is
//     not -- it is modelled as two scalar accesses in unspecified order), so a
//     reader sees the old packet or the new one, never a mix, and the packet
//     validates itself: no fence, no separate flag, no completion counter -- the
//     exchange costs one NVLink store latency after the last tile;
//   * the following residual-add + RMSNorm kernel polls (bounded) each packet until
//     its tag matches, sums the partials in rank order -- every rank adds the same
//     numbers in the same order, so the replicated residual streams stay
//     bit-identical -- and continues into the norm.
// Staging is double-buffered by the parity of the sequence number: a rank can
// only be one exchange ahead of the slowest peer, because its next push waits
// for its own reduce, which needs every peer's previous push.
// The sequence number of an exchange is (tokens decoded so far) * E + k: the token
// counter lives in device memory and is advanced once per token by the last exchange
// (the argmax), k is the exchange's fixed index inside a token and E their number, so
// producers and consumers of any grid size derive the same tag without writing it.
#pragma once

#include "common.cuh"

namespace tlb {

constexpr int TP_MAX = 8;

struct CommDev {
  int rank = 0, size = 1;
  int slot_floats = 0;            // packets per (parity, rank) slot
  uint2* stage[TP_MAX] = {};      // stage[r]: rank r's staging [2][size][slot_floats] packets
  unsigned* seq = nullptr;        // local: tokens decoded so far (advanced by the argmax exchange)
  int k = 0, E = 1;               // this exchange's index inside a token, exchanges per token
};

#ifdef __CUDACC__
__device__ __forceinline__ unsigned comm_seq(const CommDev& c) {
  return *(volatile unsigned*)c.seq * (unsigned)c.E + (unsigned)c.k;
}
// packet = (tag << 32) | value bits, little endian: .x = value, .y = tag
__device__ __forceinline__ void st_packet_sys(uint2* p, float v, unsigned tag) {
  const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
  asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 ld_packet_sys(const uint2* p) {
  unsigned long long w;
  asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return make_uint2((unsigned)(w & 0xffffffffull), (unsigned)(w >> 32));
}
// Poll a packet until its tag matches, at most the wait limit of the status block (about
// one second by default); on timeout the status block is set, later waits give up at
// once, and the (stale) payload is returned.
__device__ __forceinline__ uint2 wait_packet_bounded(const uint2* p, unsigned tag, int* status,
                                                     int where) {
  uint2 v = ld_packet_sys(p);
  if (v.y == tag) return v;
  const long long t0 = clock64();
  // the status block is a second L2 round trip: look at it (the limit, another waiter's
  // timeout) once in 32 polls, so that the common case costs one load per poll
  long long limit = 1ll << 62;
  for (unsigned spin = 1;; spin++) {
    v = ld_packet_sys(p);
    if (v.y == tag) return v;
    if ((spin & 31u) == 0) {
      limit = wait_limit(status);
      if (status && *(volatile int*)&status[ST_WAIT_TIMEOUT]) return v;
    }
    if (clock64() - t0 > limit) {
      if (status) {
        atomicExch(&status[ST_WAIT_TIMEOUT], 1);
        atomicExch(&status[ST_WAIT_WHERE], where);
      }
      return v;
    }
    __nanosleep(20);
  }
}
#endif

}  // namespace tlb
