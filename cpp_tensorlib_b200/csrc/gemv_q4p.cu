// Decode GEMV (M = 1) on the library's own tile-packed int4 layout.
// y[n] = alpha * sum_k x[k] * sc[n,k/32] * (nib[n,k]-8) + beta -- the arithmetic of
// tl_gemv_q4 (kernels/tensorlib_cuda.cu:772-796) on weights that were repacked once,
// on the device, from the reference's q4 storage (include/types.h:15-31).
//
// Why a second layout.  Read through 2-D tensor maps, the reference layout costs one
// TMA row request per 128 B of nibbles and per 32 B of scales; the request rate, not
// HBM, then bounds the stream (the scales alone cost 28 of 73 us on a 152064 x 3584
// matrix).  Packed, a work unit (16 rows x 256 k: 2048 B of nibbles + 512 B of
// scales) is one contiguous 2560-byte block, units follow each other in the order
// the kernel consumes them, and every warp streams its own contiguous byte range with
// one bulk copy per unit.
//
// Inside a unit the nibble words are stored in the order the MMA fragments want them:
// 16-byte chunk i of lane l = (g, t) holds {row g, row g+8} x {group 2i, group 2i+1},
// word 4*group + t of the row's 32 words -- four conflict-free LDS.128 per unit and
// no swizzle arithmetic.  Scales follow as [16 rows][8 groups] f32.
//
// Arithmetic.  A masked nibble word is read as two fp16 subnormals (nib * 2^-24, or
// nib * 2^-20 for the odd nibble of a byte) and is the A operand of mma.sync
// m16n8k16; the activation is the B operand.  Per slab of 256 k the activation is
// turned into 24-bit fixed point (round to nearest, relative to the slab's power-of-
// two bound) and split into two balanced 12-bit digits, which fp16 holds exactly: every
// product and every partial sum inside the MMA is a small integer multiple of 2^-24,
// so the tensor-core accumulation is exact whatever its internal rounding, and the
// only approximation is the fixed-point step (2^-24 of the slab maximum per element,
// the size of an f32 rounding error of the reference's own accumulation).  Per group of 32 k:
// acc += sc * (c_hi + 2^-12 c_lo), the -8 offset as 8 * sc * sum(x_g) from the same
// fixed-point values.
//
// Split-K falls out of the unit ranges; partial row tiles are combined by the
// last-arriving warp in worker order (deterministic, no float atomics, no spin-wait
// on another CTA).
//
// Structure of this file: the work of a launch is a device function (gemv_q4p_body) over the
// launch's parameters, a ring state and a producer cursor.  gemv_q4p_kernel calls it once.
// gemv_q4p_chain_kernel / gemv_q4p_chain_loop_kernel (opt-in) call it once per phase for up to
// four projections that depend on each other, with a grid-wide arrival counter between the
// phases -- the one place in the library where CTAs of a launch wait for each other; the
// wait is bounded and reports through the status block.
#include <cuda_bf16.h>

#include <cstdlib>
#include <cstring>

#include "gemv_q4p.cuh"
#include "q4_mma.cuh"

namespace tlb {

constexpr int PK_UNIT = 2560;
// Warps per CTA and CTAs per SM: 16 x 1 (one CTA owns the SM's shared memory), or 8 x 2 when
// built with -DTLB_PK_WARPS=8 (two half-size CTAs per SM, so that a CTA of the NEXT kernel can
// become resident, and request its weights, as soon as ONE of the two exits).
#ifndef TLB_PK_WARPS
#define TLB_PK_WARPS 16
#endif
constexpr int PK_WARPS = TLB_PK_WARPS;
constexpr int PK_CTAS_PER_SM = 16 / PK_WARPS;
static_assert(PK_WARPS == 16 || PK_WARPS == 8, "16 warps x 1 CTA or 8 warps x 2 CTAs per SM");
// dynamic shared memory a CTA may ask for: the 227 KB of an SM less the kernels' static part
// (the warps' producer cursors, the chain's epoch)
constexpr int PK_DYN_SMEM_MAX = 224 * 1024;
constexpr int PK_CTA_UNITS = 144; // most units one CTA may own in the CTA-owned modes

long long q4p_bytes(long long N, long long K) {
  const long long RT = (N + 15) / 16, SL = (K + 255) / 256;
  return RT * SL * PK_UNIT;
}

// One CTA per unit: 128 threads write the nibble chunks, 128 the scales.  Rows past N
// and k past K are filled with nibble 8 / scale 0 (weight value zero).
//
// pair_h > 0 additionally permutes the rows so that original rows r and r + pair_h of
// every block of 2*pair_h rows (a rotary pair of a head, pair_h = D/2; a gate row and
// its up row, pair_h = ff) become local rows g and g + 8 of one tile.  Both values of
// a pair then end up in the same thread of the GEMV, whose epilogue can apply
// rope / SwiGLU without another kernel.  Packed row T*16 + lr holds original row
// (pi / H) * 2H + pi % H + (lr >> 3) * H with pi = T*8 + (lr & 7).
__host__ __device__ inline int q4p_orig_row(int packed_row, int pair_h) {
  if (pair_h <= 0) return packed_row;
  const int T = packed_row >> 4, lr = packed_row & 15;
  const int pi = T * 8 + (lr & 7);
  return (pi / pair_h) * 2 * pair_h + pi % pair_h + (lr >> 3) * pair_h;
}

__global__ void q4_pack_kernel(const unsigned char* __restrict__ q4, int N, int K, int SL,
                               unsigned char* __restrict__ out, int pair_h) {
  const int unit = blockIdx.x, rt = unit / SL, s = unit - rt * SL;
  const int tid = threadIdx.x;
  const unsigned* words = (const unsigned*)q4;                       // [N][K/8]
  const float* scales = (const float*)(q4 + (size_t)N * K / 2);      // [N][K/32]
  unsigned char* u = out + (size_t)unit * PK_UNIT;
  if (tid < 128) {
    const int i = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    unsigned w[4];
#pragma unroll
    for (int c = 0; c < 4; c++) {
      const int row = q4p_orig_row(rt * 16 + g + ((c & 1) ? 8 : 0), pair_h);
      const int j = s * 32 + 4 * (2 * i + (c >> 1)) + t;
      w[c] = (row < N && j * 8 < K) ? words[(size_t)row * (K / 8) + j] : 0x88888888u;
    }
    ((uint4*)u)[i * 32 + lane] = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    const int j = tid - 128, r = j >> 3, jj = j & 7;
    const int row = q4p_orig_row(rt * 16 + r, pair_h), grp = s * 8 + jj;
    ((float*)(u + 2048))[j] = (row < N && grp * 32 < K) ? scales[(size_t)row * (K / 32) + grp] : 0.f;
  }
}

int launch_q4_pack(const void* q4, int N, int K, void* out, int pair_h, cudaStream_t s) {
  const int RT = (N + 15) / 16, SL = (K + 255) / 256;
  if (pair_h > 0 && (N % 16 != 0 || pair_h % 8 != 0 || N % (2 * pair_h) != 0))
    return set_error(TLB_ERR_ARG, "q4_pack: paired rows need N % 16 == 0, pair_h % 8 == 0, N % (2 pair_h) == 0");
  q4_pack_kernel<<<RT * SL, 256, 0, s>>>((const unsigned char*)q4, N, K, SL, (unsigned char*)out, pair_h);
  TLB_CUDA(cudaGetLastError());
  return TLB_OK;
}

struct GemvPParams {
  const unsigned char* wp;
  const float* x;
  float* y;
  int N, K, SL, RT;
  unsigned U;
  float alpha, beta;
  float* partials;  // [workers][2][16]
  int* counters;    // [row tiles]
  int* status;
  int x_vec_ok;
  int act;          // 0: x as given; 1: x = [gate(K) | up(K)] -> silu(gate)*up;
                    // 2: x = rmsnorm(x + delta) * nw, the sum also written to xout;
                    // 3: as 2 with delta = the ranks' partial vectors of a tensor-parallel
                    //    exchange, polled from this rank's staging and summed in rank order
  const float* delta;
  const float* nw;
  float* xout;
  float eps;
  int push;         // tensor-parallel: store y into every rank's staging slot (comm = that exchange)
                    // (act 3 reads comm instead: a launch pulls or pushes, never both)
  PairEpi epi;
  int cta_tiles;    // 0: warps own unit ranges.  KB >= 1: CTA-owned blocks, the grid is
                    // RB row blocks x KB slab blocks; a CTA reduces its block in shared memory.
                    // KB == 1 (small matrices): whole rows, results final.  KB > 1 (long rows):
                    // a CTA prepares only its own slabs of the activation; the KB partial blocks
                    // of a row block are folded by the last CTA to arrive
  int slabs;        // activation slabs a CTA holds in shared memory (SL, or the largest slab block)
  int grid;         // CTAs that work on this launch / phase (a chain's grid can be larger)
  // the splits of units over warps (unit ranges) or of row tiles / slabs over CTAs (owned
  // blocks), divided out on the host: a run-time division is two dozen instructions of a
  // prologue that runs from a cold instruction cache
  unsigned Wtot, RB;
  GvSplit sp, ct, cs;
  CommDev comm;
  GvStream pf;      // what the next weight-streaming kernel reads first (wp == NULL: nothing)
};

struct GemvPSmem {
  size_t ring, bars, red, ures, pslab, q, bfrag, total;
};
__host__ __device__ inline GemvPSmem gemvp_smem_layout(int stages, int SL) {
  GemvPSmem L;
  size_t o = 0;
  L.ring = o;  o += (size_t)PK_WARPS * stages * PK_UNIT;
  L.bars = o;  o += (size_t)PK_WARPS * stages * 8;
  o = (o + 15) & ~(size_t)15;
  L.red = o;   o += 32 * sizeof(float);
  L.ures = o;  o += (size_t)PK_CTA_UNITS * 16 * sizeof(float);
  L.pslab = o; o += (size_t)((SL + 3) & ~3) * sizeof(float);
  L.q = o;     o += (size_t)SL * 8 * sizeof(float);
  L.bfrag = o; o += (size_t)SL * 1024;          // [SL*8 groups][hi, lo][4] uint4
  L.total = o + 128;                            // slack for the 128-byte alignment of the base
  return L;
}

template <int OFF>
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a), "n"(OFF) : "memory");
  return v;
}
template <int OFF>
__device__ __forceinline__ float4 lds128f(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4+%5];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a), "n"(OFF) : "memory");
  return v;
}
template <int OFF>
__device__ __forceinline__ float2 lds64f(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2+%3];" : "=f"(v.x), "=f"(v.y) : "r"(a), "n"(OFF) : "memory");
  return v;
}
__device__ __forceinline__ float lds32f(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
  return v;
}

// One warp's share of a launch (or of one phase of a chain): which units it streams and how
// they map to (row tile, slab).
struct GvWarp {
  bool idle;
  unsigned u0, u1, wid, kb, rb;
  GvSplit sp;
  int n_units, tile_b, n_loc, s_b, ks, rt, s;
};
__device__ __forceinline__ void gv_warp_setup(const GemvPParams& p, int warp, GvWarp& w) {
  const int SL = p.SL;
  const unsigned grid = (unsigned)p.grid;
  const bool in_grid = blockIdx.x < grid;
  // Never more workers than units, so every worker's range is non-empty and the
  // contributors of a row tile are exactly the owners of its first..last unit.
  const unsigned Wtot = p.Wtot;
  w.wid = blockIdx.x * PK_WARPS + warp;
  w.idle = !in_grid || w.wid >= Wtot;
  w.sp = p.sp;
  w.u0 = w.idle ? 0u : gv_start(w.wid, w.sp);
  w.u1 = w.idle ? 0u : gv_start(w.wid + 1, w.sp);
  w.n_units = (int)(w.u1 - w.u0);
  // Small matrices (about two row tiles per CTA or fewer): a CTA owns whole row tiles,
  // its warps take the tiles' units round-robin and the 16-row results meet in shared
  // memory -- no partials in global memory, no ticket, no last-arriver chain.
  w.tile_b = 0; w.n_loc = 0;
  w.s_b = 0; w.ks = SL;      // the slabs this CTA prepares and indexes locally: [s_b, s_b + ks)
  w.rt = 0; w.s = 0;         // row tile and (local) slab of the unit being consumed
  w.kb = 0; w.rb = 0;
  if (p.cta_tiles) {
    if (!in_grid) {
      w.n_units = 0;
      return;
    }
    const unsigned KB = (unsigned)p.cta_tiles;
    w.rb = KB == 1 ? blockIdx.x : blockIdx.x / KB;
    w.kb = blockIdx.x - w.rb * KB;
    const GvSplit ct = p.ct, cs = p.cs;
    w.tile_b = (int)gv_start(w.rb, ct);
    w.s_b = (int)gv_start(w.kb, cs);
    w.ks = (int)gv_start(w.kb + 1, cs) - w.s_b;
    w.n_loc = ((int)gv_start(w.rb + 1, ct) - w.tile_b) * w.ks;
    w.n_units = warp < w.n_loc ? (w.n_loc - warp + PK_WARPS - 1) / PK_WARPS : 0;
    // the block's units in (tile, slab) order, dealt round-robin: this warp starts at `warp`
    w.rt = w.tile_b + warp / w.ks;
    w.s = warp % w.ks;
    w.u0 = (unsigned)(w.rt * SL + w.s_b + w.s);
  } else {
    w.rt = (int)(w.u0 / (unsigned)SL);
    w.s = (int)(w.u0 - (unsigned)w.rt * SL);
  }
}

// A warp's ring of weight units lives across the phases of a chain: the producer cursor says
// where its next unit comes from (and moves on to the next phase's range when this one's is
// issued), the ring state which slot is filled / consumed next.  Weights depend on nothing, so
// the ring is refilled for the next phase while this one's results still travel.
struct GvCursor {
  const unsigned char* src;
  int isl, ks, SL, left, own, ph;
};
struct GvRing {
  int istage, inflight, st;
  unsigned parity;
  bool dead;   // a wait ran out: consume nothing more
  uint64_t policy;   // L2 evict-first: a weight byte is read once per token
};
__device__ __forceinline__ void gv_cursor_from(GvCursor& c, const GemvPParams& p, const GvWarp& w) {
  c.src = p.wp + (size_t)w.u0 * PK_UNIT;
  c.isl = w.s;
  c.ks = w.ks;
  c.SL = p.SL;
  c.left = w.n_units;
  c.own = p.cta_tiles != 0;
}
__device__ __forceinline__ void gv_cursor_set(GvCursor& c, const GemvPParams& p, int warp) {
  GvWarp w;
  gv_warp_setup(p, warp, w);
  gv_cursor_from(c, p, w);
}
// Fill the ring up to `limit` units in flight, walking on into later phases.
// `table`: this warp's cursors of all phases (shared memory; NULL for a single launch).
template <int STAGES>
__device__ __forceinline__ void gv_top_up(GvRing& r, GvCursor& c, const GvCursor* table, int nph,
                                          unsigned char* myR, uint64_t* mybar, int lane, int limit) {
  while (r.inflight < limit) {
    while (c.left == 0 && c.ph + 1 < nph) {
      const int ph = c.ph + 1;
      c = table[ph];
      c.ph = ph;
    }
    if (c.left == 0) return;
    // lane 0 issues one 2560-byte bulk copy per unit
    if (lane == 0) {
      mbar_expect_tx(&mybar[r.istage], PK_UNIT);
      bulk_load_1d_hint(myR + r.istage * PK_UNIT, c.src, PK_UNIT, &mybar[r.istage], r.policy);
    }
    if (c.own) {
      // PK_WARPS units further on in the block; past the block's slabs the next tile's begin
      c.isl += PK_WARPS;
      c.src += (size_t)PK_WARPS * PK_UNIT;
      while (c.isl >= c.ks) {
        c.isl -= c.ks;
        c.src += (size_t)(c.SL - c.ks) * PK_UNIT;
      }
    } else {
      c.src += PK_UNIT;
    }
    c.left--;
    r.inflight++;
    if (++r.istage == STAGES) r.istage = 0;
  }
}

// PULL: the instantiation that can consume a tensor-parallel exchange in its prologue (act 3);
// kept out of the single-GPU kernel, whose register budget it would eat.
// OWN: the CTA-owned-block instantiation (p.cta_tiles != 0).  EPI: the pair epilogue
// (p.epi.kind) as a compile-time value, so the plain projections carry no rope code.
// PUSH: the tensor-parallel producer (outputs go to every rank's staging as tagged packets).
// The work of one launch, or of one phase `phi` of a chain of `nph` (phases[phi] == p).
// OWN_T / EPI_T = -1: read from the parameters at run time -- ONE instantiation for every
// single-GPU projection of a decoder, so that its code stays in the instruction cache from one
// launch to the next (four instantiations per layer do not fit, and their prologues then run
// at the speed of instruction fetches from the L2).
template <int STAGES, bool PULL, int OWN_T, int EPI_T, bool PUSH>
__device__ __forceinline__ void gemv_q4p_body(const GemvPParams& p, const GvCursor* table, int nph, int phi,
                                              GvRing& ring, GvCursor& cur, unsigned char* base) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int SL = p.SL;
  const GemvPSmem L = gemvp_smem_layout(STAGES, p.slabs);
  uint64_t* bars = (uint64_t*)(base + L.bars);
  float* red = (float*)(base + L.red);
  float* Pslab = (float*)(base + L.pslab);   // [SL]   2^(13+e) of the slab
  float* Qg = (float*)(base + L.q);          // [SL*8] 8 * sum of the group's fixed-point activations
  uint4* Bfrag = (uint4*)(base + L.bfrag);   // [SL*8][2][4]
  unsigned char* myR = base + L.ring + (size_t)warp * STAGES * PK_UNIT;
  uint64_t* mybar = bars + warp * STAGES;

  GvWarp ws;
  gv_warp_setup(p, warp, ws);
  if (nph == 1) gv_cursor_from(cur, p, ws);   // a single launch: the one setup serves the producer too
  const unsigned wid = ws.wid, u0 = ws.u0, u1 = ws.u1, kb = ws.kb, rb = ws.rb;
  const GvSplit sp = ws.sp;
  const int n_units = ring.dead ? 0 : ws.n_units;
  const bool own = OWN_T < 0 ? (p.cta_tiles != 0) : (OWN_T != 0);
  const int EPI = EPI_T < 0 ? p.epi.kind : EPI_T;
  const int tile_b = ws.tile_b, n_loc = ws.n_loc, s_b = ws.s_b, ks = ws.ks;
  int rt = ws.rt, s = ws.s;
  float* ures = (float*)(base + L.ures);

  auto top_up = [&](int limit) { gv_top_up<STAGES>(ring, cur, table, nph, myR, mybar, lane, limit); };
  // Weights do not depend on the previous kernel: the first stage streams before the
  // wait.  The other stages are issued right after the activation loads below, so
  // those small loads are not queued behind the weight traffic.  (Later phases of a chain
  // find their ring filled by the phase before.)
  if (phi == 0) {
    top_up(1);
    // While the kernel in front still runs: touch what the prep will read, so that the
    // address translations (and for the norm weights, which nobody writes, the data) are
    // there when the wait returns.  A prefetch of a line the previous kernel is still
    // writing is harmless: the L2 is where its stores land.
    {
      const int k0 = (s_b + warp) * 256 + lane * 8;
      if (warp < ks && k0 < p.K) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.x + k0));
        if (p.act == 1) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.x + p.K + k0));
        if (p.act == 2) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(p.delta + k0));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(p.nw + k0));
        }
      }
    }
    if (EPI == 2 && own && warp == 0 && ks > 0 && lane < n_loc / ks) {
      // ... and what the epilogue of this CTA's row tiles will read: the biases of the tile's
      // eight pairs (two runs of 32 bytes), the rotary table entries
      const int half = p.epi.D >> 1;
      const int pi = (tile_b + lane) * 8;
      const int h = pi / half, j = pi - h * half;
      const float* bias = h < p.epi.n_q ? p.epi.bq : (h < p.epi.n_q + p.epi.n_kv ? p.epi.bk : p.epi.bv);
      const int hh = h < p.epi.n_q ? h : (h < p.epi.n_q + p.epi.n_kv ? h - p.epi.n_q : h - p.epi.n_q - p.epi.n_kv);
      if (bias) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(bias + hh * p.epi.D + j));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(bias + hh * p.epi.D + j + half));
      }
      if (p.epi.rope_cs) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.epi.rope_cs + j));
    }
    pdl_wait();  // activations and the fix-up scratch are valid from here
  }

  // ---- activation prep.  One warp per slab of 256 k, four slabs in flight per warp.
  // Lane l covers x[256*slab + 8*l .. +8) = group jj = l/4, quad slot tt = l%4.
  float nrm_inv = 1.f;
  const bool normed = p.act == 2 || (PULL && p.act == 3);
  unsigned pull_seq = 0;
  if (PULL && p.act == 3) pull_seq = comm_seq(p.comm);
  // act 3: the exchange's reduction.  Packets validate themselves by their tag; two
  // ranks' polls (16 packets per lane) are in flight before the first check, the partials are added in rank
  // order (every rank and every CTA computes the same bits).
  auto pull8 = [&](int k0, float (&o)[8], bool on) {
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = 0.f;
    if (!on) return;
    const unsigned tag = pull_seq + 1u;
    const uint2* stb = p.comm.stage[p.comm.rank] +
                       (size_t)(pull_seq & 1u) * p.comm.size * p.comm.slot_floats + k0;
    for (int r0 = 0; r0 < p.comm.size; r0 += 2) {
      uint2 pk[2][8];
#pragma unroll
      for (int rr = 0; rr < 2; rr++)
        if (r0 + rr < p.comm.size) {
#pragma unroll
          for (int i = 0; i < 8; i++) pk[rr][i] = ld_packet_sys(stb + (size_t)(r0 + rr) * p.comm.slot_floats + i);
        }
#pragma unroll
      for (int rr = 0; rr < 2; rr++)
        if (r0 + rr < p.comm.size) {
#pragma unroll
          for (int i = 0; i < 8; i++) {
            if (pk[rr][i].y != tag)
              pk[rr][i] = wait_packet_bounded(stb + (size_t)(r0 + rr) * p.comm.slot_floats + i, tag,
                                              p.status, 300 + r0 + rr);
            o[i] += __uint_as_float(pk[rr][i].x);
          }
        }
    }
  };
  // (slab indices are local to the CTA's block [s_b, s_b + ks); the whole row unless KB > 1)
  //
  // This code runs once per launch, straight from a cold instruction cache: what it costs is
  // its LENGTH (measured: 3 us of a 5 us projection with two unrolled slab batches per warp),
  // so there is one copy of the load and one of the conversion, in loops that are not unrolled.
  float xv[8], xu[8], xw[8];   // the slab's activation, its second operand (up / delta), its norm weights
  auto load_slab = [&](int sl, bool with_w) {
    const int k0 = (s_b + sl) * 256 + lane * 8;
    const bool on = sl < ks && k0 < p.K;   // K % 32 == 0: a lane's 8 values are all in or all out
    auto load8 = [&](const float* s8, float (&o)[8]) {
      if (on) {
        if (p.x_vec_ok) {
          // .cg in a chain: the vector was written by other SMs earlier in this launch.  A
          // launch of its own reads through the L1 (measured 1 % of a decode step faster).
          float4 q0, q1;
          if (nph > 1) {
            q0 = __ldcg((const float4*)s8);
            q1 = __ldcg((const float4*)(s8 + 4));
          } else {
            q0 = *(const float4*)s8;
            q1 = *(const float4*)(s8 + 4);
          }
          o[0] = q0.x; o[1] = q0.y; o[2] = q0.z; o[3] = q0.w;
          o[4] = q1.x; o[5] = q1.y; o[6] = q1.z; o[7] = q1.w;
        } else {
#pragma unroll
          for (int i = 0; i < 8; i++) o[i] = nph > 1 ? __ldcg(s8 + i) : s8[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; i++) o[i] = 0.f;
      }
    };
    load8(p.x + k0, xv);
    if (p.act == 1) load8(p.x + p.K + k0, xu);
    if (p.act == 2) load8(p.delta + k0, xu);
    // the norm weights travel with the activation: no load left behind the block barrier
    if (normed && with_w) load8(p.nw + k0, xw);
    if constexpr (PULL) {
      if (p.act == 3) pull8(k0, xu, on);
    }
  };
  load_slab(warp, true);
  // The rest of the weight ring is queued only when this warp's activation values have
  // ARRIVED (first use below): a small load issued behind 160 KB of bulk copies per SM waits
  // until they have drained -- measured, the prep of a projection took 2 - 4 us that way, the
  // time the ring fill needs from HBM.  (An L2 prefetch of the units behind the ring was tried
  // too and lost 4 us on the 85 MB gate|up matrix for the same reason.)
  if (normed) {
    // fused residual add + RMSNorm (tl_add_rmsnorm, kernels/tensorlib_cuda.cu:155-179):
    // every CTA reduces sum((x+delta)^2) itself, slabs in the same order everywhere, so all
    // CTAs agree on the scale
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const float sv = xv[i] + xu[i];
      sq = fmaf(sv, sv, sq);
    }
    if (ks > PK_WARPS) {
      // rows longer than 16 slabs: this warp's further slabs, read once more below
      float kv[8], ku[8], kw[8];
#pragma unroll
      for (int i = 0; i < 8; i++) { kv[i] = xv[i]; ku[i] = xu[i]; kw[i] = xw[i]; }
#pragma unroll 1
      for (int sl = warp + PK_WARPS; sl < ks; sl += PK_WARPS) {
        load_slab(sl, false);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float sv = xv[i] + xu[i];
          sq = fmaf(sv, sv, sq);
        }
      }
#pragma unroll
      for (int i = 0; i < 8; i++) { xv[i] = kv[i]; xu[i] = ku[i]; xw[i] = kw[i]; }
    }
    sq = warp_sum(sq);
    top_up(STAGES);
    // The scale 1 / rms is a scalar factor of every activation, so it need not be known before
    // the digits are made: the digits are those of (x + delta) * w, and the factor multiplies
    // the outputs (with alpha, below).  That takes a block barrier and the serial sum out of
    // the prep; the warp sums meet at the barrier that ends it.
    if (lane == 0) red[warp] = sq;
  }
#pragma unroll 1
  for (int sl = warp; sl < ks; sl += PK_WARPS) {
    if (sl != warp) load_slab(sl, true);
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = xv[i];
    if (p.act == 1) {
      // fused SwiGLU (kernels/tensorlib_cuda.cu:185-192 of the reference): the row
      // holds gate then up; same expression g / (1 + exp(-g)) * u
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] = (v[i] / (1.0f + expf(-v[i]))) * xu[i];
    }
    if (normed) {
      const int k0 = sl * 256 + lane * 8;   // (the fused norm is never combined with slab blocks)
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const float sv = v[i] + xu[i];
        const bool in = k0 + i < p.K;
        if (in && blockIdx.x == 0) p.xout[k0 + i] = sv;
        v[i] = in ? sv * xw[i] : 0.f;
      }
    }
    float mx = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) mx = fmaxf(mx, fabsf(v[i]));
    // the maximum over the warp in one instruction: non-negative floats order like their bits
    mx = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(mx)));
    if (sl == warp) top_up(STAGES);
    int e = (int)((__float_as_uint(mx) >> 23) & 0xff) - 126;  // mx < 2^e
    e = mx > 0.f ? (e < -100 ? -100 : (e > 100 ? 100 : e)) : 0;
    if (!(mx < 3.0e38f)) e = 100;                              // inf / nan: keep the exponent legal
    const float s23 = __uint_as_float((unsigned)(127 + 23 - e) << 23);
    // X = rn(v * 2^(23-e)), |X| <= 2^23, as two balanced 12-bit digits X = 4096 d0 + d1 -- without
    // a float -> int conversion: those run at a sixteenth of the FMA rate, and 40 of them per
    // lane made this loop a microsecond on every CTA.  d0 = rn(y / 4096) and d1 = rn(y - 4096 d0)
    // by the add-and-subtract of 1.5 * 2^23 (round to nearest even, like cvt.rni); the
    // subtraction in between is exact, so 4096 d0 + d1 == rn(y).
    const float MAGIC = 12582912.0f;
    float d0f[8], d1f[8], sd0 = 0.f, sd1 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const float y = v[i] * s23;
      d0f[i] = fmaf(y, 0.000244140625f, MAGIC) - MAGIC;   // [-2048, 2048]
      const float r = fmaf(d0f[i], -4096.0f, y);           // exact, |r| <= 2048
      d1f[i] = (r + MAGIC) - MAGIC;                        // [-2048, 2048]
      sd0 += d0f[i];                                       // sums of at most 2^16: exact
      sd1 += d1f[i];
    }
    sd0 += __shfl_xor_sync(0xffffffffu, sd0, 1);
    sd0 += __shfl_xor_sync(0xffffffffu, sd0, 2);
    sd1 += __shfl_xor_sync(0xffffffffu, sd1, 1);
    sd1 += __shfl_xor_sync(0xffffffffu, sd1, 2);
    // the odd nibble of a byte reads as nib * 2^-20: its activation digits carry 2^-4;
    // element i pairs with i + 4 in one 32-bit word, converted as a pair
    auto pk = [](float a, float b) {
      const __half2 h = __floats2half2_rn(a, b);
      return *reinterpret_cast<const unsigned*>(&h);
    };
    uint4 fh, fl;
    fh.x = pk(d0f[0], d0f[4]);                     fl.x = pk(d1f[0], d1f[4]);
    fh.y = pk(d0f[1] * 0.0625f, d0f[5] * 0.0625f); fl.y = pk(d1f[1] * 0.0625f, d1f[5] * 0.0625f);
    fh.z = pk(d0f[2], d0f[6]);                     fl.z = pk(d1f[2], d1f[6]);
    fh.w = pk(d0f[3] * 0.0625f, d0f[7] * 0.0625f); fl.w = pk(d1f[3] * 0.0625f, d1f[7] * 0.0625f);
    const int jj = lane >> 2, tt = lane & 3;
    Bfrag[((size_t)(sl * 8 + jj) * 2 + 0) * 4 + tt] = fh;
    Bfrag[((size_t)(sl * 8 + jj) * 2 + 1) * 4 + tt] = fl;
    // 8 * sum(x_g) in the same fixed point: (8 * isum) * 2^(e-23)
    // (the correctly rounded value of the exact integer sum, what (float)isum gave)
    if (tt == 0) Qg[sl * 8 + jj] = fmaf(sd0, 4096.0f, sd1) * __uint_as_float((unsigned)(127 + 3 - 23 + e) << 23);
    // a non-finite activation makes every output of the slab NaN instead of garbage
    if (lane == 0)
      Pslab[sl] = (mx < 3.0e38f) ? __uint_as_float((unsigned)(127 + 13 + e) << 23) : __uint_as_float(0x7fc00000u);
  }
  __syncthreads();
  if (phi == 0) pdl_launch_dependents();
  if (normed) {
    // sum of the warp sums in warp order: every warp of every CTA computes the same bits
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < PK_WARPS; w++) tot += red[w];
    nrm_inv = 1.0f / sqrtf(tot / (float)p.K + p.eps);
  }
  const float alpha_n = p.alpha * nrm_inv;

  // ---- streaming loop ------------------------------------------------------
  float acc0 = 0.f, acc1 = 0.f, corr0 = 0.f, corr1 = 0.f;
  uint4 bq[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
  const bool bpred = g < 2;                  // columns 0 (hi digit) and 1 (lo digit) of B
  const uint32_t ring32 = smem_u32(myR);
  const uint32_t bh32 = smem_u32(Bfrag) + (uint32_t)((g & 1) * 4 + t) * 16u;
  const uint32_t q32 = smem_u32(Qg) + (uint32_t)t * 8u, p32 = smem_u32(Pslab);
  const uint32_t wl = (uint32_t)lane * 16u, sl_ = 2048u + (uint32_t)g * 32u;
  const uint32_t cl = 2048u + (uint32_t)g * 32u + (uint32_t)t * 8u;

  unsigned ar_seq = 0;
  if (PUSH) ar_seq = comm_seq(p.comm);
  const size_t ar_off =
      ((size_t)(ar_seq & 1u) * p.comm.size + p.comm.rank) * (size_t)p.comm.slot_floats;
  auto emit = [&](int n, float v) {
    v = v * alpha_n + p.beta;
    if (PUSH) {
      for (int r = 0; r < p.comm.size; r++) st_packet_sys(&p.comm.stage[r][ar_off + n], v, ar_seq + 1u);
    } else {
      p.y[n] = v;
    }
  };
  // pair index pi of a pair-packed matrix, a = its first row's sum, b = its second's
  auto emit_pair = [&](int pi, float a, float b) {
    a = a * alpha_n + p.beta;
    b = b * alpha_n + p.beta;
    if (EPI == 1) {
      // tl_swiglu (kernels/tensorlib_cuda.cu:185-192): silu(gate) * up, same expression
      p.epi.out[pi] = (a / (1.0f + expf(-a))) * b;
      return;
    }
    // kind 2: the seam after the fused QKV projection (bench/cuda/qwen_model.h:700-716):
    // q <- rope(q + bq), rope(k + bk) and v + bv into cache row *d_pos.  Angle in double,
    // like the CPU reference's trig (the f32 fast path drifts past 1e-3 on the low pairs).
    const int half = p.epi.D >> 1, D = p.epi.D;
    // (head sizes are powers of two in practice: a shift instead of two dozen instructions)
    const int h = (half & (half - 1)) == 0 ? pi >> (31 - __clz(half)) : pi / half;
    const int j = pi - h * half;
    const unsigned pos = *p.epi.d_pos;
    if (pos >= (unsigned)p.epi.kv_rows) {
      // the cache is full: write nothing (the attention that follows refuses the position
      // too) and tell the host through the status block
      if (p.status) atomicExch(&p.status[ST_KV_OVERFLOW], 1);
      return;
    }
    if (h >= p.epi.n_q + p.epi.n_kv) {
      const int kh = h - p.epi.n_q - p.epi.n_kv;
      if (p.epi.bv) { a += p.epi.bv[kh * D + j]; b += p.epi.bv[kh * D + j + half]; }
      const size_t row = (size_t)kh * p.epi.kv_stride + (size_t)pos * D;
      if (p.epi.kv_bf16) {
        __nv_bfloat16* dst = (__nv_bfloat16*)p.epi.Vc + row;
        dst[j] = __float2bfloat16_rn(a);
        dst[j + half] = __float2bfloat16_rn(b);
      } else {
        float* dst = p.epi.Vc + row;
        dst[j] = a;
        dst[j + half] = b;
      }
      return;
    }
    float c, sn;
    if (p.epi.rope_cs) {
      // (cos, sin) of this position, computed once per token by the same expression
      const float2 cs = p.epi.rope_cs[j];
      c = cs.x;
      sn = cs.y;
    } else {
      const double theta = exp2(-2.0 * (double)j / (double)D * log2((double)p.epi.base));
      double sd, cd;
      sincos((double)pos * theta, &sd, &cd);
      c = (float)cd;
      sn = (float)sd;
    }
    if (h < p.epi.n_q) {
      if (p.epi.bq) { a += p.epi.bq[h * D + j]; b += p.epi.bq[h * D + j + half]; }
      float* dst = p.epi.out + (size_t)h * D;
      dst[j] = a * c - b * sn;
      dst[j + half] = a * sn + b * c;
    } else {
      const int kh = h - p.epi.n_q;
      if (p.epi.bk) { a += p.epi.bk[kh * D + j]; b += p.epi.bk[kh * D + j + half]; }
      const size_t row = (size_t)kh * p.epi.kv_stride + (size_t)pos * D;
      if (p.epi.kv_bf16) {
        __nv_bfloat16* dst = (__nv_bfloat16*)p.epi.Kc + row;
        dst[j] = __float2bfloat16_rn(a * c - b * sn);
        dst[j + half] = __float2bfloat16_rn(a * sn + b * c);
      } else {
        float* dst = p.epi.Kc + row;
        dst[j] = a * c - b * sn;
        dst[j + half] = a * sn + b * c;
      }
    }
  };
  auto flush = [&](int rt) {
    // lanes t == 0 hold the row sums; the -8*sum(x_g) correction is spread over the quad
    float v0 = (t == 0 ? acc0 : 0.f) - corr0, v1 = (t == 0 ? acc1 : 0.f) - corr1;
    v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
    v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
    v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
    v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
    const unsigned t0 = (unsigned)rt * SL, t1 = t0 + SL;
    const bool complete = (u0 <= t0) && (u1 >= t1);
    const int r0 = rt * 16;
    if (complete) {
      if (t == 0) {
        if (EPI) {
          emit_pair(rt * 8 + g, v0, v1);
        } else {
          if (r0 + g < p.N) emit(r0 + g, v0);
          if (r0 + g + 8 < p.N) emit(r0 + g + 8, v1);
        }
      }
      return;
    }
    // partial: slot 0 when this tile holds the worker's first unit, else slot 1
    const int slot = (u0 >= t0) ? 0 : 1;
    float* mine = p.partials + ((size_t)wid * 2 + slot) * 16;
    if (t == 0) {
      __stcg(&mine[g], v0);
      __stcg(&mine[g + 8], v1);
    }
    __syncwarp();
    const unsigned wf = gv_owner(t0, sp), wlast = gv_owner(t1 - 1, sp);
    int old = 0;
    if (lane == 0) old = (int)atom_add_acq_rel(&p.counters[rt], 1);  // releases the warp's stores
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old != (int)(wlast - wf)) return;  // not the last contributor
    // Last contributor: lanes 0..15 own one row each and fold the partials in worker
    // order, sixteen loads in flight (one L2 round trip for up to 16 contributors).
    float s = 0.f;
    if (lane < 16) {
      for (unsigned w = wf; w <= wlast; w += 16) {
        float pv[16];
#pragma unroll
        for (int k = 0; k < 16; k++) {
          const unsigned ww = w + k;
          const bool on = ww <= wlast;
          const unsigned wz = on ? ww : wlast;
          const int sl = (gv_start(wz, sp) >= t0) ? 0 : 1;  // started inside this tile
          pv[k] = on ? __ldcg(p.partials + ((size_t)wz * 2 + sl) * 16 + lane) : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 16; k++) s += pv[k];
      }
      if (!EPI && r0 + lane < p.N) emit(r0 + lane, s);
    }
    if (EPI) {
      const float s2 = __shfl_down_sync(0xffffffffu, s, 8);   // row lane + 8 of the tile
      if (lane < 8) emit_pair(rt * 8 + lane, s, s2);
    }
    if (lane == 0) p.counters[rt] = 0;  // leave the counter clean for the next launch
  };

  for (int i = 0; i < n_units; i++) {
    const int st = ring.st;
    if (own && i > 0) {   // next unit of this warp: PK_WARPS further on
      s += PK_WARPS;
      while (s >= ks) { s -= ks; rt++; }
    }
    if (!mbar_wait_bounded(&mybar[st], ring.parity, p.status, 100 + st)) {
      ring.dead = true;
      break;
    }
    const uint32_t ust = ring32 + (uint32_t)st * PK_UNIT;
    const uint32_t wa = ust + wl, sa = ust + sl_, bs = bh32 + (uint32_t)s * 1024u;
    // the 8 group scales of rows g and g+8
    const float4 sa0 = lds128f<0>(sa), sa1 = lds128f<16>(sa), sb0 = lds128f<256>(sa), sb1 = lds128f<272>(sa);
    const float sc0[8] = {sa0.x, sa0.y, sa0.z, sa0.w, sa1.x, sa1.y, sa1.z, sa1.w};
    const float sc1[8] = {sb0.x, sb0.y, sb0.z, sb0.w, sb1.x, sb1.y, sb1.z, sb1.w};
    uint4 w[4];
    w[0] = lds128<0>(wa); w[1] = lds128<512>(wa); w[2] = lds128<1024>(wa); w[3] = lds128<1536>(wa);
    float ua0 = 0.f, ua1 = 0.f;
#define TLB_GRP(JJ, W0, W1, OFF)                                                          \
  {                                                                                       \
    if (bpred) bq[(JJ) & 1] = lds128<OFF>(bs);                                            \
    unsigned w0 = (W0), w1 = (W1);                                                        \
    float c[4];                                                                           \
    mma16816_z(c, w0 & 0x000f000fu, w1 & 0x000f000fu, w0 & 0x00f000f0u, w1 & 0x00f000f0u, \
               bq[(JJ) & 1].x, bq[(JJ) & 1].y);                                           \
    w0 >>= 8;                                                                             \
    w1 >>= 8;                                                                             \
    mma16816(c, w0 & 0x000f000fu, w1 & 0x000f000fu, w0 & 0x00f000f0u, w1 & 0x00f000f0u,   \
             bq[(JJ) & 1].z, bq[(JJ) & 1].w);                                             \
    ua0 = fmaf(sc0[JJ], fmaf(c[1], 0.000244140625f, c[0]), ua0);                          \
    ua1 = fmaf(sc1[JJ], fmaf(c[3], 0.000244140625f, c[2]), ua1);                          \
  }
    TLB_GRP(0, w[0].x, w[0].y, 0) TLB_GRP(1, w[0].z, w[0].w, 128)
    TLB_GRP(2, w[1].x, w[1].y, 256) TLB_GRP(3, w[1].z, w[1].w, 384)
    TLB_GRP(4, w[2].x, w[2].y, 512) TLB_GRP(5, w[2].z, w[2].w, 640)
    TLB_GRP(6, w[3].x, w[3].y, 768) TLB_GRP(7, w[3].z, w[3].w, 896)
#undef TLB_GRP
    {
      // lane t of the quad handles groups 2t, 2t+1 of the correction term
      const float2 q = lds64f<0>(q32 + (uint32_t)s * 32u);
      const float2 c0 = lds64f<0>(ust + cl), c1 = lds64f<256>(ust + cl);
      corr0 = fmaf(c0.x, q.x, fmaf(c0.y, q.y, corr0));
      corr1 = fmaf(c1.x, q.x, fmaf(c1.y, q.y, corr1));
    }
    const float P = lds32f(p32 + (uint32_t)s * 4u);
    acc0 = fmaf(P, ua0, acc0);
    acc1 = fmaf(P, ua1, acc1);
    __syncwarp();
    ring.inflight--;
    top_up(STAGES);   // the slot just freed: this phase's next unit, or the next phase's first
    if (++ring.st == STAGES) { ring.st = 0; ring.parity ^= 1u; }
    if (own) {
      // this unit's 16 row sums go to the CTA's table, slot = unit index inside the CTA
      float v0 = (t == 0 ? acc0 : 0.f) - corr0, v1 = (t == 0 ? acc1 : 0.f) - corr1;
      v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
      v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
      v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
      v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
      if (t == 0) {
        float* dst = ures + (size_t)((rt - tile_b) * ks + s) * 16;
        dst[g] = v0;
        dst[g + 8] = v1;
      }
      acc0 = acc1 = corr0 = corr1 = 0.f;
      continue;
    }
    if (++s == SL) {
      flush(rt);
      acc0 = acc1 = corr0 = corr1 = 0.f;
      s = 0;
      rt++;
    }
  }
  // This warp's stream has run dry: ask the L2 for the head of the next kernel's weights.
  if (p.pf.wp) {
    for (unsigned nc = blockIdx.x + (unsigned)p.grid * (unsigned)warp; nc < (unsigned)p.pf.grid;
         nc += (unsigned)p.grid * PK_WARPS)
      gv_prefetch_head(p.pf, nc, lane);
  }
  if (own) {
    __syncthreads();
    const int ntl = n_loc / ks;   // row tiles of this block
    // one thread per output row: fold the row's unit results in slab order
    if (EPI) {
      // one thread per pair: rows (lr, lr + 8) of a tile (whole rows only: KB == 1)
      for (int idx = tid; idx < ntl * 8; idx += PK_WARPS * 32) {
        const int tl = idx >> 3, lr = idx & 7;
        const float* srcp = ures + (size_t)tl * ks * 16 + lr;
        float sa = 0.f, sb = 0.f;
        for (int k = 0; k < ks; k++) { sa += srcp[k * 16]; sb += srcp[k * 16 + 8]; }
        emit_pair((tile_b + tl) * 8 + lr, sa, sb);
      }
      return;
    }
    const unsigned KB = (unsigned)p.cta_tiles;
    for (int idx = tid; idx < ntl * 16; idx += PK_WARPS * 32) {
      const int tl = idx >> 4, row = idx & 15;
      const float* srcp = ures + (size_t)tl * ks * 16 + row;
      float sum = 0.f;
      for (int k = 0; k < ks; k++) sum += srcp[k * 16];
      const int n = (tile_b + tl) * 16 + row;
      if (KB == 1) {
        if (n < p.N) emit(n, sum);
      } else {
        __stcg(p.partials + ((size_t)kb * p.RT + tile_b + tl) * 16 + row, sum);
      }
    }
    if (KB == 1) return;
    // Slab blocks: the row block's KB partial blocks meet in global memory; the CTA that
    // arrives last folds them in block order (the same bits whichever CTA that is).
    __threadfence();
    __syncthreads();
    int* flag = (int*)red;
    if (tid == 0) *flag = (int)atom_add_acq_rel(&p.counters[rb], 1);
    __syncthreads();
    if (*flag != (int)KB - 1) return;
    __threadfence();
    for (int idx = tid; idx < ntl * 16; idx += PK_WARPS * 32) {
      const size_t off = (size_t)(tile_b + (idx >> 4)) * 16 + (idx & 15);
      float sum = 0.f;
      for (unsigned b0 = 0; b0 < KB; b0 += 8) {
        float pv[8];
#pragma unroll
        for (int k = 0; k < 8; k++)
          pv[k] = b0 + k < KB ? __ldcg(p.partials + (size_t)(b0 + k) * p.RT * 16 + off) : 0.f;
#pragma unroll
        for (int k = 0; k < 8; k++) sum += pv[k];
      }
      if ((int)off < p.N) emit((int)off, sum);
    }
    if (tid == 0) p.counters[rb] = 0;  // clean for the next launch
    return;
  }
  if (n_units > 0 && s != 0) flush(rt);
}

__device__ __forceinline__ unsigned char* gv_ring_init(unsigned char* smem_raw, int stages, GvRing& ring) {
  unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint64_t* mybar = (uint64_t*)(base + gemvp_smem_layout(stages, 0).bars) + warp * stages;
  if (lane == 0) {
    for (int s = 0; s < stages; s++) mbar_init(&mybar[s], 1);
    mbar_fence_init();
  }
  __syncwarp();
  ring.istage = 0; ring.inflight = 0; ring.st = 0; ring.parity = 0u; ring.dead = false;
  ring.policy = l2_evict_first_policy();
  return base;
}

template <int STAGES, bool PULL, int OWN, int EPI, bool PUSH>
__global__ void __launch_bounds__(PK_WARPS * 32, PK_CTAS_PER_SM)
    gemv_q4p_kernel(const __grid_constant__ GemvPParams p) {
  extern __shared__ unsigned char smem_raw[];
  GvRing ring;
  unsigned char* base = gv_ring_init(smem_raw, STAGES, ring);
  GvCursor cur;
  cur.ph = 0;
  gemv_q4p_body<STAGES, PULL, OWN, EPI, PUSH>(p, nullptr, 1, 0, ring, cur, base);
}

// ---- a chain of GEMVs in one launch ------------------------------------------------------
// The projections between two attention calls of a decoder (o, gate|up, down, the next
// layer's qkv -- or the lm_head) each need the whole output of the one before, so as separate
// launches every boundary costs the drain of one kernel and the ramp of the next (about 3 us
// of an idle HBM each, against 1.3 - 13 us of streaming).  Here they are phases of one
// persistent launch: between phases the CTAs meet at a counter in global memory (bounded
// spin), and because a warp's ring of weight units is refilled across the phase boundary
// (weights depend on nothing), the HBM keeps streaming the next matrix while the last
// results of this one are folded, the barrier is crossed and the activations are prepared.
constexpr int GV_CHAIN_MAX = 4;
constexpr int GV_CHAIN_BARRIERS = GV_CHAIN_MAX - 1;   // arrivals per CTA and launch, always
struct GvChainParams {
  GemvPParams ph[GV_CHAIN_MAX];
  int nph;
  unsigned long long* cell;   // arrival counter of the device: never reset, += BARRIERS * grid per launch
};

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// All CTAs of the launch arrive; nobody leaves before the last has arrived (or the wait limit
// of the status block runs out: the status block records it and the phase runs on stale data).
// `epoch` = value of the counter when the launch began, found at the first barrier: no CTA
// can be past barrier 1 before this one has arrived at it, so the counter then lies in
// [epoch, epoch + grid).
__device__ __forceinline__ void gv_grid_barrier(unsigned long long* cell, unsigned long long& epoch, int k,
                                                int* status) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned long long per_launch = (unsigned long long)GV_CHAIN_BARRIERS * gridDim.x;
    if (k == 1) {
      const unsigned long long c0 = ld_acquire_u64(cell);
      epoch = c0 - c0 % per_launch;
    }
    __threadfence();
    atomicAdd(cell, 1ull);
    const unsigned long long target = epoch + (unsigned long long)k * gridDim.x;
    if (ld_acquire_u64(cell) < target) {
      const long long t0 = clock64();
      long long limit = 1ll << 62;
      for (unsigned spin = 1;; spin++) {
        if (ld_acquire_u64(cell) >= target) break;
        if ((spin & 63u) == 0) limit = wait_limit(status);
        if (clock64() - t0 > limit) {
          if (status) {
            atomicExch(&status[ST_WAIT_TIMEOUT], 1);
            atomicExch(&status[ST_WAIT_WHERE], 700 + k);
          }
          break;
        }
      }
    }
  }
  __syncthreads();
}

// A phase's instantiation is chosen at compile time (code 3 * own + epilogue kind), so that its
// parameters stay immediate operands from the constant bank like in a launch of its own; the
// host picks the kernel whose codes match the phases' plans.
template <int STAGES, int CODE>
__device__ __forceinline__ void gv_chain_phase(const GemvPParams& p, const GvCursor* table, int nph, int phi,
                                               GvRing& ring, GvCursor& cur, unsigned char* base,
                                               unsigned long long* cell, unsigned long long& epoch) {
  if (phi >= nph) return;
  if (phi > 0) gv_grid_barrier(cell, epoch, phi, p.status);
  if (blockIdx.x < (unsigned)p.grid) {
    gemv_q4p_body<STAGES, false, (CODE >= 3), CODE % 3, false>(p, table, nph, phi, ring, cur, base);
  } else if (phi == 0) {
    pdl_wait();
    pdl_launch_dependents();
  }
}

template <int STAGES, int C0, int C1, int C2, int C3>
__global__ void __launch_bounds__(PK_WARPS * 32, PK_CTAS_PER_SM)
    gemv_q4p_chain_kernel(const __grid_constant__ GvChainParams cp) {
  extern __shared__ unsigned char smem_raw[];
  // every warp's unit range in every phase, worked out once (phase numbers are immediates
  // here, so the parameters are plain constant-bank operands) and looked up when the ring
  // moves on to the next phase
  __shared__ GvCursor curs[PK_WARPS][GV_CHAIN_MAX];
  __shared__ unsigned long long epoch_s;
  GvRing ring;
  unsigned char* base = gv_ring_init(smem_raw, STAGES, ring);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nph = cp.nph;
  GvCursor cur;
  cur.ph = 0;
  gv_cursor_set(cur, cp.ph[0], warp);
  {
    GvCursor t;
    t.ph = 0;
#pragma unroll
    for (int i = 1; i < GV_CHAIN_MAX; i++) {
      if (i < nph) {
        gv_cursor_set(t, cp.ph[i], warp);
        if (lane == 0) curs[warp][i] = t;
      }
    }
    __syncwarp();
  }
  const GvCursor* table = curs[warp];
  unsigned long long& epoch = epoch_s;   // thread 0 alone reads and writes it
  gv_chain_phase<STAGES, C0>(cp.ph[0], table, nph, 0, ring, cur, base, cp.cell, epoch);
  gv_chain_phase<STAGES, C1>(cp.ph[1], table, nph, 1, ring, cur, base, cp.cell, epoch);
  gv_chain_phase<STAGES, C2>(cp.ph[2], table, nph, 2, ring, cur, base, cp.cell, epoch);
  gv_chain_phase<STAGES, C3>(cp.ph[3], table, nph, 3, ring, cur, base, cp.cell, epoch);
  // every launch adds the same number of arrivals, whatever its length
  __syncthreads();
  if (threadIdx.x == 0 && nph - 1 < GV_CHAIN_BARRIERS)
    atomicAdd(cp.cell, (unsigned long long)(GV_CHAIN_BARRIERS - (nph - 1)) );
}

// The same chain with ONE copy of the body in a loop over the phases (run-time modes, the
// phases' parameters in shared memory because kernel parameters cannot be indexed by a
// run-time phase number): phases after the first run from a warm instruction cache.
template <int STAGES>
__global__ void __launch_bounds__(PK_WARPS * 32, PK_CTAS_PER_SM)
    gemv_q4p_chain_loop_kernel(const __grid_constant__ GvChainParams cp) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ GvCursor curs[PK_WARPS][GV_CHAIN_MAX];
  __shared__ unsigned long long epoch_s;
  __shared__ __align__(16) GemvPParams sph[GV_CHAIN_MAX];
  GvRing ring;
  unsigned char* base = gv_ring_init(smem_raw, STAGES, ring);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nph = cp.nph;
  {
    static_assert(sizeof(GemvPParams) % 4 == 0, "copied word by word");
    constexpr int W = (int)(sizeof(GemvPParams) / 4);
    const unsigned* srcw = (const unsigned*)&cp.ph[0];
    unsigned* dstw = (unsigned*)&sph[0];
    for (int i = threadIdx.x; i < GV_CHAIN_MAX * W; i += blockDim.x) dstw[i] = srcw[i];
  }
  GvCursor cur;
  cur.ph = 0;
  gv_cursor_set(cur, cp.ph[0], warp);
  {
    GvCursor t;
    t.ph = 0;
#pragma unroll
    for (int i = 1; i < GV_CHAIN_MAX; i++) {
      if (i < nph) {
        gv_cursor_set(t, cp.ph[i], warp);
        if (lane == 0) curs[warp][i] = t;
      }
    }
  }
  __syncthreads();
  const GvCursor* table = curs[warp];
  unsigned long long& epoch = epoch_s;
#pragma unroll 1
  for (int phi = 0; phi < nph; phi++) {
    const GemvPParams& p = sph[phi];
    if (phi > 0) gv_grid_barrier(cp.cell, epoch, phi, p.status);
    if (blockIdx.x < (unsigned)p.grid) {
      gemv_q4p_body<STAGES, false, -1, -1, false>(p, table, nph, phi, ring, cur, base);
    } else if (phi == 0) {
      pdl_wait();
      pdl_launch_dependents();
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && nph - 1 < GV_CHAIN_BARRIERS)
    atomicAdd(cp.cell, (unsigned long long)(GV_CHAIN_BARRIERS - (nph - 1)));
}

static int gemvp_stages(int slabs) {
  for (int st = 4; st >= 2; st--)
    if (gemvp_smem_layout(st, slabs).total <= (size_t)(PK_DYN_SMEM_MAX / PK_CTAS_PER_SM) - (PK_CTAS_PER_SM > 1 ? 1024 : 0)) return st;
  return 0;
}

bool gemv_q4p_supported(long long N, long long K) {
  if (!(N > 0 && K > 0 && K % 32 == 0 && K <= (1 << 20))) return false;
  const int SL = (int)((K + 255) / 256);
  // whole rows in shared memory, or slab blocks of at most 2 x PK_WARPS slabs
  return gemvp_stages(SL) != 0 || (SL > 2 * PK_WARPS && gemvp_stages(2 * PK_WARPS) != 0);
}

template <int STAGES, bool PULL, int OWN, int EPI, bool PUSH>
static int gemvp_launch_t(const GemvPParams& p, int ctas, size_t smem, cudaStream_t stream) {
  static std::atomic<unsigned long long> attr_done{0};
  {
    const int rc_attr = ensure_dynamic_smem(gemv_q4p_kernel<STAGES, PULL, OWN, EPI, PUSH>, PK_DYN_SMEM_MAX, attr_done);
    if (rc_attr) return rc_attr;
  }
  LaunchCfg lc(dim3(ctas), dim3(PK_WARPS * 32), smem, stream, pdl_enabled());
  TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, gemv_q4p_kernel<STAGES, PULL, OWN, EPI, PUSH>, p));
  return TLB_OK;
}
template <int STAGES, bool PULL, bool OWN>
static int gemvp_launch_e(const GemvPParams& p, int ctas, size_t smem, cudaStream_t stream) {
  if (p.push) {   // a pushing launch has neither a pair epilogue nor a pulling prologue
    if (PULL) return set_error(TLB_ERR_ARG, "gemv_q4p: a launch pulls or pushes, not both");
    return gemvp_launch_t<STAGES, false, OWN, 0, true>(p, ctas, smem, stream);
  }
  if (p.epi.kind == 0) return gemvp_launch_t<STAGES, PULL, OWN, 0, false>(p, ctas, smem, stream);
  if (p.epi.kind == 1) return gemvp_launch_t<STAGES, PULL, OWN, 1, false>(p, ctas, smem, stream);
  return gemvp_launch_t<STAGES, PULL, OWN, 2, false>(p, ctas, smem, stream);
}
template <int STAGES, bool PULL>
static int gemvp_launch_o(const GemvPParams& p, int ctas, size_t smem, cudaStream_t stream) {
  // TLB_GEMV_UNIFIED=1: the one instantiation with run-time modes for every single-GPU launch
  // (measured 3 % slower than one instantiation per mode: the instruction cache does not carry
  // a kernel's code from one launch to the next, so sharing it buys nothing)
  static const bool unified = getenv("TLB_GEMV_UNIFIED") && atoi(getenv("TLB_GEMV_UNIFIED")) == 1;
  if (!PULL && !p.push && unified) return gemvp_launch_t<STAGES, false, -1, -1, false>(p, ctas, smem, stream);
  if (p.cta_tiles) return gemvp_launch_e<STAGES, PULL, true>(p, ctas, smem, stream);
  return gemvp_launch_e<STAGES, PULL, false>(p, ctas, smem, stream);
}

struct GemvPlan {
  int ctas = 0, cta_tiles = 0, slabs = 0, stages = 0;
};
// Grid, ownership mode and ring depth of a launch (the decisions, without the launch).
static int gemvp_plan(DeviceCtx* c, int N, int K, int act, bool has_epi, int max_ctas, GemvPlan* out) {
  GemvPlan pl;
  if (K % 32) return set_error(TLB_ERR_UNSUPPORTED, "gemv_q4p: K not supported");
  const int RT = (N + 15) / 16, SL = (K + 255) / 256;
  const bool whole_rows_fit = gemvp_stages(SL) != 0;   // else only slab blocks can run this K
  const unsigned U = (unsigned)RT * (unsigned)SL;
  if (RT > c->gemv_max_tiles)
    return set_error(TLB_ERR_UNSUPPORTED, "gemv_q4p: N exceeds the fix-up counter capacity");
  const int slots = c->sm_count * PK_CTAS_PER_SM;   // CTAs resident at once
  int ctas = max_ctas > 0 ? max_ctas : slots;
  const int need = (int)((U + PK_WARPS - 1) / PK_WARPS);
  if (ctas > need) ctas = need;
  if (ctas * PK_WARPS > c->gemv_max_workers) ctas = c->gemv_max_workers / PK_WARPS;
  {
    // CTA-owned row tiles when that leaves every CTA at most about two units per warp
    int cb = max_ctas > 0 ? max_ctas : slots;
    if (cb > RT) cb = RT;
    const int tiles_max = (RT + cb - 1) / cb;
    if (tiles_max * SL <= PK_CTA_UNITS && tiles_max * SL <= 2 * PK_WARPS + PK_WARPS / 2) {
      pl.cta_tiles = 1;
      ctas = cb;
    }
  }
  pl.slabs = SL;
  if (!pl.cta_tiles && SL > 2 * PK_WARPS && act <= 1 && !has_epi) {
    // Long rows (the down projection): every CTA would turn the whole activation into
    // digits, 16 slabs per round, before its stream can start.  Slab blocks cut that to one
    // round at the price of a KB-way fold.  Pick KB by a cost model in ns: a unit is 58 ns of a
    // CTA's share of the stream, a round of activation prep 600 ns, the fold 300 + 100 KB.
    const int cb = max_ctas > 0 ? max_ctas : slots;
    const int workers = ctas * PK_WARPS;
    const long long base_cost = (long long)((U + workers - 1) / workers) * PK_WARPS * 58 +
                                (long long)((SL + PK_WARPS - 1) / PK_WARPS) * 600;
    long long best = whole_rows_fit ? base_cost : (1ll << 60);
    int best_kb = 0;
    for (int kb = 2; kb <= 40 && kb <= SL && kb <= cb; kb++) {
      const int rbn = cb / kb < RT ? cb / kb : RT;
      const int ksm = (SL + kb - 1) / kb, tm = (RT + rbn - 1) / rbn;
      if (ksm * tm > PK_CTA_UNITS || gemvp_stages(ksm) == 0) continue;
      if ((size_t)kb * RT * 16 > (size_t)c->gemv_max_workers * 2 * 128) continue;
      const long long cost = (long long)((ksm * tm + PK_WARPS - 1) / PK_WARPS) * PK_WARPS * 58 +
                             (long long)((ksm + PK_WARPS - 1) / PK_WARPS) * 600 + 300 + 100 * kb;
      if (cost < best) { best = cost; best_kb = kb; }
    }
    if (best_kb) {
      const int rbn = cb / best_kb < RT ? cb / best_kb : RT;
      pl.cta_tiles = best_kb;
      pl.slabs = (SL + best_kb - 1) / best_kb;
      ctas = rbn * best_kb;
    }
  }
  pl.stages = gemvp_stages(pl.slabs);
  if (!pl.stages) return set_error(TLB_ERR_UNSUPPORTED, "gemv_q4p: K too large for the activation fragments");
  pl.ctas = ctas;
  *out = pl;
  return TLB_OK;
}

int gemv_q4p_stream_of(DeviceCtx* c, const void* packed, int N, int K, int act, bool has_epi, int max_ctas,
                       GvStream* out) {
  GemvPlan pl;
  const int rc = gemvp_plan(c, N, K, act, has_epi, max_ctas, &pl);
  if (rc) return rc;
  out->wp = (const unsigned char*)packed;
  out->RT = (N + 15) / 16;
  out->SL = (K + 255) / 256;
  out->U = (unsigned)out->RT * (unsigned)out->SL;
  out->KB = pl.cta_tiles;
  out->grid = pl.ctas;
  out->stages = pl.stages;
  return TLB_OK;
}

// Parameters and plan of one launch / phase from the caller's arguments.
static int gemvp_fill(DeviceCtx* c, const void* packed, const float* x, float* y, int N, int K, float alpha,
                      float beta, int max_ctas, const CommDev* push_comm, int act, const float* delta,
                      const float* nw, float* xout, float eps, const PairEpi* epi, const CommDev* pull_comm,
                      const GvStream* prefetch, GemvPParams* out, GemvPlan* plan) {
  GemvPParams& p = *out;
  memset(&p, 0, sizeof(p));
  if (prefetch) p.pf = *prefetch;
  if (pull_comm) {
    if (push_comm) return set_error(TLB_ERR_ARG, "gemv_q4p: a launch pulls or pushes, not both");
    act = 3;
  }
  if (epi) {
    p.epi = *epi;
    if (push_comm) return set_error(TLB_ERR_ARG, "gemv_q4p: a pair epilogue cannot push");
    if (N % 16) return set_error(TLB_ERR_ARG, "gemv_q4p: a pair epilogue needs N % 16 == 0");
  }
  GemvPlan pl;
  {
    const int rc = gemvp_plan(c, N, K, act, epi != nullptr, max_ctas, &pl);
    if (rc) return rc;
  }
  p.act = act;
  p.delta = delta; p.nw = nw; p.xout = xout; p.eps = eps;
  if (act == 2 && (!delta || !nw || !xout))
    return set_error(TLB_ERR_ARG, "gemv_q4p: fused add+rmsnorm needs its three buffers");
  if (act == 3 && (!nw || !xout || K > pull_comm->slot_floats))
    return set_error(TLB_ERR_ARG, "gemv_q4p: fused exchange + rmsnorm needs nw, xout and K within the staging slot");
  // the norm's sum of squares is taken from the first batch of slabs: it must cover the row
  if ((act == 2 || act == 3) && (K + 255) / 256 > PK_WARPS * 2)
    return set_error(TLB_ERR_UNSUPPORTED, "gemv_q4p: fused add+rmsnorm needs K <= 8192");
  p.push = push_comm ? 1 : 0;
  if (push_comm) p.comm = *push_comm;
  if (pull_comm) p.comm = *pull_comm;
  p.wp = (const unsigned char*)packed;
  p.x = x; p.y = y; p.N = N; p.K = K;
  p.alpha = alpha; p.beta = beta;
  p.partials = c->gemv_partials; p.counters = c->gemv_counters; p.status = c->status;
  p.RT = (N + 15) / 16; p.SL = (K + 255) / 256;
  p.U = (unsigned)p.RT * (unsigned)p.SL;
  bool vec = ((uintptr_t)x & 15) == 0 && (K % 4) == 0;
  if (act == 2) vec = vec && ((uintptr_t)delta & 15) == 0;
  if (act == 2 || act == 3) vec = vec && ((uintptr_t)nw & 15) == 0;
  p.x_vec_ok = vec ? 1 : 0;
  p.cta_tiles = pl.cta_tiles;
  p.slabs = pl.slabs;
  p.grid = pl.ctas;
  {
    const unsigned Wall = (unsigned)pl.ctas * PK_WARPS;
    p.Wtot = Wall < p.U ? Wall : p.U;
    p.sp = {p.U / p.Wtot, p.U % p.Wtot};
    if (pl.cta_tiles) {
      const unsigned KB = (unsigned)pl.cta_tiles;
      p.RB = (unsigned)pl.ctas / KB;
      p.ct = {(unsigned)p.RT / p.RB, (unsigned)p.RT % p.RB};
      p.cs = {(unsigned)p.SL / KB, (unsigned)p.SL % KB};
    }
  }
  *plan = pl;
  return TLB_OK;
}

int gemv_q4p_launch(DeviceCtx* c, const void* packed, const float* x, float* y, int N, int K,
                    float alpha, float beta, cudaStream_t stream, int max_ctas,
                    const CommDev* push_comm, int act, const float* delta, const float* nw,
                    float* xout, float eps, const PairEpi* epi, const CommDev* pull_comm,
                    const GvStream* prefetch) {
  GemvPParams p;
  GemvPlan pl;
  {
    const int rc = gemvp_fill(c, packed, x, y, N, K, alpha, beta, max_ctas, push_comm, act, delta, nw, xout, eps,
                              epi, pull_comm, prefetch, &p, &pl);
    if (rc) return rc;
  }
  const int ctas = pl.ctas, stages = pl.stages;
  const size_t smem = gemvp_smem_layout(stages, p.slabs).total;
  if (p.act == 3) {
    if (stages == 4) return gemvp_launch_o<4, true>(p, ctas, smem, stream);
    if (stages == 3) return gemvp_launch_o<3, true>(p, ctas, smem, stream);
    return gemvp_launch_o<2, true>(p, ctas, smem, stream);
  }
  if (stages == 4) return gemvp_launch_o<4, false>(p, ctas, smem, stream);
  if (stages == 3) return gemvp_launch_o<3, false>(p, ctas, smem, stream);
  return gemvp_launch_o<2, false>(p, ctas, smem, stream);
}

// Up to GV_CHAIN_MAX single-GPU GEMVs, each reading what the one before wrote, as one
// persistent launch of one CTA per SM.  *fused = false (and nothing launched) when the phases
// cannot share a ring (different ring depths): the caller then launches them one by one.
int gemv_q4p_chain_launch(DeviceCtx* c, const GvPhase* ph, int nph, cudaStream_t stream, bool* fused) {
  *fused = false;
  if (nph < 2 || nph > GV_CHAIN_MAX) return set_error(TLB_ERR_ARG, "gemv_q4p chain: 2 to 4 phases");
  if (!c->chain_cell) return TLB_OK;
  GvChainParams cp;
  memset(&cp, 0, sizeof(cp));
  size_t smem = 0;
  for (int i = 0; i < nph; i++) {
    GemvPlan pl;
    const int rc = gemvp_fill(c, ph[i].packed, ph[i].x, ph[i].y, ph[i].N, ph[i].K, 1.0f, 0.0f, 0, nullptr, ph[i].act,
                              ph[i].delta, ph[i].nw, ph[i].xout, ph[i].eps, ph[i].epi, nullptr, nullptr, &cp.ph[i],
                              &pl);
    if (rc) return rc;
    if (pl.stages != 4 || pl.ctas > c->sm_count) return TLB_OK;
    const size_t need = gemvp_smem_layout(4, cp.ph[i].slabs).total;
    if (need > smem) smem = need;
  }
  cp.nph = nph;
  cp.cell = c->chain_cell;
  // the instantiated phase signatures: o, gate|up, down, then the next qkv or the lm_head, for
  // wide (7B-like: gate|up in unit ranges) and narrow (0.5B-like: gate|up CTA-owned) shapes
  int code[GV_CHAIN_MAX] = {0, 0, 0, 0};
  for (int i = 0; i < nph; i++) code[i] = (cp.ph[i].cta_tiles ? 3 : 0) + cp.ph[i].epi.kind;
  const int sig = nph == 4 ? code[0] * 1000 + code[1] * 100 + code[2] * 10 + code[3] : -1;
  LaunchCfg lc(dim3(c->sm_count), dim3(PK_WARPS * 32), smem, stream, pdl_enabled());
#define TLB_CHAIN_CASE(A, B, C, D)                                                                         \
  case A * 1000 + B * 100 + C * 10 + D: {                                                                  \
    static std::atomic<unsigned long long> attr_done{0};                                                   \
    const int rc_attr = ensure_dynamic_smem(gemv_q4p_chain_kernel<4, A, B, C, D>, PK_DYN_SMEM_MAX, attr_done);  \
    if (rc_attr) return rc_attr;                                                                           \
    TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, gemv_q4p_chain_kernel<4, A, B, C, D>, cp));                       \
    break;                                                                                                 \
  }
  // every SM gets exactly one CTA (the kernel's shared memory allows no second one), so all
  // CTAs are resident together and the barrier between phases can complete
  const bool looped = getenv("TLB_CHAIN_LOOP") && atoi(getenv("TLB_CHAIN_LOOP")) == 1;
  if (looped) {
    static std::atomic<unsigned long long> attr_done{0};
    const int rc_attr = ensure_dynamic_smem(gemv_q4p_chain_loop_kernel<4>, PK_DYN_SMEM_MAX - 2048, attr_done);
    if (rc_attr) return rc_attr;
    TLB_CUDA(cudaLaunchKernelEx(&lc.cfg, gemv_q4p_chain_loop_kernel<4>, cp));
    *fused = true;
    return TLB_OK;
  }
  switch (sig) {
    TLB_CHAIN_CASE(3, 1, 3, 5)
    TLB_CHAIN_CASE(3, 1, 3, 0)
    TLB_CHAIN_CASE(3, 4, 3, 5)
    TLB_CHAIN_CASE(3, 4, 3, 0)
    default:
      return TLB_OK;   // not fused: the caller launches the phases one by one
  }
#undef TLB_CHAIN_CASE
  *fused = true;
  return TLB_OK;
}

}  // namespace tlb
