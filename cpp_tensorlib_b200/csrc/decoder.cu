// Native driver of the Qwen2.5-architecture int4 decoder: weights, KV caches,
// scratch, the per-token launch sequence, its CUDA graph and the tensor-parallel
// exchange.  Mirrors the structure of the reference's model driver
// (bench/cuda/qwen_model.h: Layer/Scratch/Model :175-308, run_layers_ :673-740,
// captured_decoder :791-905) with every linear held in the q4 layout.
//
// One token (all on one stream, no host sync, position and token id read from
// device memory so one instantiated graph replays as the sequence grows):
//   embed gather -> rmsnorm                                   (layer 0 only)
//   per layer: qkv GEMV -> rope+bias+KV append -> attention -> wo GEMV
//              -> residual add + rmsnorm -> gate|up GEMV -> swiglu -> down GEMV
//              -> residual add + rmsnorm (next layer's input norm / final norm)
//   lm_head GEMV -> argmax -> next token id, position + 1
// Tensor parallel (column-parallel qkv / gate|up / lm_head, row-parallel wo /
// down): the row-parallel GEMVs push their partial outputs to every rank and the
// following add+rmsnorm reduces them (comm.cuh); the lm_head shards exchange
// their local argmax keys.  Each rank is one process on one GPU.
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "comm.cuh"
#include "gemv_q4p.cuh"

namespace tlb {

extern unsigned long long* g_gemv_dbg;

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
size_t attn_partials_bytes(int n_q, int n_kv, long long kv_max, int D, int sm_count);
int attn_decode_launch(DeviceCtx* c, const float* q, const void* K, const void* V, float* out,
                       int n_q, int n_kv, int ctx, long long kv_max, int D, float scale,
                       const unsigned* d_pos, float* partials, int* counters, cudaStream_t stream,
                       int early_kv, int kv_bf16, const GvStream* prefetch = nullptr);
int launch_rmsnorm(const float*, const float*, float*, int, float, int, cudaStream_t);
int launch_embed_rows(const float*, const int*, float*, int, int, cudaStream_t);
int launch_rope(const float*, const float*, float*, int, int, int, unsigned, const unsigned*, float,
                cudaStream_t);
int launch_split_heads(const float*, const float*, float*, int, long long, long long, int, int,
                       cudaStream_t);
int launch_merge_heads(const float*, float*, int, int, int, cudaStream_t);
int launch_kv_fill(void*, void*, const float*, const float*, int, long long, int, int, int, int,
                   cudaStream_t);
int launch_attn_prefill(DeviceCtx*, const float*, const void*, const void*, float*, int, int, int,
                        long long, int, float, int, int, cudaStream_t);
int launch_add_rmsnorm(const float*, const float*, const float*, float*, float*, int, float, int,
                       cudaStream_t);
int launch_add_rmsnorm_ar(const float*, const float*, float*, float*, int, float, const CommDev&,
                          int*, cudaStream_t);
int launch_swiglu(const float*, float*, int, int, cudaStream_t);
int launch_ar_sum(float*, int, const CommDev&, int*, cudaStream_t);
int launch_incr_u32(unsigned*, cudaStream_t);
int launch_qkv_post(float*, const float*, const float*, const float*, float*, float*, int, int,
                    int, const unsigned*, long long, float, int, int*, cudaStream_t);
int launch_embed_gather(const float*, const int*, float*, int, float2*, const unsigned*, int, float,
                        const float*, float*, float, cudaStream_t);
int launch_argmax(DeviceCtx*, const float*, int, int*, int*, cudaStream_t);
int launch_argmax_tp(DeviceCtx*, const float*, int, unsigned, const CommDev&, int*, int*,
                     cudaStream_t);

struct Linear {
  const void* q4 = nullptr;
  int K = 0, N = 0;
  bool tma = false;
  CUtensorMap tmW, tmS;
  void* packed = nullptr;  // tile-packed copy for the decode GEMV (owned)
  int pair_h = 0;          // > 0: packed with rows r, r + pair_h in one thread (pair epilogues)
  const float* scales() const { return (const float*)((const char*)q4 + (size_t)N * K / 2); }
};

struct DecLayer {
  Linear wqkv, wo, wgu, wd;
  const float *bq = nullptr, *bk = nullptr, *bv = nullptr, *an = nullptr, *fn = nullptr;
  float *Kc = nullptr, *Vc = nullptr;
};

struct Decoder {
  // sizes local to this rank (hidden and vocab_offset are global notions)
  int hidden = 0, n_layers = 0, n_q = 0, n_kv = 0, hd = 0, ff = 0, vocab = 0, max_ctx = 0;
  float eps = 1e-6f, rope_base = 1e6f, scale = 1.f;
  int tp_rank = 0, tp_size = 1;
  int kv_bf16 = 0;   // caches hold bf16 (kv_cache::init with dtype::bf16, include/cuda.h:1336-1346)
  unsigned vocab_offset = 0;
  std::vector<DecLayer> layers;
  Linear lm_head;
  const float *embed = nullptr, *onorm = nullptr;
  // scratch
  float *x = nullptr, *xb = nullptr, *hb = nullptr, *qkv = nullptr, *att = nullptr, *t0 = nullptr,
        *t1 = nullptr, *gu = nullptr, *mb = nullptr, *logits = nullptr;
  void* attn_partials = nullptr;
  unsigned* d_pos = nullptr;
  float2* rope_cs = nullptr;  // [hd/2] (cos, sin) of the current position, refreshed per token
  int* d_tok = nullptr;      // token consumed by the next forward; overwritten with the result
  int* d_tok_out = nullptr;  // copy of the last result (read back by the host)
  int *h_tok = nullptr, *h_out = nullptr;  // pinned
  // tensor-parallel exchange
  CommDev comm;
  uint2* stage_local = nullptr;
  unsigned* flags_local = nullptr;  // sequence counter
  void* peer_stage_base[TP_MAX] = {};
  void* peer_flags_base[TP_MAX] = {};
  bool peers_open = false;
  void* sink[TP_MAX] = {};          // loopback drill: stand-ins for peers that never answer
  // batched prompt pass: row-batched scratch for chunks of up to PF_CHUNK tokens
  float* pf = nullptr;
  int* pf_ids = nullptr;
  int pf_rows = 0;          // rows the prefill scratch was sized for
  // graph
  cudaGraphExec_t graph = nullptr;
  long long launches_per_token = 0;
  // Host mirror of the device-resident position (captured_decoder::cur_pos of the reference,
  // bench/cuda/qwen_model.h:877-885): every entry point that advances the sequence checks it
  // against the cache capacity before anything is launched.
  long long host_pos = 0;
  long long vocab_total = 0;   // rows of the embedding table (0: unknown, ids are only checked >= 0)
};

// The reference's feed() returns false when cur_pos >= max_ctx (bench/cuda/qwen_model.h:879);
// here the refusal is an argument error and nothing is launched.
static int room_for(Decoder* d, long long n, const char* who) {
  if (d->host_pos + n > d->max_ctx)
    return set_error(TLB_ERR_ARG, std::string(who) + ": position " + std::to_string(d->host_pos) + " + " +
                                      std::to_string(n) + " token(s) exceeds the cache capacity " +
                                      std::to_string(d->max_ctx));
  return TLB_OK;
}
static int token_ok(Decoder* d, long long token, const char* who) {
  if (token < 0 || (d->vocab_total > 0 && token >= d->vocab_total))
    return set_error(TLB_ERR_ARG, std::string(who) + ": token id " + std::to_string(token) +
                                      " outside the embedding table");
  return TLB_OK;
}

static int set_linear(Linear& L, const void* q4, int K, int N, int pair_h = 0) {
  L.q4 = q4;
  L.K = K;
  L.N = N;
  L.tma = gemv_q4_tma_eligible(q4, L.scales(), N, K, 1);
  if (L.packed) { cudaFree(L.packed); L.packed = nullptr; }
  L.pair_h = 0;
  if (gemv_q4p_supported(N, K)) {
    if (pair_h > 0 && N % 16 == 0 && pair_h % 8 == 0 && N % (2 * pair_h) == 0) L.pair_h = pair_h;
    TLB_CUDA(cudaMalloc(&L.packed, (size_t)q4p_bytes(N, K)));
    int rc = launch_q4_pack(q4, N, K, L.packed, L.pair_h, nullptr);
    if (rc) return rc;
    TLB_CUDA(cudaStreamSynchronize(nullptr));
  }
  if (L.tma) return make_q4_tensor_maps(q4, L.scales(), N, K, &L.tmW, &L.tmS);
  return TLB_OK;
}

// Fused residual add + RMSNorm in front of a linear: input = rmsnorm(x + delta) * w,
// and x + delta is also written to xout (the next residual base).
struct NormIn {
  const float* delta;   // NULL with `pull`: the delta is the sum of an exchange's partial vectors
  const float* w;
  float* xout;
  const CommDev* pull = nullptr;
};

// What the decode launch of linear L will stream first (for the kernel in front of it to
// prefetch); `normed`: launched with the fused add+norm prologue.  Off unless TLB_PREFETCH=1:
// measured on the 7B decode the L2 prefetch of the next kernel's first ring fill LOSES 7 %
// (646 against 693 tokens/s) -- the prefetch competes with the demand copies of the warps that
// are still streaming, and what it brings in is not where the next launch's time goes.
static GvStream stream_of(DeviceCtx* c, const Linear& L, bool normed) {
  GvStream g;
  static const bool on = getenv("TLB_PREFETCH") && atoi(getenv("TLB_PREFETCH")) == 1;
  if (!on || !L.packed || (normed && (L.K + 255) / 256 > 32)) return g;
  if (gemv_q4p_stream_of(c, L.packed, L.N, L.K, normed ? 2 : 0, L.pair_h > 0, 0, &g)) g = GvStream();
  return g;
}

static int run_linear(DeviceCtx* c, const Linear& L, const float* x, float* y, cudaStream_t s,
                      const CommDev* push, int act = 0, const NormIn* nm = nullptr, float eps = 0.f,
                      const PairEpi* epi = nullptr, const GvStream* next = nullptr) {
  if (!L.q4) return set_error(TLB_ERR_STATE, "decoder: a linear weight was never set");
  if ((epi != nullptr) != (L.pair_h > 0))
    return set_error(TLB_ERR_STATE, "decoder: pair-packed weight and epilogue do not match");
  if (L.packed && !(nm && (L.K + 255) / 256 > 32))
    return gemv_q4p_launch(c, L.packed, x, y, L.N, L.K, 1.0f, 0.0f, s, 0, push, nm ? 2 : act,
                           nm ? nm->delta : nullptr, nm ? nm->w : nullptr, nm ? nm->xout : nullptr, eps,
                           epi, nm ? nm->pull : nullptr, next);
  if (epi) return set_error(TLB_ERR_STATE, "decoder: pair epilogue without a packed weight");
  if (nm && nm->pull) return set_error(TLB_ERR_STATE, "decoder: fused exchange without a packed weight");
  if (L.tma && nm)
    return gemv_q4_launch(c, L.tmW, L.tmS, x, L.K, 1, y, L.N, L.N, L.K, 1.0f, 0.0f, s, 0, push, 2,
                          nm->delta, nm->w, nm->xout, eps);
  if (nm) return set_error(TLB_ERR_UNSUPPORTED, "decoder: the fused add+rmsnorm needs K % 128 == 0");
  if (L.tma)
    return gemv_q4_launch(c, L.tmW, L.tmS, x, act ? 2 * L.K : L.K, 1, y, L.N, L.N, L.K, 1.0f, 0.0f,
                          s, 0, push, act, nullptr, nullptr, nullptr, 0.f);
  if (act) return set_error(TLB_ERR_UNSUPPORTED, "decoder: the fused SwiGLU needs ff % 128 == 0");
  if (push) return set_error(TLB_ERR_UNSUPPORTED, "decoder: tensor-parallel linears need K % 128 == 0");
  return gemv_q4_simt_launch(x, L.K, 1, L.q4, L.scales(), y, L.N, L.N, L.K, 1.0f, 0.0f, s);
}

static PairEpi qkv_epilogue(const Decoder* d, const DecLayer& L) {
  PairEpi e;
  e.kind = 2; e.H = d->hd / 2; e.out = d->qkv; e.Kc = L.Kc; e.Vc = L.Vc; e.kv_bf16 = d->kv_bf16;
  e.bq = L.bq; e.bk = L.bk; e.bv = L.bv; e.n_q = d->n_q; e.n_kv = d->n_kv; e.D = d->hd;
  e.d_pos = d->d_pos; e.kv_stride = (long long)d->max_ctx * d->hd; e.kv_rows = d->max_ctx;
  e.base = d->rope_base;
  e.rope_cs = d->rope_cs;
  return e;
}
static PairEpi swiglu_epilogue(const Decoder* d) {
  PairEpi e;
  e.kind = 1; e.H = d->ff; e.out = d->mb;
  return e;
}


static int forward(Decoder* d, cudaStream_t s) {
  DeviceCtx* c = nullptr;
  int rc = get_ctx(&c);
  if (rc) return rc;
  const bool tp = d->tp_size > 1;
  const int E = d->hidden;
  long long n = 0;
#define RUN(expr)        \
  do {                   \
    rc = (expr);         \
    if (rc) return rc;   \
    n++;                 \
  } while (0)
  if (!d->embed || !d->onorm) return set_error(TLB_ERR_STATE, "decoder: embed / final norm not set");
  // embedding row, the token's rotary table and the first layer's attention norm in one block
  RUN(launch_embed_gather(d->embed, d->d_tok, d->x, E, d->rope_cs, d->d_pos, d->hd, d->rope_base,
                          d->layers[0].an, d->hb, d->eps, s));
  bool all_tma = d->lm_head.tma && d->lm_head.packed;
  for (auto& L : d->layers)
    all_tma = all_tma && L.wqkv.tma && L.wo.tma && L.wgu.tma && L.wd.tma && L.wqkv.packed &&
              L.wo.packed && L.wgu.packed && L.wd.packed;
  // exchanges of one token: after wo and after wd of every layer, then the argmax
  const int EX = 2 * d->n_layers + 1;
  auto cm = [&](int k) {
    CommDev c2 = d->comm;
    c2.k = k;
    c2.E = EX;
    return c2;
  };
  // How a tensor-parallel exchange is consumed.  Default: a small multi-CTA kernel sums the
  // ranks' packets into a local vector (ar_sum_kernel) and the next projection's ordinary fused
  // add+norm prologue reads that vector -- one short extra launch per exchange, no system-scope
  // polling from 148 CTAs.  (Summing in the LAST CTA of the pushing projection instead was
  // built and measured on 2 GPUs: 494 against 732 tokens/s -- a CTA that polls while the
  // peers' stores are still arriving is far slower than one launched after them.)  TLB_TP_PULL_MAX = largest rank count whose exchanges are instead
  // consumed inside the next projection's prologue (it polls the packets itself: two kernels
  // fewer per layer, measured slower on 2 GPUs, 582 vs 589 tok/s); TLB_TP_SUM=0 selects the
  // older single-CTA add+norm consumer (add_rmsnorm_ar_kernel).
  const char* pm = getenv("TLB_TP_PULL_MAX");
  const int pull_max = pm ? atoi(pm) : 1;
  const char* ts = getenv("TLB_TP_SUM");
  const bool tp_sum = !(ts && atoi(ts) == 0);
  const bool pull = tp && d->tp_size <= pull_max;
  if (all_tma && (!tp || pull || tp_sum)) {
    // Both residual adds and norms of a layer run inside the following projection's
    // activation prep (5 launches per layer, + one packet-sum launch per exchange when tensor
    // parallel).  The residual ping-pongs between two buffers because every CTA of the
    // projection reads it while one CTA writes the new sum.
    const bool sum = tp && !pull;
    float* x = d->x;
    float* xalt = d->xb;
    // Single GPU: the four projections between two attention calls (o, gate|up, down, the
    // next layer's qkv or the lm_head) run as the phases of ONE persistent launch whose
    // weight ring streams across the phase boundaries.  Opt-in (TLB_CHAIN=1): measured on the
    // 7B shape it is SLOWER than one launch each (575 - 600 against 685 tokens/s), because
    // what a projection costs beyond its stream is the activation prep and the fold of the
    // partial sums -- about 800 instructions per warp of mostly serial code -- and a phase
    // pays those plus the barrier (1.5 us), where a launch of its own pays them plus 1.3 us.
    const char* ch = getenv("TLB_CHAIN");
    const bool chain = !tp && ch && atoi(ch) == 1;
    bool qkv_done = false;   // this layer's qkv ran as the last phase of the chain before it
    bool head_done = false;
    for (int l = 0; l < d->n_layers; l++) {
      DecLayer& L = d->layers[l];
      const PairEpi eq = qkv_epilogue(d, L), eg = swiglu_epilogue(d);
      const PairEpi* pq = L.wqkv.pair_h > 0 ? &eq : nullptr;
      const PairEpi* pg = L.wgu.pair_h > 0 ? &eg : nullptr;
      const CommDev c_prev = cm(2 * l - 1), c_wo = cm(2 * l), c_wd = cm(2 * l + 1);
      // each weight-streaming kernel asks the L2 for the head of the next one's stream
      const GvStream s_wo = stream_of(c, L.wo, false), s_gu = stream_of(c, L.wgu, true),
                     s_wd = stream_of(c, L.wd, false),
                     s_nx = l + 1 < d->n_layers ? stream_of(c, d->layers[l + 1].wqkv, true)
                                                : stream_of(c, d->lm_head, true);
      if (qkv_done) {
        qkv_done = false;
      } else if (l == 0) {
        RUN(run_linear(c, L.wqkv, d->hb, d->qkv, s, nullptr, 0, nullptr, 0.f, pq));
      } else {
        NormIn nm{pull ? nullptr : d->t1, L.an, xalt, pull ? &c_prev : nullptr};
        RUN(run_linear(c, L.wqkv, x, d->qkv, s, nullptr, 0, &nm, d->eps, pq));
        float* t = x; x = xalt; xalt = t;
      }
      if (!pq)
        RUN(launch_qkv_post(d->qkv, L.bq, L.bk, L.bv, L.Kc, L.Vc, d->n_q, d->n_kv, d->hd, d->d_pos,
                            d->max_ctx, d->rope_base, d->kv_bf16, c->status, s));
      RUN(attn_decode_launch(c, d->qkv, L.Kc, L.Vc, d->att, d->n_q, d->n_kv, 0, d->max_ctx, d->hd,
                             d->scale, d->d_pos, (float*)((char*)d->attn_partials + 256),
                             (int*)d->attn_partials, s, 1, d->kv_bf16, &s_wo));
      if (chain && pg && (E + 255) / 256 <= 32) {
        const bool last = l + 1 == d->n_layers;
        const Linear& nx = last ? d->lm_head : d->layers[l + 1].wqkv;
        PairEpi eqn;
        if (!last) eqn = qkv_epilogue(d, d->layers[l + 1]);
        const bool nx_pair = nx.pair_h > 0;
        if (last ? !nx_pair : nx_pair) {
          GvPhase ph[4];
          ph[0].packed = L.wo.packed; ph[0].x = d->att; ph[0].y = d->t0; ph[0].N = L.wo.N; ph[0].K = L.wo.K;
          ph[1].packed = L.wgu.packed; ph[1].x = x; ph[1].y = d->gu; ph[1].N = L.wgu.N; ph[1].K = L.wgu.K;
          ph[1].act = 2; ph[1].delta = d->t0; ph[1].nw = L.fn; ph[1].xout = xalt; ph[1].eps = d->eps; ph[1].epi = pg;
          ph[2].packed = L.wd.packed; ph[2].x = d->mb; ph[2].y = d->t1; ph[2].N = L.wd.N; ph[2].K = L.wd.K;
          // after gate|up the residual lives in xalt: the fourth phase reads it and writes x
          ph[3].packed = nx.packed; ph[3].x = xalt; ph[3].y = last ? d->logits : d->qkv; ph[3].N = nx.N; ph[3].K = nx.K;
          ph[3].act = 2; ph[3].delta = d->t1; ph[3].nw = last ? d->onorm : d->layers[l + 1].an; ph[3].xout = x;
          ph[3].eps = d->eps; ph[3].epi = last ? nullptr : &eqn;
          bool fused = false;
          rc = gemv_q4p_chain_launch(c, ph, 4, s, &fused);
          if (rc) return rc;
          if (fused) {
            n++;
            // two swaps (gate|up, then the fourth phase): x is the residual again
            if (last) head_done = true; else qkv_done = true;
            continue;
          }
        }
      }
      RUN(run_linear(c, L.wo, d->att, tp ? nullptr : d->t0, s, tp ? &c_wo : nullptr, 0, nullptr, 0.f, nullptr,
                     &s_gu));
      if (sum) RUN(launch_ar_sum(d->t0, E, c_wo, c->status, s));
      NormIn nf{pull ? nullptr : d->t0, L.fn, xalt, pull ? &c_wo : nullptr};
      RUN(run_linear(c, L.wgu, x, d->gu, s, nullptr, 0, &nf, d->eps, pg, &s_wd));
      { float* t = x; x = xalt; xalt = t; }
      if (pg) {
        RUN(run_linear(c, L.wd, d->mb, tp ? nullptr : d->t1, s, tp ? &c_wd : nullptr, 0, nullptr, 0.f, nullptr,
                       &s_nx));
      } else {
        RUN(run_linear(c, L.wd, d->gu, tp ? nullptr : d->t1, s, tp ? &c_wd : nullptr, 1, nullptr, 0.f, nullptr,
                       &s_nx));
      }
      if (sum) RUN(launch_ar_sum(d->t1, E, c_wd, c->status, s));
    }
    const CommDev c_last = cm(2 * d->n_layers - 1);
    NormIn no{pull ? nullptr : d->t1, d->onorm, xalt, pull ? &c_last : nullptr};
    // the next token starts with layer 0's QKV projection (plain prologue: its norm is done
    // by the embedding gather)
    const GvStream s_q0 = stream_of(c, d->layers[0].wqkv, false);
    if (!head_done) RUN(run_linear(c, d->lm_head, x, d->logits, s, nullptr, 0, &no, d->eps, nullptr, &s_q0));
    if (tp) {
      RUN(launch_argmax_tp(c, d->logits, d->vocab, d->vocab_offset, cm(2 * d->n_layers), d->d_tok,
                           d->d_tok_out, s));
      n++;  // two kernels
    } else {
      RUN(launch_argmax(c, d->logits, d->vocab, d->d_tok, d->d_tok_out, s));
    }
    RUN(launch_incr_u32(d->d_pos, s));
    d->launches_per_token = n;
    return TLB_OK;
  }
  for (int l = 0; l < d->n_layers; l++) {
    DecLayer& L = d->layers[l];
    const PairEpi eq = qkv_epilogue(d, L), eg = swiglu_epilogue(d);
    const PairEpi* pq = L.wqkv.pair_h > 0 ? &eq : nullptr;
    const PairEpi* pg = L.wgu.pair_h > 0 ? &eg : nullptr;
    const CommDev c_wo = cm(2 * l), c_wd = cm(2 * l + 1);
    RUN(run_linear(c, L.wqkv, d->hb, d->qkv, s, nullptr, 0, nullptr, 0.f, pq));
    if (!pq)
      RUN(launch_qkv_post(d->qkv, L.bq, L.bk, L.bv, L.Kc, L.Vc, d->n_q, d->n_kv, d->hd, d->d_pos,
                          d->max_ctx, d->rope_base, d->kv_bf16, c->status, s));
    RUN(attn_decode_launch(c, d->qkv, L.Kc, L.Vc, d->att, d->n_q, d->n_kv, 0, d->max_ctx, d->hd,
                           d->scale, d->d_pos, (float*)((char*)d->attn_partials + 256),
                           (int*)d->attn_partials, s, 1, d->kv_bf16));
    if (tp) {
      RUN(run_linear(c, L.wo, d->att, nullptr, s, &c_wo));
      RUN(launch_add_rmsnorm_ar(d->x, L.fn, d->x, d->hb, E, d->eps, c_wo, c->status, s));
    } else {
      RUN(run_linear(c, L.wo, d->att, d->t0, s, nullptr));
      RUN(launch_add_rmsnorm(d->x, d->t0, L.fn, d->x, d->hb, E, d->eps, 1, s));
    }
    RUN(run_linear(c, L.wgu, d->hb, d->gu, s, nullptr, 0, nullptr, 0.f, pg));
    // SwiGLU: in the gate|up epilogue (pair-packed), else inside the down projection's
    // activation prep, else its own kernel
    const bool fuse_act = !pg && L.wd.tma;
    if (!pg && !fuse_act) RUN(launch_swiglu(d->gu, d->mb, d->ff, 1, s));
    const float* nextw = (l + 1 < d->n_layers) ? d->layers[l + 1].an : d->onorm;
    if (tp) {
      RUN(run_linear(c, L.wd, fuse_act ? d->gu : d->mb, nullptr, s, &c_wd, fuse_act ? 1 : 0));
      RUN(launch_add_rmsnorm_ar(d->x, nextw, d->x, d->hb, E, d->eps, c_wd, c->status, s));
    } else {
      RUN(run_linear(c, L.wd, fuse_act ? d->gu : d->mb, d->t0, s, nullptr, fuse_act ? 1 : 0));
      RUN(launch_add_rmsnorm(d->x, d->t0, nextw, d->x, d->hb, E, d->eps, 1, s));
    }
  }
  RUN(run_linear(c, d->lm_head, d->hb, d->logits, s, nullptr));
  if (tp) {
    RUN(launch_argmax_tp(c, d->logits, d->vocab, d->vocab_offset, cm(2 * d->n_layers), d->d_tok,
                         d->d_tok_out, s));
    n++;  // two kernels
  } else {
    RUN(launch_argmax(c, d->logits, d->vocab, d->d_tok, d->d_tok_out, s));
  }
  RUN(launch_incr_u32(d->d_pos, s));
#undef RUN
  d->launches_per_token = n;
  return TLB_OK;
}

}  // namespace tlb

using namespace tlb;

extern "C" {

// cfg: hidden, n_layers, n_q, n_kv, hd, ff, vocab, max_ctx (sizes LOCAL to the
// rank except hidden), then tp_rank, tp_size, vocab_offset.
int tlb_decoder_create(const int64_t* cfg, int n_cfg, float eps, float rope_base, void** out) {
  TLB_REQUIRE(cfg && out && n_cfg >= 11, "tlb_decoder_create: bad arguments");
  DeviceCtx* c = nullptr;
  int rc = get_ctx(&c);
  if (rc) return rc;
  auto* d = new Decoder();
  d->hidden = (int)cfg[0]; d->n_layers = (int)cfg[1]; d->n_q = (int)cfg[2]; d->n_kv = (int)cfg[3];
  d->hd = (int)cfg[4]; d->ff = (int)cfg[5]; d->vocab = (int)cfg[6]; d->max_ctx = (int)cfg[7];
  d->tp_rank = (int)cfg[8]; d->tp_size = (int)cfg[9]; d->vocab_offset = (unsigned)cfg[10];
  // cfg[11] (optional): rows of the embedding table; without it a single-GPU decoder knows it
  // from its own vocabulary, a tensor-parallel shard does not
  d->vocab_total = n_cfg >= 12 ? cfg[11] : (d->tp_size == 1 ? d->vocab : 0);
  // cfg[12] (optional): 1 = the KV caches hold bf16 (half the KV stream; values rounded to
  // nearest even on append, widened exactly for the dot and the accumulate)
  d->kv_bf16 = n_cfg >= 13 && cfg[12] != 0 ? 1 : 0;
  d->eps = eps; d->rope_base = rope_base; d->scale = 1.0f / sqrtf((float)d->hd);
  TLB_REQUIRE(d->hd == 64 || d->hd == 128, "tlb_decoder_create: head_dim must be 64 or 128");
  TLB_REQUIRE(d->n_kv > 0 && d->n_q % d->n_kv == 0 && d->n_kv <= 64, "tlb_decoder_create: bad head counts");
  TLB_REQUIRE(d->tp_size >= 1 && d->tp_size <= TP_MAX && d->tp_rank >= 0 && d->tp_rank < d->tp_size,
              "tlb_decoder_create: bad tensor-parallel rank/size");
  TLB_REQUIRE(d->n_layers > 0 && d->hidden > 0 && d->max_ctx > 0, "tlb_decoder_create: bad sizes");
  d->layers.resize(d->n_layers);
  const size_t kvb = (size_t)d->n_kv * d->max_ctx * d->hd * (d->kv_bf16 ? 2 : sizeof(float));
  for (auto& L : d->layers) {
    TLB_CUDA(cudaMalloc(&L.Kc, kvb));
    TLB_CUDA(cudaMalloc(&L.Vc, kvb));
    TLB_CUDA(cudaMemset(L.Kc, 0, kvb));
    TLB_CUDA(cudaMemset(L.Vc, 0, kvb));
  }
  auto fa = [&](float** p, size_t n) { return cudaMalloc(p, n * sizeof(float)); };
  TLB_CUDA(fa(&d->x, d->hidden));
  TLB_CUDA(fa(&d->xb, d->hidden));
  TLB_CUDA(fa(&d->t1, d->hidden));
  TLB_CUDA(fa(&d->hb, d->hidden));
  TLB_CUDA(fa(&d->qkv, (size_t)(d->n_q + 2 * d->n_kv) * d->hd));
  TLB_CUDA(fa(&d->att, (size_t)d->n_q * d->hd));
  TLB_CUDA(fa(&d->t0, d->hidden));
  TLB_CUDA(fa(&d->gu, (size_t)2 * d->ff));
  TLB_CUDA(fa(&d->mb, d->ff));
  TLB_CUDA(fa(&d->logits, d->vocab));
  size_t pb = 256 + attn_partials_bytes(d->n_q, d->n_kv, d->max_ctx, d->hd, c->sm_count);
  TLB_CUDA(cudaMalloc(&d->attn_partials, pb));
  TLB_CUDA(cudaMemset(d->attn_partials, 0, pb));
  TLB_CUDA(cudaMalloc(&d->rope_cs, (size_t)(d->hd / 2) * sizeof(float2)));
  TLB_CUDA(cudaMalloc(&d->d_pos, 16));
  TLB_CUDA(cudaMemset(d->d_pos, 0, 16));
  TLB_CUDA(cudaMalloc(&d->d_tok, 16));
  TLB_CUDA(cudaMemset(d->d_tok, 0, 16));
  d->d_tok_out = d->d_tok + 1;
  TLB_CUDA(cudaMallocHost(&d->h_tok, 64));
  d->h_out = d->h_tok + 4;
  // exchange buffers (allocated even at tp_size 1: tiny)
  d->comm.rank = d->tp_rank;
  d->comm.size = d->tp_size;
  d->comm.slot_floats = (d->hidden + 3) & ~3;
  const size_t sb = (size_t)2 * d->tp_size * d->comm.slot_floats * sizeof(uint2);
  TLB_CUDA(cudaMalloc(&d->stage_local, sb));
  TLB_CUDA(cudaMemset(d->stage_local, 0, sb));
  TLB_CUDA(cudaMalloc(&d->flags_local, 256));
  TLB_CUDA(cudaMemset(d->flags_local, 0, 256));
  d->comm.stage[d->tp_rank] = d->stage_local;
  d->comm.seq = d->flags_local;
  TLB_CUDA(cudaDeviceSynchronize());
  *out = d;
  return TLB_OK;
}

int tlb_decoder_destroy(void* h) {
  auto* d = (Decoder*)h;
  if (!d) return TLB_OK;
  cudaDeviceSynchronize();
  if (d->graph) cudaGraphExecDestroy(d->graph);
  if (d->peers_open)
    for (int r = 0; r < d->tp_size; r++)
      if (r != d->tp_rank) {
        if (d->peer_stage_base[r]) cudaIpcCloseMemHandle(d->peer_stage_base[r]);
        if (d->peer_flags_base[r]) cudaIpcCloseMemHandle(d->peer_flags_base[r]);
      }
  for (auto& L : d->layers) {
    cudaFree(L.Kc); cudaFree(L.Vc);
    cudaFree(L.wqkv.packed); cudaFree(L.wo.packed); cudaFree(L.wgu.packed); cudaFree(L.wd.packed);
  }
  cudaFree(d->lm_head.packed);
  float* bufs[] = {d->x, d->xb, d->t1, d->hb, d->qkv, d->att, d->t0, d->gu, d->mb, d->logits};
  for (float* b : bufs) cudaFree(b);
  cudaFree(d->stage_local);
  for (void* sk : d->sink) cudaFree(sk);
  cudaFree(d->rope_cs);
  cudaFree(d->pf); cudaFree(d->pf_ids);
  cudaFree(d->attn_partials); cudaFree(d->d_pos); cudaFree(d->d_tok); cudaFree(d->flags_local);
  cudaFreeHost(d->h_tok);
  delete d;
  return TLB_OK;
}

// which: 0 wqkv [hidden -> (n_q+2n_kv)hd]  1 wo [n_q*hd -> hidden]  2 wgu [hidden -> 2ff]
//        3 wd [ff -> hidden]  4 lm_head [hidden -> vocab] (layer ignored).
// q4 is a DEVICE pointer to a buffer in the q4 layout, borrowed for the decoder's life.
int tlb_decoder_set_linear(void* h, int64_t layer, int which, const void* q4, int64_t K, int64_t N) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d && q4 && K > 0 && N > 0 && K % 32 == 0, "tlb_decoder_set_linear: bad arguments");
  const int E = d->hidden, QKV = (d->n_q + 2 * d->n_kv) * d->hd;
  Linear* L = nullptr;
  int64_t wantK = 0, wantN = 0;
  if (which == 4) { L = &d->lm_head; wantK = E; wantN = d->vocab; }
  else {
    TLB_REQUIRE(layer >= 0 && layer < d->n_layers, "tlb_decoder_set_linear: layer out of range");
    DecLayer& Y = d->layers[layer];
    if (which == 0) { L = &Y.wqkv; wantK = E; wantN = QKV; }
    else if (which == 1) { L = &Y.wo; wantK = (int64_t)d->n_q * d->hd; wantN = E; }
    else if (which == 2) { L = &Y.wgu; wantK = E; wantN = 2 * d->ff; }
    else if (which == 3) { L = &Y.wd; wantK = d->ff; wantN = E; }
    else return set_error(TLB_ERR_ARG, "tlb_decoder_set_linear: unknown weight id");
  }
  TLB_REQUIRE(K == wantK && N == wantN, "tlb_decoder_set_linear: shape does not match the config");
  // q/k/v rows are packed as rotary pairs and gate/up rows as (gate, up) pairs, so the
  // projection's epilogue finishes rope / SwiGLU itself
  const int pair_h = which == 0 ? d->hd / 2 : (which == 2 ? d->ff : 0);
  return set_linear(*L, q4, (int)K, (int)N, pair_h);
}

// which: 0 attn norm  1 ffn norm  2 bq  3 bk  4 bv (may be NULL: no bias)  5 final norm
//        6 embedding table [vocab_total, hidden] (layer ignored for 5 and 6). Device pointers.
int tlb_decoder_set_vector(void* h, int64_t layer, int which, const float* v) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d, "tlb_decoder_set_vector: null decoder");
  if (which == 5) { d->onorm = v; return TLB_OK; }
  if (which == 6) { d->embed = v; return TLB_OK; }
  TLB_REQUIRE(layer >= 0 && layer < d->n_layers, "tlb_decoder_set_vector: layer out of range");
  DecLayer& L = d->layers[layer];
  if (which == 0) L.an = v; else if (which == 1) L.fn = v; else if (which == 2) L.bq = v;
  else if (which == 3) L.bk = v; else if (which == 4) L.bv = v;
  else return set_error(TLB_ERR_ARG, "tlb_decoder_set_vector: unknown vector id");
  return TLB_OK;
}

// Device pointers of one layer's K and V cache ([n_kv, max_ctx, hd] f32) so the
// caller can pre-fill a context.
int tlb_decoder_kv(void* h, int64_t layer, void** K, void** V) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d && K && V && layer >= 0 && layer < d->n_layers, "tlb_decoder_kv: bad arguments");
  *K = d->layers[layer].Kc;
  *V = d->layers[layer].Vc;
  return TLB_OK;
}
int tlb_decoder_logits(void* h, void** logits) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d && logits, "tlb_decoder_logits: bad arguments");
  *logits = d->logits;
  return TLB_OK;
}
int tlb_decoder_set_pos(void* h, int64_t pos, void* stream) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d && pos >= 0 && pos < d->max_ctx, "tlb_decoder_set_pos: position outside the cache");
  d->h_tok[8] = (int)pos;
  TLB_CUDA(cudaMemcpyAsync(d->d_pos, &d->h_tok[8], 4, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  TLB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  d->host_pos = pos;
  return TLB_OK;
}
int tlb_decoder_set_token(void* h, int64_t token, void* stream) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d, "tlb_decoder_set_token: null decoder");
  {
    const int rc = token_ok(d, token, "tlb_decoder_set_token");
    if (rc) return rc;
  }
  d->h_tok[0] = (int)token;
  TLB_CUDA(cudaMemcpyAsync(d->d_tok, d->h_tok, 4, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  TLB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return TLB_OK;
}


// Enqueue one token's launches on `stream` (capturable: no sync, no allocation).
int tlb_decoder_forward(void* h, void* stream) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d, "tlb_decoder_forward: null decoder");
  int rc = room_for(d, 1, "tlb_decoder_forward");
  if (rc) return rc;
  rc = forward(d, (cudaStream_t)stream);
  if (!rc) d->host_pos++;
  return rc;
}
int64_t tlb_decoder_launches_per_token(void* h) {
  auto* d = (Decoder*)h;
  return d ? d->launches_per_token : 0;
}

// Capture one forward into an executable graph owned by the decoder
// (qwen_model.h:791-905 captured_decoder::init_).
int tlb_decoder_capture(void* h) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d, "tlb_decoder_capture: null decoder");
  if (d->graph) { cudaGraphExecDestroy(d->graph); d->graph = nullptr; }
  cudaStream_t s;
  TLB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  TLB_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
  int rc = forward(d, s);
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(s, &g);
  cudaStreamDestroy(s);
  if (rc) { if (g) cudaGraphDestroy(g); return rc; }
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture");
  e = cudaGraphInstantiate(&d->graph, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
  return TLB_OK;
}

// Replay the captured token `n` times back to back; the token id feeds back on
// the device (greedy decoding with no host round trip).
int tlb_decoder_run(void* h, int64_t n, void* stream) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d && d->graph, "tlb_decoder_run: capture the decoder first");
  TLB_REQUIRE(n >= 0, "tlb_decoder_run: negative token count");
  const int rc = room_for(d, n, "tlb_decoder_run");
  if (rc) return rc;
  for (int64_t i = 0; i < n; i++) {
    TLB_CUDA(cudaGraphLaunch(d->graph, (cudaStream_t)stream));
    d->host_pos++;
  }
  return TLB_OK;
}

// End-to-end step with HOST buffers: token id in (host), next token id out (host).
// H2D of the id, one graph replay (or eager launches when not captured), D2H of
// the result, stream synchronised.  token_in < 0 keeps the device-resident token.
int tlb_decoder_step(void* h, const int32_t* token_in, int32_t* token_out, void* stream) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d && token_out, "tlb_decoder_step: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  {
    int rc = room_for(d, 1, "tlb_decoder_step");
    if (!rc && token_in && *token_in >= 0) rc = token_ok(d, *token_in, "tlb_decoder_step");
    if (rc) return rc;
  }
  if (token_in && *token_in >= 0) {
    d->h_tok[0] = *token_in;
    TLB_CUDA(cudaMemcpyAsync(d->d_tok, d->h_tok, 4, cudaMemcpyHostToDevice, s));
  }
  if (d->graph) TLB_CUDA(cudaGraphLaunch(d->graph, s));
  else {
    int rc = forward(d, s);
    if (rc) return rc;
  }
  d->host_pos++;
  TLB_CUDA(cudaMemcpyAsync(d->h_out, d->d_tok_out, 4, cudaMemcpyDeviceToHost, s));
  TLB_CUDA(cudaStreamSynchronize(s));
  *token_out = d->h_out[0];
  return TLB_OK;
}
// ---- batched prompt pass (bench/cuda/qwen_model.h:357-442 prefill_chunk_ / prefill_batched):
// the same forward as the decode step with one row per prompt token -- every projection is a
// GEMM on the int4 weights (tensor cores for more than 8 rows), attention is one tiled causal
// pass over the cache -- in chunks of up to 1024 tokens starting at the decoder's current
// position.  Leaves the caches and the position at pos + T, the greedy next token in the
// device-resident token cell (so tlb_decoder_run continues from there) and in *next_token.
// Single GPU; the weights are read in the reference layout the caller handed to
// tlb_decoder_set_linear, which must still be alive.
int tlb_decoder_prefill(void* h, const int32_t* tokens, int64_t T, int32_t* next_token, void* stream) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d && tokens && T > 0, "tlb_decoder_prefill: bad arguments");
  if (d->tp_size != 1) return set_error(TLB_ERR_UNSUPPORTED, "tlb_decoder_prefill: single GPU only");
  if (!d->embed || !d->onorm) return set_error(TLB_ERR_STATE, "decoder: embed / final norm not set");
  DeviceCtx* c = nullptr;
  int rc = get_ctx(&c);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  // rows per pass: enough CTAs for the narrow (hidden-wide) projections; TLB_PREFILL_CHUNK overrides
  int CH = 1024;
  if (const char* e = getenv("TLB_PREFILL_CHUNK")) CH = atoi(e) < 16 ? 16 : (atoi(e) > 8192 ? 8192 : atoi(e));
  const int E = d->hidden, D = d->hd, NQ = d->n_q, NKV = d->n_kv, FF = d->ff;
  const int QKV = (NQ + 2 * NKV) * D;
  unsigned pos0 = 0;
  TLB_CUDA(cudaMemcpyAsync(&pos0, d->d_pos, 4, cudaMemcpyDeviceToHost, s));
  TLB_CUDA(cudaStreamSynchronize(s));
  if ((long long)pos0 + T > d->max_ctx)
    return set_error(TLB_ERR_ARG, "tlb_decoder_prefill: the prompt does not fit the cache");
  for (int64_t i = 0; i < T; i++) {
    rc = token_ok(d, tokens[i], "tlb_decoder_prefill");
    if (rc) return rc;
  }
  // row-batched scratch, carved from one allocation
  const size_t n_emb = (size_t)CH * E, n_qkv = (size_t)CH * QKV, n_att = (size_t)CH * NQ * D,
               n_gu = (size_t)CH * 2 * FF, n_mb = (size_t)CH * FF;
  const size_t total = 5 * n_emb /* res0 res1 h h2 md */ + 2 * n_qkv + 2 * n_att + n_gu + n_mb;
  if (d->pf && d->pf_rows < CH) {
    TLB_CUDA(cudaStreamSynchronize(s));
    TLB_CUDA(cudaFree(d->pf));
    TLB_CUDA(cudaFree(d->pf_ids));
    d->pf = nullptr;
    d->pf_ids = nullptr;
  }
  if (!d->pf) {
    TLB_CUDA(cudaMalloc(&d->pf, total * sizeof(float)));
    TLB_CUDA(cudaMalloc(&d->pf_ids, CH * sizeof(int)));
    d->pf_rows = CH;
  }
  float* p = d->pf;
  float* res[2] = {p, p + n_emb};
  p += 2 * n_emb;
  float* hrow = p; p += n_emb;
  float* h2 = p; p += n_emb;
  float* md = p; p += n_emb;
  float* qkv = p; p += n_qkv;
  float* qkvh = p; p += n_qkv;
  float* ah = p; p += n_att;
  float* at = p; p += n_att;
  float* gu = p; p += n_gu;
  float* mb = p;
  auto gemm = [&](const Linear& L, const float* x, float* y, int rows) -> int {
    if (!L.q4) return set_error(TLB_ERR_STATE, "decoder: a linear weight was never set");
    return tlb_gemm_q4(x, rows, L.K, L.q4, L.scales(), y, L.N, L.N, L.K, 1.0f, 0.0f, s);
  };
#define PF(expr) do { rc = (expr); if (rc) return rc; } while (0)
  int last_rows = 0;
  for (int64_t t0 = 0; t0 < T; t0 += CH) {
    const int rows = (int)((T - t0) < CH ? (T - t0) : CH);
    const unsigned pos = pos0 + (unsigned)t0;
    last_rows = rows;
    TLB_CUDA(cudaMemcpyAsync(d->pf_ids, tokens + t0, (size_t)rows * sizeof(int), cudaMemcpyHostToDevice, s));
    float* x = res[1];   // the chunk's embeddings; layer l writes its residual into res[l & 1]
    PF(launch_embed_rows(d->embed, d->pf_ids, x, E, rows, s));
    PF(launch_rmsnorm(x, d->layers[0].an, hrow, E, d->eps, rows, s));
    for (int l = 0; l < d->n_layers; l++) {
      DecLayer& L = d->layers[l];
      float* ro = res[l & 1];
      PF(gemm(L.wqkv, hrow, qkv, rows));
      // token-major [rows, q|k|v] -> head-major [n_q + 2 n_kv, rows, D], biases riding along
      float* kh = qkvh + (size_t)NQ * rows * D;
      float* vh = qkvh + (size_t)(NQ + NKV) * rows * D;
      PF(launch_split_heads(qkv, L.bq, qkvh, rows, QKV, 0, NQ, D, s));
      PF(launch_split_heads(qkv, L.bk, kh, rows, QKV, (long long)NQ * D, NKV, D, s));
      PF(launch_split_heads(qkv, L.bv, vh, rows, QKV, (long long)(NQ + NKV) * D, NKV, D, s));
      // [H, rows, D] flattened: row r = h*rows + t, so rope's position is pos + r % rows
      PF(launch_rope(qkvh, nullptr, qkvh, NQ * rows, rows, D, pos, nullptr, d->rope_base, s));
      PF(launch_rope(kh, nullptr, kh, NKV * rows, rows, D, pos, nullptr, d->rope_base, s));
      PF(launch_kv_fill(L.Kc, L.Vc, kh, vh, rows, d->max_ctx, NKV, D, (int)pos, d->kv_bf16, s));
      PF(launch_attn_prefill(c, qkvh, L.Kc, L.Vc, ah, NQ, NKV, rows, d->max_ctx, D, d->scale, (int)pos,
                             d->kv_bf16, s));
      PF(launch_merge_heads(ah, at, rows, NQ, D, s));
      PF(gemm(L.wo, at, md, rows));
      PF(launch_add_rmsnorm(x, md, L.fn, ro, h2, E, d->eps, rows, s));
      PF(gemm(L.wgu, h2, gu, rows));
      PF(launch_swiglu(gu, mb, FF, rows, s));
      PF(gemm(L.wd, mb, md, rows));
      const float* nextw = (l + 1 < d->n_layers) ? d->layers[l + 1].an : d->onorm;
      PF(launch_add_rmsnorm(ro, md, nextw, ro, hrow, E, d->eps, rows, s));
      x = ro;
    }
  }
  // logits only for the last row of the last chunk (hrow holds its final norm)
  PF(run_linear(c, d->lm_head, hrow + (size_t)(last_rows - 1) * E, d->logits, s, nullptr));
  PF(launch_argmax(c, d->logits, d->vocab, d->d_tok, d->d_tok_out, s));
#undef PF
  const unsigned newpos = pos0 + (unsigned)T;
  d->h_tok[1] = (int)newpos;
  TLB_CUDA(cudaMemcpyAsync(d->d_pos, &d->h_tok[1], 4, cudaMemcpyHostToDevice, s));
  TLB_CUDA(cudaMemcpyAsync(d->h_out, d->d_tok_out, 4, cudaMemcpyDeviceToHost, s));
  TLB_CUDA(cudaStreamSynchronize(s));
  d->host_pos = (long long)newpos;
  if (next_token) *next_token = d->h_out[0];
  return TLB_OK;
}

int tlb_decoder_last_token(void* h, int32_t* token_out, void* stream) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d && token_out, "tlb_decoder_last_token: bad arguments");
  TLB_CUDA(cudaMemcpyAsync(d->h_out, d->d_tok_out, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  TLB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  *token_out = d->h_out[0];
  return TLB_OK;
}

// ---- tensor-parallel wiring: exchange 128-byte records between the ranks (any
// host channel), then open the peers' buffers.  Record = two CUDA IPC handles.
int tlb_decoder_ipc_export(void* h, void* record128) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d && record128, "tlb_decoder_ipc_export: bad arguments");
  cudaIpcMemHandle_t a, b;
  TLB_CUDA(cudaIpcGetMemHandle(&a, d->stage_local));
  TLB_CUDA(cudaIpcGetMemHandle(&b, d->flags_local));
  memcpy(record128, &a, 64);
  memcpy((char*)record128 + 64, &b, 64);
  return TLB_OK;
}
// records: tp_size consecutive 128-byte records, index = rank.
int tlb_decoder_ipc_open(void* h, const void* records) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d && records, "tlb_decoder_ipc_open: bad arguments");
  for (int r = 0; r < d->tp_size; r++) {
    if (r == d->tp_rank) continue;
    cudaIpcMemHandle_t a, b;
    memcpy(&a, (const char*)records + (size_t)r * 128, 64);
    memcpy(&b, (const char*)records + (size_t)r * 128 + 64, 64);
    TLB_CUDA(cudaIpcOpenMemHandle(&d->peer_stage_base[r], a, cudaIpcMemLazyEnablePeerAccess));
    TLB_CUDA(cudaIpcOpenMemHandle(&d->peer_flags_base[r], b, cudaIpcMemLazyEnablePeerAccess));
    d->comm.stage[r] = (uint2*)d->peer_stage_base[r];
  }
  d->peers_open = true;
  return TLB_OK;
}

// Fault drill on ONE GPU: wire a tensor-parallel rank to peers that never answer.  Every other
// rank's staging pointer is aimed at a private, zeroed sink of the right size in this GPU's own
// memory, so the rank's pushes land somewhere harmless and nobody ever writes the packets it
// polls for: its next exchange runs into the bounded wait, the kernels return, and
// tlb_device_status reports TLB_ERR_DEVICE_WAIT.  Nothing faults or hangs.
int tlb_decoder_loopback_peers(void* h) {
  auto* d = (Decoder*)h;
  TLB_REQUIRE(d, "tlb_decoder_loopback_peers: null decoder");
  if (d->peers_open) return set_error(TLB_ERR_STATE, "tlb_decoder_loopback_peers: real peers are open already");
  const size_t sb = (size_t)2 * d->tp_size * d->comm.slot_floats * sizeof(uint2);
  for (int r = 0; r < d->tp_size; r++) {
    if (r == d->tp_rank) continue;
    if (!d->sink[r]) TLB_CUDA(cudaMalloc(&d->sink[r], sb));
    TLB_CUDA(cudaMemset(d->sink[r], 0, sb));
    d->comm.stage[r] = (uint2*)d->sink[r];
  }
  TLB_CUDA(cudaDeviceSynchronize());
  return TLB_OK;
}

}  // extern "C"
