// TEST INFRASTRUCTURE ONLY -- never linked into, loaded by, or shipped with the
// product library.  This file is a thin extern "C" wrapper that is compiled
// AGAINST THE UNMODIFIED REFERENCE HEADERS where they lie (the build recipe in
// this directory passes -I<reference>/include) and exposes the reference's own
// CPU implementation of the quantized-decode path as plain C functions, so the
// parity tests and the CPU-baseline leg of the benchmark can call "the real
// thing".  No reference source is copied here: every numeric result below is
// produced by tl::array code from the reference tree.
//
// Reference entry points exercised (paths inside the reference project):
//   include/array.h:703-742   array::to_q4      (int4 packing contract)
//   include/array.h:666-684   array::to_f32     (dequantised-f32 definition)
//   include/array.h:2414      array::dot  -> graph::dot -> cpu::sgemm
//   include/array.h:1654-1687 graph::ref_attn_  (via array::attn_decode)
//   include/array.h:1709-1734 graph::ref_rope_  (via array::rope)
//   include/array.h:2429-2439 array::rmsnorm / silu / swiglu compositions
//   bench/cuda/qwen_model.h:642-647 host argmax (first maximum wins)
// The decoder below is assembled from those ops following the block structure
// of bench/cuda/qwen_model.h:673-740 and bench/cuda/check/check_llm_decode.cpp
// :172-222 (weights dequantised once with to_q4().to_f32(), K/V kept on the
// host, GQA expanded by repeating KV heads because array::attn_decode is
// MHA-only).
//
// Built with -fno-access-control so the packed bytes of a q4 array can be read
// out of its private storage without touching the reference sources.

#include <tensorlib.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

using tl::array;

namespace {

array wrap(const float* p, tl::shape_t shape) {
  int64_t n = 1;
  for (auto d : shape) n *= d;
  return array::from(std::vector<float>(p, p + n), std::move(shape));
}

void copy_out(const array& a, float* out) {
  array c = a.contiguous() ? a : a.clone();
  const float* p = c.raw();
  std::memcpy(out, p, sizeof(float) * static_cast<size_t>(c.size()));
}

struct RefLayer {
  array wqkv, wo, wgu, wd;  // dequantised f32, logical [K,N]
  array bq, bk, bv;         // biases, f32
  array an, fn;             // norm weights
  std::vector<float> Kc, Vc;  // [n_kv, max_ctx, hd]
};

struct RefDecoder {
  int64_t hidden, n_layers, n_q, n_kv, hd, ff, vocab, max_ctx;
  float eps, rope_base, scale;
  std::vector<float> embed;  // [vocab, hidden]
  array onorm, lm_head;
  std::vector<RefLayer> layers;
};

}  // namespace

extern "C" {

int ref_threads() {
  unsigned hc = std::thread::hardware_concurrency();
  return hc > 1 ? static_cast<int>(hc) : 1;
}

// W is logical [K,N] row-major f32.  out receives q4_bytes(N,K) bytes:
// packed nibbles [N][K/2] followed by f32 scales [N][K/32].
int ref_to_q4(const float* w_kn, int64_t K, int64_t N, uint8_t* out) {
  tl::use_cpu();
  try {
    array wq = wrap(w_kn, {K, N}).to_q4();
    std::memcpy(out, wq.storage_.data(), static_cast<size_t>(tl::q4_bytes(N, K)));
  } catch (...) {
    return 1;
  }
  return 0;
}

// Round trip through the reference: to_q4 then to_f32, result logical [K,N].
int ref_q4_roundtrip_f32(const float* w_kn, int64_t K, int64_t N, float* out_kn) {
  tl::use_cpu();
  try {
    array deq = wrap(w_kn, {K, N}).to_q4().to_f32();
    copy_out(deq, out_kn);
  } catch (...) {
    return 1;
  }
  return 0;
}

// out[M,N] = (X[M,K] . Wq) * alpha + beta with Wq = to_q4(w_kn).
// predequant == 0: the shipped funnel X.dot(Wq) (re-dequantises inside dot).
// predequant == 1: X.dot(Wq.to_f32()) -- the "dequantised-f32 reference".
// reps > 1 repeats the timed expression (for the CPU-baseline timing loop).
int ref_dot_q4(const float* x, int64_t M, int64_t K, const float* w_kn, int64_t N,
               float alpha, float beta, int predequant, int reps, float* out,
               double* seconds_best) {
  tl::use_cpu();
  try {
    array X = wrap(x, {M, K});
    array Wq = wrap(w_kn, {K, N}).to_q4();
    array Wf = predequant ? Wq.to_f32() : array();
    double best = 1e30;
    array y;
    for (int r = 0; r < std::max(1, reps); r++) {
      auto t0 = std::chrono::steady_clock::now();
      y = (predequant ? X.dot(Wf) : X.dot(Wq)) * alpha + beta;
      y.eval();
      auto t1 = std::chrono::steady_clock::now();
      best = std::min(best, std::chrono::duration<double>(t1 - t0).count());
    }
    if (seconds_best) *seconds_best = best;
    copy_out(y, out);
  } catch (...) {
    return 1;
  }
  return 0;
}

int ref_attn_decode(const float* q, const float* K, const float* V, int64_t H,
                    int64_t ctx, int64_t D, float scale, int reps, float* out,
                    double* seconds_best) {
  tl::use_cpu();
  try {
    array aq = wrap(q, {H, D}), aK = wrap(K, {H, ctx, D}), aV = wrap(V, {H, ctx, D});
    double best = 1e30;
    array o;
    for (int r = 0; r < std::max(1, reps); r++) {
      auto t0 = std::chrono::steady_clock::now();
      o = array::attn_decode(aq, aK, aV, scale);
      o.eval();
      auto t1 = std::chrono::steady_clock::now();
      best = std::min(best, std::chrono::duration<double>(t1 - t0).count());
    }
    if (seconds_best) *seconds_best = best;
    copy_out(o, out);
  } catch (...) {
    return 1;
  }
  return 0;
}

// x is [H,D] when T == 1, else [H,T,D].
int ref_rope(const float* x, int64_t H, int64_t T, int64_t D, int64_t pos,
             float base, float* out) {
  tl::use_cpu();
  try {
    array ax = T == 1 ? wrap(x, {H, D}) : wrap(x, {H, T, D});
    array o = array::rope(ax, pos, base);
    o.eval();
    copy_out(o, out);
  } catch (...) {
    return 1;
  }
  return 0;
}

int ref_rmsnorm(const float* x, const float* w, int64_t rows, int64_t n, float eps,
                float* out) {
  tl::use_cpu();
  try {
    array o = array::rmsnorm(wrap(x, {rows, n}), wrap(w, {n}), eps);
    o.eval();
    copy_out(o, out);
  } catch (...) {
    return 1;
  }
  return 0;
}

int ref_swiglu(const float* gate, const float* up, int64_t rows, int64_t n,
               float* out) {
  tl::use_cpu();
  try {
    array o = array::swiglu(wrap(gate, {rows, n}), wrap(up, {rows, n}));
    o.eval();
    copy_out(o, out);
  } catch (...) {
    return 1;
  }
  return 0;
}

int64_t ref_argmax(const float* v, int64_t n) {
  tl::use_cpu();
  return wrap(v, {n}).argmax();
}

// ---- decoder assembled from reference ops --------------------------------

void* ref_decoder_create(int64_t hidden, int64_t n_layers, int64_t n_q,
                         int64_t n_kv, int64_t hd, int64_t ff, int64_t vocab,
                         int64_t max_ctx, float eps, float rope_base) {
  auto* d = new RefDecoder();
  d->hidden = hidden; d->n_layers = n_layers; d->n_q = n_q; d->n_kv = n_kv;
  d->hd = hd; d->ff = ff; d->vocab = vocab; d->max_ctx = max_ctx;
  d->eps = eps; d->rope_base = rope_base;
  d->scale = 1.0f / std::sqrt(static_cast<float>(hd));
  d->layers.resize(static_cast<size_t>(n_layers));
  for (auto& L : d->layers) {
    L.Kc.assign(static_cast<size_t>(n_kv * max_ctx * hd), 0.0f);
    L.Vc.assign(static_cast<size_t>(n_kv * max_ctx * hd), 0.0f);
  }
  return d;
}

void ref_decoder_destroy(void* h) { delete static_cast<RefDecoder*>(h); }

// which: 0 wqkv [hidden,(n_q+2n_kv)hd]  1 wo [n_q*hd,hidden]
//        2 wgu [hidden,2ff]             3 wd [ff,hidden]     4 lm_head [hidden,vocab]
// w_kn is the f32 master weight, logical [K,N]; it is quantised with the
// reference's to_q4 and kept dequantised (to_f32) as the reference CPU path
// multiplies it.  layer is ignored for lm_head.
int ref_decoder_set_linear(void* h, int64_t layer, int which, const float* w_kn,
                           int64_t K, int64_t N) {
  tl::use_cpu();
  auto* d = static_cast<RefDecoder*>(h);
  try {
    array wf = wrap(w_kn, {K, N}).to_q4().to_f32();
    if (which == 4) { d->lm_head = wf; return 0; }
    RefLayer& L = d->layers.at(static_cast<size_t>(layer));
    if (which == 0) L.wqkv = wf;
    else if (which == 1) L.wo = wf;
    else if (which == 2) L.wgu = wf;
    else if (which == 3) L.wd = wf;
    else return 2;
  } catch (...) {
    return 1;
  }
  return 0;
}

// which: 0 attn-norm  1 ffn-norm  2 bq  3 bk  4 bv  5 final norm (layer ignored)
int ref_decoder_set_vector(void* h, int64_t layer, int which, const float* v,
                           int64_t n) {
  auto* d = static_cast<RefDecoder*>(h);
  try {
    array a = wrap(v, {n});
    if (which == 5) { d->onorm = a; return 0; }
    RefLayer& L = d->layers.at(static_cast<size_t>(layer));
    if (which == 0) L.an = a;
    else if (which == 1) L.fn = a;
    else if (which == 2) L.bq = a;
    else if (which == 3) L.bk = a;
    else if (which == 4) L.bv = a;
    else return 2;
  } catch (...) {
    return 1;
  }
  return 0;
}

int ref_decoder_set_embed(void* h, const float* e) {
  auto* d = static_cast<RefDecoder*>(h);
  d->embed.assign(e, e + d->vocab * d->hidden);
  return 0;
}

// Overwrite rows [0,n) of one layer's K and V cache ([n_kv, n, hd] each).
int ref_decoder_fill_kv(void* h, int64_t layer, const float* K, const float* V,
                        int64_t n) {
  auto* d = static_cast<RefDecoder*>(h);
  RefLayer& L = d->layers.at(static_cast<size_t>(layer));
  for (int64_t kh = 0; kh < d->n_kv; kh++) {
    std::memcpy(&L.Kc[(kh * d->max_ctx) * d->hd], K + kh * n * d->hd,
                sizeof(float) * n * d->hd);
    std::memcpy(&L.Vc[(kh * d->max_ctx) * d->hd], V + kh * n * d->hd,
                sizeof(float) * n * d->hd);
  }
  return 0;
}

// One token through the decoder at position pos; logits[vocab] out; returns
// the greedy token (first maximum), or -1 on error.
int64_t ref_decoder_step(void* h, int64_t token, int64_t pos, float* logits) {
  tl::use_cpu();
  auto* d = static_cast<RefDecoder*>(h);
  try {
    const int64_t E = d->hidden, HD = d->hd, NQ = d->n_q, NKV = d->n_kv;
    const int64_t grp = NQ / NKV, ctx = pos + 1;
    array x = wrap(&d->embed[token * E], {1, E});
    for (auto& L : d->layers) {
      array hb = array::rmsnorm(x, L.an, d->eps);
      array qkv = hb.dot(L.wqkv).reshape({(NQ + 2 * NKV) * HD});
      array q = array::rope((qkv.slice(0, NQ * HD) + L.bq).reshape({NQ, HD}), pos,
                            d->rope_base);
      array k = array::rope((qkv.slice(NQ * HD, NKV * HD) + L.bk).reshape({NKV, HD}),
                            pos, d->rope_base);
      array v = qkv.slice((NQ + NKV) * HD, NKV * HD) + L.bv;
      k.eval();
      v.eval();
      const float* pk = k.raw();
      const float* pv = v.raw();
      for (int64_t kh = 0; kh < NKV; kh++) {
        std::memcpy(&L.Kc[(kh * d->max_ctx + pos) * HD], pk + kh * HD, sizeof(float) * HD);
        std::memcpy(&L.Vc[(kh * d->max_ctx + pos) * HD], pv + kh * HD, sizeof(float) * HD);
      }
      std::vector<float> Ke(static_cast<size_t>(NQ * ctx * HD)), Ve(Ke.size());
      for (int64_t qh = 0; qh < NQ; qh++) {
        int64_t kh = qh / grp;
        std::memcpy(&Ke[qh * ctx * HD], &L.Kc[kh * d->max_ctx * HD], sizeof(float) * ctx * HD);
        std::memcpy(&Ve[qh * ctx * HD], &L.Vc[kh * d->max_ctx * HD], sizeof(float) * ctx * HD);
      }
      array att = array::attn_decode(q, array::from(std::move(Ke), {NQ, ctx, HD}),
                                     array::from(std::move(Ve), {NQ, ctx, HD}),
                                     d->scale);
      array x1 = x + att.reshape({1, NQ * HD}).dot(L.wo);
      array h2 = array::rmsnorm(x1, L.fn, d->eps);
      array gu = h2.dot(L.wgu).reshape({2 * d->ff});
      array m = array::swiglu(gu.slice(0, d->ff), gu.slice(d->ff, d->ff))
                    .reshape({1, d->ff})
                    .dot(L.wd);
      array x2 = x1 + m;
      x2.eval();
      x = x2;
    }
    array lg = array::rmsnorm(x, d->onorm, d->eps).dot(d->lm_head);
    lg.eval();
    const float* p = lg.raw();
    if (logits) std::memcpy(logits, p, sizeof(float) * d->vocab);
    int64_t bi = 0;
    for (int64_t i = 1; i < d->vocab; i++)
      if (p[i] > p[bi]) bi = i;
    return bi;
  } catch (...) {
    return -1;
  }
}

}  // extern "C"
