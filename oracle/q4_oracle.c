/* TEST INFRASTRUCTURE ONLY -- a CPU restatement ("port") of the reference
 * algorithms on the quantized-decode path.  It is the checker that the parity
 * tests, the smoke test and the CPU-baseline leg of the benchmark compare the
 * CUDA library against.  Nothing in the product library includes, links or
 * loads this file, and it contains no GPU code.
 *
 * Pinning: every function here is checked by the CPU test-suite against (a)
 * the reference itself, compiled from its own headers into the sibling
 * reference shim when the reference tree is present, and (b) the committed
 * golden vectors that were produced by that shim.
 *
 * Each function cites the reference file:line it restates (paths inside the
 * reference project).  Where the reference accumulates in float with a blocked
 * order (cpu::sgemm) this port accumulates the same float products in double:
 * it is a tighter oracle for the same mathematical value, and the tests allow
 * the tolerance the reference's own tests allow (1e-4 GEMV/GEMM, 1e-3
 * attention/logits).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define Q4_GROUP 32 /* include/types.h:28  kQ4Group */

/* include/types.h:29-31  q4_bytes */
int64_t orc_q4_bytes(int64_t N, int64_t K) { return N * K / 2 + N * (K / Q4_GROUP) * 4; }

/* include/array.h:703-742  array::to_q4.
 * w is logical [K,N] row-major.  For each output row n and each group of 32
 * along k: maxabs (floor 1e-8f), scale = maxabs/7, q = clamp(lround(w/scale),
 * -8, 7), stored nibble q+8; byte k/2, low nibble for even k.  Scales follow
 * the packed block at byte N*K/2. */
int orc_to_q4(const float* w, int64_t K, int64_t N, uint8_t* out) {
  if (K % Q4_GROUP) return 1;
  memset(out, 0, (size_t)orc_q4_bytes(N, K));
  float* sc = (float*)(out + N * K / 2);
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    uint8_t* qrow = out + n * (K / 2);
    float* srow = sc + n * (K / Q4_GROUP);
    for (int64_t g = 0; g < K / Q4_GROUP; g++) {
      float maxabs = 1e-8f;
      for (int64_t j = 0; j < Q4_GROUP; j++) {
        float a = fabsf(w[(g * Q4_GROUP + j) * N + n]);
        if (a > maxabs) maxabs = a;
      }
      float scale = maxabs / 7.0f;
      srow[g] = scale;
      for (int64_t j = 0; j < Q4_GROUP; j++) {
        int64_t k = g * Q4_GROUP + j;
        long q = lroundf(w[k * N + n] / scale);
        if (q < -8) q = -8;
        if (q > 7) q = 7;
        unsigned nib = (unsigned)(q + 8);
        if (k & 1) qrow[k / 2] = (uint8_t)((qrow[k / 2] & 0x0F) | (nib << 4));
        else qrow[k / 2] = (uint8_t)((qrow[k / 2] & 0xF0) | nib);
      }
    }
  }
  return 0;
}

/* include/array.h:666-684  array::to_f32 (q4 branch): out[k,n] = scale*(nib-8) */
void orc_q4_to_f32(const uint8_t* q4, int64_t K, int64_t N, float* out_kn) {
  const float* sc = (const float*)(q4 + N * K / 2);
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    const uint8_t* qrow = q4 + n * (K / 2);
    const float* srow = sc + n * (K / Q4_GROUP);
    for (int64_t k = 0; k < K; k++) {
      uint8_t b = qrow[k / 2];
      int nib = (k & 1) ? (b >> 4) : (b & 0xF);
      out_kn[k * N + n] = srow[k / Q4_GROUP] * (float)(nib - 8);
    }
  }
}

/* out[M,N] = (X[M,K] . dequant(Wq)) * alpha + beta.
 * The "dequantised-f32 reference" of include/array.h:1980-1984 (widen) followed
 * by the dot and the fused affine epilogue (array.h:1305-1311, 1511-1518);
 * kernels/tensorlib_cuda.cu:786-794 multiplies the same float values
 * a[k]*(sc*(float)q) at M==1. */
void orc_gemm_q4(const float* x, int64_t M, int64_t K, const uint8_t* q4, int64_t N,
                 float alpha, float beta, float* out) {
  const float* sc = (const float*)(q4 + N * K / 2);
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    const uint8_t* qrow = q4 + n * (K / 2);
    const float* srow = sc + n * (K / Q4_GROUP);
    for (int64_t m = 0; m < M; m++) {
      const float* xr = x + m * K;
      double acc = 0.0;
      for (int64_t k = 0; k < K; k++) {
        uint8_t b = qrow[k / 2];
        int nib = (k & 1) ? (b >> 4) : (b & 0xF);
        float wv = srow[k / Q4_GROUP] * (float)(nib - 8);
        acc += (double)xr[k] * (double)wv;
      }
      out[m * N + n] = (float)acc * alpha + beta;
    }
  }
}

/* include/array.h:1654-1687  graph::ref_attn_, extended with the GQA / cache
 * addressing of include/cuda.h:966-984: q head h reads kv head h/(Hq/Hkv); K,V
 * are [Hkv, kv_max, D] read over the prefix [0,ctx). */
void orc_attn_decode(const float* q, const float* K, const float* V, int64_t Hq,
                     int64_t Hkv, int64_t ctx, int64_t kv_max, int64_t D, float scale,
                     float* out) {
  int64_t grp = Hq / Hkv;
#pragma omp parallel for schedule(static)
  for (int64_t h = 0; h < Hq; h++) {
    const float* qh = q + h * D;
    const float* Kh = K + (h / grp) * kv_max * D;
    const float* Vh = V + (h / grp) * kv_max * D;
    float* s = (float*)malloc(sizeof(float) * (size_t)(ctx > 0 ? ctx : 1));
    float mx = -INFINITY;
    for (int64_t j = 0; j < ctx; j++) {
      float acc = 0;
      for (int64_t d = 0; d < D; d++) acc += qh[d] * Kh[j * D + d];
      s[j] = acc * scale;
      if (s[j] > mx) mx = s[j];
    }
    float sum = 0;
    for (int64_t j = 0; j < ctx; j++) {
      s[j] = expf(s[j] - mx);
      sum += s[j];
    }
    for (int64_t d = 0; d < D; d++) {
      float acc = 0;
      for (int64_t j = 0; j < ctx; j++) acc += s[j] * Vh[j * D + d];
      out[h * D + d] = acc / sum;
    }
    free(s);
  }
}

/* include/array.h:1709-1734  graph::ref_rope_ (double trig, half-split pairs
 * (j, j+D/2), row r at position pos + r%T), with the optional bias added before
 * the rotation as kernels/tensorlib_cuda.cu:1374-1377 does. bias may be NULL;
 * it has the same [rows,D] layout as x. */
void orc_rope(const float* x, const float* bias, int64_t rows, int64_t T, int64_t D,
              int64_t pos, float base, float* out) {
  int64_t half = D / 2;
  for (int64_t r = 0; r < rows; r++) {
    int64_t t = T ? r % T : 0;
    double position = (double)(pos + t);
    for (int64_t j = 0; j < half; j++) {
      double theta = pow((double)base, -2.0 * (double)j / (double)D);
      double ang = position * theta;
      float c = (float)cos(ang), s = (float)sin(ang);
      float x0 = x[r * D + j], x1 = x[r * D + j + half];
      if (bias) {
        x0 += bias[r * D + j];
        x1 += bias[r * D + j + half];
      }
      out[r * D + j] = x0 * c - x1 * s;
      out[r * D + j + half] = x0 * s + x1 * c;
    }
  }
}

/* include/array.h:2429-2433 array::rmsnorm == kernels/tensorlib_cuda.cu:131-149:
 * x * (1/sqrtf(mean(x^2)+eps)) * w per row. */
void orc_rmsnorm(const float* x, const float* w, int64_t rows, int64_t n, float eps,
                 float* out) {
  for (int64_t r = 0; r < rows; r++) {
    double ms = 0;
    for (int64_t i = 0; i < n; i++) ms += (double)x[r * n + i] * x[r * n + i];
    float inv = 1.0f / sqrtf((float)(ms / (double)n) + eps);
    for (int64_t i = 0; i < n; i++) out[r * n + i] = x[r * n + i] * inv * w[i];
  }
}

/* kernels/tensorlib_cuda.cu:155-179 tl_add_rmsnorm: xout = a+b; hout = rmsnorm(xout)*w.
 * xout may alias a. */
void orc_add_rmsnorm(const float* a, const float* b, const float* w, int64_t rows,
                     int64_t n, float eps, float* xout, float* hout) {
  for (int64_t r = 0; r < rows; r++) {
    double ms = 0;
    for (int64_t i = 0; i < n; i++) {
      float v = a[r * n + i] + b[r * n + i];
      xout[r * n + i] = v;
      ms += (double)v * v;
    }
    float inv = 1.0f / sqrtf((float)(ms / (double)n) + eps);
    for (int64_t i = 0; i < n; i++) hout[r * n + i] = xout[r * n + i] * inv * w[i];
  }
}

/* kernels/tensorlib_cuda.cu:185-192 tl_swiglu on the fused [rows, 2*ff] buffer
 * (gate then up); include/array.h:2435-2439 gives the same g/(1+exp(-g))*u. */
void orc_swiglu(const float* gu, int64_t rows, int64_t ff, float* out) {
  for (int64_t r = 0; r < rows; r++)
    for (int64_t f = 0; f < ff; f++) {
      float g = gu[r * 2 * ff + f];
      out[r * ff + f] = (g / (1.0f + expf(-g))) * gu[r * 2 * ff + ff + f];
    }
}

/* bench/cuda/qwen_model.h:642-647 host argmax == kernels/tensorlib_cuda.cu:90-119:
 * the smallest index among the maxima. */
int64_t orc_argmax(const float* v, int64_t n) {
  int64_t bi = 0;
  for (int64_t i = 1; i < n; i++)
    if (v[i] > v[bi]) bi = i;
  return bi;
}

/* ---- decoder: bench/cuda/qwen_model.h:673-740 run_layers_ restated on the host,
 * every linear held in the q4 layout (BASELINE quantises all of them). ---- */
typedef struct {
  const uint8_t *wqkv, *wo, *wgu, *wd;
  const float *bq, *bk, *bv, *an, *fn;
  float *Kc, *Vc; /* [n_kv, max_ctx, hd] */
} orc_layer;

typedef struct {
  int64_t hidden, n_layers, n_q, n_kv, hd, ff, vocab, max_ctx;
  float eps, rope_base, scale;
  const float* embed;
  const float* onorm;
  const uint8_t* lm_head;
  orc_layer* layers;
  float *x, *hb, *qkv, *att, *t0, *gu, *mb;
  int kv_bf16; /* cache rows are rounded to bf16 when stored (kv_st, kernels/tensorlib_cuda.cu:828-831) */
} orc_decoder;

/* f32 -> bf16 -> f32, round to nearest even: what __float2bfloat16 does in kv_st
 * (kernels/tensorlib_cuda.cu:831) followed by the exact widening of kv_ld (:828-830). */
static float orc_bf16_round(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return x; /* NaN stays NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  memcpy(&x, &u, 4);
  return x;
}
void orc_bf16_round_array(const float* in, int64_t n, float* out) {
  for (int64_t i = 0; i < n; i++) out[i] = orc_bf16_round(in[i]);
}
static void orc_store_row(const orc_decoder* d, float* dst, const float* src, int64_t n) {
  if (d->kv_bf16)
    for (int64_t i = 0; i < n; i++) dst[i] = orc_bf16_round(src[i]);
  else
    memcpy(dst, src, sizeof(float) * (size_t)n);
}
/* kv_cache::init with dtype::bf16 (include/cuda.h:1336-1346): the host model keeps f32 storage
 * holding bf16-representable values, which is what the bf16 cache widens to. */
void orc_decoder_set_kv_bf16(void* h, int on) { ((orc_decoder*)h)->kv_bf16 = on ? 1 : 0; }

void* orc_decoder_create(int64_t hidden, int64_t n_layers, int64_t n_q, int64_t n_kv,
                         int64_t hd, int64_t ff, int64_t vocab, int64_t max_ctx,
                         float eps, float rope_base) {
  orc_decoder* d = (orc_decoder*)calloc(1, sizeof(orc_decoder));
  d->hidden = hidden; d->n_layers = n_layers; d->n_q = n_q; d->n_kv = n_kv;
  d->hd = hd; d->ff = ff; d->vocab = vocab; d->max_ctx = max_ctx;
  d->eps = eps; d->rope_base = rope_base; d->scale = 1.0f / sqrtf((float)hd);
  d->layers = (orc_layer*)calloc((size_t)n_layers, sizeof(orc_layer));
  for (int64_t l = 0; l < n_layers; l++) {
    d->layers[l].Kc = (float*)calloc((size_t)(n_kv * max_ctx * hd), sizeof(float));
    d->layers[l].Vc = (float*)calloc((size_t)(n_kv * max_ctx * hd), sizeof(float));
  }
  d->x = (float*)malloc(sizeof(float) * hidden);
  d->hb = (float*)malloc(sizeof(float) * hidden);
  d->qkv = (float*)malloc(sizeof(float) * (n_q + 2 * n_kv) * hd);
  d->att = (float*)malloc(sizeof(float) * n_q * hd);
  d->t0 = (float*)malloc(sizeof(float) * hidden);
  d->gu = (float*)malloc(sizeof(float) * 2 * ff);
  d->mb = (float*)malloc(sizeof(float) * ff);
  return d;
}

void orc_decoder_destroy(void* h) {
  orc_decoder* d = (orc_decoder*)h;
  for (int64_t l = 0; l < d->n_layers; l++) { free(d->layers[l].Kc); free(d->layers[l].Vc); }
  free(d->layers); free(d->x); free(d->hb); free(d->qkv); free(d->att);
  free(d->t0); free(d->gu); free(d->mb); free(d);
}

/* Pointers are borrowed: the caller keeps the buffers alive.  Linear weights
 * are q4 byte buffers (orc_to_q4 layout).  which as in the reference shim:
 * linear 0 wqkv 1 wo 2 wgu 3 wd 4 lm_head; vector 0 an 1 fn 2 bq 3 bk 4 bv 5 onorm. */
void orc_decoder_set_linear(void* h, int64_t layer, int which, const uint8_t* q4) {
  orc_decoder* d = (orc_decoder*)h;
  if (which == 4) { d->lm_head = q4; return; }
  orc_layer* L = &d->layers[layer];
  if (which == 0) L->wqkv = q4; else if (which == 1) L->wo = q4;
  else if (which == 2) L->wgu = q4; else if (which == 3) L->wd = q4;
}
void orc_decoder_set_vector(void* h, int64_t layer, int which, const float* v) {
  orc_decoder* d = (orc_decoder*)h;
  if (which == 5) { d->onorm = v; return; }
  orc_layer* L = &d->layers[layer];
  if (which == 0) L->an = v; else if (which == 1) L->fn = v; else if (which == 2) L->bq = v;
  else if (which == 3) L->bk = v; else if (which == 4) L->bv = v;
}
void orc_decoder_set_embed(void* h, const float* e) { ((orc_decoder*)h)->embed = e; }

void orc_decoder_fill_kv(void* h, int64_t layer, const float* K, const float* V, int64_t n) {
  orc_decoder* d = (orc_decoder*)h;
  orc_layer* L = &d->layers[layer];
  for (int64_t kh = 0; kh < d->n_kv; kh++) {
    orc_store_row(d, L->Kc + kh * d->max_ctx * d->hd, K + kh * n * d->hd, n * d->hd);
    orc_store_row(d, L->Vc + kh * d->max_ctx * d->hd, V + kh * n * d->hd, n * d->hd);
  }
}

int64_t orc_decoder_step(void* h, int64_t token, int64_t pos, float* logits) {
  orc_decoder* d = (orc_decoder*)h;
  const int64_t E = d->hidden, HD = d->hd, NQ = d->n_q, NKV = d->n_kv, FF = d->ff;
  memcpy(d->x, d->embed + token * E, sizeof(float) * E);
  for (int64_t l = 0; l < d->n_layers; l++) {
    orc_layer* L = &d->layers[l];
    orc_rmsnorm(d->x, L->an, 1, E, d->eps, d->hb);
    orc_gemm_q4(d->hb, 1, E, L->wqkv, (NQ + 2 * NKV) * HD, 1.0f, 0.0f, d->qkv);
    float* q = d->qkv;
    float* k = d->qkv + NQ * HD;
    float* v = d->qkv + (NQ + NKV) * HD;
    orc_rope(q, L->bq, NQ, 1, HD, pos, d->rope_base, q);
    orc_rope(k, L->bk, NKV, 1, HD, pos, d->rope_base, k);
    for (int64_t i = 0; i < NKV * HD; i++) v[i] += L->bv[i];
    for (int64_t kh = 0; kh < NKV; kh++) {
      orc_store_row(d, L->Kc + (kh * d->max_ctx + pos) * HD, k + kh * HD, HD);
      orc_store_row(d, L->Vc + (kh * d->max_ctx + pos) * HD, v + kh * HD, HD);
    }
    orc_attn_decode(q, L->Kc, L->Vc, NQ, NKV, pos + 1, d->max_ctx, HD, d->scale, d->att);
    orc_gemm_q4(d->att, 1, NQ * HD, L->wo, E, 1.0f, 0.0f, d->t0);
    orc_add_rmsnorm(d->x, d->t0, L->fn, 1, E, d->eps, d->x, d->hb);
    orc_gemm_q4(d->hb, 1, E, L->wgu, 2 * FF, 1.0f, 0.0f, d->gu);
    orc_swiglu(d->gu, 1, FF, d->mb);
    orc_gemm_q4(d->mb, 1, FF, L->wd, E, 1.0f, 0.0f, d->t0);
    for (int64_t i = 0; i < E; i++) d->x[i] += d->t0[i];
  }
  orc_rmsnorm(d->x, d->onorm, 1, E, d->eps, d->hb);
  float* lg = logits ? logits : (float*)malloc(sizeof(float) * d->vocab);
  orc_gemm_q4(d->hb, 1, E, d->lm_head, d->vocab, 1.0f, 0.0f, lg);
  int64_t tok = orc_argmax(lg, d->vocab);
  if (!logits) free(lg);
  return tok;
}
