/* tlb200 -- C-ABI of the B200 (sm_100a) implementation of cpp-tensorlib's
 * quantized-decode hot path.
 *
 * Every entry point is plain C: raw device pointers, sizes, a CUDA stream passed
 * as void* (NULL = the legacy default stream).  No C++ or torch types cross this
 * boundary.  Functions return 0 on success or a non-zero tlb status code;
 * tlb_last_error() gives the message.  Each declaration names the reference
 * interface it replaces (paths inside the reference project; "cu.h" =
 * include/cuda.h, ".cu" = kernels/tensorlib_cuda.cu, "arr" = include/array.h,
 * "qm" = bench/cuda/qwen_model.h).
 *
 * The library links the CUDA runtime statically; consumers dlopen this one
 * shared object and link nothing else.  There is no CPU fallback: when no
 * usable device exists every call fails with a status code.
 */
#ifndef TLB200_H_
#define TLB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define TLB_OK 0
#define TLB_ERR_CUDA 1
#define TLB_ERR_ARG 2
#define TLB_ERR_UNSUPPORTED 3
#define TLB_ERR_DEVICE_WAIT 4
#define TLB_ERR_STATE 5

/* ---- context / memory ------------------------------------------------------ */
/* cu.h:235-321 context::get -- bind the calling thread to `device` and create the
 * per-device state (scratch, status block).  Called implicitly by every op for
 * the current device. */
int tlb_init(int device);
int tlb_device_count(void);                 /* cu.h:493 available() (count > 0) */
const char* tlb_last_error(void);           /* message of the last failing call on this thread */
int tlb_version(void);
/* Bounded device-side waits record a timeout here instead of hanging:
 * out[0] = 1 when any wait expired since the last clear, out[1] = where. */
int tlb_device_status(int* out2, int clear);
/* The limit of those waits in GPU clock ticks (clock64) for the current device;
 * default 2e9, about one second.  No counterpart in the reference, whose kernels never
 * wait on one another.  Synchronises the device. */
int tlb_set_wait_limit_cycles(int64_t cycles);
int tlb_set_pdl(int enabled);               /* programmatic dependent launch on/off (default on) */

int tlb_alloc(int64_t bytes, void** dptr);  /* cu.h:586-603 alloc */
int tlb_free(void* dptr);                   /* cu.h:605-624 release */
int tlb_h2d(void* dst, const void* src, int64_t bytes, void* stream); /* cu.h:559-580 upload */
int tlb_d2h(void* dst, const void* src, int64_t bytes, void* stream); /* cu.h:626-637 sync_to_host */
int tlb_memset(void* dst, int value, int64_t bytes, void* stream);
int tlb_sync(void* stream);                 /* cu.h:501-506 flush */

/* ---- int4 storage ---------------------------------------------------------- */
int64_t tlb_q4_bytes(int64_t N, int64_t K); /* include/types.h:29-31 q4_bytes */
/* arr:703-742 array::to_q4 on the device: w is f32 logical [K,N] row-major; q4
 * receives packed nibbles [N][K/2] then f32 scales [N][K/32].  K % 32 == 0. */
int tlb_to_q4(const float* w_kn, int64_t K, int64_t N, void* q4, void* stream);
/* arr:666-684 array::to_f32 (q4 branch): out is f32 logical [K,N]. */
int tlb_q4_to_f32(const void* q4, int64_t K, int64_t N, float* out_kn, void* stream);

/* ---- int4 dequant-matmul --------------------------------------------------- */
/* cu.h:770-785 cuda::gemv_bf16_row: y[n] = sum_k a[k] * W[n][k], W bf16 row-major [N][K] (the
 * decode projection of the reference's bf16-weight models); K % 8 == 0. */
int tlb_gemv_bf16_row(const float* a, const void* W, float* y, int64_t N, int64_t K, void* stream);

/* ---- tile-packed int4 weights: the library's own HBM layout for the decode GEMV.
 * No counterpart in the reference.  A matrix in the reference layout (types.h:15-31) is
 * repacked once, on the device, into 2560-byte units (16 rows x 256 k: nibble words in
 * MMA-fragment order, then the unit's f32 scales), N padded to 16 and K to 256 with
 * zero weights.  tlb_gemv_q4p then computes what cuda::gemv_q4 (cu.h:886-905) computes,
 * y[n] = alpha * sum_k x[k] * dequant(W)[k,n] + beta, from one contiguous byte stream
 * per warp. ---- */
int64_t tlb_q4p_bytes(int64_t N, int64_t K);                 /* size of the packed copy; -1 on bad shape */
int tlb_q4_pack(const void* q4, int64_t N, int64_t K, void* packed, void* stream);
int tlb_gemv_q4p(const float* x, const void* packed, float* y, int64_t N, int64_t K, float alpha,
                 float beta, void* stream);

/* cu.h:886-905 cuda::gemv_q4 / .cu:772-796 tl_gemv_q4:  y[N] = a[K] . dequant(W).
 * group must be 32. */
int tlb_gemv_q4(const float* a, const void* qw, const float* scales, float* y, int64_t N,
                int64_t K, int64_t group, void* stream);
/* The M >= 1 contraction with the fused affine epilogue the lazy graph composes
 * into a dot node (arr:1305-1311, arr:2109-2141; the reference routes M > 1
 * through host dequant + tl_sgemm_rb, arr:1980-1984, .cu:310-421):
 *   y[M,N] = (x[M,K] . dequant(W)) * alpha + beta,  x row stride ldx, y row stride ldy. */
int tlb_gemm_q4(const float* x, int64_t M, int64_t ldx, const void* qw, const float* scales,
                float* y, int64_t ldy, int64_t N, int64_t K, float alpha, float beta,
                void* stream);
/* Same contraction forced through the general-shape CUDA-core kernel (any
 * K % 32 == 0, no alignment rules); used as an independent cross-check. */
int tlb_gemm_q4_simt(const float* x, int64_t M, int64_t ldx, const void* qw, const float* scales,
                     float* y, int64_t ldy, int64_t N, int64_t K, float alpha, float beta,
                     void* stream);

/* ---- decode attention ------------------------------------------------------ */
/* cu.h:966-1009 cuda::attn_decode (f32 cache).  q,out [n_q,D]; K,V [n_kv,kv_max,D]
 * read over [0,ctx).  Split partials live in library-owned scratch. */
int tlb_attn_decode(const float* q, const float* K, const float* V, float* out, int64_t n_q,
                    int64_t n_kv, int64_t ctx, int64_t kv_max, int64_t D, float scale,
                    void* stream);
/* cu.h:1084-1114 cuda::attn_decode_dpos: ctx = *d_pos + 1, capacity-sized grid,
 * caller-owned partials of tlb_attn_partials_bytes() (first 256 bytes must be
 * zero before the first call: they hold the merge counters). */
int tlb_attn_decode_dpos(const float* q, const float* K, const float* V, float* out, int64_t n_q,
                         int64_t n_kv, const void* d_pos, int64_t kv_max, int64_t D, float scale,
                         void* partials, void* stream);
/* bf16 KV cache (cu.h:1326-1346 kv_cache::init with dtype::bf16; kernels .cu:828-831 kv_ld /
 * kv_st): K, V are bf16 [n_kv, kv_max, D], widened to f32 for the dot and the accumulate;
 * q, out and the split partials stay f32.  Same arguments otherwise. */
int tlb_attn_decode_bf16(const float* q, const void* K, const void* V, float* out, int64_t n_q,
                         int64_t n_kv, int64_t ctx, int64_t kv_max, int64_t D, float scale,
                         void* stream);
int tlb_attn_decode_dpos_bf16(const float* q, const void* K, const void* V, float* out, int64_t n_q,
                              int64_t n_kv, const void* d_pos, int64_t kv_max, int64_t D, float scale,
                              void* partials, void* stream);
/* No counterpart in the reference.  Same result as tlb_attn_decode, for callers
 * that must not allocate device memory when they call (an embedder that owns the
 * whole device heap, a region where cudaMalloc's implicit device synchronisation
 * is not allowed, a fixed memory budget): the split partials live in a 4 MiB array
 * inside the library image, which every GPU that loads the library holds until
 * exit.  Limits: n_kv <= 64 and n_q * splits * (D + 4) * 4 bytes <= 4 MiB - 256
 * (TLB_ERR_UNSUPPORTED beyond that).  The first call on a device looks the array's
 * device address up; make that call before any stream capture.  All calls share
 * the one array: calls that overlap on the GPU (different streams) race. */
int tlb_attn_decode_noalloc(const float* q, const float* K, const float* V, float* out,
                            int64_t n_q, int64_t n_kv, int64_t ctx, int64_t kv_max, int64_t D,
                            float scale, void* stream);
int64_t tlb_attn_partials_bytes(int64_t n_q, int64_t n_kv, int64_t kv_max, int64_t D); /* cu.h:948-960 */

/* ---- fused row ops --------------------------------------------------------- */
int tlb_rmsnorm(const float* x, const float* w, float* out, int64_t n, float eps, int64_t rows,
                void* stream);                                   /* cu.h:1287-1302 */
int tlb_rmsnorm_res(const float* x, const float* delta, const float* w, float* xout, float* hout,
                    int64_t n, float eps, int64_t rows, void* stream); /* cu.h:1233-1252 */
int tlb_swiglu(const float* gu, float* out, int64_t ff, int64_t rows, void* stream); /* cu.h:1306-1319 */
/* arr:2435-2439 array::swiglu(gate, up) = silu(gate) * up on two separate [rows, ff] operands with
 * row strides ldg / ldu (the lazy graph's composition; tlb_swiglu is the fused-buffer form). */
int tlb_swiglu_split(const float* gate, int64_t ldg, const float* up, int64_t ldu, float* out,
                     int64_t ff, int64_t rows, void* stream);
int tlb_rope(const float* x, float* out, int64_t rows, int64_t T, int64_t D, int64_t pos,
             float base, const float* bias, void* stream);       /* cu.h:1205-1222 */
int tlb_rope_dpos(const float* x, float* out, int64_t rows, int64_t T, int64_t D,
                  const void* d_pos, float base, const float* bias, void* stream); /* cu.h:1018-1035 */
int tlb_kv_append(float* Kc, float* Vc, const float* k_new, const float* v_new, int64_t pos,
                  int64_t kv_max, int64_t n_kv, int64_t D, void* stream); /* cu.h:1118-1138 */
int tlb_kv_append_dpos(float* Kc, float* Vc, const float* k_new, const float* v_new,
                       const void* d_pos, int64_t kv_max, int64_t n_kv, int64_t D,
                       void* stream);                             /* cu.h:1050-1070 */
/* the same two with a bf16 cache (kv_st, kernels/tensorlib_cuda.cu:831: round to nearest even) */
int tlb_kv_append_bf16(void* Kc, void* Vc, const float* k_new, const float* v_new, int64_t pos,
                       int64_t kv_max, int64_t n_kv, int64_t D, void* stream);
int tlb_kv_append_dpos_bf16(void* Kc, void* Vc, const float* k_new, const float* v_new,
                            const void* d_pos, int64_t kv_max, int64_t n_kv, int64_t D, void* stream);
int tlb_incr_u32(void* d_pos, void* stream);                      /* cu.h:1038-1047 */
/* cu.h:1261-1282 cuda::argmax: reduces on the device, synchronises the stream and
 * returns the index (smallest index among the maxima). */
int tlb_argmax(const float* in, int64_t n, int64_t* out_idx, void* stream);
/* Asynchronous form: the int32 index is written to d_out (device), no sync. */
int tlb_argmax_dev(const float* in, int64_t n, void* d_out, void* stream);

/* ---- the rest of the evaluator's GPU surface (elementwise, broadcast, row ops, f32 GEMM,
 * [K,N]-layout GEMVs, bf16 prefill GEMM).  Every kernel computes out = expr * scale + offset
 * like the reference's (.cu:25-82). ---- */
#define TLB_OP_ADD 0
#define TLB_OP_SUB 1
#define TLB_OP_MUL 2
#define TLB_OP_DIV 3
#define TLB_OP_POW 4   /* the reference declines pow on CUDA (cu.h:642); here it runs on the device */
#define TLB_UOP_EXP 0
#define TLB_UOP_LOG 1
#define TLB_UOP_SQRT 2
#define TLB_UOP_SIGMOID 3
#define TLB_UOP_RELU 4
#define TLB_UOP_AFFINE 5
#define TLB_ROW_SOFTMAX 0
#define TLB_ROW_SUM 1
#define TLB_ROW_MAX 2
/* cu.h:640-655 cuda::binary / .cu:25-36: out[i] = (a[i] OP b[i]) * scale + offset */
int tlb_binary(int op, const float* a, const float* b, float* out, int64_t n, float scale, float offset,
               void* stream);
/* cu.h:658-662 cuda::binary_bcast (declined by the reference's CUDA backend; arr:1487-1506 gives
 * the contract): out[r,c] = (a[r*a_rs + c*a_cs] OP b[r*b_rs + c*b_cs]) * scale + offset,
 * strides in elements, 0 for a broadcast axis */
int tlb_binary_bcast(int op, const float* a, int64_t a_rs, int64_t a_cs, const float* b, int64_t b_rs,
                     int64_t b_cs, float* out, int64_t rows, int64_t cols, float scale, float offset,
                     void* stream);
/* cu.h:664-675 cuda::unary / .cu:38-51 */
int tlb_unary(int op, const float* a, float* out, int64_t n, float scale, float offset, void* stream);
/* cu.h:1487-1503 cuda::row_op / .cu:53-82, 222-258: softmax writes rows x cols (scale / offset
 * ignored), row_sum / row_max one value per row */
int tlb_row_op(int op, const float* in, float* out, int64_t rows, int64_t cols, float scale, float offset,
               void* stream);
/* cu.h:1409-1483 cuda::gemm / .cu:262-421: C[m,n] = (A . B) * scale + offset, C contiguous,
 * A(i,k) = ta ? A[k*lda+i] : A[i*lda+k], B(k,j) = tb ? B[j*ldb+k] : B[k*ldb+j] */
int tlb_gemm_f32(const float* a, int64_t lda, int ta, const float* b, int64_t ldb, int tb, float* out,
                 int64_t m, int64_t n, int64_t k, float scale, float offset, void* stream);
/* cu.h:790-841 cuda::gemm_bf16_nt / .cu:474-595: C[M,N] = A[M,K] . W^T, W bf16 row-major [N,K] */
int tlb_gemm_bf16_nt(const float* a, const void* w, float* c, int64_t M, int64_t N, int64_t K, void* stream);
/* cu.h:719-742 cuda::gemv_f32 / gemv_bf16, .cu:611-682: y[n] = sum_k a[k] * B[k*n_cols + n],
 * B row-major [K,N] f32 or bf16 */
int tlb_gemv_f32(const float* a, const float* B, float* y, int64_t n, int64_t k, void* stream);
int tlb_gemv_bf16(const float* a, const void* B, float* y, int64_t n, int64_t k, void* stream);

/* ---- batched prefill (the "next" row: prompt chunks instead of token-by-token) ---- */
/* cu.h:848-864 split_heads: [T, ld] token-major (column block at `off`) -> [H, T, D], + bias[H*D] */
int tlb_split_heads(const float* src, const float* bias, float* dst, int64_t T, int64_t ld,
                    int64_t off, int64_t H, int64_t D, void* stream);
/* cu.h:867-879 merge_heads: [H, T, D] -> [T, H*D] */
int tlb_merge_heads(const float* src, float* dst, int64_t T, int64_t H, int64_t D, void* stream);
/* cu.h:1143-1164 kv_fill: k, v [n_kv, T, D] into cache rows [pos0, pos0 + T) (f32 cache) */
int tlb_kv_fill(float* Kc, float* Vc, const float* K, const float* V, int64_t T, int64_t kv_max,
                int64_t n_kv, int64_t D, int64_t pos0, void* stream);
int tlb_kv_fill_bf16(void* Kc, void* Vc, const float* K, const float* V, int64_t T, int64_t kv_max,
                     int64_t n_kv, int64_t D, int64_t pos0, void* stream);   /* bf16 cache */
/* cu.h:1171-1201 attn_prefill: causal attention of a prompt chunk; q, out [n_q, T, D];
 * query p is at position pos0 + p and attends keys 0..pos0+p of the cache. */
int tlb_attn_prefill(const float* q, const float* K, const float* V, float* out, int64_t n_q,
                     int64_t n_kv, int64_t T, int64_t kv_max, int64_t D, float scale, int64_t pos0,
                     void* stream);
int tlb_attn_prefill_bf16(const float* q, const void* K, const void* V, float* out, int64_t n_q,
                          int64_t n_kv, int64_t T, int64_t kv_max, int64_t D, float scale, int64_t pos0,
                          void* stream);                          /* bf16 cache */

/* ---- CUDA-graph capture (cu.h:512-551) ------------------------------------- */
int tlb_capture_begin(void** stream_out);   /* capture_begin: returns the stream to launch on */
int tlb_capture_end(void** graph_exec_out); /* capture_end */
int tlb_graph_launch(void* graph_exec, void* stream); /* graph_launch */
int tlb_graph_destroy(void* graph_exec);    /* graph_destroy */

/* ---- Qwen2.5-architecture int4 decoder (native driver) ----------------------
 * Replaces the model driver of qm:175-308 (Layer/Scratch/Model), qm:673-740
 * (run_layers_) and qm:791-905 (captured_decoder) with every linear in the q4
 * layout, plus the tensor-parallel path the reference does not have.
 * cfg[0..10] = hidden, n_layers, n_q, n_kv, head_dim, ff, vocab, max_ctx (sizes
 * local to the rank, hidden global), tp_rank, tp_size, vocab_offset; optional cfg[11] =
 * rows of the embedding table (token ids are checked against it); optional cfg[12] = 1: the KV
 * caches hold bf16 (cu.h:1336-1346 kv_cache::init with dtype::bf16; tlb_decoder_kv then returns
 * bf16 buffers).
 * Capacity: set_pos / forward / run / step / prefill keep a host mirror of the position and
 * refuse (TLB_ERR_ARG, nothing launched) to advance past max_ctx, as captured_decoder::feed
 * does (qm:877-885).  A graph replayed behind the library's back is caught on the device:
 * the append epilogue and the attention skip the row and tlb_device_status reports it. */
int tlb_decoder_create(const int64_t* cfg, int n_cfg, float eps, float rope_base, void** out);
int tlb_decoder_destroy(void* dec);
/* which: 0 wqkv 1 wo 2 wgu 3 wd 4 lm_head; q4 = device pointer, borrowed (qm:85-153). */
int tlb_decoder_set_linear(void* dec, int64_t layer, int which, const void* q4, int64_t K, int64_t N);
/* which: 0 attn norm 1 ffn norm 2 bq 3 bk 4 bv 5 final norm 6 embedding table (device f32). */
int tlb_decoder_set_vector(void* dec, int64_t layer, int which, const float* v);
int tlb_decoder_kv(void* dec, int64_t layer, void** K, void** V);     /* cu.h:1326-1346 kv_cache K,V */
int tlb_decoder_logits(void* dec, void** logits);                      /* qm Scratch.logitsb */
int tlb_decoder_set_pos(void* dec, int64_t pos, void* stream);         /* qm:877-885 feed / cu.h:559 upload_u32 */
int tlb_decoder_set_token(void* dec, int64_t token, void* stream);
int tlb_decoder_forward(void* dec, void* stream);                      /* qm:673-740 run_layers_ + argmax */
int64_t tlb_decoder_launches_per_token(void* dec);
int tlb_decoder_capture(void* dec);                                    /* qm:791-860 captured_decoder::init_ */
int tlb_decoder_run(void* dec, int64_t n_tokens, void* stream);        /* qm:862-905 step, device-resident ids */
/* qm:747-752 step_imperative with HOST buffers: token id in, next id out. */
int tlb_decoder_step(void* dec, const int32_t* token_in, int32_t* token_out, void* stream);
int tlb_decoder_last_token(void* dec, int32_t* token_out, void* stream);
/* qm:357-442 prefill_chunk_ / prefill_batched: T prompt tokens (HOST ids) as row-batched GEMMs on
 * the int4 weights + tiled causal attention, in chunks of 1024 (TLB_PREFILL_CHUNK overrides), from the current position; leaves
 * position += T and the greedy next token on the device and in *next_token.  Single GPU. */
int tlb_decoder_prefill(void* dec, const int32_t* tokens, int64_t T, int32_t* next_token, void* stream);
/* Tensor-parallel wiring (no counterpart in the reference, which is single-device):
 * each rank exports a 128-byte record, the ranks exchange them over any host
 * channel, and every rank opens the others' exchange buffers. */
int tlb_decoder_ipc_export(void* dec, void* record128);
int tlb_decoder_ipc_open(void* dec, const void* records);
/* Fault drill on one GPU (no counterpart in the reference): aim every peer's staging pointer
 * at a private sink nobody writes, so the rank's next exchange runs into its bounded wait
 * and tlb_device_status reports TLB_ERR_DEVICE_WAIT; nothing faults or hangs. */
int tlb_decoder_loopback_peers(void* dec);

#ifdef __cplusplus
}
#endif
#endif /* TLB200_H_ */
