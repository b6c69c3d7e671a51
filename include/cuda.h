// tl::cuda facade for cpp-tensorlib backed by libtlb200.so (B200, sm_100a).
//
// Drop-in replacement for the reference's include/cuda.h: put THIS directory before
// the reference's include directory on the include path and build with
// -DTENSORLIB_CUDA; storage.h -> gpu.h -> "cuda.h" then resolves here, while every
// other reference header (array.h, storage.h, metal.h for the kop enum, ...) is
// consumed unmodified.  The facade keeps the reference's names and signatures
// (reference include/cuda.h:496-1405); below it there is no driver table and no
// embedded PTX, only dlopen("libtlb200.so") and the C-ABI of tlb200.h.
//
// Scope: the quantized-decode path -- gemv_q4, attn_decode(+_dpos), rope(+_dpos),
// rmsnorm, rmsnorm_res, swiglu, argmax, kv_append(+_dpos), kv_cache (f32 or bf16), incr_u32, graph
// capture, the host/device mirror (alloc / release / sync_to_host / upload) -- and the rest of
// the evaluator's GPU surface (elementwise and broadcast binaries, unary ops, row reductions and
// softmax, f32 GEMM, f32 / bf16 GEMVs and the bf16 prefill GEMM), so a graph evaluated under
// tl::use_gpu() stays on the device between hot ops.  An op the library refuses is NOT
// declined: it throws, because silently computing a decode op on the CPU is exactly what
// this backend exists to prevent.
#pragma once

#include <dlfcn.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "metal.h"  // tl::metal::kop, the op enum every backend shares
#include "types.h"  // tl::dtype

namespace tl {
namespace cuda {

using kop = tl::metal::kop;
struct CUgraphExec_st;
using CUgraphExec = CUgraphExec_st*;

#if defined(TENSORLIB_CUDA) && !defined(__APPLE__)

namespace detail {

// One process-wide binding to the shared library plus the host/device mirror table.
struct backend {
  void* so = nullptr;
  bool ready = false;
  bool work_pending = false;
  void* stream = nullptr;  // nullptr = default stream; the capture stream while recording

  // ---- C-ABI entry points (signatures of tlb200.h) ----
  int (*init)(int) = nullptr;
  int (*device_count)() = nullptr;
  const char* (*last_error)() = nullptr;
  int (*alloc_)(int64_t, void**) = nullptr;
  int (*free_)(void*) = nullptr;
  int (*h2d)(void*, const void*, int64_t, void*) = nullptr;
  int (*d2h)(void*, const void*, int64_t, void*) = nullptr;
  int (*sync)(void*) = nullptr;
  int (*gemv_q4)(const float*, const void*, const float*, float*, int64_t, int64_t, int64_t, void*) = nullptr;
  int (*attn_decode)(const float*, const float*, const float*, float*, int64_t, int64_t, int64_t,
                     int64_t, int64_t, float, void*) = nullptr;
  int (*attn_decode_dpos)(const float*, const float*, const float*, float*, int64_t, int64_t,
                          const void*, int64_t, int64_t, float, void*, void*) = nullptr;
  int64_t (*attn_partials_bytes)(int64_t, int64_t, int64_t, int64_t) = nullptr;
  int (*rmsnorm)(const float*, const float*, float*, int64_t, float, int64_t, void*) = nullptr;
  int (*rmsnorm_res)(const float*, const float*, const float*, float*, float*, int64_t, float,
                     int64_t, void*) = nullptr;
  int (*swiglu)(const float*, float*, int64_t, int64_t, void*) = nullptr;
  int (*swiglu_split)(const float*, int64_t, const float*, int64_t, float*, int64_t, int64_t, void*) = nullptr;
  int (*gemm_q4)(const float*, int64_t, int64_t, const void*, const float*, float*, int64_t, int64_t,
                 int64_t, float, float, void*) = nullptr;
  int (*rope)(const float*, float*, int64_t, int64_t, int64_t, int64_t, float, const float*, void*) = nullptr;
  int (*rope_dpos)(const float*, float*, int64_t, int64_t, int64_t, const void*, float, const float*,
                   void*) = nullptr;
  int (*kv_append)(float*, float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t,
                   void*) = nullptr;
  int (*kv_append_dpos)(float*, float*, const float*, const float*, const void*, int64_t, int64_t,
                        int64_t, void*) = nullptr;
  int (*incr_u32)(void*, void*) = nullptr;
  int (*argmax)(const float*, int64_t, int64_t*, void*) = nullptr;
  int (*memset_)(void*, int, int64_t, void*) = nullptr;
  int (*attn_decode_bf16)(const float*, const void*, const void*, float*, int64_t, int64_t, int64_t,
                          int64_t, int64_t, float, void*) = nullptr;
  int (*kv_append_bf16)(void*, void*, const float*, const float*, int64_t, int64_t, int64_t, int64_t,
                        void*) = nullptr;
  int (*kv_fill_bf16)(void*, void*, const float*, const float*, int64_t, int64_t, int64_t, int64_t,
                      int64_t, void*) = nullptr;
  int (*attn_prefill_bf16)(const float*, const void*, const void*, float*, int64_t, int64_t, int64_t,
                           int64_t, int64_t, float, int64_t, void*) = nullptr;
  int (*gemv_bf16_row_)(const float*, const void*, float*, int64_t, int64_t, void*) = nullptr;
  int64_t (*q4p_bytes)(int64_t, int64_t) = nullptr;
  int (*q4_pack)(const void*, int64_t, int64_t, void*, void*) = nullptr;
  int (*gemv_q4p)(const float*, const void*, float*, int64_t, int64_t, float, float, void*) = nullptr;
  int (*split_heads)(const float*, const float*, float*, int64_t, int64_t, int64_t, int64_t, int64_t, void*) = nullptr;
  int (*merge_heads)(const float*, float*, int64_t, int64_t, int64_t, void*) = nullptr;
  int (*kv_fill)(float*, float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t, int64_t, void*) = nullptr;
  int (*attn_prefill)(const float*, const float*, const float*, float*, int64_t, int64_t, int64_t, int64_t,
                      int64_t, float, int64_t, void*) = nullptr;
  int (*binary_)(int, const float*, const float*, float*, int64_t, float, float, void*) = nullptr;
  int (*binary_bcast_)(int, const float*, int64_t, int64_t, const float*, int64_t, int64_t, float*, int64_t,
                       int64_t, float, float, void*) = nullptr;
  int (*unary_)(int, const float*, float*, int64_t, float, float, void*) = nullptr;
  int (*row_op_)(int, const float*, float*, int64_t, int64_t, float, float, void*) = nullptr;
  int (*gemm_f32_)(const float*, int64_t, int, const float*, int64_t, int, float*, int64_t, int64_t, int64_t,
                   float, float, void*) = nullptr;
  int (*gemm_bf16_nt_)(const float*, const void*, float*, int64_t, int64_t, int64_t, void*) = nullptr;
  int (*gemv_f32_)(const float*, const float*, float*, int64_t, int64_t, void*) = nullptr;
  int (*gemv_bf16_)(const float*, const void*, float*, int64_t, int64_t, void*) = nullptr;
  int (*capture_begin)(void**) = nullptr;
  int (*capture_end)(void**) = nullptr;
  int (*graph_launch)(void*, void*) = nullptr;
  int (*graph_destroy)(void*) = nullptr;

  // ---- mirror: every allocation is a device buffer plus a malloc'd host twin;
  // `where` says which side holds the live copy (reference cuda.h:199-233) ----
  enum side { HOST, DEVICE, BOTH };
  struct twin {
    float* host = nullptr;
    size_t bytes = 0;
    side where = HOST;
  };
  std::unordered_map<void*, twin> twins;                                  // key: device pointer
  std::unordered_map<size_t, std::vector<std::pair<void*, float*>>> pool;  // recycled, by size

  // Weights seen by gemv_q4 are repacked once into the library's tile-packed layout (the
  // fast decode GEMV reads that); key: the q4 buffer's device pointer.  An entry dies when
  // the mirror uploads new host contents into the buffer, a kernel writes it, or it is
  // released.  TLB200_SEAM_PACK=0 keeps the reference layout (half the weight memory).
  struct packed_w {
    void* dev = nullptr;
    int64_t N = 0, K = 0;
  };
  std::unordered_map<void*, packed_w> packed;
  int pack_enabled = -1;
  void drop_packed(void* native) {
    auto it = packed.find(native);
    if (it == packed.end()) return;
    sync(stream);   // a launch may still read it
    free_(it->second.dev);
    packed.erase(it);
  }
  const void* packed_for(void* qw, int64_t N, int64_t K) {
    if (pack_enabled < 0) {
      const char* e = std::getenv("TLB200_SEAM_PACK");
      pack_enabled = (e && e[0] == '0') ? 0 : 1;
    }
    if (!pack_enabled) return nullptr;
    auto it = packed.find(qw);
    if (it != packed.end()) {
      if (it->second.N == N && it->second.K == K) return it->second.dev;
      drop_packed(qw);
    }
    const int64_t nb = q4p_bytes(N, K);
    packed_w w;
    if (nb <= 0 || alloc_(nb, &w.dev) != 0) return nullptr;
    if (q4_pack(qw, N, K, w.dev, stream) != 0) {
      free_(w.dev);
      return nullptr;
    }
    w.N = N;
    w.K = K;
    packed.emplace(qw, w);
    return w.dev;
  }

  template <class F>
  bool bind(F& fn, const char* name) {
    fn = reinterpret_cast<F>(dlsym(so, name));
    return fn != nullptr;
  }

  static backend& get() {
    static backend* b = new backend();  // leaked on purpose, like the reference context
    static bool tried = false;
    if (!tried) {
      tried = true;
      b->open_();
    }
    return *b;
  }

  void open_() {
    const char* env = std::getenv("TLB200_LIB");
    const char* names[] = {env, "libtlb200.so", "cpp_tensorlib_b200/libtlb200.so"};
    for (const char* n : names) {
      if (n && (so = dlopen(n, RTLD_NOW | RTLD_LOCAL))) break;
    }
    if (!so) return;
    bool ok = bind(init, "tlb_init") && bind(device_count, "tlb_device_count") &&
              bind(last_error, "tlb_last_error") && bind(alloc_, "tlb_alloc") &&
              bind(free_, "tlb_free") && bind(h2d, "tlb_h2d") && bind(d2h, "tlb_d2h") &&
              bind(sync, "tlb_sync") && bind(gemv_q4, "tlb_gemv_q4") &&
              bind(attn_decode, "tlb_attn_decode") && bind(attn_decode_dpos, "tlb_attn_decode_dpos") &&
              bind(attn_partials_bytes, "tlb_attn_partials_bytes") && bind(rmsnorm, "tlb_rmsnorm") &&
              bind(rmsnorm_res, "tlb_rmsnorm_res") && bind(swiglu, "tlb_swiglu") &&
              bind(rope, "tlb_rope") && bind(rope_dpos, "tlb_rope_dpos") &&
              bind(kv_append, "tlb_kv_append") && bind(kv_append_dpos, "tlb_kv_append_dpos") &&
              bind(incr_u32, "tlb_incr_u32") && bind(argmax, "tlb_argmax") &&
              bind(memset_, "tlb_memset") && bind(q4p_bytes, "tlb_q4p_bytes") &&
              bind(q4_pack, "tlb_q4_pack") && bind(gemv_q4p, "tlb_gemv_q4p") &&
              bind(gemv_bf16_row_, "tlb_gemv_bf16_row") &&
              bind(attn_decode_bf16, "tlb_attn_decode_bf16") && bind(kv_append_bf16, "tlb_kv_append_bf16") &&
              bind(kv_fill_bf16, "tlb_kv_fill_bf16") && bind(attn_prefill_bf16, "tlb_attn_prefill_bf16") && bind(split_heads, "tlb_split_heads") &&
              bind(merge_heads, "tlb_merge_heads") && bind(kv_fill, "tlb_kv_fill") &&
              bind(attn_prefill, "tlb_attn_prefill") && bind(capture_begin, "tlb_capture_begin") &&
              bind(capture_end, "tlb_capture_end") && bind(graph_launch, "tlb_graph_launch") &&
              bind(graph_destroy, "tlb_graph_destroy") && bind(swiglu_split, "tlb_swiglu_split") &&
              bind(gemm_q4, "tlb_gemm_q4") && bind(binary_, "tlb_binary") &&
              bind(binary_bcast_, "tlb_binary_bcast") && bind(unary_, "tlb_unary") && bind(row_op_, "tlb_row_op") &&
              bind(gemm_f32_, "tlb_gemm_f32") && bind(gemm_bf16_nt_, "tlb_gemm_bf16_nt") &&
              bind(gemv_f32_, "tlb_gemv_f32") && bind(gemv_bf16_, "tlb_gemv_bf16");
    if (!ok || device_count() <= 0) return;
    ready = init(0) == 0;
  }

  // A hot-path call the library refused: report it, never fall back.
  [[noreturn]] void fail(const char* what) const {
    throw std::runtime_error(std::string("tl::cuda::") + what + ": " +
                             (last_error ? last_error() : "libtlb200.so not loaded"));
  }
  void must(int rc, const char* what) {
    if (rc != 0) fail(what);
    work_pending = true;
  }

  twin* find(void* native) {
    auto it = twins.find(native);
    return it == twins.end() ? nullptr : &it->second;
  }
  // A kernel is about to read / write the buffer (mid-buffer pointers are not keys:
  // their base must already be current, as in the reference).
  void reads(void* native) {
    twin* t = find(native);
    if (t && t->where == HOST) {
      if (h2d(native, t->host, (int64_t)t->bytes, stream) != 0) fail("upload");
      t->where = BOTH;
      drop_packed(native);   // new contents: a packed copy of the old ones is stale
    }
  }
  void writes(void* native) {
    if (twin* t = find(native)) t->where = DEVICE;
    drop_packed(native);
  }
};

inline const float* f(void* p) { return static_cast<const float*>(p); }
inline float* fw(void* p) { return static_cast<float*>(p); }

}  // namespace detail

inline bool available() { return detail::backend::get().ready; }
inline bool pending() { return detail::backend::get().work_pending; }
inline void set_no_splitk(bool) {}  // diagnostic knob of the reference kernels; no meaning here

inline void flush() {
  auto& b = detail::backend::get();
  if (!b.ready || !b.work_pending) return;
  if (b.sync(b.stream) != 0) b.fail("flush");
  b.work_pending = false;
}

inline void* alloc(int64_t bytes, float** contents) {
  auto& b = detail::backend::get();
  if (!b.ready) return nullptr;
  const size_t nb = bytes > 0 ? (size_t)bytes : 4;
  void* dev = nullptr;
  float* host = nullptr;
  auto it = b.pool.find(nb);
  if (it != b.pool.end() && !it->second.empty()) {
    dev = it->second.back().first;
    host = it->second.back().second;
    it->second.pop_back();
  } else {
    if (b.alloc_((int64_t)nb, &dev) != 0) return nullptr;
    host = static_cast<float*>(std::malloc(nb));
    if (!host) {
      b.free_(dev);
      return nullptr;
    }
  }
  b.twins[dev] = detail::backend::twin{host, nb, detail::backend::HOST};
  if (contents) *contents = host;
  return dev;
}

inline void release(void* buf, int64_t, float*) {
  auto& b = detail::backend::get();
  if (!b.ready || !buf) return;
  b.drop_packed(buf);
  auto it = b.twins.find(buf);
  if (it == b.twins.end()) {
    b.free_(buf);
    return;
  }
  b.pool[it->second.bytes].push_back({buf, it->second.host});
  b.twins.erase(it);
}

inline void sync_to_host(void* native, bool for_write) {
  auto& b = detail::backend::get();
  if (!b.ready || !native) return;
  auto* t = b.find(native);
  if (!t) return;
  if (b.work_pending) flush();
  if (t->where == detail::backend::DEVICE) {
    if (b.d2h(t->host, native, (int64_t)t->bytes, b.stream) != 0) b.fail("sync_to_host");
    t->where = detail::backend::BOTH;
  }
  if (for_write) t->where = detail::backend::HOST;
}

// Blocking upload of the first n floats (reference cuda.h:559-570).
inline void upload(void* native, const float* src, int64_t n) {
  auto& b = detail::backend::get();
  if (!b.ready || !native || n <= 0) return;
  auto* t = b.find(native);
  if (!t) return;
  if (src != t->host) std::memcpy(t->host, src, (size_t)n * 4);
  if (b.h2d(native, t->host, n * 4, b.stream) != 0 || b.sync(b.stream) != 0) b.fail("upload");
  t->where = detail::backend::BOTH;
}
inline void upload_u32(void* native, unsigned val) {
  auto& b = detail::backend::get();
  if (!b.ready || !native) return;
  auto* t = b.find(native);
  if (!t || t->bytes < 4) return;
  std::memcpy(t->host, &val, 4);
  if (b.h2d(native, t->host, 4, b.stream) != 0 || b.sync(b.stream) != 0) b.fail("upload_u32");
  t->where = detail::backend::BOTH;
}

// ---- the rest of the evaluator's surface (reference cuda.h:640-742, 1409-1503): on the device
// too, so a graph evaluated under tl::use_gpu() does not bounce to the host between hot ops.
// Offsets are in BYTES (reference array.h:1480-1482 passes offset_ * 4). ----
namespace detail {
inline const float* at(void* p, int64_t byte_off) {
  return reinterpret_cast<const float*>(static_cast<const char*>(p) + byte_off);
}
inline float* at_w(void* p, int64_t byte_off) { return reinterpret_cast<float*>(static_cast<char*>(p) + byte_off); }
inline int bin_code(kop op) {
  switch (op) {
    case kop::add: case kop::badd: return 0;
    case kop::sub: case kop::bsub: return 1;
    case kop::mul: case kop::bmul: return 2;
    case kop::div: case kop::bdiv: return 3;
    case kop::pow_: case kop::bpow: return 4;
    default: return -1;
  }
}
inline int una_code(kop op) {
  switch (op) {
    case kop::exp_: return 0;
    case kop::log_: return 1;
    case kop::sqrt_: return 2;
    case kop::sigmoid: return 3;
    case kop::relu: return 4;
    case kop::affine: return 5;
    default: return -1;
  }
}
}  // namespace detail

inline bool binary(kop op, void* a, int64_t ao, void* b_, int64_t bo, void* out, int64_t oo, int64_t n,
                   float scale, float offset) {
  auto& b = detail::backend::get();
  const int code = detail::bin_code(op);
  if (!b.ready || code < 0) return false;
  b.reads(a); b.reads(b_); b.writes(out);
  b.must(b.binary_(code, detail::at(a, ao), detail::at(b_, bo), detail::at_w(out, oo), n, scale, offset, b.stream),
         "binary");
  return true;
}
inline bool binary_bcast(kop op, void* a, int64_t ao, int64_t ars, int64_t acs, void* b_, int64_t bo, int64_t brs,
                         int64_t bcs, void* out, int64_t oo, int64_t rows, int64_t cols, float scale,
                         float offset) {
  auto& b = detail::backend::get();
  const int code = detail::bin_code(op);
  if (!b.ready || code < 0) return false;
  b.reads(a); b.reads(b_); b.writes(out);
  b.must(b.binary_bcast_(code, detail::at(a, ao), ars, acs, detail::at(b_, bo), brs, bcs, detail::at_w(out, oo),
                         rows, cols, scale, offset, b.stream), "binary_bcast");
  return true;
}
inline bool unary(kop op, void* a, int64_t ao, void* out, int64_t oo, int64_t n, float scale, float offset) {
  auto& b = detail::backend::get();
  const int code = detail::una_code(op);
  if (!b.ready || code < 0) return false;
  b.reads(a); b.writes(out);
  b.must(b.unary_(code, detail::at(a, ao), detail::at_w(out, oo), n, scale, offset, b.stream), "unary");
  return true;
}
inline bool gemm(void* a, int64_t ao, int64_t lda, bool ta, void* b_, int64_t bo, int64_t ldb, bool tb,
                 void* out, int64_t oo, int64_t m, int64_t n, int64_t k, float scale, float offset) {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  b.reads(a); b.reads(b_); b.writes(out);
  b.must(b.gemm_f32_(detail::at(a, ao), lda, ta ? 1 : 0, detail::at(b_, bo), ldb, tb ? 1 : 0,
                     detail::at_w(out, oo), m, n, k, scale, offset, b.stream), "gemm");
  return true;
}
inline bool row_op(kop op, void* in, int64_t io, void* out, int64_t oo, int64_t rows, int64_t cols, float scale,
                   float offset) {
  auto& b = detail::backend::get();
  const int code = op == kop::softmax ? 0 : (op == kop::row_sum ? 1 : (op == kop::row_max ? 2 : -1));
  if (!b.ready || code < 0 || cols <= 0) return false;
  b.reads(in); b.writes(out);
  b.must(b.row_op_(code, detail::at(in, io), detail::at_w(out, oo), rows, cols, scale, offset, b.stream), "row_op");
  return true;
}
// decode GEMV on [K,N] weights (reference cuda.h:719-742)
inline bool gemv_f32(void* a, void* B, void* y, int64_t n, int64_t k) {
  auto& b = detail::backend::get();
  if (!b.ready || n <= 0 || k <= 0) return false;
  b.reads(a); b.reads(B); b.writes(y);
  b.must(b.gemv_f32_(detail::f(a), detail::f(B), detail::fw(y), n, k, b.stream), "gemv_f32");
  return true;
}
inline bool gemv_bf16(void* a, void* B, void* y, int64_t n, int64_t k) {
  auto& b = detail::backend::get();
  if (!b.ready || n <= 0 || k <= 0) return false;
  b.reads(a); b.reads(B); b.writes(y);
  b.must(b.gemv_bf16_(detail::f(a), B, detail::fw(y), n, k, b.stream), "gemv_bf16");
  return true;
}
// bf16 row-major weights [N][K] (reference cuda.h:770-785): the decode projection of the
// reference's bf16-weight models
inline bool gemv_bf16_row(void* a, void* B, void* y, int64_t n, int64_t k) {
  auto& b = detail::backend::get();
  if (!b.ready || (k % 8) != 0) return false;
  b.reads(a); b.reads(B); b.writes(y);
  b.must(b.gemv_bf16_row_(detail::f(a), B, detail::fw(y), n, k, b.stream), "gemv_bf16_row");
  return true;
}
// weight-native prefill GEMM on bf16 [N,K] weights (reference cuda.h:790-841)
inline bool gemm_bf16_nt(void* A, void* W, void* C, int64_t M, int64_t N, int64_t K) {
  auto& b = detail::backend::get();
  if (!b.ready || M <= 0 || N <= 0 || K <= 0) return false;
  b.reads(A); b.reads(W); b.writes(C);
  b.must(b.gemm_bf16_nt_(detail::f(A), W, detail::fw(C), M, N, K, b.stream), "gemm_bf16_nt");
  return true;
}

// ---- the quantized-decode path ----
inline bool gemv_q4(void* a, void* qw, void* scales, void* y, int64_t N, int64_t K, int64_t group) {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  b.reads(a); b.reads(qw); b.reads(scales); b.writes(y);
  // scales sit inside the same buffer at qw + N*K/2 (reference array.h:1621-1622): only then
  // is qw the whole weight, and only then may the packed copy stand in for it
  if (group == 32 && static_cast<char*>(scales) == static_cast<char*>(qw) + N * K / 2) {
    if (const void* pk = b.packed_for(qw, N, K)) {
      b.must(b.gemv_q4p(detail::f(a), pk, detail::fw(y), N, K, 1.0f, 0.0f, b.stream), "gemv_q4 (packed)");
      return true;
    }
  }
  b.must(b.gemv_q4(detail::f(a), qw, detail::f(scales), detail::fw(y), N, K, group, b.stream), "gemv_q4");
  return true;
}

inline bool attn_decode(void* q, void* K, void* V, void* out, int64_t n_q_heads, int64_t n_kv_heads,
                        int64_t ctx, int64_t kv_max, int64_t D, float scale, bool kv_bf16 = false) {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  b.reads(q); b.reads(K); b.reads(V); b.writes(out);
  if (kv_bf16)
    b.must(b.attn_decode_bf16(detail::f(q), K, V, detail::fw(out), n_q_heads, n_kv_heads, ctx, kv_max,
                              D, scale, b.stream), "attn_decode (bf16 cache)");
  else
    b.must(b.attn_decode(detail::f(q), detail::f(K), detail::f(V), detail::fw(out), n_q_heads,
                         n_kv_heads, ctx, kv_max, D, scale, b.stream), "attn_decode");
  return true;
}

inline bool rope(void* x, void* out, int64_t rows, int64_t T, int64_t D, int64_t pos, float base,
                 void* bias = nullptr) {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  b.reads(x); if (bias) b.reads(bias); b.writes(out);
  b.must(b.rope(detail::f(x), detail::fw(out), rows, T, D, pos, base, detail::f(bias), b.stream), "rope");
  return true;
}
inline bool rope_dpos(void* x, void* out, int64_t rows, int64_t T, int64_t D, void* d_pos, float base,
                      void* bias = nullptr) {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  b.reads(x); if (bias) b.reads(bias); b.reads(d_pos); b.writes(out);
  b.must(b.rope_dpos(detail::f(x), detail::fw(out), rows, T, D, d_pos, base, detail::f(bias), b.stream),
         "rope_dpos");
  return true;
}
inline bool incr_u32(void* d_pos) {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  b.writes(d_pos);
  b.must(b.incr_u32(d_pos, b.stream), "incr_u32");
  return true;
}
inline bool rmsnorm(void* x, void* w, void* out, int64_t n, float eps, int64_t rows = 1) {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  b.reads(x); b.reads(w); b.writes(out);
  b.must(b.rmsnorm(detail::f(x), detail::f(w), detail::fw(out), n, eps, rows, b.stream), "rmsnorm");
  return true;
}
inline bool rmsnorm_res(void* x, void* delta, void* w, void* xout, void* hout, int64_t n, float eps,
                        int64_t rows = 1) {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  b.reads(x); b.reads(delta); b.reads(w); b.writes(xout); b.writes(hout);
  b.must(b.rmsnorm_res(detail::f(x), detail::f(delta), detail::f(w), detail::fw(xout), detail::fw(hout),
                       n, eps, rows, b.stream), "rmsnorm_res");
  return true;
}
inline bool swiglu(void* gu, void* out, int64_t ff, int64_t rows = 1) {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  b.reads(gu); b.writes(out);
  b.must(b.swiglu(detail::f(gu), detail::fw(out), ff, rows, b.stream), "swiglu");
  return true;
}
inline bool argmax(void* in, int64_t n, int64_t* out_idx) {
  auto& b = detail::backend::get();
  if (!b.ready || !in || n <= 0 || !out_idx) return false;
  b.reads(in);
  b.must(b.argmax(detail::f(in), n, out_idx, b.stream), "argmax");
  b.work_pending = false;  // tlb_argmax synchronises the stream
  return true;
}
inline bool kv_append(void* Kc, void* Vc, void* k_new, void* v_new, int64_t pos, int64_t kv_max,
                      int64_t n_kv_heads, int64_t D, bool kv_bf16 = false) {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  b.reads(k_new); b.reads(v_new); b.reads(Kc); b.reads(Vc); b.writes(Kc); b.writes(Vc);
  if (kv_bf16)
    b.must(b.kv_append_bf16(Kc, Vc, detail::f(k_new), detail::f(v_new), pos, kv_max, n_kv_heads, D,
                            b.stream), "kv_append (bf16 cache)");
  else
    b.must(b.kv_append(detail::fw(Kc), detail::fw(Vc), detail::f(k_new), detail::f(v_new), pos, kv_max,
                       n_kv_heads, D, b.stream), "kv_append");
  return true;
}
inline bool kv_append_dpos(void* Kc, void* Vc, void* k_new, void* v_new, void* d_pos, int64_t kv_max,
                           int64_t n_kv_heads, int64_t D) {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  b.reads(k_new); b.reads(v_new); b.reads(d_pos); b.reads(Kc); b.reads(Vc); b.writes(Kc); b.writes(Vc);
  b.must(b.kv_append_dpos(detail::fw(Kc), detail::fw(Vc), detail::f(k_new), detail::f(v_new), d_pos,
                          kv_max, n_kv_heads, D, b.stream), "kv_append_dpos");
  return true;
}
inline bool attn_decode_dpos(void* q, void* K, void* V, void* out, int64_t n_q_heads,
                             int64_t n_kv_heads, void* d_pos, int64_t kv_max, int64_t D, float scale,
                             void* partials) {
  auto& b = detail::backend::get();
  if (!b.ready || !partials) return false;
  b.reads(q); b.reads(K); b.reads(V); b.reads(d_pos); b.writes(out);
  b.must(b.attn_decode_dpos(detail::f(q), detail::f(K), detail::f(V), detail::fw(out), n_q_heads,
                            n_kv_heads, d_pos, kv_max, D, scale, partials, b.stream), "attn_decode_dpos");
  return true;
}
// ---- batched prefill (reference cuda.h:848-879, 1143-1201), f32 cache ----
inline bool split_heads(void* src, void* bias, void* dst, int64_t T, int64_t ld, int64_t off,
                        int64_t H, int64_t D) {
  auto& b = detail::backend::get();
  if (!b.ready || T <= 0 || H <= 0 || D <= 0) return false;
  b.reads(src); if (bias) b.reads(bias); b.writes(dst);
  b.must(b.split_heads(detail::f(src), detail::f(bias), detail::fw(dst), T, ld, off, H, D, b.stream), "split_heads");
  return true;
}
inline bool merge_heads(void* src, void* dst, int64_t T, int64_t H, int64_t D) {
  auto& b = detail::backend::get();
  if (!b.ready || T <= 0 || H <= 0 || D <= 0) return false;
  b.reads(src); b.writes(dst);
  b.must(b.merge_heads(detail::f(src), detail::fw(dst), T, H, D, b.stream), "merge_heads");
  return true;
}
inline bool kv_fill(void* Kc, void* Vc, void* K, void* V, int64_t T, int64_t kv_max,
                    int64_t n_kv_heads, int64_t D, bool kv_bf16 = false, int64_t pos0 = 0) {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  b.reads(K); b.reads(V); b.reads(Kc); b.reads(Vc); b.writes(Kc); b.writes(Vc);
  if (kv_bf16)
    b.must(b.kv_fill_bf16(Kc, Vc, detail::f(K), detail::f(V), T, kv_max, n_kv_heads, D, pos0, b.stream),
           "kv_fill (bf16 cache)");
  else
    b.must(b.kv_fill(detail::fw(Kc), detail::fw(Vc), detail::f(K), detail::f(V), T, kv_max, n_kv_heads, D,
                     pos0, b.stream), "kv_fill");
  return true;
}
inline bool attn_prefill(void* q, void* K, void* V, void* out, int64_t n_q_heads, int64_t n_kv_heads,
                         int64_t T, int64_t kv_max, int64_t D, float scale, bool kv_bf16 = false,
                         int64_t pos0 = 0) {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  b.reads(q); b.reads(K); b.reads(V); b.writes(out);
  if (kv_bf16)
    b.must(b.attn_prefill_bf16(detail::f(q), K, V, detail::fw(out), n_q_heads, n_kv_heads, T, kv_max, D,
                               scale, pos0, b.stream), "attn_prefill (bf16 cache)");
  else
    b.must(b.attn_prefill(detail::f(q), detail::f(K), detail::f(V), detail::fw(out), n_q_heads, n_kv_heads,
                          T, kv_max, D, scale, pos0, b.stream), "attn_prefill");
  return true;
}

// ---- CUDA-graph capture (reference cuda.h:512-551) ----
inline bool graph_available() { return detail::backend::get().ready; }
inline bool capture_begin() {
  auto& b = detail::backend::get();
  if (!b.ready) return false;
  if (b.work_pending) flush();
  void* s = nullptr;
  if (b.capture_begin(&s) != 0) return false;
  b.stream = s;
  return true;
}
inline CUgraphExec capture_end() {
  auto& b = detail::backend::get();
  void* e = nullptr;
  int rc = b.capture_end(&e);
  b.stream = nullptr;
  return rc == 0 ? static_cast<CUgraphExec>(e) : nullptr;
}
inline bool graph_launch(CUgraphExec e) {
  auto& b = detail::backend::get();
  if (!b.ready || !e) return false;
  if (b.graph_launch(e, nullptr) != 0) return false;
  b.work_pending = true;
  return true;
}
inline void graph_destroy(CUgraphExec e) {
  auto& b = detail::backend::get();
  if (e && b.ready) b.graph_destroy(e);
}

// Persistent KV cache (reference cuda.h:1326-1405), f32 or bf16 storage.  The device-position
// forms read an f32 cache only (as in the reference) and decline on a bf16 one.
struct kv_cache {
  void* K = nullptr;
  void* V = nullptr;
  int64_t n_kv_heads = 0, max_ctx = 0, D = 0, pos = 0;
  bool kv_bf16 = false;
  void* dpos_partials = nullptr;

  bool init(int64_t kv_heads, int64_t maxctx, int64_t d, dtype kv_dt = dtype::f32) {
    if (kv_dt != dtype::f32 && kv_dt != dtype::bf16) return false;
    n_kv_heads = kv_heads; max_ctx = maxctx; D = d; pos = 0;
    kv_bf16 = (kv_dt == dtype::bf16);
    const int64_t w = kv_bf16 ? 2 : 4;  // bytes per K/V element
    K = alloc(n_kv_heads * max_ctx * D * w, nullptr);
    V = alloc(n_kv_heads * max_ctx * D * w, nullptr);
    return K && V;
  }
  bool append(void* k_new, void* v_new) {
    if (pos >= max_ctx) return false;
    if (!kv_append(K, V, k_new, v_new, pos, max_ctx, n_kv_heads, D, kv_bf16)) return false;
    pos++;
    return true;
  }
  bool attn(void* q, void* out, int64_t n_q_heads, float scale) {
    return attn_decode(q, K, V, out, n_q_heads, n_kv_heads, pos, max_ctx, D, scale, kv_bf16);
  }
  bool append_dpos(void* k_new, void* v_new, void* d_pos) {
    if (kv_bf16) return false;
    return kv_append_dpos(K, V, k_new, v_new, d_pos, max_ctx, n_kv_heads, D);
  }
  bool attn_dpos(void* q, void* out, int64_t n_q_heads, void* d_pos, float scale) {
    auto& b = detail::backend::get();
    if (kv_bf16) return false;
    if (!dpos_partials) {
      int64_t nb = b.attn_partials_bytes(n_q_heads, n_kv_heads, max_ctx, D);
      if (nb <= 0) return false;
      dpos_partials = alloc(nb, nullptr);
      if (!dpos_partials) return false;
      if (b.memset_(dpos_partials, 0, nb, b.stream) != 0) return false;
      b.writes(dpos_partials);
    }
    return attn_decode_dpos(q, K, V, out, n_q_heads, n_kv_heads, d_pos, max_ctx, D, scale, dpos_partials);
  }
  bool prefill(void* q, void* k_src, void* v_src, void* out, int64_t T, int64_t n_q_heads, float scale) {
    if (T <= 0 || pos + T > max_ctx) return false;
    if (!kv_fill(K, V, k_src, v_src, T, max_ctx, n_kv_heads, D, kv_bf16, pos)) return false;
    const int64_t p0 = pos;
    pos += T;
    return attn_prefill(q, K, V, out, n_q_heads, n_kv_heads, T, max_ctx, D, scale, kv_bf16, p0);
  }
  void destroy() {
    if (K) release(K, 0, nullptr);
    if (V) release(V, 0, nullptr);
    if (dpos_partials) release(dpos_partials, 0, nullptr);
    K = V = dpos_partials = nullptr;
  }
};

#else  // no TENSORLIB_CUDA: the same inert surface the reference's stubs give

inline bool available() { return false; }
inline bool pending() { return false; }
inline void flush() {}
inline void* alloc(int64_t, float**) { return nullptr; }
inline void release(void*, int64_t, float*) {}
inline void sync_to_host(void*, bool) {}
inline bool binary(kop, void*, int64_t, void*, int64_t, void*, int64_t, int64_t, float, float) { return false; }
inline bool binary_bcast(kop, void*, int64_t, int64_t, int64_t, void*, int64_t, int64_t, int64_t,
                         void*, int64_t, int64_t, int64_t, float, float) { return false; }
inline bool unary(kop, void*, int64_t, void*, int64_t, int64_t, float, float) { return false; }
inline bool gemm(void*, int64_t, int64_t, bool, void*, int64_t, int64_t, bool, void*, int64_t,
                 int64_t, int64_t, int64_t, float, float) { return false; }
inline bool row_op(kop, void*, int64_t, void*, int64_t, int64_t, int64_t, float, float) { return false; }
inline bool gemv_f32(void*, void*, void*, int64_t, int64_t) { return false; }
inline bool gemv_bf16(void*, void*, void*, int64_t, int64_t) { return false; }
inline bool gemv_q4(void*, void*, void*, void*, int64_t, int64_t, int64_t) { return false; }
inline bool attn_decode(void*, void*, void*, void*, int64_t, int64_t, int64_t, int64_t, int64_t, float,
                        bool = false) { return false; }
inline bool rope(void*, void*, int64_t, int64_t, int64_t, int64_t, float, void* = nullptr) { return false; }

#endif

// CPU-read barrier: sync the GPU before any host read of a managed buffer.
inline void cpu_barrier() {
  if (pending()) flush();
}

}  // namespace cuda
}  // namespace tl
