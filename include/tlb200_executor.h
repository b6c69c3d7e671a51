// Lazy-graph executor of cpp-tensorlib for the B200 backend (libtlb200.so).
//
// The reference offers embedders an official plug point for graph evaluation: built with
// -DTL_RUNTIME_HOOKS, every evaluation goes through detail::run_hook / run_noflush_hook
// (reference include/array.h:190-195, 2244-2256; installed by tl::install_runtime_hooks(),
// array.h:2525-2532; storage hooks in storage.h:95-110).  This header installs an executor
// there that keeps the quantized-decode path on the device where the reference's own
// evaluator leaves it:
//
//   * a `dot` node whose weight is q4 runs as ONE launch of the int4 contraction at ANY
//     number of rows M, with the node's fused affine epilogue (node.scale / node.offset,
//     array.h:1305-1311) applied in the kernel's store.  The reference evaluator offers only
//     M == 1 to the device (array.h:1607-1628) and applies the epilogue on the CPU after a
//     D2H (array.h:2218-2225); for M > 1 it widens the weight to f32 on the host
//     (array.h:1978-1984) and multiplies on the CPU or with an f32 GEMM;
//   * the RMSNorm composition  (x * 1/sqrt(mean(x*x, last) + eps)) * w  (array.h:2429-2433)
//     and the SwiGLU composition  (g * sigmoid(g)) * u  (array.h:2435-2439) are recognised
//     in the graph and run as the fused kernels behind tl::cuda::rmsnorm / swiglu (the
//     reference's composition leaves the device half way: it has no reciprocal kernel and
//     its broadcast multiplies decline);
//   * every other node is handed to the reference's own detail::graph::eval_one, in the
//     same topological order, so attention / rope nodes still reach tl::cuda::attn_decode /
//     rope through the facade and the rest of the array surface behaves as before.
//
// Use (a translation unit built with -DTL_RUNTIME_HOOKS -DTENSORLIB_CUDA and this
// repository's include directory before the reference's):
//     #include <tensorlib.h>
//     #include <tlb200_executor.h>
//     tl::tlb200::install_executor();     // instead of tl::install_runtime_hooks()
//     tl::use_gpu();
// Nothing in the reference headers is edited.
#pragma once

#if !defined(TL_RUNTIME_HOOKS)
#error "tlb200_executor.h needs -DTL_RUNTIME_HOOKS (the reference's runtime-hook build)"
#endif

#include <tensorlib.h>

#include <cstdint>
#include <vector>

namespace tl {
namespace tlb200 {

#if defined(TENSORLIB_CUDA) && !defined(__APPLE__)

// What the executor did since the last reset; a consumer (or a test) reads it to see that
// the hot path stayed on the device.
struct executor_stats {
  long q4_dots_on_device = 0;     // dot nodes with a q4 weight run by the int4 kernels
  long q4_dot_rows = 0;           // rows (M) those launches covered
  long rmsnorm_fused = 0;         // RMSNorm compositions run as one kernel
  long swiglu_fused = 0;          // SwiGLU compositions run as one kernel
  long nodes_fused_away = 0;      // interior nodes of those compositions never evaluated
  long delegated = 0;             // nodes handed to the reference evaluator
  long q4_dots_delegated = 0;     // q4 dots the executor could NOT take (host operands, views)
};
inline executor_stats& stats() {
  static executor_stats s;
  return s;
}

namespace detail_ {

using node = tl::detail::node;
using node_ptr = tl::detail::node_ptr;
using op_t = node::op_t;
using backend = tl::cuda::detail::backend;

inline bool plain(const node& n) { return n.scale == 1.0f && n.offset == 0.0f; }
inline bool contiguous(const node& n) {
  return n.strides == tl::detail::contiguous_strides(n.shape);
}
// device address of an evaluated node's first element, or nullptr when it lives on the heap
inline const float* dev_ptr(const node& n) {
  if (!n.stor.native) return nullptr;
  return reinterpret_cast<const float*>(static_cast<const char*>(n.stor.native)) + n.soffset;
}
inline int64_t count(const shape_t& s) {
  int64_t c = 1;
  for (auto d : s) c *= d;
  return c;
}

// ---- q4 dot: y[M,N] = (x[M,K] . dequant(Wq)) * scale + offset ------------------------
inline bool run_q4_dot(node& n) {
  if (n.op != op_t::dot || n.inputs.size() != 2) return false;
  node& a = *n.inputs[0];
  node& w = *n.inputs[1];
  if (!a.evaluated || !w.evaluated || w.stor.dt != tl::dtype::q4 || w.shape.size() != 2) return false;
  auto& b = backend::get();
  const bool ok = b.ready && a.stor.dt == tl::dtype::f32 && (a.shape.size() == 1 || a.shape.size() == 2) &&
                  contiguous(a) && a.stor.native && w.stor.native && w.soffset == 0;
  if (!ok) {
    stats().q4_dots_delegated++;
    return false;
  }
  const int64_t K = w.shape[0], N = w.shape[1];
  const int64_t M = a.shape.size() == 1 ? 1 : a.shape[0];
  if ((a.shape.size() == 1 ? a.shape[0] : a.shape[1]) != K || K % tl::kQ4Group != 0) {
    stats().q4_dots_delegated++;
    return false;
  }
  tl::storage out = tl::storage::make(M * N);
  if (!out.native) {
    stats().q4_dots_delegated++;
    return false;
  }
  if (M > 0 && N > 0) {
    b.reads(a.stor.native);
    b.reads(w.stor.native);
    b.writes(out.native);
    const float* x = dev_ptr(a);
    float* y = static_cast<float*>(out.native);
    const void* pk = (M == 1) ? b.packed_for(w.stor.native, N, K) : nullptr;
    if (pk) {
      b.must(b.gemv_q4p(x, pk, y, N, K, n.scale, n.offset, b.stream), "executor: q4 dot (packed GEMV)");
    } else {
      const float* scales =
          reinterpret_cast<const float*>(static_cast<const char*>(w.stor.native) + N * K / 2);
      b.must(b.gemm_q4(x, M, K, w.stor.native, scales, y, N, N, K, n.scale, n.offset, b.stream),
             "executor: q4 dot");
    }
  }
  tl::detail::graph::store_raw_(n, std::move(out));
  stats().q4_dots_on_device++;
  stats().q4_dot_rows += M;
  return true;
}

// ---- pattern matching -----------------------------------------------------------------
// An interior node of a composition may be skipped only if nothing outside the composition
// can ever ask for its value: every owner of the node is one of the composition's own edges.
inline bool only_owned_by_edges(const node_ptr& p, long edges) { return p.use_count() == edges; }

struct rms_match {
  node* x = nullptr;
  node* w = nullptr;
  float eps = 0.f;
  std::vector<node*> interior;
};
// root = mul(mul(x, recip(sqrt(mean_ax(mul(x, x), last, keepdims) + eps))), w)
inline bool match_rmsnorm(node& root, rms_match& m) {
  if (root.op != op_t::mul || root.inputs.size() != 2 || !plain(root)) return false;
  for (int side = 0; side < 2; side++) {
    const node_ptr& xi = root.inputs[side];
    const node_ptr& wn = root.inputs[1 - side];
    if (xi->evaluated || xi->op != op_t::mul || xi->inputs.size() != 2 || !plain(*xi)) continue;
    for (int s2 = 0; s2 < 2; s2++) {
      const node_ptr& x = xi->inputs[s2];
      const node_ptr& inv = xi->inputs[1 - s2];
      if (inv->evaluated || inv->op != op_t::recip || !plain(*inv) || inv->inputs.size() != 1) continue;
      const node_ptr& sq = inv->inputs[0];
      if (sq->evaluated || sq->op != op_t::sqrt_ || !plain(*sq) || sq->inputs.size() != 1) continue;
      const node_ptr& ms = sq->inputs[0];
      if (ms->evaluated || ms->op != op_t::mean_ax || ms->scale != 1.0f || !ms->keepdims ||
          ms->inputs.size() != 1)
        continue;
      const node_ptr& xx = ms->inputs[0];
      if (xx->evaluated || xx->op != op_t::mul || !plain(*xx) || xx->inputs.size() != 2) continue;
      if (xx->inputs[0].get() != x.get() || xx->inputs[1].get() != x.get()) continue;
      const int rank = (int)x->shape.size();
      if (rank < 1 || ms->axis != rank - 1) continue;
      const int64_t nlast = x->shape[rank - 1];
      if (count(wn->shape) != nlast || wn->shape.empty() || wn->shape.back() != nlast) continue;
      if (root.shape != x->shape || xi->shape != x->shape) continue;
      if (!only_owned_by_edges(xi, 1) || !only_owned_by_edges(inv, 1) || !only_owned_by_edges(sq, 1) ||
          !only_owned_by_edges(ms, 1) || !only_owned_by_edges(xx, 1))
        continue;
      m.x = x.get();
      m.w = wn.get();
      m.eps = ms->offset;
      m.interior = {xi.get(), inv.get(), sq.get(), ms.get(), xx.get()};
      return true;
    }
  }
  return false;
}

struct swiglu_match {
  node* g = nullptr;
  node* u = nullptr;
  std::vector<node*> interior;
};
// root = mul(mul(g, sigmoid(g)), u)
inline bool match_swiglu(node& root, swiglu_match& m) {
  if (root.op != op_t::mul || root.inputs.size() != 2 || !plain(root)) return false;
  for (int side = 0; side < 2; side++) {
    const node_ptr& si = root.inputs[side];
    const node_ptr& u = root.inputs[1 - side];
    if (si->evaluated || si->op != op_t::mul || si->inputs.size() != 2 || !plain(*si)) continue;
    for (int s2 = 0; s2 < 2; s2++) {
      const node_ptr& g = si->inputs[s2];
      const node_ptr& sg = si->inputs[1 - s2];
      if (sg->evaluated || sg->op != op_t::sigmoid || !plain(*sg) || sg->inputs.size() != 1) continue;
      if (sg->inputs[0].get() != g.get()) continue;
      if (g->shape != u->shape || root.shape != g->shape || g->shape.empty()) continue;
      if (!only_owned_by_edges(si, 1) || !only_owned_by_edges(sg, 1)) continue;
      m.g = g.get();
      m.u = u.get();
      m.interior = {si.get(), sg.get()};
      return true;
    }
  }
  return false;
}

// rows x n view of an evaluated f32 node: last dim contiguous, one row stride (or one row)
inline bool row_view(const node& t, int64_t& rows, int64_t& n, int64_t& ld) {
  if (!t.evaluated || t.stor.dt != tl::dtype::f32 || !t.stor.native || t.shape.empty()) return false;
  if (t.strides.size() != t.shape.size()) return false;
  n = t.shape.back();
  rows = n > 0 ? count(t.shape) / n : 0;
  if (t.strides.back() != 1 && n > 1) return false;
  if (contiguous(t)) {
    ld = n;
    return true;
  }
  if (t.shape.size() == 2) {
    ld = t.strides[0];
    return ld >= n;
  }
  return false;
}

inline bool run_rmsnorm(node& root, const rms_match& m) {
  auto& b = backend::get();
  if (!b.ready) return false;
  int64_t rows, n, ld;
  if (!row_view(*m.x, rows, n, ld) || ld != n) return false;
  if (!m.w->evaluated || m.w->stor.dt != tl::dtype::f32 || !m.w->stor.native || !contiguous(*m.w)) return false;
  tl::storage out = tl::storage::make(rows * n);
  if (!out.native) return false;
  if (rows > 0 && n > 0) {
    b.reads(m.x->stor.native);
    b.reads(m.w->stor.native);
    b.writes(out.native);
    b.must(b.rmsnorm(dev_ptr(*m.x), dev_ptr(*m.w), static_cast<float*>(out.native), n, m.eps, rows, b.stream),
           "executor: rmsnorm");
  }
  tl::detail::graph::store_raw_(root, std::move(out));
  stats().rmsnorm_fused++;
  return true;
}

inline bool run_swiglu(node& root, const swiglu_match& m) {
  auto& b = backend::get();
  if (!b.ready) return false;
  int64_t rows, ff, ldg, rows2, ff2, ldu;
  if (!row_view(*m.g, rows, ff, ldg) || !row_view(*m.u, rows2, ff2, ldu)) return false;
  if (rows != rows2 || ff != ff2 || rows > 65535) return false;
  tl::storage out = tl::storage::make(rows * ff);
  if (!out.native) return false;
  if (rows > 0 && ff > 0) {
    b.reads(m.g->stor.native);
    b.reads(m.u->stor.native);
    b.writes(out.native);
    b.must(b.swiglu_split(dev_ptr(*m.g), ldg, dev_ptr(*m.u), ldu, static_cast<float*>(out.native), ff, rows,
                          b.stream),
           "executor: swiglu");
  }
  tl::detail::graph::store_raw_(root, std::move(out));
  stats().swiglu_fused++;
  return true;
}

// One evaluation batch: the reference's traversal (array.h:1785-1811) with the three device
// routes in front of eval_one.
inline void run_batch(const std::vector<node_ptr>& roots, bool do_flush) {
  thread_local std::vector<node*> order;
  thread_local std::vector<std::pair<node*, size_t>> stack;
  order.clear();
  stack.clear();
  const uint64_t stamp = ++tl::detail::visit_counter;
  for (const auto& root : roots) {
    if (!root || root->evaluated || root->visit_mark == stamp) continue;
    root->visit_mark = stamp;
    stack.emplace_back(root.get(), 0);
    while (!stack.empty()) {
      auto& top = stack.back();
      node* n = top.first;
      if (top.second < n->inputs.size()) {
        node* in = n->inputs[top.second++].get();
        if (!in->evaluated && in->visit_mark != stamp) {
          in->visit_mark = stamp;
          stack.emplace_back(in, 0);
        }
      } else {
        order.push_back(n);
        stack.pop_back();
      }
    }
  }
  const bool device = tl::device_ != tl::device_type::cpu && tl::cuda::available();
  // Pass 1: find the compositions; their interior nodes are never evaluated.
  struct fused {
    node* root;
    int kind;  // 1 rmsnorm, 2 swiglu
    rms_match rm;
    swiglu_match sw;
  };
  std::vector<fused> plan;
  std::vector<node*> skip;
  if (device) {
    for (node* n : order) {
      if (n->op != op_t::mul) continue;
      fused f{n, 0, {}, {}};
      if (match_rmsnorm(*n, f.rm)) f.kind = 1;
      else if (match_swiglu(*n, f.sw)) f.kind = 2;
      if (!f.kind) continue;
      // a composition's interior must not be another batch root
      bool clash = false;
      const auto& inner = f.kind == 1 ? f.rm.interior : f.sw.interior;
      for (const auto& r : roots)
        for (node* i : inner) clash = clash || r.get() == i;
      if (clash) continue;
      for (node* i : inner) skip.push_back(i);
      plan.push_back(std::move(f));
    }
  }
  auto skipped = [&](node* n) {
    for (node* s : skip)
      if (s == n) return true;
    return false;
  };
  auto planned = [&](node* n) -> fused* {
    for (auto& f : plan)
      if (f.root == n) return &f;
    return nullptr;
  };
  // Pass 2: evaluate in order.
  for (node* n : order) {
    if (n->evaluated) continue;
    if (skipped(n)) {
      stats().nodes_fused_away++;
      continue;
    }
    if (device) {
      if (fused* f = planned(n)) {
        const bool done = f->kind == 1 ? run_rmsnorm(*n, f->rm) : run_swiglu(*n, f->sw);
        if (done) continue;
        // the operands were not device rows after all: evaluate the interior the ordinary way
        const auto& inner = f->kind == 1 ? f->rm.interior : f->sw.interior;
        for (auto it = inner.rbegin(); it != inner.rend(); ++it) {
          if (!(*it)->evaluated) {
            tl::detail::graph::eval_one(**it);
            stats().delegated++;
            stats().nodes_fused_away--;
          }
        }
      } else if (n->op == op_t::dot && run_q4_dot(*n)) {
        continue;
      }
    }
    tl::detail::graph::eval_one(*n);
    stats().delegated++;
  }
  if (do_flush) tl::gpu::flush();
}

inline void run_hook_(const std::vector<node_ptr>& roots) { run_batch(roots, true); }
inline void run_noflush_hook_(const std::vector<node_ptr>& roots) { run_batch(roots, false); }

}  // namespace detail_

// Install the reference's storage / barrier / host-sync hooks as tl::install_runtime_hooks()
// does, and this executor as the evaluation hook.
inline void install_executor() {
  tl::install_runtime_hooks();
  tl::detail::run_hook = &detail_::run_hook_;
  tl::detail::run_noflush_hook = &detail_::run_noflush_hook_;
}

#else  // no CUDA build: the reference evaluator as it is

struct executor_stats {
  long q4_dots_on_device = 0, q4_dot_rows = 0, rmsnorm_fused = 0, swiglu_fused = 0, nodes_fused_away = 0,
       delegated = 0, q4_dots_delegated = 0;
};
inline executor_stats& stats() {
  static executor_stats s;
  return s;
}
inline void install_executor() { tl::install_runtime_hooks(); }

#endif

}  // namespace tlb200
}  // namespace tl
