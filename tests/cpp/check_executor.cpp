// Check of the runtime-hook executor (include/tlb200_executor.h) against the reference's own
// CPU evaluation, through the reference's public tl::array API only.  Built with
//   -DTL_RUNTIME_HOOKS -DTENSORLIB_CUDA -I<this repository>/include -I<reference>/include
// so every reference header except gpu.h / cuda.h is the unmodified original.
//
//  1. BASELINE config 4: y = X.dot(Wq) * 0.5f + 1.0f with X [M, 3584] ~ N(0,1), W [3584, 18944]
//     ~ N(0, 0.02) quantised by the reference's own to_q4, M in {1, 8, 64, 512}, evaluated under
//     tl::use_gpu() by the executor: one int4 launch per dot with the epilogue in the kernel
//     (counted), no host dequantisation (the whole evaluation must take less time than the
//     reference's host to_f32 of that weight alone), 1e-4 against
//     X.dot(Wq.to_f32()) * 0.5f + 1.0f under tl::use_cpu().
//  2. The RMSNorm and SwiGLU compositions of include/array.h:2429-2439 are recognised and run
//     as one kernel each (counted), 1e-5 against the CPU evaluation; operands that are views
//     or kept alive elsewhere fall back to the reference evaluator and still give its numbers.
//  3. A block-shaped chain (norm -> q4 dot -> swiglu -> q4 dot) in ONE evaluation batch.
// Prints "ALL OK" and returns 0 on success.
#include <tensorlib.h>
#include <tlb200_executor.h>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

using tl::array;
using clk = std::chrono::steady_clock;

static int g_fail = 0;
#define CHECK(cond, ...)                 \
  do {                                   \
    if (!(cond)) {                       \
      std::printf("FAIL: " __VA_ARGS__); \
      std::printf("\n");                 \
      g_fail++;                          \
    }                                    \
  } while (0)

static array randn(tl::shape_t shape, float std, uint32_t seed) {
  std::mt19937 rng(seed);
  int64_t n = 1;
  for (auto d : shape) n *= d;
  std::vector<float> v((size_t)n);
  // Box-Muller on the raw engine output (std::normal_distribution is implementation-defined)
  for (int64_t i = 0; i < n; i += 2) {
    const double u1 = (rng() + 1.0) / 4294967297.0, u2 = (rng() + 1.0) / 4294967297.0;
    const double r = std::sqrt(-2.0 * std::log(u1));
    v[(size_t)i] = (float)(r * std::cos(6.283185307179586 * u2) * std);
    if (i + 1 < n) v[(size_t)i + 1] = (float)(r * std::sin(6.283185307179586 * u2) * std);
  }
  return array::from(std::move(v), shape);
}

static double max_err(const array& got, const array& want, double rtol_scale) {
  auto g = got.clone(), w = want.clone();
  const float *pg = g.data(), *pw = w.data();
  double worst = 0;
  for (int64_t i = 0; i < g.size(); i++) {
    const double e = std::fabs((double)pg[i] - pw[i]) / (1.0 + rtol_scale * std::fabs((double)pw[i]));
    if (!(e <= worst)) worst = e;  // NaN propagates
  }
  return worst;
}

int main(int argc, char** argv) {
  const bool small = argc > 1 && std::string(argv[1]) == "--small";
  tl::tlb200::install_executor();
  if (!tl::cuda::available()) {
    std::printf("no CUDA device -- the executor only delegates here\n");
  }
  auto& st = tl::tlb200::stats();
  const int64_t K = 3584, N = small ? 1024 : 18944;

  // ---- 1. config 4 -------------------------------------------------------------------
  tl::use_gpu();
  array W = randn({K, N}, 0.02f, 3);
  array Wq = W.to_q4();
  tl::use_cpu();
  array Wd = Wq.to_f32();
  const auto t_dq0 = clk::now();
  array Wd2 = Wq.to_f32();   // timed: what a host dequant of this weight costs
  const double dequant_ms = std::chrono::duration<double, std::milli>(clk::now() - t_dq0).count();
  (void)Wd2;
  const int64_t Ms[] = {1, 8, 64, 512};
  for (int64_t M : Ms) {
    array X = randn({M, K}, 1.0f, 100 + (uint32_t)M);
    tl::use_cpu();
    array want = X.dot(Wd) * 0.5f + 1.0f;
    want.eval();
    tl::use_gpu();
    const long dots0 = st.q4_dots_on_device, deleg0 = st.q4_dots_delegated;
    array warm = X.dot(Wq) * 0.5f + 1.0f;   // first touch uploads the weight
    warm.eval();
    const auto t0 = clk::now();
    array y = X.dot(Wq) * 0.5f + 1.0f;
    y.eval();
    const double ms = std::chrono::duration<double, std::milli>(clk::now() - t0).count();
    const double e = max_err(y, want, 1.0);
    std::printf("config 4  M=%-4lld  err %.2e  eval %.3f ms (host dequant alone: %.0f ms)  device dots %ld\n",
                (long long)M, e, ms, dequant_ms, st.q4_dots_on_device - dots0);
    CHECK(e < 1e-4, "config 4 M=%lld: error %.3e >= 1e-4", (long long)M, e);
    if (tl::cuda::available()) {
      CHECK(st.q4_dots_on_device - dots0 == 2 && st.q4_dots_delegated == deleg0,
            "config 4 M=%lld: the dot did not run on the device", (long long)M);
      CHECK(ms < 0.5 * dequant_ms, "config 4 M=%lld: %.1f ms is not faster than a host dequant (%.1f ms)",
            (long long)M, ms, dequant_ms);
    }
  }

  // ---- 2. compositions ---------------------------------------------------------------
  {
    array x = randn({5, K}, 1.0f, 7), w = randn({K}, 0.02f, 8) + 1.0f;
    w.eval();
    tl::use_cpu();
    array want = array::rmsnorm(x, w, 1e-6f);
    want.eval();
    tl::use_gpu();
    const long f0 = st.rmsnorm_fused;
    array got = array::rmsnorm(x, w, 1e-6f);
    got.eval();
    const double e = max_err(got, want, 1.0);
    std::printf("rmsnorm composition  err %.2e  fused %ld\n", e, st.rmsnorm_fused - f0);
    CHECK(e < 1e-5, "rmsnorm composition: error %.3e", e);
    if (tl::cuda::available()) CHECK(st.rmsnorm_fused - f0 == 1, "rmsnorm composition was not fused");
    // an intermediate that somebody else holds: no fusion, same numbers
    array ms = (x * x).mean(1, true);
    array inv = 1.0f / (ms + 1e-6f).sqrt();
    array got2 = (x * inv) * w;
    const long f1 = st.rmsnorm_fused;
    got2.eval();
    CHECK(st.rmsnorm_fused == f1, "a composition with a shared intermediate must not be fused");
    CHECK(max_err(got2, want, 1.0) < 1e-5, "unfused rmsnorm differs");
    CHECK(inv.size() == 5, "the kept intermediate must still be usable");
  }
  {
    const int64_t FF = small ? 512 : 18944;
    array g = randn({3, FF}, 1.0f, 9), u = randn({3, FF}, 1.0f, 10);
    tl::use_cpu();
    array want = array::swiglu(g, u);
    want.eval();
    tl::use_gpu();
    const long f0 = st.swiglu_fused;
    array got = array::swiglu(g, u);
    got.eval();
    const double e = max_err(got, want, 1.0);
    std::printf("swiglu composition   err %.2e  fused %ld\n", e, st.swiglu_fused - f0);
    CHECK(e < 1e-5, "swiglu composition: error %.3e", e);
    if (tl::cuda::available()) CHECK(st.swiglu_fused - f0 == 1, "swiglu composition was not fused");
  }

  // ---- 3. one batch: norm -> q4 dot -> swiglu -> q4 dot --------------------------------
  {
    const int64_t E = 896, FF = 1024, M = 4;
    array x = randn({M, E}, 1.0f, 20), w = randn({E}, 0.02f, 21) + 1.0f;
    tl::use_gpu();
    array Wg = randn({E, FF}, 0.02f, 22).to_q4(), Wu = randn({E, FF}, 0.02f, 23).to_q4();
    array Wdn = randn({FF, E}, 0.02f, 24).to_q4();
    tl::use_cpu();
    array Wgf = Wg.to_f32(), Wuf = Wu.to_f32(), Wdf = Wdn.to_f32();
    array hc = array::rmsnorm(x, w, 1e-6f);
    array want = array::swiglu(hc.dot(Wgf), hc.dot(Wuf)).dot(Wdf) + x;
    want.eval();
    tl::use_gpu();
    const long d0 = st.q4_dots_on_device, r0 = st.rmsnorm_fused, s0 = st.swiglu_fused;
    array h = array::rmsnorm(x, w, 1e-6f);
    array y = array::swiglu(h.dot(Wg), h.dot(Wu)).dot(Wdn) + x;
    y.eval();
    const double e = max_err(y, want, 1.0);
    std::printf("block chain          err %.2e  dots %ld  rmsnorm %ld  swiglu %ld\n", e,
                st.q4_dots_on_device - d0, st.rmsnorm_fused - r0, st.swiglu_fused - s0);
    CHECK(e < 1e-4, "block chain: error %.3e", e);
    if (tl::cuda::available())
      CHECK(st.q4_dots_on_device - d0 == 3 && st.rmsnorm_fused - r0 == 1 && st.swiglu_fused - s0 == 1,
            "block chain: not every hot op ran on the device");
  }
  std::printf("executor: q4 dots on device %ld (rows %ld), rmsnorm fused %ld, swiglu fused %ld, interior nodes "
              "skipped %ld, delegated %ld, q4 dots delegated %ld\n",
              st.q4_dots_on_device, st.q4_dot_rows, st.rmsnorm_fused, st.swiglu_fused, st.nodes_fused_away,
              st.delegated, st.q4_dots_delegated);
  std::printf(g_fail ? "FAILED (%d)\n" : "ALL OK\n", g_fail);
  return g_fail ? 1 : 0;
}
