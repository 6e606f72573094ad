// CPU optimizer kernels for optimizer-state offloading: multi-threaded (std::thread), vectorised
// by the compiler for AVX-512 / AVX2 / baseline through function multi-versioning, so one
// binary runs on the build host and on the GPU box.
//
//   prb_cpu_adamw_step     fp32 master / moments, fp32 or bf16 gradient (read-only, scaled),
//                          optional bf16 or fp32 "compute" copy written in the same pass
//   prb_cpu_sign_sgd_step  p = p * (1 - lr wd) - lr sign(g), sign(0) = 0
//   prb_cpu_bf16_to_fp32   dst = src or dst += src (gradient accumulation on the host)
//
// Same update rules as the reference's C++ extension
// (src/prime_rl/trainer/optim/cpu_adam/kernel.cpp:58-483); written against raw pointers and a
// C ABI instead of ATen.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <algorithm>
#include <cstdlib>
#include <thread>
#include <vector>

#define PRB_API extern "C" __attribute__((visibility("default")))
#define PRB_CLONES __attribute__((target_clones("avx512f", "avx2", "default")))

namespace {

inline float bf16_to_f32(uint16_t v) {
  uint32_t u = static_cast<uint32_t>(v) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // NaN
  u += 0x7fffu + ((u >> 16) & 1u);  // round to nearest even
  return static_cast<uint16_t>(u >> 16);
}

constexpr long long kGrain = 32 * 1024;

// Static partition of [0, chunks) over worker threads (PRB_CPU_THREADS overrides the count).
template <class F>
void parallel_chunks(long long chunks, F&& fn) {
  unsigned hw = std::thread::hardware_concurrency();
  if (const char* e = std::getenv("PRB_CPU_THREADS")) hw = static_cast<unsigned>(std::max(1, std::atoi(e)));
  const long long nt = std::max<long long>(1, std::min<long long>(hw ? hw : 1, chunks));
  if (nt == 1) {
    for (long long c = 0; c < chunks; ++c) fn(c);
    return;
  }
  std::vector<std::thread> workers;
  workers.reserve(nt - 1);
  auto run = [&](long long t) {
    const long long lo = chunks * t / nt, hi = chunks * (t + 1) / nt;
    for (long long c = lo; c < hi; ++c) fn(c);
  };
  for (long long t = 1; t < nt; ++t) workers.emplace_back(run, t);
  run(0);
  for (auto& w : workers) w.join();
}

PRB_CLONES void adamw_span(float* p, float* m, float* v, const float* g32, const uint16_t* g16, uint16_t* out16,
                           float* out32, long long n, float lr, float b1, float b2, float eps, float wd, float bc1,
                           float bc2_sqrt, float gscale) {
  const float decay = 1.f - lr * wd;
  const float step = lr / bc1;
  for (long long i = 0; i < n; ++i) {
    const float g = (g32 ? g32[i] : bf16_to_f32(g16[i])) * gscale;
    const float mi = b1 * m[i] + (1.f - b1) * g;
    const float vi = b2 * v[i] + (1.f - b2) * g * g;
    const float pi = p[i] * decay - step * mi / (std::sqrt(vi) / bc2_sqrt + eps);
    m[i] = mi;
    v[i] = vi;
    p[i] = pi;
    if (out16) out16[i] = f32_to_bf16(pi);
    if (out32) out32[i] = pi;
  }
}

PRB_CLONES void sign_sgd_span(float* p, const float* g32, const uint16_t* g16, uint16_t* out16, float* out32,
                              long long n, float lr, float wd, float gscale) {
  for (long long i = 0; i < n; ++i) {
    const float g = (g32 ? g32[i] : bf16_to_f32(g16[i])) * gscale;
    const float s = (g > 0.f) - (g < 0.f);
    const float pi = p[i] + p[i] * (-lr * wd) + s * (-lr);
    p[i] = pi;
    if (out16) out16[i] = f32_to_bf16(pi);
    if (out32) out32[i] = pi;
  }
}

PRB_CLONES void bf16_span(float* dst, const uint16_t* src, long long n, int accumulate) {
  if (accumulate)
    for (long long i = 0; i < n; ++i) dst[i] += bf16_to_f32(src[i]);
  else
    for (long long i = 0; i < n; ++i) dst[i] = bf16_to_f32(src[i]);
}

}  // namespace

// step is 1-based. grad_is_bf16 selects how `grad` is read. out_param may be null;
// out_is_bf16 selects its type. Returns 0.
PRB_API int prb_cpu_adamw_step(float* p, float* m, float* v, const void* grad, int grad_is_bf16, void* out_param,
                               int out_is_bf16, long long n, int step, float lr, float b1, float b2, float eps,
                               float wd, float grad_scale) {
  const float bc1 = 1.f - std::pow(b1, static_cast<float>(step));
  const float bc2_sqrt = std::sqrt(1.f - std::pow(b2, static_cast<float>(step)));
  const long long chunks = (n + kGrain - 1) / kGrain;
  parallel_chunks(chunks, [&](long long c) {
    const long long o = c * kGrain;
    const long long len = (o + kGrain <= n) ? kGrain : n - o;
    adamw_span(p + o, m + o, v + o, grad_is_bf16 ? nullptr : static_cast<const float*>(grad) + o,
               grad_is_bf16 ? static_cast<const uint16_t*>(grad) + o : nullptr,
               (out_param && out_is_bf16) ? static_cast<uint16_t*>(out_param) + o : nullptr,
               (out_param && !out_is_bf16) ? static_cast<float*>(out_param) + o : nullptr, len, lr, b1, b2, eps, wd,
               bc1, bc2_sqrt, grad_scale);
  });
  return 0;
}

PRB_API int prb_cpu_sign_sgd_step(float* p, const void* grad, int grad_is_bf16, void* out_param, int out_is_bf16,
                                  long long n, float lr, float wd, float grad_scale) {
  const long long chunks = (n + kGrain - 1) / kGrain;
  parallel_chunks(chunks, [&](long long c) {
    const long long o = c * kGrain;
    const long long len = (o + kGrain <= n) ? kGrain : n - o;
    sign_sgd_span(p + o, grad_is_bf16 ? nullptr : static_cast<const float*>(grad) + o,
                  grad_is_bf16 ? static_cast<const uint16_t*>(grad) + o : nullptr,
                  (out_param && out_is_bf16) ? static_cast<uint16_t*>(out_param) + o : nullptr,
                  (out_param && !out_is_bf16) ? static_cast<float*>(out_param) + o : nullptr, len, lr, wd, grad_scale);
  });
  return 0;
}

PRB_API int prb_cpu_bf16_to_fp32(float* dst, const void* src, long long n, int accumulate) {
  const long long chunks = (n + kGrain - 1) / kGrain;
  parallel_chunks(chunks, [&](long long c) {
    const long long o = c * kGrain;
    const long long len = (o + kGrain <= n) ? kGrain : n - o;
    bf16_span(dst + o, static_cast<const uint16_t*>(src) + o, len, accumulate);
  });
  return 0;
}
