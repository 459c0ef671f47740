// Host-side AdamW for the offloaded optimizer tier: fp32 master / m / v in pinned host memory,
// gradient arriving as bf16 or fp32, refreshed parameters leaving as bf16 or fp32. One pass over
// the data, OpenMP across cores, inner loop written so the compiler vectorises it.
// Takes the place of the ~12 single-threaded NumPy passes of the reference
// (model/optimizer.py:74-99).
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define B200_API extern "C" __attribute__((visibility("default")))

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);   // NaN stays NaN
  u += 0x7fffu + ((u >> 16) & 1u);                                                         // round to nearest even
  return static_cast<uint16_t>(u >> 16);
}

B200_API int b200_cpu_adamw(const void* grad, int grad_fp32, float* m, float* v, float* master, void* out,
                            int out_fp32, long long n, float lr, float beta1, float beta2, float eps,
                            float weight_decay, float m_corr, float v_corr, float gmul, int threads) {
  if (n <= 0) return 0;
  const float decay = weight_decay > 0.f ? (1.f - lr * weight_decay) : 1.f;
  const float ombeta1 = 1.f - beta1, ombeta2 = 1.f - beta2;
  const float step = lr * m_corr;
  const long long block = 4096;
  const long long nblocks = (n + block - 1) / block;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#endif
#pragma omp parallel for schedule(static)
  for (long long b = 0; b < nblocks; ++b) {
    const long long lo = b * block;
    const long long hi = lo + block < n ? lo + block : n;
    float g[4096];
    if (grad_fp32) {
      const float* gp = static_cast<const float*>(grad);
      for (long long i = lo; i < hi; ++i) g[i - lo] = gp[i] * gmul;
    } else {
      const uint16_t* gp = static_cast<const uint16_t*>(grad);
      for (long long i = lo; i < hi; ++i) g[i - lo] = bf16_to_f32(gp[i]) * gmul;
    }
    for (long long i = lo; i < hi; ++i) {
      const float gi = g[i - lo];
      const float mi = beta1 * m[i] + ombeta1 * gi;
      const float vi = beta2 * v[i] + ombeta2 * gi * gi;
      float w = master[i] * decay;
      w -= step * mi / (sqrtf(vi * v_corr) + eps);
      m[i] = mi;
      v[i] = vi;
      master[i] = w;
    }
    if (out_fp32) {
      float* op = static_cast<float*>(out);
      for (long long i = lo; i < hi; ++i) op[i] = master[i];
    } else {
      uint16_t* op = static_cast<uint16_t*>(out);
      for (long long i = lo; i < hi; ++i) op[i] = f32_to_bf16(master[i]);
    }
  }
  return 0;
}
