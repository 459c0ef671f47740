// Optimizer-side kernels: sharded AdamW, gradient statistics (sum of squares + non-finite flag),
// gradient-shard accumulation, and the cross-entropy row kernels (online log-sum-exp over vocab
// chunks, loss, d-logits).
//
// Reference counterparts: adam_update_kernel (model/optimizer.py:112-151), grad_stats_f16_kernel
// (model/ZeRO3.py:746-796), ChunkedCrossEntropy_Share row math (model/fast_layers.py:1322-1470).
// Differences by design: gradients may arrive as bf16 or fp32, the clip coefficient and the
// skip-on-non-finite decision are taken on the device from the statistics buffer (no host
// round trip between the norm and the update), and everything is 128-bit vectorised.
#include "common.cuh"

namespace b200 {

template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p, size_t i);
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_as_float<bf16>(const bf16* p, size_t i) { return __bfloat162float(p[i]); }

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, m_corr, v_corr;
  float grad_scale;       // host-known multiplier: 1 / (world * accum * loss_scale)
  float max_grad_norm;    // <= 0 disables clipping
};

// stats[0] = sum of squares of the *unscaled* global gradient, stats[1] = non-finite flag.
// When stats is null no clipping / skipping happens on the device.
__device__ __forceinline__ bool adam_prologue(const AdamArgs& a, const float* stats, float& gmul) {
  gmul = a.grad_scale;
  if (stats != nullptr) {
    if (stats[1] != 0.f) return false;   // non-finite gradient somewhere: skip the whole step
    if (a.max_grad_norm > 0.f) {
      const float norm = sqrtf(stats[0]) * a.grad_scale;
      gmul *= fminf(1.f, a.max_grad_norm / (norm + 1e-6f));
    }
  }
  return true;
}

__device__ __forceinline__ void adam_one(float g, float& m, float& v, float& w, const AdamArgs& a) {
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  if (a.weight_decay > 0.f) w *= (1.f - a.lr * a.weight_decay);
  w -= a.lr * (m * a.m_corr) / (sqrtf(v * a.v_corr) + a.eps);
}

template <typename TG>
__global__ void __launch_bounds__(256)
adamw_kernel(const TG* __restrict__ grad, float* __restrict__ m, float* __restrict__ v, float* __restrict__ master,
             bf16* __restrict__ param, size_t n, AdamArgs a, const float* __restrict__ stats, int vec,
             const float* __restrict__ hyper) {
  // hyper = {lr, m_corr, v_corr, grad_scale} in device memory: the step-dependent values of a launch
  // that is replayed from a CUDA graph, where kernel arguments are frozen at capture time
  if (hyper != nullptr) {
    a.lr = hyper[0];
    a.m_corr = hyper[1];
    a.v_corr = hyper[2];
    a.grad_scale = hyper[3];
  }
  float gmul;
  if (!adam_prologue(a, stats, gmul)) return;
  const size_t n4 = vec ? (n >> 2) : 0;   // unaligned shards take the scalar loop for everything
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += size_t(gridDim.x) * blockDim.x) {
    // Streaming accesses throughout: the optimizer touches every byte once and runs beside the next
    // forward pass, whose GEMM operands should stay in L2.
    float g[4];
    if constexpr (sizeof(TG) == 4) {
      const float4 t = __ldcs(reinterpret_cast<const float4*>(grad) + i);
      g[0] = t.x; g[1] = t.y; g[2] = t.z; g[3] = t.w;
    } else {
      const uint2 t = __ldcs(reinterpret_cast<const uint2*>(grad) + i);
      const float2 lo = __bfloat1622float2(*reinterpret_cast<const bf162*>(&t.x));
      const float2 hi = __bfloat1622float2(*reinterpret_cast<const bf162*>(&t.y));
      g[0] = lo.x; g[1] = lo.y; g[2] = hi.x; g[3] = hi.y;
    }
    float4 mm = __ldcs(reinterpret_cast<const float4*>(m) + i);
    float4 vv = __ldcs(reinterpret_cast<const float4*>(v) + i);
    float4 ww = __ldcs(reinterpret_cast<const float4*>(master) + i);
    adam_one(g[0] * gmul, mm.x, vv.x, ww.x, a);
    adam_one(g[1] * gmul, mm.y, vv.y, ww.y, a);
    adam_one(g[2] * gmul, mm.z, vv.z, ww.z, a);
    adam_one(g[3] * gmul, mm.w, vv.w, ww.w, a);
    __stcs(reinterpret_cast<float4*>(m) + i, mm);
    __stcs(reinterpret_cast<float4*>(v) + i, vv);
    __stcs(reinterpret_cast<float4*>(master) + i, ww);
    uint2 o;
    *reinterpret_cast<bf162*>(&o.x) = __floats2bfloat162_rn(ww.x, ww.y);
    *reinterpret_cast<bf162*>(&o.y) = __floats2bfloat162_rn(ww.z, ww.w);
    reinterpret_cast<uint2*>(param)[i] = o;          // the parameters are read again right away: default policy
  }
  {
    for (size_t i = (n4 << 2) + size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += size_t(gridDim.x) * blockDim.x) {
      float mm = m[i], vv = v[i], ww = master[i];
      adam_one(ld_as_float<TG>(grad, i) * gmul, mm, vv, ww, a);
      m[i] = mm; v[i] = vv; master[i] = ww;
      param[i] = __float2bfloat16(ww);
    }
  }
}

// stats[0] += sum over finite g of g^2 ; stats[1] = 1 if any g is NaN/Inf.
template <typename TG>
__global__ void __launch_bounds__(256)
grad_stats_kernel(const TG* __restrict__ g, size_t n, float* __restrict__ stats) {
  float ss = 0.f;
  int bad = 0;
  auto take = [&](float x) {
    if (isfinite(x)) ss += x * x;
    else bad = 1;
  };
  // 16-byte loads over the aligned body, scalar loads for the unaligned head and the tail
  constexpr int PER = 16 / int(sizeof(TG));
  const size_t mis = (reinterpret_cast<uintptr_t>(g) & 15) / sizeof(TG);
  size_t head = mis ? size_t(PER) - mis : 0;
  if (head > n) head = n;
  const size_t nvec = (n - head) / PER;
  const uint4* gv = reinterpret_cast<const uint4*>(g + head);
  const size_t tid = size_t(blockIdx.x) * blockDim.x + threadIdx.x, nthr = size_t(gridDim.x) * blockDim.x;
  size_t i = tid;
  for (; i + 3 * nthr < nvec; i += 4 * nthr) {
    uint4 t[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) t[u] = gv[i + u * nthr];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if constexpr (sizeof(TG) == 4) {
        take(__uint_as_float(t[u].x)); take(__uint_as_float(t[u].y));
        take(__uint_as_float(t[u].z)); take(__uint_as_float(t[u].w));
      } else {
        const bf162* h = reinterpret_cast<const bf162*>(&t[u]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          take(f.x); take(f.y);
        }
      }
    }
  }
  for (; i < nvec; i += nthr) {
    const uint4 t = gv[i];
    if constexpr (sizeof(TG) == 4) {
      take(__uint_as_float(t.x)); take(__uint_as_float(t.y)); take(__uint_as_float(t.z)); take(__uint_as_float(t.w));
    } else {
      const bf162* h = reinterpret_cast<const bf162*>(&t);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        take(f.x); take(f.y);
      }
    }
  }
  for (size_t j = tid; j < head; j += nthr) take(ld_as_float<TG>(g, j));
  for (size_t j = head + nvec * PER + tid; j < n; j += nthr) take(ld_as_float<TG>(g, j));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
    bad |= __shfl_xor_sync(0xffffffffu, bad, o);
  }
  __shared__ float sss[8];
  __shared__ int sbad[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sss[warp] = ss; sbad[warp] = bad; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    int b = 0;
    for (int w = 0; w < int(blockDim.x >> 5); ++w) { t += sss[w]; b |= sbad[w]; }
    atomicAdd(&stats[0], t);
    if (b) stats[1] = 1.f;
  }
}

// acc (fp32) += g (bf16|fp32) * scale   — gradient-shard accumulation across micro-batches.
template <typename TG>
__global__ void accumulate_kernel(float* __restrict__ acc, const TG* __restrict__ g, size_t n, float scale) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x)
    acc[i] += ld_as_float<TG>(g, i) * scale;
}

// ------------------------------------------------------------------ cross-entropy rows
// Online update of (row max, row sum-exp, target logit) with one vocab chunk of fp32 logits
// [M, C] (pitch ld) that covers vocabulary ids [col0, col0 + C). One warp per row.
__global__ void __launch_bounds__(256)
ce_stats_kernel(const float* __restrict__ logits, const int* __restrict__ targets, float* __restrict__ rmax,
                float* __restrict__ rsum, float* __restrict__ tlogit, int M, int C, int ld, int col0, int first) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= M) return;
  const float* lr = logits + size_t(row) * ld;
  float mx = -INFINITY;
  for (int c = lane; c < C; c += 32) mx = fmaxf(mx, lr[c]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const float old_max = first ? -INFINITY : rmax[row];
  const float new_max = fmaxf(old_max, mx);
  float s = 0.f;
  for (int c = lane; c < C; c += 32) s += __expf(lr[c] - new_max);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) {
    const float old_sum = first ? 0.f : rsum[row];
    rsum[row] = old_sum * __expf(old_max - new_max) + s;
    rmax[row] = new_max;
    const int t = targets[row] - col0;
    if (t >= 0 && t < C) tlogit[row] = lr[t];
  }
}

// out[0] = sum over valid rows of (log-sum-exp - target logit), out[1] = number of valid rows.
__global__ void __launch_bounds__(256)
ce_loss_kernel(const float* __restrict__ rmax, const float* __restrict__ rsum, const float* __restrict__ tlogit,
               const int* __restrict__ targets, float* __restrict__ out, int M, int pad_id) {
  float loss = 0.f, cnt = 0.f;
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < M; r += gridDim.x * blockDim.x) {
    const int t = targets[r];
    if (t != pad_id && t >= 0) {
      loss += rmax[r] + __logf(rsum[r]) - tlogit[r];
      cnt += 1.f;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    loss += __shfl_xor_sync(0xffffffffu, loss, o);
    cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(&out[0], loss);
    atomicAdd(&out[1], cnt);
  }
}

// dlogits[r, c] = (softmax - onehot) * valid(r) * gscale / count   as bf16. loss_cnt[1] is the
// valid-row count written by ce_loss_kernel (read on the device: no host sync in between).
__global__ void __launch_bounds__(256)
ce_dlogits_kernel(const float* __restrict__ logits, const int* __restrict__ targets, const float* __restrict__ rmax,
                  const float* __restrict__ rsum, const float* __restrict__ loss_cnt, bf16* __restrict__ dlogits,
                  int M, int C, int ld, int ldd, int col0, int pad_id, float gscale) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= M) return;
  const int t = targets[row];
  const bool valid = (t != pad_id && t >= 0);
  const float scale = valid ? gscale / fmaxf(loss_cnt[1], 1.f) : 0.f;
  const float mx = rmax[row], inv = 1.f / rsum[row];
  const float* lr = logits + size_t(row) * ld;
  bf16* dr = dlogits + size_t(row) * ldd;
  const int tc = t - col0;
  for (int c = lane; c < C; c += 32) {
    float p = __expf(lr[c] - mx) * inv;
    if (c == tc) p -= 1.f;
    dr[c] = __float2bfloat16(p * scale);
  }
}

// Rows of the fused LM-head path. The logits GEMM leaves, per 256-column tile, the row maximum and the sum
// of exp(logit - maximum) ([nt][M]); this kernel merges the nt partials of a row into (rmax, rsum).
__global__ void __launch_bounds__(256)
ce_merge_kernel(const float* __restrict__ pmax, const float* __restrict__ psum, float* __restrict__ rmax,
                float* __restrict__ rsum, int M, int nt) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  float mx = -INFINITY;
  for (int t = 0; t < nt; ++t) mx = fmaxf(mx, pmax[size_t(t) * M + row]);
  float s = 0.f;
  for (int t = 0; t < nt; ++t) s += psum[size_t(t) * M + row] * __expf(pmax[size_t(t) * M + row] - mx);
  rmax[row] = mx;
  rsum[row] = s;
}

// What the logit-gradient epilogue needs per row: lse = rmax + log(rsum) and
// coef = valid(row) * gscale / max(number of valid rows, 1) (the count is read on the device).
__global__ void __launch_bounds__(256)
ce_row_coef_kernel(const float* __restrict__ rmax, const float* __restrict__ rsum, const int* __restrict__ targets,
                   const float* __restrict__ loss_cnt, float* __restrict__ lse, float* __restrict__ coef, int M,
                   int pad_id, float gscale) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  const int t = targets[row];
  lse[row] = rmax[row] + logf(rsum[row]);
  coef[row] = (t != pad_id && t >= 0) ? gscale / fmaxf(loss_cnt[1], 1.f) : 0.f;
}

static inline int grid_cap(size_t items, int block) {
  size_t g = (items + block - 1) / block;
  const size_t cap = size_t(num_sms()) * 8;
  return int(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace b200

using namespace b200;

// Upper bound on the CTAs of one AdamW launch (0 = none). A caller that runs AdamW beside compute
// kernels keeps it to a couple of CTAs per SM so that those kernels still find thread slots.
static int g_adam_max_blocks = 0;

static int adamw_launch(const void* grad, int grad_fp32, void* m, void* v, void* master, void* param, long long n,
                        float lr, float beta1, float beta2, float eps, float weight_decay, float m_corr, float v_corr,
                        float grad_scale, float max_grad_norm, const void* stats, const void* hyper_dev,
                        cudaStream_t st) {
  if (n <= 0) return 0;
  const float* hyper = static_cast<const float*>(hyper_dev);
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, m_corr, v_corr, grad_scale, max_grad_norm};
  int grid = grid_cap(size_t(n) / 4 + 1, 256);
  if (g_adam_max_blocks > 0 && grid > g_adam_max_blocks) grid = g_adam_max_blocks;
  const uintptr_t all = reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(m) |
                        reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(master) |
                        (reinterpret_cast<uintptr_t>(param) << 1);
  const int vec = (all & 15) == 0;
  // AdamW runs beside the next forward's GEMMs (pipelined optimizer): same carve-out as their CTAs
  if (grad_fp32) {
    B200_PREFER_MAX_SMEM(adamw_kernel<float>);
    adamw_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(grad), static_cast<float*>(m),
                                              static_cast<float*>(v), static_cast<float*>(master),
                                              static_cast<bf16*>(param), size_t(n), a,
                                              static_cast<const float*>(stats), vec, hyper);
  } else {
    B200_PREFER_MAX_SMEM(adamw_kernel<bf16>);
    adamw_kernel<bf16><<<grid, 256, 0, st>>>(static_cast<const bf16*>(grad), static_cast<float*>(m),
                                             static_cast<float*>(v), static_cast<float*>(master),
                                             static_cast<bf16*>(param), size_t(n), a,
                                             static_cast<const float*>(stats), vec, hyper);
  }
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_adamw(const void* grad, int grad_fp32, void* m, void* v, void* master, void* param, long long n,
                        float lr, float beta1, float beta2, float eps, float weight_decay, float m_corr, float v_corr,
                        float grad_scale, float max_grad_norm, const void* stats, cudaStream_t st) {
  return adamw_launch(grad, grad_fp32, m, v, master, param, n, lr, beta1, beta2, eps, weight_decay, m_corr, v_corr,
                      grad_scale, max_grad_norm, stats, nullptr, st);
}

B200_API int b200_adamw_max_blocks(int n) {
  const int old = g_adam_max_blocks;
  if (n >= 0) g_adam_max_blocks = n;
  return old;
}

// As b200_adamw, with lr, m_corr, v_corr and grad_scale read from hyper[0..3] in device memory.
B200_API int b200_adamw_dev(const void* grad, int grad_fp32, void* m, void* v, void* master, void* param, long long n,
                            float beta1, float beta2, float eps, float weight_decay, float max_grad_norm,
                            const void* stats, const void* hyper, cudaStream_t st) {
  if (hyper == nullptr) return static_cast<int>(cudaErrorInvalidValue);
  return adamw_launch(grad, grad_fp32, m, v, master, param, n, 0.f, beta1, beta2, eps, weight_decay, 1.f, 1.f, 1.f,
                      max_grad_norm, stats, hyper, st);
}

// Adds into stats[0..1]; the caller zeroes stats once per step.
B200_API int b200_grad_stats(const void* g, int fp32, long long n, void* stats, cudaStream_t st) {
  if (n <= 0) return 0;
  const int grid = grid_cap(size_t(n), 256 * 8);
  if (fp32) grad_stats_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(g), size_t(n),
                                                           static_cast<float*>(stats));
  else grad_stats_kernel<bf16><<<grid, 256, 0, st>>>(static_cast<const bf16*>(g), size_t(n),
                                                     static_cast<float*>(stats));
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_accumulate(void* acc, const void* g, int g_fp32, long long n, float scale, cudaStream_t st) {
  if (n <= 0) return 0;
  const int grid = grid_cap(size_t(n), 256 * 4);
  if (g_fp32) accumulate_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(acc), static_cast<const float*>(g),
                                                             size_t(n), scale);
  else accumulate_kernel<bf16><<<grid, 256, 0, st>>>(static_cast<float*>(acc), static_cast<const bf16*>(g),
                                                     size_t(n), scale);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_ce_stats(const void* logits, const void* targets, void* rmax, void* rsum, void* tlogit, int M, int C,
                           int ld, int col0, int first, cudaStream_t st) {
  if (M <= 0 || C <= 0) return 0;
  ce_stats_kernel<<<(M + 7) / 8, 256, 0, st>>>(static_cast<const float*>(logits), static_cast<const int*>(targets),
                                               static_cast<float*>(rmax), static_cast<float*>(rsum),
                                               static_cast<float*>(tlogit), M, C, ld, col0, first);
  return static_cast<int>(cudaGetLastError());
}

// out (2 floats) must be zeroed by the caller.
B200_API int b200_ce_loss(const void* rmax, const void* rsum, const void* tlogit, const void* targets, void* out,
                          int M, int pad_id, cudaStream_t st) {
  if (M <= 0) return 0;
  int grid = (M + 255) / 256;
  if (grid > 256) grid = 256;
  ce_loss_kernel<<<grid, 256, 0, st>>>(static_cast<const float*>(rmax), static_cast<const float*>(rsum),
                                       static_cast<const float*>(tlogit), static_cast<const int*>(targets),
                                       static_cast<float*>(out), M, pad_id);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_ce_dlogits(const void* logits, const void* targets, const void* rmax, const void* rsum,
                             const void* loss_cnt, void* dlogits, int M, int C, int ld, int ldd, int col0, int pad_id,
                             float gscale, cudaStream_t st) {
  if (M <= 0 || C <= 0) return 0;
  ce_dlogits_kernel<<<(M + 7) / 8, 256, 0, st>>>(static_cast<const float*>(logits), static_cast<const int*>(targets),
                                                 static_cast<const float*>(rmax), static_cast<const float*>(rsum),
                                                 static_cast<const float*>(loss_cnt), static_cast<bf16*>(dlogits), M, C,
                                                 ld, ldd, col0, pad_id, gscale);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_ce_merge(const void* pmax, const void* psum, void* rmax, void* rsum, int M, int nt, cudaStream_t st) {
  if (M <= 0 || nt <= 0) return 0;
  ce_merge_kernel<<<(M + 255) / 256, 256, 0, st>>>(static_cast<const float*>(pmax), static_cast<const float*>(psum),
                                                   static_cast<float*>(rmax), static_cast<float*>(rsum), M, nt);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_ce_row_coef(const void* rmax, const void* rsum, const void* targets, const void* loss_cnt, void* lse,
                              void* coef, int M, int pad_id, float gscale, cudaStream_t st) {
  if (M <= 0) return 0;
  ce_row_coef_kernel<<<(M + 255) / 256, 256, 0, st>>>(static_cast<const float*>(rmax), static_cast<const float*>(rsum),
                                                      static_cast<const int*>(targets),
                                                      static_cast<const float*>(loss_cnt), static_cast<float*>(lse),
                                                      static_cast<float*>(coef), M, pad_id, gscale);
  return static_cast<int>(cudaGetLastError());
}
