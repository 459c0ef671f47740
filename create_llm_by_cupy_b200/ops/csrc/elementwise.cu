// Bandwidth-bound kernels of the transformer block: RMSNorm (fwd, dx, dgamma), SwiGLU (fwd, bwd),
// rotary embedding, embedding gather / scatter-add, residual add. All are 128-bit vectorised,
// do their arithmetic in fp32 and read every input exactly once.
//
// They take the place of the NVRTC-compiled kernels of the reference:
//   rope_inplace_kernel      model/fast_layers.py:27-61
//   swiglu_fwd/bwd_kernel    model/fast_layers.py:681-704   (those evaluate exp in fp16; fp32 here)
//   rmsnorm_fwd/dgamma/dx    model/fast_layers.py:834-1092  (dgamma there walks columns uncoalesced)
//   TimeEmbedding_shard      model/fast_layers.py:1494-1512
#include "common.cuh"

namespace b200 {

struct alignas(16) Pack8 {
  bf162 v[4];
};

__device__ __forceinline__ void unpack8(const Pack8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ Pack8 pack8(const float (&f)[8]) {
  Pack8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------ RMSNorm forward
// One warp per row; the row stays in registers between the reduction and the scaling pass when
// it fits (H <= 32 * 8 * NV), otherwise it is read a second time (served by L1/L2).
template <int NV>
__global__ void __launch_bounds__(128)
rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gamma, bf16* __restrict__ y,
                   float* __restrict__ rstd, int M, int H, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + warp;
  if (row >= M) return;
  const int nchunk = H >> 3;
  const Pack8* xr = reinterpret_cast<const Pack8*>(x + size_t(row) * H);
  const Pack8* gr = reinterpret_cast<const Pack8*>(gamma);
  Pack8* yr = reinterpret_cast<Pack8*>(y + size_t(row) * H);
  Pack8 cache[NV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + i * 32;
    if (c < nchunk) {
      cache[i] = xr[c];
      float f[8];
      unpack8(cache[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
    }
  }
  for (int c = lane + NV * 32; c < nchunk; c += 32) {
    float f[8];
    unpack8(xr[c], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / float(H) + eps);
  if (lane == 0) rstd[row] = r;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + i * 32;
    if (c < nchunk) {
      float f[8], g[8];
      unpack8(cache[i], f);
      unpack8(gr[c], g);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = f[e] * r * g[e];
      yr[c] = pack8(f);
    }
  }
  for (int c = lane + NV * 32; c < nchunk; c += 32) {
    float f[8], g[8];
    unpack8(xr[c], f);
    unpack8(gr[c], g);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = f[e] * r * g[e];
    yr[c] = pack8(f);
  }
}

// Wide rows (1024 < H <= 8192): the whole CTA works on R rows at a time, every thread owning NV
// 8-column chunks of each; all loads are issued before the first use and the R sums of squares are
// combined with one block-wide exchange per step.
template <int NV, int R>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_cta_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gamma, bf16* __restrict__ y,
                       float* __restrict__ rstd, int M, int H, float eps) {
  __shared__ float sss[2][R][8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nchunk = H >> 3;
  const float inv_h = 1.f / float(H);
  float g[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = tid + i * 256;
    if (c < nchunk) unpack8(reinterpret_cast<const Pack8*>(gamma)[c], g[i]);
  }
  int it = 0;
  for (int row0 = blockIdx.x * R; row0 < M; row0 += gridDim.x * R, ++it) {
    Pack8 px[R][NV];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = row0 + r;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = tid + i * 256;
        if (row < M && c < nchunk) px[r][i] = reinterpret_cast<const Pack8*>(x + size_t(row) * H)[c];
        else px[r][i] = Pack8{};
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        float f[8];
        unpack8(px[r][i], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
      }
      ss = warp_sum(ss);
      if (lane == 0) sss[it & 1][r][warp] = ss;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = row0 + r;
      if (row >= M) continue;
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += sss[it & 1][r][w];
      const float rs = rsqrtf(t * inv_h + eps);
      if (tid == 0) rstd[row] = rs;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = tid + i * 256;
        if (c >= nchunk) continue;
        float f[8];
        unpack8(px[r][i], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = f[e] * rs * g[i][e];
        reinterpret_cast<Pack8*>(y + size_t(row) * H)[c] = pack8(f);
      }
    }
  }
}

// Any H (used when H is not a multiple of 8).
__global__ void rmsnorm_fwd_scalar_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gamma,
                                          bf16* __restrict__ y, float* __restrict__ rstd, int M, int H, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + warp;
  if (row >= M) return;
  const bf16* xr = x + size_t(row) * H;
  float ss = 0.f;
  for (int c = lane; c < H; c += 32) {
    const float f = __bfloat162float(xr[c]);
    ss += f * f;
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / float(H) + eps);
  if (lane == 0) rstd[row] = r;
  for (int c = lane; c < H; c += 32)
    y[size_t(row) * H + c] = __float2bfloat16(__bfloat162float(xr[c]) * r * __bfloat162float(gamma[c]));
}

// ------------------------------------------------------------------ RMSNorm backward
// dx = rstd * (dy*g - xhat * mean(dy*g*xhat)), xhat = x * rstd; optionally dx += add (the
// residual-stream gradient). dgamma partials: every warp walks rows grid-stride and keeps its
// column sums in registers; warps of a CTA are combined in shared memory and each CTA writes one
// row of `partial` [gridDim.x, H] (coalesced), reduced by rmsnorm_dgamma_reduce_kernel.
template <int NV>
__global__ void __launch_bounds__(256, 2)
rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ gamma,
                   const float* __restrict__ rstd, const bf16* __restrict__ add, bf16* __restrict__ dx,
                   float* __restrict__ partial, int M, int H) {
  extern __shared__ float sred[];   // [warps per block][H]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nchunk = H >> 3;
  const Pack8* gr = reinterpret_cast<const Pack8*>(gamma);
  float dg[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) dg[i][e] = 0.f;

  for (int row = blockIdx.x * wpb + warp; row < M; row += gridDim.x * wpb) {
    const Pack8* dyr = reinterpret_cast<const Pack8*>(dy + size_t(row) * H);
    const Pack8* xr = reinterpret_cast<const Pack8*>(x + size_t(row) * H);
    const Pack8* ar = add ? reinterpret_cast<const Pack8*>(add + size_t(row) * H) : nullptr;
    Pack8* dxr = reinterpret_cast<Pack8*>(dx + size_t(row) * H);
    const float r = rstd[row];
    constexpr bool kCache = NV <= 4;   // wider rows are re-read in the second pass (L1/L2 hits)
    float wdy[kCache ? NV : 1][8], xh[kCache ? NV : 1][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + i * 32;
      if (c < nchunk) {
        float d[8], xv[8], g[8];
        unpack8(dyr[c], d);
        unpack8(xr[c], xv);
        unpack8(gr[c], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xhe = xv[e] * r, w = d[e] * g[e];
          if (kCache) { xh[i][e] = xhe; wdy[i][e] = w; }
          dot += w * xhe;
          dg[i][e] += d[e] * xhe;
        }
      }
    }
    dot = warp_sum(dot) / float(H);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + i * 32;
      if (c < nchunk) {
        float o[8];
        if (kCache) {
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = r * (wdy[i][e] - xh[i][e] * dot);
        } else {
          float d[8], xv[8], g[8];
          unpack8(dyr[c], d);
          unpack8(xr[c], xv);
          unpack8(gr[c], g);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = r * (d[e] * g[e] - xv[e] * r * dot);
        }
        if (ar) {
          float a[8];
          unpack8(ar[c], a);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += a[e];
        }
        dxr[c] = pack8(o);
      }
    }
  }
  // combine the warps of this CTA
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + i * 32;
    if (c < nchunk) {
#pragma unroll
      for (int e = 0; e < 8; ++e) sred[warp * H + c * 8 + e] = dg[i][e];
    }
  }
  __syncthreads();
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float t = 0.f;
    for (int w = 0; w < wpb; ++w) t += sred[w * H + h];
    partial[size_t(blockIdx.x) * H + h] = t;
  }
}

// Wide rows (1024 < H <= 8192): the whole CTA works on R rows at a time, every thread owning NV
// fixed 8-column chunks. All loads of the R rows are issued before the first use, the R row dots
// are combined with one block-wide exchange, and each thread's dgamma columns stay in its own
// registers for the whole kernel, so no cross-warp combine is needed at the end.
template <int NV, int R>
__global__ void __launch_bounds__(256, 2)
rmsnorm_bwd_cta_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ gamma,
                       const float* __restrict__ rstd, const bf16* __restrict__ add, bf16* __restrict__ dx,
                       float* __restrict__ partial, int M, int H) {
  __shared__ float sdot[2][R][8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nchunk = H >> 3;
  const float inv_h = 1.f / float(H);
  float g[NV][8], dg[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = tid + i * 256;
    if (c < nchunk) unpack8(reinterpret_cast<const Pack8*>(gamma)[c], g[i]);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      dg[i][e] = 0.f;
      if (c >= nchunk) g[i][e] = 0.f;
    }
  }
  int it = 0;
  for (int row0 = blockIdx.x * R; row0 < M; row0 += gridDim.x * R, ++it) {
    Pack8 pd[R][NV], px[R][NV], pa[R][NV];
    float rs[R], dot[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = row0 + r;
      const bool valid = row < M;
      rs[r] = valid ? rstd[row] : 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = tid + i * 256;
        if (valid && c < nchunk) {
          pd[r][i] = reinterpret_cast<const Pack8*>(dy + size_t(row) * H)[c];
          px[r][i] = reinterpret_cast<const Pack8*>(x + size_t(row) * H)[c];
          if (add) pa[r][i] = reinterpret_cast<const Pack8*>(add + size_t(row) * H)[c];
        } else {
          pd[r][i] = Pack8{};
          px[r][i] = Pack8{};
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        float d[8], xv[8];
        unpack8(pd[r][i], d);
        unpack8(px[r][i], xv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xhe = xv[e] * rs[r];
          acc += d[e] * g[i][e] * xhe;
          dg[i][e] += d[e] * xhe;
        }
      }
      acc = warp_sum(acc);
      if (lane == 0) sdot[it & 1][r][warp] = acc;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += sdot[it & 1][r][w];
      dot[r] = t * inv_h;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = row0 + r;
      if (row >= M) continue;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = tid + i * 256;
        if (c >= nchunk) continue;
        float d[8], xv[8], o[8];
        unpack8(pd[r][i], d);
        unpack8(px[r][i], xv);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rs[r] * (d[e] * g[i][e] - xv[e] * rs[r] * dot[r]);
        if (add) {
          float a[8];
          unpack8(pa[r][i], a);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += a[e];
        }
        reinterpret_cast<Pack8*>(dx + size_t(row) * H)[c] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = tid + i * 256;
    if (c < nchunk) {
      float4* dst = reinterpret_cast<float4*>(partial + size_t(blockIdx.x) * H + size_t(c) * 8);
      dst[0] = make_float4(dg[i][0], dg[i][1], dg[i][2], dg[i][3]);
      dst[1] = make_float4(dg[i][4], dg[i][5], dg[i][6], dg[i][7]);
    }
  }
}

// Generic-H variant: two passes over the row, atomics for dgamma partial rows.
__global__ void rmsnorm_bwd_scalar_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                          const bf16* __restrict__ gamma, const float* __restrict__ rstd,
                                          const bf16* __restrict__ add, bf16* __restrict__ dx,
                                          float* __restrict__ partial, int M, int H) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * 4 + warp; row < M; row += gridDim.x * 4) {
    const float r = rstd[row];
    float dot = 0.f;
    for (int c = lane; c < H; c += 32) {
      const float d = __bfloat162float(dy[size_t(row) * H + c]);
      const float xh = __bfloat162float(x[size_t(row) * H + c]) * r;
      dot += d * __bfloat162float(gamma[c]) * xh;
      atomicAdd(&partial[size_t(blockIdx.x) * H + c], d * xh);
    }
    dot = warp_sum(dot) / float(H);
    for (int c = lane; c < H; c += 32) {
      const float d = __bfloat162float(dy[size_t(row) * H + c]);
      const float xh = __bfloat162float(x[size_t(row) * H + c]) * r;
      float o = r * (d * __bfloat162float(gamma[c]) - xh * dot);
      if (add) o += __bfloat162float(add[size_t(row) * H + c]);
      dx[size_t(row) * H + c] = __float2bfloat16(o);
    }
  }
}

__global__ void __launch_bounds__(256)
rmsnorm_dgamma_reduce_kernel(const float* __restrict__ partial, bf16* __restrict__ dgamma, int nrows, int H,
                             int accumulate) {
  // block = 32 columns x 8 row-groups: coalesced 128-byte reads, rows split over the warps
  __shared__ float red[8][33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int h = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (h < H)
    for (int r = w; r < nrows; r += 8) s += partial[size_t(r) * H + h];
  red[w][lane] = s;
  __syncthreads();
  if (w == 0 && h < H) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i][lane];
    if (accumulate) t += __bfloat162float(dgamma[h]);
    dgamma[h] = __float2bfloat16(t);
  }
}

// ------------------------------------------------------------------ SwiGLU
// gate_val is [M, 2I] with pitch ld: gate = [:, :I], value = [:, I:]. act = silu(gate) * value.
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gv, bf16* __restrict__ act, int M, int I, int ld) {
  const int chunks = I >> 3;
  const size_t total = size_t(M) * chunks;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const int row = int(i / chunks), c = int(i % chunks);
    float g[8], v[8];
    unpack8(*reinterpret_cast<const Pack8*>(gv + size_t(row) * ld + c * 8), g);
    unpack8(*reinterpret_cast<const Pack8*>(gv + size_t(row) * ld + I + c * 8), v);
#pragma unroll
    for (int e = 0; e < 8; ++e) g[e] = g[e] / (1.f + __expf(-g[e])) * v[e];
    *reinterpret_cast<Pack8*>(act + size_t(row) * I + c * 8) = pack8(g);
  }
}
__global__ void swiglu_fwd_scalar_kernel(const bf16* __restrict__ gv, bf16* __restrict__ act, int M, int I, int ld) {
  const size_t total = size_t(M) * I;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const int row = int(i / I), c = int(i % I);
    const float g = __bfloat162float(gv[size_t(row) * ld + c]);
    const float v = __bfloat162float(gv[size_t(row) * ld + I + c]);
    act[i] = __float2bfloat16(g / (1.f + __expf(-g)) * v);
  }
}
// d_gate = dact * value * s * (1 + gate * (1 - s)),  d_value = dact * gate * s,  s = sigmoid(gate)
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ dact, const bf16* __restrict__ gv, bf16* __restrict__ dgv,
                                  int M, int I, int ld) {
  const int chunks = I >> 3;
  const size_t total = size_t(M) * chunks;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const int row = int(i / chunks), c = int(i % chunks);
    float g[8], v[8], d[8], dg[8], dv[8];
    unpack8(*reinterpret_cast<const Pack8*>(gv + size_t(row) * ld + c * 8), g);
    unpack8(*reinterpret_cast<const Pack8*>(gv + size_t(row) * ld + I + c * 8), v);
    unpack8(*reinterpret_cast<const Pack8*>(dact + size_t(row) * I + c * 8), d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float s = 1.f / (1.f + __expf(-g[e]));
      dg[e] = d[e] * v[e] * s * (1.f + g[e] * (1.f - s));
      dv[e] = d[e] * g[e] * s;
    }
    *reinterpret_cast<Pack8*>(dgv + size_t(row) * ld + c * 8) = pack8(dg);
    *reinterpret_cast<Pack8*>(dgv + size_t(row) * ld + I + c * 8) = pack8(dv);
  }
}
__global__ void swiglu_bwd_scalar_kernel(const bf16* __restrict__ dact, const bf16* __restrict__ gv,
                                         bf16* __restrict__ dgv, int M, int I, int ld) {
  const size_t total = size_t(M) * I;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const int row = int(i / I), c = int(i % I);
    const float g = __bfloat162float(gv[size_t(row) * ld + c]);
    const float v = __bfloat162float(gv[size_t(row) * ld + I + c]);
    const float d = __bfloat162float(dact[i]);
    const float s = 1.f / (1.f + __expf(-g));
    dgv[size_t(row) * ld + c] = __float2bfloat16(d * v * s * (1.f + g * (1.f - s)));
    dgv[size_t(row) * ld + I + c] = __float2bfloat16(d * g * s);
  }
}

// ------------------------------------------------------------------ rotary embedding
// cos/sin table [T, D/2] fp32 with freq_j = base^(-2j/D).
__global__ void rope_table_kernel(float* __restrict__ cs, float* __restrict__ sn, int T, int half, float base) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * half) return;
  const int t = i / half, j = i % half;
  const float freq = powf(base, -float(2 * j) / float(2 * half));
  float s, c;
  sincosf(float(t) * freq, &s, &c);
  cs[i] = c;
  sn[i] = s;
}
// In place on `nheads` heads of width D that start at column col0 of a [M, ld] buffer; token m
// has position pos0 + (m % T). Half-split pairing (j, j + D/2). sign = +1 rotates, -1 un-rotates.
__global__ void rope_inplace_kernel(bf16* __restrict__ buf, const float* __restrict__ cs, const float* __restrict__ sn,
                                    int M, int T, int nheads, int D, int ld, int col0, int pos0, float sign) {
  const int half = D >> 1;
  const size_t total = size_t(M) * nheads * half;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const int j = int(i % half);
    const int h = int((i / half) % nheads);
    const int m = int(i / (size_t(half) * nheads));
    const int pos = pos0 + (m % T);
    bf16* p = buf + size_t(m) * ld + col0 + h * D + j;
    const float x1 = __bfloat162float(p[0]), x2 = __bfloat162float(p[half]);
    const float c = cs[size_t(pos) * half + j], s = sn[size_t(pos) * half + j] * sign;
    p[0] = __float2bfloat16(x1 * c - x2 * s);
    p[half] = __float2bfloat16(x2 * c + x1 * s);
  }
}

// 128-bit version: one thread rotates 8 pairs (two 16-byte chunks). Needs D/2 % 8 == 0 and 16-byte
// aligned rows / column offset.
__global__ void rope_inplace_vec_kernel(bf16* __restrict__ buf, const float* __restrict__ cs,
                                        const float* __restrict__ sn, int M, int T, int nheads, int D, int ld, int col0,
                                        int pos0, float sign) {
  const int half = D >> 1;
  const int cph = half >> 3;                        // 8-element chunks per half head
  const size_t total = size_t(M) * nheads * cph;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const int jc = int(i % cph);
    const int h = int((i / cph) % nheads);
    const int m = int(i / (size_t(cph) * nheads));
    const int pos = pos0 + (m % T);
    bf16* p = buf + size_t(m) * ld + col0 + h * D + jc * 8;
    Pack8 a = *reinterpret_cast<const Pack8*>(p);
    Pack8 b = *reinterpret_cast<const Pack8*>(p + half);
    const float4* c4 = reinterpret_cast<const float4*>(cs + size_t(pos) * half + jc * 8);
    const float4* s4 = reinterpret_cast<const float4*>(sn + size_t(pos) * half + jc * 8);
    const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    float x1[8], x2[8], y1[8], y2[8];
    unpack8(a, x1);
    unpack8(b, x2);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = sv[e] * sign;
      y1[e] = x1[e] * c[e] - x2[e] * sg;
      y2[e] = x2[e] * c[e] + x1[e] * sg;
    }
    *reinterpret_cast<Pack8*>(p) = pack8(y1);
    *reinterpret_cast<Pack8*>(p + half) = pack8(y2);
  }
}

// ------------------------------------------------------------------ embedding
// An id outside [0, V) never touches W: the row is written as zeros (forward) or skipped (backward) and
// the status word gets error 4 with the kernel id 401 / 402, which the host raises on its next check.
__device__ __forceinline__ void embedding_bad_id(int* status, int kid) {
  if (status != nullptr && atomicCAS(status, 0, 4) == 0) status[1] = kid;
}

__global__ void embedding_fwd_kernel(const bf16* __restrict__ W, const int* __restrict__ idx, bf16* __restrict__ out,
                                     int M, int H, int pad_id, int V, int* status) {
  const int chunks = H >> 3;
  const size_t total = size_t(M) * chunks;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const int row = int(i / chunks), c = int(i % chunks);
    const int id = idx[row];
    Pack8 v;
    if (id >= V && c == 0) embedding_bad_id(status, 401);
    if (id == pad_id || id < 0 || id >= V) {
#pragma unroll
      for (int e = 0; e < 4; ++e) v.v[e] = __floats2bfloat162_rn(0.f, 0.f);
    } else {
      v = *reinterpret_cast<const Pack8*>(W + size_t(id) * H + c * 8);
    }
    *reinterpret_cast<Pack8*>(out + size_t(row) * H + c * 8) = v;
  }
}
__global__ void embedding_fwd_scalar_kernel(const bf16* __restrict__ W, const int* __restrict__ idx,
                                            bf16* __restrict__ out, int M, int H, int pad_id, int V, int* status) {
  const size_t total = size_t(M) * H;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const int row = int(i / H), c = int(i % H);
    const int id = idx[row];
    if (id >= V && c == 0) embedding_bad_id(status, 401);
    out[i] = (id == pad_id || id < 0 || id >= V) ? __float2bfloat16(0.f) : W[size_t(id) * H + c];
  }
}
// dW[idx[m], :] += dout[m, :] for idx != pad. dW is bf16 (packed atomics) or fp32.
template <typename TW>
__global__ void embedding_bwd_kernel(TW* __restrict__ dW, const int* __restrict__ idx, const bf16* __restrict__ dout,
                                     int M, int H, int pad_id, int V, int* status) {
  const int pairs = H >> 1;
  const size_t total = size_t(M) * pairs;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const int row = int(i / pairs), c = int(i % pairs);
    const int id = idx[row];
    if (id >= V) {
      if (c == 0) embedding_bad_id(status, 402);
      continue;
    }
    if (id == pad_id || id < 0) continue;
    const bf162 d = *reinterpret_cast<const bf162*>(dout + size_t(row) * H + 2 * c);
    if constexpr (sizeof(TW) == 2) {
      atomicAdd(reinterpret_cast<bf162*>(dW + size_t(id) * H + 2 * c), d);
    } else {
      const float2 f = __bfloat1622float2(d);
      atomicAdd(reinterpret_cast<float*>(dW) + size_t(id) * H + 2 * c, f.x);
      atomicAdd(reinterpret_cast<float*>(dW) + size_t(id) * H + 2 * c + 1, f.y);
    }
  }
}

// out = a + b (bf16, n multiple of 8 handled vectorised; tail scalar)
__global__ void add_bf16_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ out,
                                size_t n) {
  const size_t chunks = n >> 3;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < chunks; i += size_t(gridDim.x) * blockDim.x) {
    float x[8], y[8];
    unpack8(reinterpret_cast<const Pack8*>(a)[i], x);
    unpack8(reinterpret_cast<const Pack8*>(b)[i], y);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] += y[e];
    reinterpret_cast<Pack8*>(out)[i] = pack8(x);
  }
  if (blockIdx.x == 0)
    for (size_t i = (chunks << 3) + threadIdx.x; i < n; i += blockDim.x)
      out[i] = __float2bfloat16(__bfloat162float(a[i]) + __bfloat162float(b[i]));
}

static inline int grid_for(size_t work_items, int block) {
  size_t g = (work_items + block - 1) / block;
  const size_t cap = size_t(num_sms()) * 16;
  return int(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace b200

using namespace b200;

B200_API int b200_rmsnorm_fwd(const void* x, const void* gamma, void* y, void* rstd, int M, int H, float eps,
                              cudaStream_t st) {
  if (M <= 0) return 0;
  const dim3 grid((M + 3) / 4), block(128);
  const bf16* xp = static_cast<const bf16*>(x);
  const bf16* gp = static_cast<const bf16*>(gamma);
  bf16* yp = static_cast<bf16*>(y);
  float* rp = static_cast<float*>(rstd);
  if (H % 8 != 0) {
    rmsnorm_fwd_scalar_kernel<<<grid, block, 0, st>>>(xp, gp, yp, rp, M, H, eps);
  } else if (H <= 256) {
    rmsnorm_fwd_kernel<1><<<grid, block, 0, st>>>(xp, gp, yp, rp, M, H, eps);
  } else if (H <= 1024) {
    rmsnorm_fwd_kernel<4><<<grid, block, 0, st>>>(xp, gp, yp, rp, M, H, eps);
  } else if (H <= 8192) {
    const int cap = num_sms() * 4;
    if (H <= 2048) {
      const int ctas = min((M + 3) / 4, cap);
      rmsnorm_fwd_cta_kernel<1, 4><<<ctas, 256, 0, st>>>(xp, gp, yp, rp, M, H, eps);
    } else if (H <= 4096) {
      const int ctas = min((M + 1) / 2, cap);
      rmsnorm_fwd_cta_kernel<2, 2><<<ctas, 256, 0, st>>>(xp, gp, yp, rp, M, H, eps);
    } else {
      rmsnorm_fwd_cta_kernel<4, 1><<<min(M, cap), 256, 0, st>>>(xp, gp, yp, rp, M, H, eps);
    }
  } else {
    rmsnorm_fwd_kernel<16><<<grid, block, 0, st>>>(xp, gp, yp, rp, M, H, eps);
  }
  return static_cast<int>(cudaGetLastError());
}

// Number of partial rows rmsnorm_bwd writes; the caller provides `partial` of [that, H] fp32.
B200_API int b200_rmsnorm_bwd_partial_rows(int M) {
  int g = (M + 7) / 8;
  const int cap = num_sms() * 2;
  return g < cap ? (g < 1 ? 1 : g) : cap;
}

B200_API int b200_rmsnorm_bwd(const void* dy, const void* x, const void* gamma, const void* rstd, const void* add,
                              void* dx, void* dgamma, void* partial, int M, int H, int accumulate_dgamma,
                              cudaStream_t st) {
  if (M <= 0) return 0;
  const int rows = b200_rmsnorm_bwd_partial_rows(M);
  const bf16* dyp = static_cast<const bf16*>(dy);
  const bf16* xp = static_cast<const bf16*>(x);
  const bf16* gp = static_cast<const bf16*>(gamma);
  const float* rp = static_cast<const float*>(rstd);
  const bf16* ap = static_cast<const bf16*>(add);
  bf16* dxp = static_cast<bf16*>(dx);
  float* pp = static_cast<float*>(partial);
  const size_t smem = size_t(8) * H * sizeof(float);   // 8 warps per CTA in the vector kernels
  if (H % 8 != 0 || H > 8192) {
    B200_CHECK(cudaMemsetAsync(pp, 0, size_t(rows) * H * sizeof(float), st));
    rmsnorm_bwd_scalar_kernel<<<rows, 128, 0, st>>>(dyp, xp, gp, rp, ap, dxp, pp, M, H);
  } else if (H <= 256) {
    rmsnorm_bwd_kernel<1><<<rows, 256, smem, st>>>(dyp, xp, gp, rp, ap, dxp, pp, M, H);
  } else if (H <= 1024) {
    rmsnorm_bwd_kernel<4><<<rows, 256, smem, st>>>(dyp, xp, gp, rp, ap, dxp, pp, M, H);
  } else if (H <= 2048) {
    rmsnorm_bwd_cta_kernel<1, 4><<<rows, 256, 0, st>>>(dyp, xp, gp, rp, ap, dxp, pp, M, H);
  } else if (H <= 4096) {
    rmsnorm_bwd_cta_kernel<2, 2><<<rows, 256, 0, st>>>(dyp, xp, gp, rp, ap, dxp, pp, M, H);
  } else {
    rmsnorm_bwd_cta_kernel<4, 1><<<rows, 256, 0, st>>>(dyp, xp, gp, rp, ap, dxp, pp, M, H);
  }
  B200_CHECK(cudaGetLastError());
  rmsnorm_dgamma_reduce_kernel<<<(H + 31) / 32, 256, 0, st>>>(pp, static_cast<bf16*>(dgamma), rows, H,
                                                                 accumulate_dgamma);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_swiglu_fwd(const void* gate_val, void* act, int M, int I, int ld, cudaStream_t st) {
  if (M <= 0 || I <= 0) return 0;
  const bf16* g = static_cast<const bf16*>(gate_val);
  const bool vec = (I % 8 == 0) && (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(g) & 15) == 0);
  if (vec) swiglu_fwd_kernel<<<grid_for(size_t(M) * (I / 8), 256), 256, 0, st>>>(g, static_cast<bf16*>(act), M, I, ld);
  else swiglu_fwd_scalar_kernel<<<grid_for(size_t(M) * I, 256), 256, 0, st>>>(g, static_cast<bf16*>(act), M, I, ld);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_swiglu_bwd(const void* dact, const void* gate_val, void* d_gate_val, int M, int I, int ld,
                             cudaStream_t st) {
  if (M <= 0 || I <= 0) return 0;
  const bf16* g = static_cast<const bf16*>(gate_val);
  const bool vec = (I % 8 == 0) && (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(g) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(d_gate_val) & 15) == 0);
  if (vec)
    swiglu_bwd_kernel<<<grid_for(size_t(M) * (I / 8), 256), 256, 0, st>>>(static_cast<const bf16*>(dact), g,
                                                                           static_cast<bf16*>(d_gate_val), M, I, ld);
  else
    swiglu_bwd_scalar_kernel<<<grid_for(size_t(M) * I, 256), 256, 0, st>>>(static_cast<const bf16*>(dact), g,
                                                                            static_cast<bf16*>(d_gate_val), M, I, ld);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_rope_table(void* cs, void* sn, int T, int D, float base, cudaStream_t st) {
  const int half = D / 2;
  const int n = T * half;
  if (n <= 0) return 0;
  rope_table_kernel<<<(n + 255) / 256, 256, 0, st>>>(static_cast<float*>(cs), static_cast<float*>(sn), T, half, base);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_rope_inplace(void* buf, const void* cs, const void* sn, int M, int T, int nheads, int D, int ld,
                               int col0, int pos0, int inverse, cudaStream_t st) {
  const size_t total = size_t(M) * nheads * (D / 2);
  if (total == 0) return 0;
  const bool vec = ((D / 2) % 8 == 0) && (ld % 8 == 0) && (col0 % 8 == 0) &&
                   ((reinterpret_cast<uintptr_t>(buf) & 15) == 0);
  if (vec)
    rope_inplace_vec_kernel<<<grid_for(total / 8, 256), 256, 0, st>>>(
        static_cast<bf16*>(buf), static_cast<const float*>(cs), static_cast<const float*>(sn), M, T, nheads, D, ld,
        col0, pos0, inverse ? -1.f : 1.f);
  else
    rope_inplace_kernel<<<grid_for(total, 256), 256, 0, st>>>(static_cast<bf16*>(buf), static_cast<const float*>(cs),
                                                              static_cast<const float*>(sn), M, T, nheads, D, ld, col0,
                                                              pos0, inverse ? -1.f : 1.f);
  return static_cast<int>(cudaGetLastError());
}

// V: rows of W (vocabulary size).
B200_API int b200_embedding_fwd(const void* W, const void* idx, void* out, int M, int H, int pad_id, int V,
                                cudaStream_t st) {
  if (M <= 0) return 0;
  if (H % 8 == 0)
    embedding_fwd_kernel<<<grid_for(size_t(M) * (H / 8), 256), 256, 0, st>>>(
        static_cast<const bf16*>(W), static_cast<const int*>(idx), static_cast<bf16*>(out), M, H, pad_id, V,
        status_ptr());
  else
    embedding_fwd_scalar_kernel<<<grid_for(size_t(M) * H, 256), 256, 0, st>>>(
        static_cast<const bf16*>(W), static_cast<const int*>(idx), static_cast<bf16*>(out), M, H, pad_id, V,
        status_ptr());
  return static_cast<int>(cudaGetLastError());
}

// H must be even. dw_fp32 selects the dtype of dW.
B200_API int b200_embedding_bwd(void* dW, const void* idx, const void* dout, int M, int H, int pad_id, int V,
                                int dw_fp32, cudaStream_t st) {
  if (M <= 0) return 0;
  if (H % 2 != 0) return static_cast<int>(cudaErrorInvalidValue);
  const int grid = grid_for(size_t(M) * (H / 2), 256);
  if (dw_fp32)
    embedding_bwd_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(dW), static_cast<const int*>(idx),
                                                      static_cast<const bf16*>(dout), M, H, pad_id, V,
                                                      status_ptr());
  else
    embedding_bwd_kernel<bf16><<<grid, 256, 0, st>>>(static_cast<bf16*>(dW), static_cast<const int*>(idx),
                                                     static_cast<const bf16*>(dout), M, H, pad_id, V,
                                                     status_ptr());
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  add_bf16_kernel<<<grid_for(size_t(n) / 8 + 1, 256), 256, 0, st>>>(static_cast<const bf16*>(a),
                                                                    static_cast<const bf16*>(b),
                                                                    static_cast<bf16*>(out), size_t(n));
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ dropout with a bit-packed mask
// Inverted dropout (model/fast_layers.py:616-673 of the reference keeps the mask as packed bits too). The keep
// decision of element i is a pure function of (seed, i): a 64-bit mix of the seed and i / 4 yields four 16-bit
// lanes, element i keeps when its lane >= round(p * 65536). Eight consecutive elements share one mask byte,
// first element in the most significant bit (the order of numpy.packbits). The forward writes the mask bytes,
// the backward only reads them: nothing of the size of the activations is kept besides one bit per element.
__device__ __forceinline__ unsigned long long drop_mix(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <typename T>
__global__ void __launch_bounds__(256)
dropout_fwd_kernel(const T* __restrict__ x, T* __restrict__ out, uint8_t* __restrict__ mask, size_t n,
                   unsigned long long seed, unsigned long long offset, unsigned int threshold, float scale) {
  const size_t nbytes = (n + 7) / 8;
  for (size_t b = size_t(blockIdx.x) * blockDim.x + threadIdx.x; b < nbytes; b += size_t(gridDim.x) * blockDim.x) {
    const size_t i0 = b * 8;
    const unsigned long long r0 = drop_mix(seed ^ ((offset + i0) >> 2) * 0xD1342543DE82EF95ull);
    const unsigned long long r1 = drop_mix(seed ^ (((offset + i0) >> 2) + 1) * 0xD1342543DE82EF95ull);
    unsigned int bits = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const unsigned int lane = unsigned((j < 4 ? r0 >> (16 * j) : r1 >> (16 * (j - 4))) & 0xffffull);
      const bool keep = lane >= threshold;
      if (i0 + j < n) {
        bits |= (keep ? 1u : 0u) << (7 - j);
        out[i0 + j] = keep ? T(float(x[i0 + j]) * scale) : T(0.f);
      }
    }
    mask[b] = uint8_t(bits);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
dropout_bwd_kernel(const T* __restrict__ dout, const uint8_t* __restrict__ mask, T* __restrict__ out, size_t n,
                   float scale) {
  const size_t nbytes = (n + 7) / 8;
  for (size_t b = size_t(blockIdx.x) * blockDim.x + threadIdx.x; b < nbytes; b += size_t(gridDim.x) * blockDim.x) {
    const unsigned int bits = mask[b];
    const size_t i0 = b * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (i0 + j < n) out[i0 + j] = ((bits >> (7 - j)) & 1u) ? T(float(dout[i0 + j]) * scale) : T(0.f);
  }
}

// x, out: n elements of bf16 (is_f32 == 0) or fp32; mask: (n + 7) / 8 bytes; offset must be a multiple of 8 (the
// caller advances it by the padded element count of every call, so no two calls share random lanes).
B200_API int b200_dropout_fwd(const void* x, void* out, void* mask, long long n, int is_f32, unsigned long long seed,
                              unsigned long long offset, float p, cudaStream_t st) {
  if (n <= 0) return 0;
  if (!(p >= 0.f && p < 1.f) || (offset & 7ull) != 0) return static_cast<int>(cudaErrorInvalidValue);
  const unsigned int thr = static_cast<unsigned int>(p * 65536.f + 0.5f);
  const float scale = 1.f / (1.f - p);
  const int grid = grid_for(size_t(n + 7) / 8, 256);
  if (is_f32)
    dropout_fwd_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(out),
                                                    static_cast<uint8_t*>(mask), size_t(n), seed, offset, thr, scale);
  else
    dropout_fwd_kernel<bf16><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), static_cast<bf16*>(out),
                                                   static_cast<uint8_t*>(mask), size_t(n), seed, offset, thr, scale);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_dropout_bwd(const void* dout, const void* mask, void* out, long long n, int is_f32, float p,
                              cudaStream_t st) {
  if (n <= 0) return 0;
  if (!(p >= 0.f && p < 1.f)) return static_cast<int>(cudaErrorInvalidValue);
  const float scale = 1.f / (1.f - p);
  const int grid = grid_for(size_t(n + 7) / 8, 256);
  if (is_f32)
    dropout_bwd_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(dout), static_cast<const uint8_t*>(mask),
                                                    static_cast<float*>(out), size_t(n), scale);
  else
    dropout_bwd_kernel<bf16><<<grid, 256, 0, st>>>(static_cast<const bf16*>(dout), static_cast<const uint8_t*>(mask),
                                                   static_cast<bf16*>(out), size_t(n), scale);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ allocation-free RMSNorm backward
// See b200_noalloc.h. The scratch for the dgamma partial sums lives in this translation unit; in
// host code the array's name only stands for the symbol, so its device address is looked up once
// per device and that pointer is what the kernels receive.
#include "b200_noalloc.h"

static __device__ __align__(256) float g_noalloc_rms_partial[B200_NOALLOC_RMS_ROWS * B200_NOALLOC_RMS_MAX_H];

static int noalloc_rms_scratch(float** out) {
  static float* per_device[64] = {nullptr};
  int dev = 0;
  B200_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return static_cast<int>(cudaErrorInvalidDevice);
  if (per_device[dev] == nullptr) {
    float* p = nullptr;
    B200_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_rms_partial));
    per_device[dev] = p;
  }
  *out = per_device[dev];
  return 0;
}

B200_API int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const void* rstd,
                                      const void* add, void* dx, void* dgamma, int M, int H, int accumulate_dgamma,
                                      cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H <= 0 || H > B200_NOALLOC_RMS_MAX_H) {
    fprintf(stderr, "[b200] rmsnorm_bwd_noalloc: hidden size %d is outside 1..%d, the size its built-in scratch "
                    "was compiled for; use b200_rmsnorm_bwd with your own scratch\n", H, B200_NOALLOC_RMS_MAX_H);
    return static_cast<int>(cudaErrorInvalidValue);
  }
  const int rows = b200_rmsnorm_bwd_partial_rows(M);
  if (rows > B200_NOALLOC_RMS_ROWS) {
    fprintf(stderr, "[b200] rmsnorm_bwd_noalloc: %d partial rows needed, built-in scratch holds %d\n", rows,
            B200_NOALLOC_RMS_ROWS);
    return static_cast<int>(cudaErrorInvalidValue);
  }
  float* scratch = nullptr;
  const int rc = noalloc_rms_scratch(&scratch);
  if (rc != 0) return rc;
  // Every partial row the kernels read is fully rewritten first (vector path) or zeroed with a
  // memset on `stream` (generic-H path), so stale contents of an earlier call are never summed.
  return b200_rmsnorm_bwd(dy, x, gamma, rstd, add, dx, dgamma, scratch, M, H, accumulate_dgamma, stream);
}
