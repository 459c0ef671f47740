// Causal GQA flash-attention forward on tcgen05, second generation (head_dim 128).
//
// Same data flow as flash_attn_tc.cu (TMA ring for K/V, S = Q K^T and PV = P V on the tensor core,
// P handed to the second MMA through TMEM) but the softmax work of every 128 x 128 score tile is
// shared by TWO warpgroups: warpgroup A owns key columns 0..63 and output columns 0..63 of each
// query row, warpgroup B the other halves. A thread therefore keeps 64 scores in registers (one
// pass over TMEM instead of two), 64 output accumulators instead of 128, and the per-row maximum
// is agreed through shared memory and an mbarrier (bounded wait) once per tile. Twice the exp2 / FMA issue
// slots per SM and a third of the TMEM reads per thread compared with the first kernel.
#include "common.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int F2_THREADS = 384;
constexpr int F2_TILE = 128 * 128 * 2;               // 32 KiB
constexpr float kF2Log2e = 1.4426950408889634f;

struct Flash2Params {
  bf16* o;
  float* lse;
  const int* valid_len;
  long long o_bs, o_ts, o_hs;
  int B, T, QH, KVH;
  float scale;
  int* status;
};

struct F2Smem {
  static constexpr int kQ = 0;
  static constexpr int kKV = F2_TILE;                                   // stage s: K then V
  static constexpr int kMax = kKV + 2 * 2 * F2_TILE;                    // float [2 parity][2 halves][128]
  static constexpr int kBar = kMax + 2 * 2 * 128 * 4;
  // q_full, kv_full[2], kv_empty[2], s_full[2], p_full[2], pv_full, pv_empty, mx_bar[2], sum_bar = 14
  static constexpr int kTotal = kBar + 14 * 8 + 16 + 1024;
};

__global__ void __launch_bounds__(F2_THREADS, 1)
flash_fwd_tc2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const Flash2Params p) {
  extern __shared__ uint8_t f2_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(f2_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + F2Smem::kBar);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 3;
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 7;
  uint64_t* pv_full = bars + 9;
  uint64_t* pv_empty = bars + 10;
  uint64_t* mx_bar = bars + 11;      // the two softmax warpgroups exchange row maxima (bounded wait, no bar.sync)
  uint64_t* sum_bar = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* smax = reinterpret_cast<float*>(smem + F2Smem::kMax);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mtile = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.QH / p.KVH);
  const int m0 = mtile * 128;
  const int T = p.T;
  const int vlen = p.valid_len ? min(p.valid_len[b], T) : T;
  const int n_tiles = min(mtile + 1, (max(vlen, 1) + 127) / 128);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 256);
    }
    mbar_init(pv_full, 1);
    mbar_init(pv_empty, 256);
    mbar_init(&mx_bar[0], 256);
    mbar_init(&mx_bar[1], 256);
    mbar_init(sum_bar, 256);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 2) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColS = 0, kColPV = 256;

  if (warp < 4) {
    if (warp == 0 && lane == 0) {
      mbar_expect_tx(q_full, F2_TILE);
      tma_load_4d(smem + F2Smem::kQ, &tmQ, q_full, 0, h, m0, b);
      tma_load_4d(smem + F2Smem::kQ + 16384, &tmQ, q_full, 64, h, m0, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) break;
        uint8_t* sK = smem + F2Smem::kKV + s * 2 * F2_TILE;
        uint8_t* sV = sK + F2_TILE;
        mbar_expect_tx(&kv_full[s], 2 * F2_TILE);
        tma_load_4d(sK, &tmK, &kv_full[s], 0, kvh, j * 128, b);
        tma_load_4d(sK + 16384, &tmK, &kv_full[s], 64, kvh, j * 128, b);
        tma_load_4d(sV, &tmV, &kv_full[s], 0, kvh, j * 128, b);
        tma_load_4d(sV + 16384, &tmV, &kv_full[s], 64, kvh, j * 128, b);
      }
    } else if (warp == 1 && lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);
      const uint32_t aQ = smem_u32(smem + F2Smem::kQ);
      auto issue_s = [&](int j) {
        const uint32_t aK = smem_u32(smem + F2Smem::kKV + (j & 1) * 2 * F2_TILE);
        const uint32_t td = tmem_base + kColS + (j & 1) * 128;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16_ss(td, umma_smem_desc(aQ + off, 16, 1024), umma_smem_desc(aK + off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(&s_full[j & 1]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j == 0) {
          if (!mbar_wait(&kv_full[0], 0, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_s(0);
        }
        if (j + 1 < n_tiles) {
          if (!mbar_wait(&kv_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_s(j + 1);
        }
        if (!mbar_wait(&p_full[j & 1], (j >> 1) & 1, abort_flag)) { ok = false; break; }
        if (j > 0 && !mbar_wait(pv_empty, (j - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t aV = smem_u32(smem + F2Smem::kKV + (j & 1) * 2 * F2_TILE + F2_TILE);
        const uint32_t tP = tmem_base + kColS + (j & 1) * 128;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16_ts(tmem_base + kColPV, tP + kk * 8, umma_smem_desc(aV + kk * 2048, 16384, 1024), idesc_pv, kk != 0);
        umma_commit(pv_full);
        umma_commit(&kv_empty[j & 1]);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + O (two warpgroups)
    const int q = warp & 3;
    const int half = (warp - 4) >> 2;              // key columns / output columns [64 * half, 64 * half + 64)
    const int rloc = q * 32 + lane;
    const int row = m0 + rloc;
    const uint32_t lane_sel = uint32_t(q * 32) << 16;
    const float sl2 = p.scale * kF2Log2e;
    float o[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, corr_prev = 1.f;
    bool ok = true;
    auto accumulate_pv = [&](int j, float corr) {
      if (!mbar_wait(pv_full, j & 1, abort_flag)) { ok = false; return; }
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(tmem_base + lane_sel + kColPV + half * 64, r0);
      tmem_ld_32x32b_x32(tmem_base + lane_sel + kColPV + half * 64 + 32, r1);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        o[e] = fmaf(o[e], corr, __uint_as_float(r0[e]));
        o[32 + e] = fmaf(o[32 + e], corr, __uint_as_float(r1[e]));
      }
      tc_fence_before();
      mbar_arrive(pv_empty);
    };
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int buf = j & 1;
      if (!mbar_wait(&s_full[buf], (j >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tS = tmem_base + lane_sel + kColS + buf * 128;
      const int n0 = j * 128 + half * 64;
      const bool need_mask = (j == mtile) || (j * 128 + 128 > vlen);
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(tS + half * 64, r0);
      tmem_ld_32x32b_x32(tS + half * 64 + 32, r1);
      tmem_ld_wait();
      float s[64];
      float mx = -INFINITY;
#pragma unroll
      for (int e = 0; e < 64; ++e) {
        float v = __uint_as_float(e < 32 ? r0[e] : r1[e - 32]) * sl2;
        if (need_mask) {
          const int key = n0 + e;
          if (key > row || key >= vlen) v = -INFINITY;
        }
        s[e] = v;
        mx = fmaxf(mx, v);
      }
      // agree on the row maximum with the thread of the other warpgroup that owns the same row
      float* mslot = smax + (buf * 2) * 128;
      mslot[half * 128 + rloc] = mx;
      mbar_arrive(&mx_bar[buf]);
      if (!mbar_wait(&mx_bar[buf], (j >> 1) & 1, abort_flag)) { ok = false; break; }
      mx = fmaxf(mx, mslot[(half ^ 1) * 128 + rloc]);
      const float m_new = fmaxf(m_run, mx);
      const float msafe = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = exp2f(m_run - msafe);
      float rs = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int e = 0; e < 64; e += 2) {
        const float p0 = exp2f(s[e] - msafe), p1 = exp2f(s[e + 1] - msafe);
        rs += p0 + p1;
        const bf162 t = __floats2bfloat162_rn(p0, p1);
        pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&t);
      }
      // both warpgroups have read all of S (they passed mx_bar after their loads): P may overwrite it
      {
        uint32_t a[16], c[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) { a[e] = pk[e]; c[e] = pk[16 + e]; }
        tmem_st_32x32b_x16(tS + half * 32, a);
        tmem_st_32x32b_x16(tS + half * 32 + 16, c);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[buf]);
      l_run = l_run * corr + rs;
      m_run = m_new;
      if (j > 0) accumulate_pv(j - 1, corr_prev);
      corr_prev = corr;
    }
    if (ok && n_tiles > 0) accumulate_pv(n_tiles - 1, corr_prev);
    if (ok) {
      // total row sum = the two warpgroups' partial sums (both relative to the same running maximum)
      float* lslot = smax;      // all maxima exchanges are over
      lslot[half * 128 + rloc] = l_run;
      mbar_arrive(sum_bar);
      if (mbar_wait(sum_bar, 0, abort_flag)) {
        const float l_tot = l_run + lslot[(half ^ 1) * 128 + rloc];
        if (row < T) {
          const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
          bf16* orow = p.o + b * p.o_bs + (long long)row * p.o_ts + h * p.o_hs + half * 64;
#pragma unroll
          for (int i = 0; i < 64; i += 8) {
            uint4 v;
            bf162* v2 = reinterpret_cast<bf162*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) v2[e] = __floats2bfloat162_rn(o[i + 2 * e] * inv, o[i + 2 * e + 1] * inv);
            *reinterpret_cast<uint4*>(orow + i) = v;
          }
          if (half == 0)
            p.lse[(size_t(b) * p.QH + h) * T + row] =
                l_tot > 0.f ? m_run * 0.6931471805599453f + logf(l_tot) : -INFINITY;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, int(*abort_flag)) == 0) p.status[1] = 301;
  }
}

}  // namespace b200

using namespace b200;

// Same contract as b200_flash_fwd_tc (inputs already rotated, head_dim 128).
B200_API int b200_flash_fwd_tc2(const void* q, const void* k, const void* v, void* o, void* lse, const void* valid_len,
                                const long long* strides, int B, int T, int QH, int KVH, int D, float scale,
                                cudaStream_t st) {
  if (B <= 0 || T <= 0) return 0;
  if (D != 128 || QH % KVH != 0) return static_cast<int>(cudaErrorInvalidValue);
  for (int i = 0; i < 12; ++i)
    if (strides[i] % 8 != 0) return static_cast<int>(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(o) & 15) != 0) return static_cast<int>(cudaErrorInvalidValue);
  const CUtensorMap* tq = get_tensor_map_bthd(q, B, T, QH, D, strides[0], strides[1], strides[2], 128, 64);
  const CUtensorMap* tk = get_tensor_map_bthd(k, B, T, KVH, D, strides[3], strides[4], strides[5], 128, 64);
  const CUtensorMap* tv = get_tensor_map_bthd(v, B, T, KVH, D, strides[6], strides[7], strides[8], 128, 64);
  if (!tq || !tk || !tv) return static_cast<int>(cudaErrorInvalidValue);
  Flash2Params p;
  p.o = static_cast<bf16*>(o);
  p.lse = static_cast<float*>(lse);
  p.valid_len = static_cast<const int*>(valid_len);
  p.o_bs = strides[9]; p.o_ts = strides[10]; p.o_hs = strides[11];
  p.B = B; p.T = T; p.QH = QH; p.KVH = KVH; p.scale = scale;
  p.status = status_ptr();
  static bool configured = false;
  if (!configured) {
    B200_CHECK(cudaFuncSetAttribute(flash_fwd_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F2Smem::kTotal));
    configured = true;
  }
  dim3 grid((T + 127) / 128, QH, B);
  flash_fwd_tc2_kernel<<<grid, F2_THREADS, F2Smem::kTotal, st>>>(*tq, *tk, *tv, p);
  return static_cast<int>(cudaGetLastError());
}
