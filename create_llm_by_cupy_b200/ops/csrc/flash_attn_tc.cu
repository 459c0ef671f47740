// Causal GQA flash-attention FORWARD on the 5th-generation tensor cores (head_dim 128).
//
// One CTA per 128-query tile of one (batch, head); key/value tiles of 128 stream through a
// two-stage TMA ring. Warp roles (256 threads):
//   warp 0      TMA producer : Q once, then K_j / V_j tiles (4-D tensor maps over the strided
//                              [B, T, heads, D] views of the packed K|Q|V buffer, 128B swizzle)
//   warp 1      MMA issuer   : S_j = Q K_j^T   (tcgen05.mma, both operands from shared memory)
//                              PV_j = P_j V_j  (A = P_j read straight from TMEM, B = V_j MN-major)
//   warp 2      TMEM allocator (512 columns: S double-buffered, P aliases S, one PV buffer)
//   warps 4..7  softmax      : one query row per thread; tcgen05.ld of S in 32-column chunks, online
//                              softmax in the exp2 domain, P written back to TMEM as packed bf16
//                              with tcgen05.st, O kept in registers and updated from PV_j
// S_{j+1} is issued before PV_j so the tensor core computes the next scores while the softmax
// warps work on the current ones. Q and K are expected already rotated (the rotary embedding is
// applied by the caller); the log-sum-exp is written for the backward pass.
//
// Reference counterpart: cupy_flash_gqa_forward (model/flash_attention.py:51-106) and the Triton
// forward (:195-282).
#include "common.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int FT_BM = 128;
constexpr int FT_BN = 128;
constexpr int FT_D = 128;
constexpr int FT_THREADS = 256;
constexpr int FT_STAGES = 2;
constexpr int FT_TILE_BYTES = 128 * FT_D * 2;            // 32 KiB: one Q, K or V tile
constexpr float kFtLog2e = 1.4426950408889634f;

struct FlashTcParams {
  bf16* o;
  float* lse;
  const int* valid_len;
  long long o_bs, o_ts, o_hs;
  int B, T, QH, KVH;
  float scale;
  int* status;
};

struct FtSmem {
  static constexpr int kQ = 0;
  static constexpr int kKV = FT_TILE_BYTES;                               // stage s: K at +0, V at +32 KiB
  static constexpr int kBar = kKV + FT_STAGES * 2 * FT_TILE_BYTES;
  // q_full, kv_full[2], kv_empty[2], s_full[2], p_full[2], pv_full, pv_empty  = 11 barriers
  static constexpr int kTotal = kBar + 11 * 8 + 16 + 1024;
};

__global__ void __launch_bounds__(FT_THREADS, 1)
flash_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const FlashTcParams p) {
  extern __shared__ uint8_t ft_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ft_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FtSmem::kBar);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 3;
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 7;
  uint64_t* pv_full = bars + 9;
  uint64_t* pv_empty = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mtile = gridDim.x - 1 - blockIdx.x;       // long (late) tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.QH / p.KVH);
  const int m0 = mtile * FT_BM;
  const int T = p.T;
  const int vlen = p.valid_len ? min(p.valid_len[b], T) : T;
  const int n_tiles = min(mtile + 1, (max(vlen, 1) + FT_BN - 1) / FT_BN);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
    }
    mbar_init(pv_full, 1);
    mbar_init(pv_empty, 128);
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

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, FT_TILE_BYTES);
      tma_load_4d(smem + FtSmem::kQ, &tmQ, q_full, 0, h, m0, b);
      tma_load_4d(smem + FtSmem::kQ + 16384, &tmQ, q_full, 64, h, m0, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) break;
        uint8_t* sK = smem + FtSmem::kKV + s * 2 * FT_TILE_BYTES;
        uint8_t* sV = sK + FT_TILE_BYTES;
        mbar_expect_tx(&kv_full[s], 2 * FT_TILE_BYTES);
        tma_load_4d(sK, &tmK, &kv_full[s], 0, kvh, j * FT_BN, b);
        tma_load_4d(sK + 16384, &tmK, &kv_full[s], 64, kvh, j * FT_BN, b);
        tma_load_4d(sV, &tmV, &kv_full[s], 0, kvh, j * FT_BN, b);
        tma_load_4d(sV + 16384, &tmV, &kv_full[s], 64, kvh, j * FT_BN, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(FT_BM, FT_BN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(FT_BM, FT_D, 0, 1);
      const uint32_t aQ = smem_u32(smem + FtSmem::kQ);
      auto issue_s = [&](int j) {
        const uint32_t aK = smem_u32(smem + FtSmem::kKV + (j & 1) * 2 * FT_TILE_BYTES);
        const uint32_t td = tmem_base + kColS + (j & 1) * 128;
#pragma unroll
        for (int kk = 0; kk < FT_D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16_ss(td, umma_smem_desc(aQ + off, 16, 1024), umma_smem_desc(aK + off, 16, 1024), idesc_s,
                       kk != 0 ? 1u : 0u);
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
        const uint32_t aV = smem_u32(smem + FtSmem::kKV + (j & 1) * 2 * FT_TILE_BYTES + FT_TILE_BYTES);
        const uint32_t tP = tmem_base + kColS + (j & 1) * 128;
#pragma unroll
        for (int kk = 0; kk < FT_BN / 16; ++kk) {
          umma_bf16_ts(tmem_base + kColPV, tP + kk * 8, umma_smem_desc(aV + kk * 2048, 16384, 1024), idesc_pv,
                       kk != 0 ? 1u : 0u);
        }
        umma_commit(pv_full);
        umma_commit(&kv_empty[j & 1]);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ softmax + O
    const int q = warp & 3;
    const int row = m0 + q * 32 + lane;
    const uint32_t lane_sel = uint32_t(q * 32) << 16;
    const float sl2 = p.scale * kFtLog2e;
    float o[FT_D];
#pragma unroll
    for (int i = 0; i < FT_D; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, corr_prev = 1.f;
    bool ok = true;
    auto accumulate_pv = [&](int j, float corr) {
      if (!mbar_wait(pv_full, j & 1, abort_flag)) { ok = false; return; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < FT_D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + lane_sel + kColPV + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[c * 32 + e] = fmaf(o[c * 32 + e], corr, __uint_as_float(r[e]));
      }
      tc_fence_before();
      mbar_arrive(pv_empty);
    };
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int buf = j & 1;
      if (!mbar_wait(&s_full[buf], (j >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tS = tmem_base + lane_sel + kColS + buf * 128;
      const int n0 = j * FT_BN;
      const bool need_mask = (j == mtile) || (n0 + FT_BN > vlen);
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < FT_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tS + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float v = __uint_as_float(r[e]) * sl2;
          if (need_mask) {
            const int key = n0 + c * 32 + e;
            if (key > row || key >= vlen) v = -INFINITY;
          }
          mx = fmaxf(mx, v);
        }
      }
      const float m_new = fmaxf(m_run, mx);
      const float msafe = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = exp2f(m_run - msafe);
      float rs = 0.f;
#pragma unroll 1
      for (int c = 0; c < FT_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tS + c * 32, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float p0 = exp2f(__uint_as_float(r[e]) * sl2 - msafe);
          float p1 = exp2f(__uint_as_float(r[e + 1]) * sl2 - msafe);
          if (need_mask) {
            const int key = n0 + c * 32 + e;
            if (key > row || key >= vlen) p0 = 0.f;
            if (key + 1 > row || key + 1 >= vlen) p1 = 0.f;
          }
          rs += p0 + p1;
          const bf162 t = __floats2bfloat162_rn(p0, p1);
          pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&t);
        }
        // P chunk c (16 packed columns) lands on S columns [16c, 16c + 16), all of them already read
        tmem_st_32x32b_x16(tS + c * 16, pk);
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
    if (ok && row < T) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      bf16* orow = p.o + b * p.o_bs + (long long)row * p.o_ts + h * p.o_hs;
#pragma unroll
      for (int i = 0; i < FT_D; i += 8) {
        uint4 v;
        bf162* v2 = reinterpret_cast<bf162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) v2[e] = __floats2bfloat162_rn(o[i + 2 * e] * inv, o[i + 2 * e + 1] * inv);
        *reinterpret_cast<uint4*>(orow + i) = v;
      }
      p.lse[(size_t(b) * p.QH + h) * T + row] = l_run > 0.f ? m_run * 0.6931471805599453f + logf(l_run) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, int(*abort_flag)) == 0) p.status[1] = 300;
  }
}

}  // namespace b200

using namespace b200;

// q [B,T,QH,128], k/v [B,T,KVH,128] with element strides (batch, token, head), last dim contiguous,
// already rotated. o [B,T,QH,128]; lse [B,QH,T] fp32. strides: q(3) k(3) v(3) o(3).
B200_API int b200_flash_fwd_tc(const void* q, const void* k, const void* v, void* o, void* lse, const void* valid_len,
                               const long long* strides, int B, int T, int QH, int KVH, int D, float scale,
                               cudaStream_t st) {
  if (B <= 0 || T <= 0) return 0;
  if (D != FT_D || QH % KVH != 0) return static_cast<int>(cudaErrorInvalidValue);
  for (int i = 0; i < 12; ++i)
    if (strides[i] % 8 != 0) return static_cast<int>(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(o) & 15) != 0) return static_cast<int>(cudaErrorInvalidValue);
  const CUtensorMap* tq = get_tensor_map_bthd(q, B, T, QH, D, strides[0], strides[1], strides[2], 128, 64);
  const CUtensorMap* tk = get_tensor_map_bthd(k, B, T, KVH, D, strides[3], strides[4], strides[5], 128, 64);
  const CUtensorMap* tv = get_tensor_map_bthd(v, B, T, KVH, D, strides[6], strides[7], strides[8], 128, 64);
  if (!tq || !tk || !tv) return static_cast<int>(cudaErrorInvalidValue);
  FlashTcParams p;
  p.o = static_cast<bf16*>(o);
  p.lse = static_cast<float*>(lse);
  p.valid_len = static_cast<const int*>(valid_len);
  p.o_bs = strides[9]; p.o_ts = strides[10]; p.o_hs = strides[11];
  p.B = B; p.T = T; p.QH = QH; p.KVH = KVH; p.scale = scale;
  p.status = status_ptr();
  static bool configured = false;
  if (!configured) {
    B200_CHECK(cudaFuncSetAttribute(flash_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FtSmem::kTotal));
    configured = true;
  }
  dim3 grid((T + FT_BM - 1) / FT_BM, QH, B);
  flash_fwd_tc_kernel<<<grid, FT_THREADS, FtSmem::kTotal, st>>>(*tq, *tk, *tv, p);
  return static_cast<int>(cudaGetLastError());
}
