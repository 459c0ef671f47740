// Causal GQA flash-attention forward on tcgen05 (head_dim 128 or 64).
//
// One CTA owns TWO consecutive 128-row query tiles of one (batch, head) and walks the key tiles
// once for both. Each query tile has its own softmax warpgroup, its own score buffer and its own
// output accumulator in tensor memory:
//
//   TMEM columns   0..127  S_0 (fp32 scores of query tile 0; P_0 as bf16 overwrites columns 0..63)
//                128..255  S_1
//                256..383  O_0 (fp32, accumulated by the P V MMAs themselves)
//                384..511  O_1
//
// A thread of a softmax warpgroup owns one query row (one TMEM lane) and all 128 key columns of
// the tile, so the row maximum and the row sum never leave the thread. While warpgroup 0 is in
// its exp2 pass the tensor core runs P_1 V and the next S_1, and the other way round; neither
// side waits for the other except through the data it needs.
//
// The running maximum is applied lazily: the reference point m of a row only moves when the new
// tile maximum exceeds it by more than 8 (log2 units), so exp2(s - m) stays below 2^8 and the
// output accumulator has to be rescaled (TMEM load, multiply, TMEM store by the row's own thread)
// only on the rare tiles where that happens. The final 1 / l normalisation uses the same m.
//
// K and V travel through separate 2-deep rings: the K slot of tile j is free as soon as both
// S(j) MMAs have run, long before the V slot, so the TMA load of K(j+2) gets a full iteration of
// lead. The output tile is staged in the (by then unused) Q tile in the 128-byte swizzle and
// stored with cp.async.bulk.tensor. Every wait is bounded (see ptx.cuh).
//
// head_dim 64 (template parameter) uses the same layout with half of everything that depends on it:
// one 64-column box per Q / K / V / O tile instead of two, four k-steps in S = Q K^T, N = 64 in O += P V,
// 64 live columns in each O accumulator.
#include "common.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int F3_THREADS = 384;                      // warps 0-3: TMA / MMA / TMEM; 4-7: WG 0; 8-11: WG 1
constexpr int F3_TILE = 128 * 128 * 2;               // 32 KiB
constexpr float kF3Log2e = 1.4426950408889634f;
constexpr float kF3RescaleStep = 8.f;

struct Flash3Params {
  float* lse;
  const int* valid_len;
  int B, T, QH, KVH;
  float scale;
  int* status;
};

struct F3Smem {
  static constexpr int kQ = 0;                                         // Q_0, Q_1
  static constexpr int kK = 2 * F3_TILE;                               // K ring [2]
  static constexpr int kV = 4 * F3_TILE;                               // V ring [2]
  static constexpr int kBar = 6 * F3_TILE;
  // q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], pv_done[2], stage_bar[2] = 17
  static constexpr int kTotal = kBar + 17 * 8 + 16 + 1024;
};

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2,
                                             int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

struct TrueTag { static constexpr bool value = true; };
struct FalseTag { static constexpr bool value = false; };

__device__ __forceinline__ float f3_max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Raw maximum of the 128 scores of one row; masked keys (beyond the diagonal or the valid length) are
// set to -inf in place so that the exponential pass needs no mask.
template <bool kMask>
__device__ __forceinline__ float f3_row_max(uint32_t (&sc)[128], int key0, int row, int vlen) {
  float mx = -INFINITY;
#pragma unroll
  for (int e = 0; e < 128; e += 2) {
    if (kMask) {
      const int key = key0 + e;
      if (key > row || key >= vlen) sc[e] = 0xff800000u;
      if (key + 1 > row || key + 1 >= vlen) sc[e + 1] = 0xff800000u;
    }
    mx = f3_max3(mx, __uint_as_float(sc[e]), __uint_as_float(sc[e + 1]));
  }
  return mx;
}

// P = exp2(s * sl2 - m_ref) for the 128 scores of one row, packed to bf16 pairs IN PLACE (pair e / 2 lands in
// register e / 2, which has been consumed by then); returns the row sum.
__device__ __forceinline__ float f3_row_p(uint32_t (&sc)[128], float sl2, float m_ref) {
  float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
  for (int e = 0; e < 128; e += 2) {
    const float p0 = exp2f(fmaf(__uint_as_float(sc[e]), sl2, -m_ref));
    const float p1 = exp2f(fmaf(__uint_as_float(sc[e + 1]), sl2, -m_ref));
    rs0 += p0;
    rs1 += p1;
    const bf162 t = __floats2bfloat162_rn(p0, p1);
    sc[e >> 1] = *reinterpret_cast<const uint32_t*>(&t);
  }
  return rs0 + rs1;
}

template <int kD>
__global__ void __launch_bounds__(F3_THREADS, 1)
flash_fwd_tc3_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                     const Flash3Params p) {
  extern __shared__ uint8_t f3_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(f3_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + F3Smem::kBar);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 3;
  uint64_t* v_full = bars + 5;
  uint64_t* v_empty = bars + 7;
  uint64_t* s_full = bars + 9;       // [w]: S_w of the current key tile is in TMEM
  uint64_t* p_full = bars + 11;      // [w]: warpgroup w has written P_w (128 arrivals)
  uint64_t* pv_done = bars + 13;     // [w]: O_w includes the key tile whose P V was committed last
  uint64_t* stage_bar = bars + 15;   // [w]: the output tile of warpgroup w is staged in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pt = gridDim.x - 1 - blockIdx.x;             // pair of query tiles; the longest rows start first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.QH / p.KVH);
  const int T = p.T;
  const int vlen = p.valid_len ? checked_index(p.valid_len[b], T, p.status, 301) : T;
  const int kv_tiles = (max(vlen, 1) + 127) / 128;
  int nt[2];
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    const int mt = 2 * pt + w;
    nt[w] = (mt * 128 < T) ? min(mt + 1, kv_tiles) : 0;
  }
  const int nmax = max(nt[0], nt[1]);
  constexpr uint32_t kTileBytes = 128 * kD * 2;          // live bytes of a Q / K / V tile (its slot stays 32 KiB)

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
      mbar_init(&pv_done[s], 1);
      mbar_init(&stage_bar[s], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO);
  }
  if (warp == 2) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColS = 0, kColO = 256;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, (nt[1] > 0 ? 2 : 1) * kTileBytes);
      for (int w = 0; w < 2; ++w) {
        if (nt[w] == 0) continue;
        uint8_t* sQ = smem + F3Smem::kQ + w * F3_TILE;
        tma_load_4d(sQ, &tmQ, q_full, 0, h, (2 * pt + w) * 128, b);
        if (kD == 128) tma_load_4d(sQ + 16384, &tmQ, q_full, 64, h, (2 * pt + w) * 128, b);
      }
      for (int j = 0; j < nmax; ++j) {
        const int s = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&k_empty[s], par, abort_flag)) break;
        uint8_t* sK = smem + F3Smem::kK + s * F3_TILE;
        mbar_expect_tx(&k_full[s], kTileBytes);
        tma_load_4d(sK, &tmK, &k_full[s], 0, kvh, j * 128, b);
        if (kD == 128) tma_load_4d(sK + 16384, &tmK, &k_full[s], 64, kvh, j * 128, b);
        if (!mbar_wait(&v_empty[s], par, abort_flag)) break;
        uint8_t* sV = smem + F3Smem::kV + s * F3_TILE;
        mbar_expect_tx(&v_full[s], kTileBytes);
        tma_load_4d(sV, &tmV, &v_full[s], 0, kvh, j * 128, b);
        if (kD == 128) tma_load_4d(sV + 16384, &tmV, &v_full[s], 64, kvh, j * 128, b);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, kD, 0, 1);
      auto issue_s = [&](int w, int j) {
        const uint32_t aQ = smem_u32(smem + F3Smem::kQ + w * F3_TILE);
        const uint32_t aK = smem_u32(smem + F3Smem::kK + (j & 1) * F3_TILE);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16_ss(tmem_base + kColS + w * 128, umma_smem_desc(aQ + off, 16, 1024),
                       umma_smem_desc(aK + off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(&s_full[w]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (ok && nmax > 0) {
        ok = mbar_wait(&k_full[0], 0, abort_flag);
        if (ok) {
          tc_fence_after();
          for (int w = 0; w < 2; ++w)
            if (nt[w] > 0) issue_s(w, 0);
          umma_commit(&k_empty[0]);
        }
      }
      for (int j = 0; j < nmax && ok; ++j) {
        bool v_ready = false, k_ready = false;
        for (int w = 0; w < 2 && ok; ++w) {
          if (j >= nt[w]) continue;
          if (!mbar_wait(&p_full[w], j & 1, abort_flag)) { ok = false; break; }
          if (!v_ready) {
            if (!mbar_wait(&v_full[j & 1], (j >> 1) & 1, abort_flag)) { ok = false; break; }
            v_ready = true;
          }
          tc_fence_after();
          const uint32_t aV = smem_u32(smem + F3Smem::kV + (j & 1) * F3_TILE);
          const uint32_t tP = tmem_base + kColS + w * 128;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_bf16_ts(tmem_base + kColO + w * 128, tP + kk * 8, umma_smem_desc(aV + kk * 2048, 16384, 1024),
                         idesc_pv, (j | kk) != 0);
          umma_commit(&pv_done[w]);
          if (j + 1 < nt[w]) {
            if (!k_ready) {
              if (!mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
              k_ready = true;
              tc_fence_after();
            }
            issue_s(w, j + 1);
          }
        }
        if (!ok) break;
        if (j + 1 < nmax) umma_commit(&k_empty[(j + 1) & 1]);
        umma_commit(&v_empty[j & 1]);
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- softmax warpgroup w: one query tile
    const int w = (warp - 4) >> 2;
    const int q = warp & 3;
    const int rloc = q * 32 + lane;
    const int mt = 2 * pt + w;
    const int row = mt * 128 + rloc;
    const int my_tiles = nt[w];
    const uint32_t lane_sel = uint32_t(q * 32) << 16;
    const uint32_t tS = tmem_base + lane_sel + kColS + w * 128;
    const uint32_t tO = tmem_base + lane_sel + kColO + w * 128;
    const float sl2 = p.scale * kF3Log2e;
    float m_ref = 0.f, l_run = 0.f;          // reference maximum (log2 units) and the row sum relative to it
    bool ok = true;
    for (int j = 0; j < my_tiles && ok; ++j) {
      if (!mbar_wait(&s_full[w], j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool need_mask = (j == mt) || (j * 128 + 128 > vlen);
      const int key0 = j * 128;
      // The whole row (128 raw scores) is read in one go: four loads, one wait. A tensor-memory load queues
      // behind the MMAs the other warpgroup has in flight, so every separate round trip costs that wait again.
      uint32_t sc[128];
      tmem_ld_32x32b_x32(tS, *reinterpret_cast<uint32_t(*)[32]>(&sc[0]));
      tmem_ld_32x32b_x32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&sc[32]));
      tmem_ld_32x32b_x32(tS + 64, *reinterpret_cast<uint32_t(*)[32]>(&sc[64]));
      tmem_ld_32x32b_x32(tS + 96, *reinterpret_cast<uint32_t(*)[32]>(&sc[96]));
      tmem_ld_wait();
      float mx = (need_mask ? f3_row_max<true>(sc, key0, row, vlen) : f3_row_max<false>(sc, key0, row, vlen)) * sl2;
      // The reference maximum is set by the first tile and afterwards moves only when a tile exceeds it by
      // more than 2^8; then O_w and the row sum are rescaled by the row's own thread.
      if (j == 0) {
        m_ref = (mx == -INFINITY) ? 0.f : mx;
      } else {
        const bool need = mx > m_ref + kF3RescaleStep;
        if (__any_sync(0xffffffffu, need)) {
          // O_w holds the key tiles up to j - 1 once their P V has completed
          if (!mbar_wait(&pv_done[w], (j - 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const float corr = need ? exp2f(m_ref - mx) : 1.f;
          l_run *= corr;
#pragma unroll 1
          for (int c = 0; c < kD / 16; ++c) {
            uint32_t t[16];
            tmem_ld_32x32b_x16(tO + c * 16, t);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) t[e] = __float_as_uint(__uint_as_float(t[e]) * corr);
            tmem_st_32x32b_x16(tO + c * 16, t);
          }
          tmem_st_wait();
          if (need) m_ref = mx;
        }
      }
      // P = exp2(s * scale - m_ref) as bf16 pairs, packed in place over the first 64 registers, and its row sum
      const float rs = f3_row_p(sc, sl2, m_ref);
      // P over the first 64 columns of S_w
#pragma unroll
      for (int c = 0; c < 4; ++c)
        tmem_st_32x32b_x16(tS + c * 16, *reinterpret_cast<const uint32_t(*)[16]>(&sc[16 * c]));
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[w]);
      l_run += rs;
    }
    if (ok && my_tiles > 0) {
      if (mbar_wait(&pv_done[w], (my_tiles - 1) & 1, abort_flag)) {
        tc_fence_after();
        // all MMAs of this query tile have completed: its Q tile in shared memory is free and becomes
        // the staging area of the output (two 128 x 64 boxes, 128-byte swizzle)
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        uint8_t* stg = smem + F3Smem::kQ + w * F3_TILE;
        const uint32_t swz = uint32_t(rloc & 7);
#pragma unroll 1
        for (int c = 0; c < kD / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tO + c * 32, r);
          tmem_ld_wait();
          uint8_t* rowp = stg + (c >> 1) * 16384 + rloc * 128;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 o;
            bf162* o2 = reinterpret_cast<bf162*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              o2[e] = __floats2bfloat162_rn(__uint_as_float(r[8 * k + 2 * e]) * inv,
                                            __uint_as_float(r[8 * k + 2 * e + 1]) * inv);
            *reinterpret_cast<uint4*>(rowp + ((uint32_t((c & 1) * 4 + k) ^ swz) << 4)) = o;
          }
        }
        if (row < T)
          p.lse[(size_t(b) * p.QH + h) * T + row] =
              l_run > 0.f ? m_ref * 0.6931471805599453f + logf(l_run) : -INFINITY;
        fence_proxy_async_smem();
        mbar_arrive(&stage_bar[w]);
        if (q == 0 && lane == 0) {
          if (mbar_wait(&stage_bar[w], 0, abort_flag)) {
            tma_store_4d(&tmO, stg, 0, h, mt * 128, b);
            if (kD == 128) tma_store_4d(&tmO, stg + 16384, 64, h, mt * 128, b);
            tma_store_commit();
            tma_store_wait_read<0>();
          }
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
    if (atomicCAS(p.status, 0, int(*abort_flag)) == 0) p.status[1] = 302;
  }
}

}  // namespace b200

using namespace b200;

// Same contract as b200_flash_fwd_tc (inputs already rotated) for head_dim 128 or 64; the output must be
// TMA-addressable (16-byte aligned base, strides that are multiples of 8 elements).
B200_API int b200_flash_fwd_tc3(const void* q, const void* k, const void* v, void* o, void* lse, const void* valid_len,
                                const long long* strides, int B, int T, int QH, int KVH, int D, float scale,
                                cudaStream_t st) {
  if (B <= 0 || T <= 0) return 0;
  if ((D != 128 && D != 64) || QH % KVH != 0) return static_cast<int>(cudaErrorInvalidValue);
  for (int i = 0; i < 12; ++i)
    if (strides[i] % 8 != 0) return static_cast<int>(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(o) & 15) != 0) return static_cast<int>(cudaErrorInvalidValue);
  const CUtensorMap* tq = get_tensor_map_bthd(q, B, T, QH, D, strides[0], strides[1], strides[2], 128, 64);
  const CUtensorMap* tk = get_tensor_map_bthd(k, B, T, KVH, D, strides[3], strides[4], strides[5], 128, 64);
  const CUtensorMap* tv = get_tensor_map_bthd(v, B, T, KVH, D, strides[6], strides[7], strides[8], 128, 64);
  const CUtensorMap* to = get_tensor_map_bthd(o, B, T, QH, D, strides[9], strides[10], strides[11], 128, 64);
  if (!tq || !tk || !tv || !to) return static_cast<int>(cudaErrorInvalidValue);
  Flash3Params p;
  p.lse = static_cast<float*>(lse);
  p.valid_len = static_cast<const int*>(valid_len);
  p.B = B; p.T = T; p.QH = QH; p.KVH = KVH; p.scale = scale;
  p.status = status_ptr();
  static bool configured = false;
  if (!configured) {
    B200_CHECK(cudaFuncSetAttribute(flash_fwd_tc3_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    F3Smem::kTotal));
    B200_CHECK(cudaFuncSetAttribute(flash_fwd_tc3_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    F3Smem::kTotal));
    configured = true;
  }
  dim3 grid((T + 255) / 256, QH, B);
  if (D == 128)
    flash_fwd_tc3_kernel<128><<<grid, F3_THREADS, F3Smem::kTotal, st>>>(*tq, *tk, *tv, *to, p);
  else
    flash_fwd_tc3_kernel<64><<<grid, F3_THREADS, F3Smem::kTotal, st>>>(*tq, *tk, *tv, *to, p);
  return static_cast<int>(cudaGetLastError());
}
