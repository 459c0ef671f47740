// Causal GQA flash-attention BACKWARD on the 5th-generation tensor cores (head_dim 128; dK/dV also 64).
//
// Two kernels, both TMA-fed with accumulators in TMEM and the element-wise softmax-gradient math
// done by two warpgroups that split the columns of each score tile:
//
//   flash_bwd_dq_tc  : CTA = 128 queries of one (batch, head); loops over 128-key tiles.
//        S  = Q K_j^T          (SS MMA)            dP = dO V_j^T        (SS MMA)
//        dS = exp2(S*c - lse) * (dP - delta) * scale   -> bf16 into TMEM
//        dQ += dS K_j          (A = dS from TMEM, B = K_j MN-major), accumulated in TMEM over j
//   flash_bwd_dkv_tc : CTA = 128 keys of one (batch, kv head); loops over the query heads of the
//        group and over 64-query tiles at or below the diagonal, working on transposed scores so
//        that key rows are TMEM lanes:
//        S^T = K Q_i^T (SS)    dP^T = V dO_i^T (SS)   P^T, dS^T -> bf16 into TMEM
//        dV += P^T dO_i        dK += dS^T Q_i      (A from TMEM, B = the same Q_i / dO_i tiles read
//                                                   MN-major), accumulated in TMEM over all i
//   flash_bwd_dkv_wide : the same for head_dim 128 with 128-query iterations: every product is an N = 128 MMA, S^T,
//        dP^T, dV and dK take all 512 tensor-memory columns, and the products of consecutive iterations are
//        interleaved instead of double-buffered (see the comment above that kernel). The default for head_dim 128.
// Q and K are expected already rotated; dQ and dK are gradients w.r.t. the rotated tensors unless the
// caller passes the rotary tables, in which case the epilogues apply the inverse rotation
// (flash_rope_epilogue.cuh). No atomics and no fp32 scratch. When the caller gives a workspace the
// dK/dV kernel also stores its dS^T tiles there and dQ is computed from them by a GEMM kernel
// (flash_attn_bwd_dq.cu) instead of flash_bwd_dq_tc, which recomputes S and dP. The dK/dV kernel and
// that GEMM are templates on the head dimension (128 or 64).
//
// Reference counterpart: cupy_flash_gqa_backward (model/flash_attention.py:109-176).
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"
#include "flash_rope_epilogue.cuh"

namespace b200 {

constexpr int FB_D = 128;
constexpr int FBT_THREADS = 384;          // warps 0-3: producer / MMA / TMEM; warps 4-11: two math warpgroups
constexpr int FB_TILE = 128 * FB_D * 2;   // 32 KiB
constexpr float kFbLog2e = 1.4426950408889634f;

struct FlashBwdTcParams {
  bf16* dq; bf16* dk; bf16* dv;
  const float* lse;      // [B, QH, T]
  const float* delta;    // [B, QH, T]
  const int* valid_len;
  long long dq_bs, dq_ts, dq_hs;
  long long dk_bs, dk_ts, dk_hs;
  long long dv_bs, dv_ts, dv_hs;
  int B, T, QH, KVH;
  int n_tiles;           // 128-row tiles per sequence
  int bchunk;            // batch elements whose Q, dO, K, V stay in L2 together
  int pairing;           // dK/dV kernel: 1 = a CTA owns key tiles i and n_tiles - 1 - i, 0 = one key tile per CTA
  bf16* ds;              // optional: dS^T written by the dK/dV kernel, [B][QH][ds_tp][ds_tp] (key, query)
  long long ds_tp;       // its pitch: T rounded up to 128
  const float* unrot_cos;   // optional fp32 tables, transposed [D / 2][unrot_ld >= T]: dQ and dK leave with the
  const float* unrot_sin;   // inverse rotary embedding applied (gradients of the un-rotated q and k)
  int unrot_ld;
  float scale;
  int* status;
};

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Store one accumulator row (fp32 columns of this thread's TMEM lane) as bf16 to global. The TMEM
// load is warp-collective (.sync.aligned): every lane of the warp must call this; `active` only
// predicates the global stores (rows past the end of the sequence).
__device__ __forceinline__ void store_row_from_tmem(uint32_t taddr, bf16* grow, int col_lo, int col_hi, bool active) {
  for (int c = col_lo; c < col_hi; c += 32) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(taddr + c, r);
    tmem_ld_wait();
    if (!active) continue;
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      uint4 v;
      bf162* v2 = reinterpret_cast<bf162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        v2[e] = __floats2bfloat162_rn(__uint_as_float(r[i + 2 * e]), __uint_as_float(r[i + 2 * e + 1]));
      *reinterpret_cast<uint4*>(grow + c + i) = v;
    }
  }
}

// dS for 16 key columns of one query row: P = exp2(s * sl2 - lse2), dS = P * (dP * scale - delta * scale),
// packed to bf16 pairs. Masked keys (beyond the diagonal or the valid length) give 0.
template <bool kMask>
__device__ __forceinline__ void fb_ds_chunk(const uint32_t (&rs)[16], const uint32_t (&rp)[16], uint32_t (&pk)[8],
                                            float sl2, float lse2, float scale, float dlt_s, int key_base, int row,
                                            int vlen) {
#pragma unroll
  for (int e = 0; e < 16; e += 2) {
    float p0 = exp2f(fmaf(__uint_as_float(rs[e]), sl2, -lse2));
    float p1 = exp2f(fmaf(__uint_as_float(rs[e + 1]), sl2, -lse2));
    if (kMask) {
      const int key = key_base + e;
      if (key > row || key >= vlen) p0 = 0.f;
      if (key + 1 > row || key + 1 >= vlen) p1 = 0.f;
    }
    const float d0 = p0 * fmaf(__uint_as_float(rp[e]), scale, -dlt_s);
    const float d1 = p1 * fmaf(__uint_as_float(rp[e + 1]), scale, -dlt_s);
    const bf162 t = __floats2bfloat162_rn(d0, d1);
    pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&t);
  }
}

// P^T and dS^T for 16 query columns of one key row; lse2 / dlt_s point at the 16 per-query values.
template <bool kMask>
__device__ __forceinline__ void fb_pds_chunk(const uint32_t (&rs)[16], const uint32_t (&rp)[16], uint32_t (&pk)[8],
                                             uint32_t (&dk)[8], float sl2, float scale, const float* lse2,
                                             const float* dlt_s, int q_base, int key, bool key_dead) {
#pragma unroll
  for (int e = 0; e < 16; e += 4) {
    const float4 l4 = *reinterpret_cast<const float4*>(lse2 + e);
    const float4 d4 = *reinterpret_cast<const float4*>(dlt_s + e);
    const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dl[4] = {d4.x, d4.y, d4.z, d4.w};
    float pv[4], dv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float pe = exp2f(fmaf(__uint_as_float(rs[e + u]), sl2, -lv[u]));
      if (kMask) {
        if (key_dead || key > q_base + e + u) pe = 0.f;
      }
      pv[u] = pe;
      dv[u] = pe * fmaf(__uint_as_float(rp[e + u]), scale, -dl[u]);
    }
#pragma unroll
    for (int u = 0; u < 4; u += 2) {
      const bf162 t0 = __floats2bfloat162_rn(pv[u], pv[u + 1]);
      const bf162 t1 = __floats2bfloat162_rn(dv[u], dv[u + 1]);
      pk[(e + u) >> 1] = *reinterpret_cast<const uint32_t*>(&t0);
      dk[(e + u) >> 1] = *reinterpret_cast<const uint32_t*>(&t1);
    }
  }
}

// =================================================================== dQ
struct FdqSmem {
  static constexpr int kQ = 0, kDO = FB_TILE, kKV = 2 * FB_TILE;           // KV stage s: K, V
  static constexpr int kBar = kKV + 2 * 2 * FB_TILE;
  // qdo_full, kv_full[2], kv_empty[2], sdp_full[2], ds_full[2], (2 unused), dq_done = 12 barriers
  static constexpr int kTotal = kBar + 12 * 8 + 16 + 1024;
};

__global__ void __launch_bounds__(FBT_THREADS, 1)
flash_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                       const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                       const FlashBwdTcParams p) {
  extern __shared__ uint8_t fb_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fb_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FdqSmem::kBar);
  uint64_t* qdo_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 3;
  uint64_t* sdp_full = bars + 5;     // [2]: scores of 64-key sub-tile u live in TMEM buffer u & 1
  uint64_t* ds_full = bars + 7;      // [2]: math warpgroup `sub` has written dS of a sub-tile into buffer `sub`
  uint64_t* dq_done = bars + 11;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 1-D grid over chunks of p.bchunk batch elements (what the L2 holds of Q / dO / K / V); inside a
  // chunk the longest rows come first: every (head, batch) of the last query tile, then the one before
  int mtile, h, b;
  {
    const int per_chunk = p.n_tiles * p.QH * p.bchunk;
    const int chunk = int(blockIdx.x) / per_chunk, r = int(blockIdx.x) - chunk * per_chunk;
    const int hb = p.QH * min(p.bchunk, p.B - chunk * p.bchunk);
    mtile = p.n_tiles - 1 - r / hb;
    h = (r % hb) % p.QH;
    b = chunk * p.bchunk + (r % hb) / p.QH;
  }
  const int kvh = h / (p.QH / p.KVH);
  const int m0 = mtile * 128;
  const int T = p.T;
  const int vlen = p.valid_len ? checked_index(p.valid_len[b], T, p.status, 302) : T;
  const int n_tiles = min(mtile + 1, (max(vlen, 1) + 127) / 128);

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&sdp_full[s], 1); mbar_init(&ds_full[s], 128); }
    mbar_init(dq_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmDO); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 2) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Every 128-key tile is processed as two 64-key sub-tiles so that S and dP (64 columns each) can
  // be double-buffered, and each buffer has its own math warpgroup: warpgroup w turns the scores of
  // sub-tiles u = w, w + 2, ... into dS while the other warpgroup and the tensor core are on u + 1.
  // A thread owns one query row (one TMEM lane) and walks its 64 key columns in two halves; dS
  // (bf16, 32 packed columns) overwrites, lane by lane, score columns that thread has already read.
  constexpr uint32_t kColS = 0, kColDP = 128, kColDQ = 384;
  const int n_sub = 2 * n_tiles;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(qdo_full, 2 * FB_TILE);
      tma_load_4d(smem + FdqSmem::kQ, &tmQ, qdo_full, 0, h, m0, b);
      tma_load_4d(smem + FdqSmem::kQ + 16384, &tmQ, qdo_full, 64, h, m0, b);
      tma_load_4d(smem + FdqSmem::kDO, &tmDO, qdo_full, 0, h, m0, b);
      tma_load_4d(smem + FdqSmem::kDO + 16384, &tmDO, qdo_full, 64, h, m0, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) break;
        uint8_t* sK = smem + FdqSmem::kKV + s * 2 * FB_TILE;
        uint8_t* sV = sK + FB_TILE;
        mbar_expect_tx(&kv_full[s], 2 * FB_TILE);
        tma_load_4d(sK, &tmK, &kv_full[s], 0, kvh, j * 128, b);
        tma_load_4d(sK + 16384, &tmK, &kv_full[s], 64, kvh, j * 128, b);
        tma_load_4d(sV, &tmV, &kv_full[s], 0, kvh, j * 128, b);
        tma_load_4d(sV + 16384, &tmV, &kv_full[s], 64, kvh, j * 128, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = umma_idesc_bf16(128, 64, 0, 0);    // [128 q x 64 keys], K-major operands
      constexpr uint32_t idesc_mn = umma_idesc_bf16(128, 128, 0, 1);   // [128 q x 128 d], B MN-major
      const uint32_t aQ = smem_u32(smem + FdqSmem::kQ), aDO = smem_u32(smem + FdqSmem::kDO);
      auto issue_scores = [&](int u) {
        const int j = u >> 1, sub = u & 1;
        const uint32_t aK = smem_u32(smem + FdqSmem::kKV + (j & 1) * 2 * FB_TILE) + sub * 8192, aV = aK + FB_TILE;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16_ss(tmem_base + kColS + sub * 64, umma_smem_desc(aQ + off, 16, 1024),
                       umma_smem_desc(aK + off, 16, 1024), idesc_kk, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16_ss(tmem_base + kColDP + sub * 64, umma_smem_desc(aDO + off, 16, 1024),
                       umma_smem_desc(aV + off, 16, 1024), idesc_kk, kk != 0);
        }
        umma_commit(&sdp_full[sub]);
      };
      bool ok = mbar_wait(qdo_full, 0, abort_flag);
      if (ok && n_sub > 0) {
        ok = mbar_wait(&kv_full[0], 0, abort_flag);
        if (ok) { tc_fence_after(); issue_scores(0); }
      }
      for (int u = 0; u < n_sub && ok; ++u) {
        const int j = u >> 1, sub = u & 1;
        if (u + 1 < n_sub) {
          if (((u + 1) & 1) == 0) {       // first sub-tile of the next key tile: its K / V must have landed
            const int jn = (u + 1) >> 1;
            if (!mbar_wait(&kv_full[jn & 1], (jn >> 1) & 1, abort_flag)) { ok = false; break; }
          }
          tc_fence_after();
          issue_scores(u + 1);
        }
        if (!mbar_wait(&ds_full[sub], (u >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t aK = smem_u32(smem + FdqSmem::kKV + (j & 1) * 2 * FB_TILE) + sub * 8192;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ts(tmem_base + kColDQ, tmem_base + kColS + sub * 64 + kk * 8,
                       umma_smem_desc(aK + kk * 2048, 16384, 1024), idesc_mn, (u | kk) != 0);
        if (sub == 1) umma_commit(&kv_empty[j & 1]);
      }
      if (ok) umma_commit(dq_done);
    }
  } else if (warp >= 4) {
    const int q = warp & 3;                   // TMEM lane quarter
    const int wg = (warp - 4) >> 2;           // math warpgroup = score buffer it serves
    const int half = wg;                      // dQ columns this warpgroup stores at the end
    const int row = m0 + q * 32 + lane;
    const uint32_t lane_sel = uint32_t(q * 32) << 16;
    const float sl2 = p.scale * kFbLog2e;
    const size_t sidx = (size_t(b) * p.QH + h) * T + min(row, T - 1);
    const float lse2 = (row < T) ? p.lse[sidx] * kFbLog2e : INFINITY;
    const float dlt_s = (row < T) ? p.delta[sidx] * p.scale : 0.f;
    bool ok = true;
    for (int u = wg; u < n_sub && ok; u += 2) {
      const int j = u >> 1, sub = wg;
      if (!mbar_wait(&sdp_full[sub], (u >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int n0 = j * 128 + sub * 64;
      const bool need_mask = (j == mtile) || (j * 128 + 128 > vlen);
      // 16 key columns at a time, the next 16 already in flight while these are converted
      const uint32_t tS = tmem_base + lane_sel + kColS + sub * 64, tP = tmem_base + lane_sel + kColDP + sub * 64;
      uint32_t sa[16], pa[16], sb[16], pb[16];
      auto chunk = [&](const uint32_t (&rs)[16], const uint32_t (&rp)[16], int c) {
        uint32_t pk[8];
        if (need_mask) fb_ds_chunk<true>(rs, rp, pk, sl2, lse2, p.scale, dlt_s, n0 + c * 16, row, vlen);
        else fb_ds_chunk<false>(rs, rp, pk, sl2, lse2, p.scale, dlt_s, 0, 0, 0);
        tmem_st_32x32b_x8(tS + c * 8, pk);
      };
      tmem_ld_32x32b_x16(tS, sa);
      tmem_ld_32x32b_x16(tP, pa);
      tmem_ld_wait();
      tmem_ld_32x32b_x16(tS + 16, sb);
      tmem_ld_32x32b_x16(tP + 16, pb);
      chunk(sa, pa, 0);
      tmem_ld_wait();
      tmem_ld_32x32b_x16(tS + 32, sa);
      tmem_ld_32x32b_x16(tP + 32, pa);
      chunk(sb, pb, 1);
      tmem_ld_wait();
      tmem_ld_32x32b_x16(tS + 48, sb);
      tmem_ld_32x32b_x16(tP + 48, pb);
      chunk(sa, pa, 2);
      tmem_ld_wait();
      chunk(sb, pb, 3);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&ds_full[sub]);
    }
    if (ok) {
      if (mbar_wait(dq_done, 0, abort_flag)) {
        tc_fence_after();
        const int pos = min(row, T - 1);
        bf16* grow = p.dq + b * p.dq_bs + (long long)pos * p.dq_ts + h * p.dq_hs;
        if (p.unrot_cos != nullptr)
          store_row_unrot_from_tmem<128>(tmem_base + lane_sel + kColDQ, grow, half * 32, 32, p.unrot_cos + pos,
                                         p.unrot_sin + pos, p.unrot_ld, row < T);
        else
          store_row_from_tmem(tmem_base + lane_sel + kColDQ, grow, half * 64, half * 64 + 64, row < T);
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
    if (atomicCAS(p.status, 0, int(*abort_flag)) == 0) p.status[1] = 310;
  }
}

// =================================================================== dK, dV
constexpr int FKV_BQ = 64;                       // query rows per iteration
constexpr int FKV_QTILE = FKV_BQ * FB_D * 2;     // 16 KiB
constexpr int FKV_ST = 3;                        // Q / dO / statistics ring depth
constexpr int FKV_STG = 128 * 128;               // dS^T staging tile of one math warpgroup: 128 keys x 64 queries bf16
struct FdkvSmem {
  static constexpr int kK = 0, kV = FB_TILE, kQ = 2 * FB_TILE;            // stage s: Q_i (16 KiB), dO_i (16 KiB)
  static constexpr int kStats = kQ + FKV_ST * 2 * FKV_QTILE;               // stage s: lse2[64], delta * scale [64]
  static constexpr int kStage = (kStats + FKV_ST * 2 * FKV_BQ * 4 + 1023) / 1024 * 1024;   // [2] dS^T staging tiles
  static constexpr int kBar = kStage + 2 * FKV_STG;
  // kv_full, q_full[3], q_empty[3], st_full[3] (stats staged), sdp_full[2], pds_full[2], acc_done, acc_free,
  // stg_full[2], stg_free[2] = 20
  static constexpr int kTotal = kBar + 20 * 8 + 16 + 1024;
};

__device__ __forceinline__ void tma_store_4d_ds(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2,
                                                int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

// What one pass of the dK/dV kernel works on: a key tile and the query tiles at or below it.
struct DkvPass {
  int n0, i_first, n_qt, iters;
};
__device__ __forceinline__ DkvPass dkv_pass(int ntile, int T, int R, int vlen) {
  DkvPass d;
  d.n0 = ntile * 128;
  d.i_first = d.n0 / FKV_BQ;                                  // first 64-query tile at / below the diagonal
  d.n_qt = (T + FKV_BQ - 1) / FKV_BQ - d.i_first;
  d.iters = (d.n0 < vlen) ? R * d.n_qt : 0;                  // keys past valid_len: zero gradients
  return d;
}

// kD: head dimension (128, or 64: one 64-column box per K / V / Q / dO tile, four k-steps in the score
// products, N = 64 in the gradient products, 64 live columns in dV and dK).
template <int kD>
__global__ void __launch_bounds__(FBT_THREADS, 1)
flash_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                        const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                        const __grid_constant__ CUtensorMap tmDS, const FlashBwdTcParams p) {
  extern __shared__ uint8_t fb_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fb_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FdkvSmem::kBar);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;                    // [FKV_ST]
  uint64_t* q_empty = q_full + FKV_ST;            // [FKV_ST]
  uint64_t* st_full = q_empty + FKV_ST;           // [FKV_ST]
  uint64_t* sdp_full = st_full + FKV_ST;          // [2]: S^T / dP^T of iteration g live in TMEM buffer g & 1
  uint64_t* pds_full = sdp_full + 2;              // [2]: math warpgroup g & 1 has written P^T / dS^T
  uint64_t* acc_done = pds_full + 2;              // every MMA of a pass has completed
  uint64_t* acc_free = acc_done + 1;              // the dK / dV accumulators of a pass have been stored
  uint64_t* stg_full = acc_free + 1;              // [2]: warpgroup w has written its dS^T tile into its staging tile
  uint64_t* stg_free = stg_full + 2;              // [2]: the TMA store of that tile has read it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stg_free + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A CTA owns the key tiles `pair` and `n_tiles - 1 - pair` of one (kv head, batch element), one after
  // the other: key tile 0 sees every query tile and the last one only two, so each pair adds up to the
  // same number of iterations and no CTA is left working alone at the end of the kernel. 1-D grid over
  // chunks of p.bchunk batch elements (what the L2 holds of Q / dO).
  // With many CTAs per SM (p.pairing == 0) a CTA owns ONE key tile instead and the grid is ordered
  // longest first.
  int pair, kvh, b;
  {
    const int n_pairs = p.pairing ? (p.n_tiles + 1) / 2 : p.n_tiles;
    const int per_chunk = n_pairs * p.KVH * p.bchunk;
    const int chunk = int(blockIdx.x) / per_chunk, r = int(blockIdx.x) - chunk * per_chunk;
    const int hb = p.KVH * min(p.bchunk, p.B - chunk * p.bchunk);
    pair = r / hb;
    kvh = (r % hb) % p.KVH;
    b = chunk * p.bchunk + (r % hb) / p.KVH;
  }
  const int T = p.T;
  const int R = p.QH / p.KVH;
  const int vlen = p.valid_len ? checked_index(p.valid_len[b], T, p.status, 302) : T;
  const int tile_of_pass[2] = {pair, p.pairing ? p.n_tiles - 1 - pair : pair};
  const int n_pass = tile_of_pass[0] == tile_of_pass[1] ? 1 : 2;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < FKV_ST; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); mbar_init(&st_full[s], 32); }
    for (int s = 0; s < 2; ++s) { mbar_init(&sdp_full[s], 1); mbar_init(&pds_full[s], 128); }
    mbar_init(acc_done, 1);
    mbar_init(acc_free, 256);
    for (int s = 0; s < 2; ++s) { mbar_init(&stg_full[s], 128); mbar_init(&stg_free[s], 1); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmDO); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDS);
  }
  if (warp == 2) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // S^T and dP^T are double-buffered (64 columns each per buffer) and each buffer has its own math
  // warpgroup: warpgroup w handles iterations g = w, w + 2, ... (g counts on across the two passes)
  // while the other warpgroup and the tensor core are on g + 1. A thread owns one key row (one TMEM
  // lane) and walks the 64 query columns in 16-column chunks; P^T / dS^T (bf16, 32 packed columns)
  // overwrite, lane by lane, columns of S^T / dP^T that the thread has already read. Q, dO and the
  // row statistics of the next query tiles are prefetched through a 3-stage ring.
  constexpr uint32_t kColST = 0, kColDPT = 128, kColDV = 256, kColDK = 384;

  if (warp == 0) {
    if (lane == 0) {
      int g = 0, kv_loads = 0;
      bool ok = true;
      for (int ps = 0; ps < n_pass && ok; ++ps) {
        const DkvPass d = dkv_pass(tile_of_pass[ps], T, R, vlen);
        if (d.iters == 0) continue;
        if (ps > 0) {             // K / V of the previous pass are read by its MMAs until they have all completed
          if (!mbar_wait(acc_done, (ps - 1) & 1, abort_flag)) break;
        }
        mbar_expect_tx(kv_full, 2 * 128 * kD * 2);
        tma_load_4d(smem + FdkvSmem::kK, &tmK, kv_full, 0, kvh, d.n0, b);
        if (kD == 128) tma_load_4d(smem + FdkvSmem::kK + 16384, &tmK, kv_full, 64, kvh, d.n0, b);
        tma_load_4d(smem + FdkvSmem::kV, &tmV, kv_full, 0, kvh, d.n0, b);
        if (kD == 128) tma_load_4d(smem + FdkvSmem::kV + 16384, &tmV, kv_full, 64, kvh, d.n0, b);
        ++kv_loads;
        for (int it = 0; it < d.iters; ++it, ++g) {
          const int s = g % FKV_ST;
          const int h = kvh * R + it / d.n_qt;
          const int m0 = (d.i_first + it % d.n_qt) * FKV_BQ;
          if (!mbar_wait(&q_empty[s], ((g / FKV_ST) & 1) ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sQ = smem + FdkvSmem::kQ + s * 2 * FKV_QTILE;
          uint8_t* sDO = sQ + FKV_QTILE;
          mbar_expect_tx(&q_full[s], 2 * FKV_BQ * kD * 2);
          tma_load_4d(sQ, &tmQ, &q_full[s], 0, h, m0, b);
          if (kD == 128) tma_load_4d(sQ + 8192, &tmQ, &q_full[s], 64, h, m0, b);
          tma_load_4d(sDO, &tmDO, &q_full[s], 0, h, m0, b);
          if (kD == 128) tma_load_4d(sDO + 8192, &tmDO, &q_full[s], 64, h, m0, b);
        }
      }
      (void)kv_loads;
    }
  } else if (warp == 3) {
    // stages the per-query statistics (lse in log2 units, delta * scale) of each query tile in shared memory
    int g = 0;
    bool ok = true;
    for (int ps = 0; ps < n_pass && ok; ++ps) {
      const DkvPass d = dkv_pass(tile_of_pass[ps], T, R, vlen);
      for (int it = 0; it < d.iters; ++it, ++g) {
        const int s = g % FKV_ST;
        const int h = kvh * R + it / d.n_qt;
        const int m0 = (d.i_first + it % d.n_qt) * FKV_BQ;
        if (!mbar_wait(&q_empty[s], ((g / FKV_ST) & 1) ^ 1, abort_flag)) { ok = false; break; }
        float* st = reinterpret_cast<float*>(smem + FdkvSmem::kStats + s * 2 * FKV_BQ * 4);
        float lv[FKV_BQ / 32], dv[FKV_BQ / 32];      // every load in flight before the first store
#pragma unroll
        for (int j = 0; j < FKV_BQ / 32; ++j) {
          const int row = m0 + lane + 32 * j;
          const size_t idx = (size_t(b) * p.QH + h) * T + min(row, T - 1);
          lv[j] = __ldg(p.lse + idx);
          dv[j] = __ldg(p.delta + idx);
        }
#pragma unroll
        for (int j = 0; j < FKV_BQ / 32; ++j) {
          const int r = lane + 32 * j;
          st[r] = (m0 + r < T) ? lv[j] * kFbLog2e : INFINITY;       // +inf => P = 0 for rows past T
          st[FKV_BQ + r] = (m0 + r < T) ? dv[j] * p.scale : 0.f;
        }
        mbar_arrive(&st_full[s]);
      }
    }
  } else if (warp == 2) {
    // stores the dS^T staging tiles: iteration g belongs to warpgroup g & 1 (g counts on across the passes)
    if (lane == 0 && p.ds != nullptr) {
      int g = 0;
      bool ok = true;
      for (int ps = 0; ps < n_pass && ok; ++ps) {
        const DkvPass d = dkv_pass(tile_of_pass[ps], T, R, vlen);
        for (int it = 0; it < d.iters && ok; ++it, ++g) {
          const int w = g & 1;
          const int m0 = (d.i_first + it % d.n_qt) * FKV_BQ;
          if (!mbar_wait(&stg_full[w], (g >> 1) & 1, abort_flag)) { ok = false; break; }
          tma_store_4d_ds(&tmDS, smem + FdkvSmem::kStage + w * FKV_STG, m0, kvh * R + it / d.n_qt, d.n0, b);
          tma_store_commit();
          tma_store_wait_read<0>();
          mbar_arrive(&stg_free[w]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, FKV_BQ, 0, 0);   // [128 keys x 64 q], K-major operands
      constexpr uint32_t idesc_g = umma_idesc_bf16(128, kD, 0, 1);       // [128 keys x d], B MN-major
      const uint32_t aK = smem_u32(smem + FdkvSmem::kK), aV = smem_u32(smem + FdkvSmem::kV);
      auto issue_scores = [&](int g) {
        const int s = g & 1;
        const uint32_t aQ = smem_u32(smem + FdkvSmem::kQ + (g % FKV_ST) * 2 * FKV_QTILE), aDO = aQ + FKV_QTILE;
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t offk = (kk >> 2) * 16384 + (kk & 3) * 32;     // 128-row tiles
          const uint32_t offq = (kk >> 2) * 8192 + (kk & 3) * 32;      // 64-row tiles
          umma_bf16_ss(tmem_base + kColST + s * 64, umma_smem_desc(aK + offk, 16, 1024),
                       umma_smem_desc(aQ + offq, 16, 1024), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t offk = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t offq = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16_ss(tmem_base + kColDPT + s * 64, umma_smem_desc(aV + offk, 16, 1024),
                       umma_smem_desc(aDO + offq, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(&sdp_full[s]);
      };
      bool ok = true;
      int g0 = 0, kv_loads = 0;
      for (int ps = 0; ps < n_pass && ok; ++ps) {
        const DkvPass d = dkv_pass(tile_of_pass[ps], T, R, vlen);
        if (d.iters > 0) {
          if (!mbar_wait(kv_full, kv_loads & 1, abort_flag)) { ok = false; break; }
          ++kv_loads;
          if (!mbar_wait(&q_full[g0 % FKV_ST], (g0 / FKV_ST) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_scores(g0);
          if (ps > 0) {           // the accumulators still hold the previous pass until its rows are stored
            if (!mbar_wait(acc_free, (ps - 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
          }
        }
        for (int it = 0; it < d.iters && ok; ++it) {
          const int g = g0 + it, s = g & 1;
          if (it + 1 < d.iters) {
            // scores of the next query tile go to the other TMEM buffer while the math warps work on
            // this one (its previous contents were consumed by the gradient MMAs issued earlier)
            if (!mbar_wait(&q_full[(g + 1) % FKV_ST], ((g + 1) / FKV_ST) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            issue_scores(g + 1);
          }
          if (!mbar_wait(&pds_full[s], (g >> 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t aQ = smem_u32(smem + FdkvSmem::kQ + (g % FKV_ST) * 2 * FKV_QTILE), aDO = aQ + FKV_QTILE;
          // B = dO_i / Q_i read MN-major: 64 query rows (k), 128 d (n); 64-d chunks are 8 KiB apart
#pragma unroll
          for (int kk = 0; kk < FKV_BQ / 16; ++kk) {
            umma_bf16_ts(tmem_base + kColDV, tmem_base + kColST + s * 64 + kk * 8,
                         umma_smem_desc(aDO + kk * 2048, 8192, 1024), idesc_g, (it | kk) != 0);
          }
#pragma unroll
          for (int kk = 0; kk < FKV_BQ / 16; ++kk) {
            umma_bf16_ts(tmem_base + kColDK, tmem_base + kColDPT + s * 64 + kk * 8,
                         umma_smem_desc(aQ + kk * 2048, 8192, 1024), idesc_g, (it | kk) != 0);
          }
          umma_commit(&q_empty[g % FKV_ST]);
        }
        if (ok && d.iters == 0 && ps > 0) {
          // nothing to do in this pass: still do not complete acc_done a second time before every math
          // thread has seen its first completion (a waiter two phases behind would never wake up)
          if (!mbar_wait(acc_free, (ps - 1) & 1, abort_flag)) { ok = false; break; }
        }
        if (ok) umma_commit(acc_done);
        g0 += d.iters;
      }
    }
  } else if (warp >= 4) {
    const int q = warp & 3;
    const int wg = (warp - 4) >> 2;           // math warpgroup = score buffer it serves
    const int half = wg;                      // dK / dV columns this warpgroup stores at the end of a pass
    const uint32_t lane_sel = uint32_t(q * 32) << 16;
    const float sl2 = p.scale * kFbLog2e;
    // dS^T goes to global memory through this warpgroup's staging tile (128-byte swizzle) and a TMA store
    uint8_t* stg_row = smem + FdkvSmem::kStage + wg * FKV_STG + (q * 32 + lane) * 128;
    const uint32_t swz = uint32_t(lane & 7);
    const bool ds_on = p.ds != nullptr;
    uint32_t stg_uses = 0;
    bool ok = true;
    int g0 = 0;
    for (int ps = 0; ps < n_pass && ok; ++ps) {
      const DkvPass d = dkv_pass(tile_of_pass[ps], T, R, vlen);
      const int n0 = d.n0;
      const int key = n0 + q * 32 + lane;
      const bool key_dead = key >= vlen;
      for (int it = ((g0 & 1) == wg ? 0 : 1); it < d.iters && ok; it += 2) {
        const int g = g0 + it;
        const int s = wg, s4 = g % FKV_ST;
        const int m0 = (d.i_first + it % d.n_qt) * FKV_BQ;
        if (!mbar_wait(&st_full[s4], (g / FKV_ST) & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait(&sdp_full[s], (g >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const float* st = reinterpret_cast<const float*>(smem + FdkvSmem::kStats + s4 * 2 * FKV_BQ * 4);
        const bool need_mask = (m0 < n0 + 128) || (n0 + 128 > vlen);     // the diagonal or the padded tail
        // 16 query columns at a time, the next 16 already in flight while these are converted
        const uint32_t tS = tmem_base + lane_sel + kColST + s * 64, tP = tmem_base + lane_sel + kColDPT + s * 64;
        uint32_t sa[16], pa[16], sb[16], pb[16];
        if (ds_on) {              // the store of this warpgroup's previous tile must have read the staging tile
          if (!mbar_wait(&stg_free[wg], (stg_uses & 1) ^ 1, abort_flag)) { ok = false; break; }
        }
        auto chunk = [&](const uint32_t (&rs)[16], const uint32_t (&rp)[16], int c) {
          uint32_t pk[8], dk_[8];
          if (need_mask)
            fb_pds_chunk<true>(rs, rp, pk, dk_, sl2, p.scale, st + c * 16, st + FKV_BQ + c * 16, m0 + c * 16, key,
                               key_dead);
          else
            fb_pds_chunk<false>(rs, rp, pk, dk_, sl2, p.scale, st + c * 16, st + FKV_BQ + c * 16, 0, 0, false);
          tmem_st_32x32b_x8(tS + c * 8, pk);
          tmem_st_32x32b_x8(tP + c * 8, dk_);
          if (ds_on) {            // 16 queries = two 16-byte chunks of this key's 128-byte staging row
            *reinterpret_cast<uint4*>(stg_row + ((uint32_t(2 * c) ^ swz) << 4)) = make_uint4(dk_[0], dk_[1], dk_[2], dk_[3]);
            *reinterpret_cast<uint4*>(stg_row + ((uint32_t(2 * c + 1) ^ swz) << 4)) = make_uint4(dk_[4], dk_[5], dk_[6], dk_[7]);
          }
        };
        tmem_ld_32x32b_x16(tS, sa);
        tmem_ld_32x32b_x16(tP, pa);
        tmem_ld_wait();
        tmem_ld_32x32b_x16(tS + 16, sb);
        tmem_ld_32x32b_x16(tP + 16, pb);
        chunk(sa, pa, 0);
        tmem_ld_wait();
        tmem_ld_32x32b_x16(tS + 32, sa);
        tmem_ld_32x32b_x16(tP + 32, pa);
        chunk(sb, pb, 1);
        tmem_ld_wait();
        tmem_ld_32x32b_x16(tS + 48, sb);
        tmem_ld_32x32b_x16(tP + 48, pb);
        chunk(sa, pa, 2);
        tmem_ld_wait();
        chunk(sb, pb, 3);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&pds_full[s]);
        if (ds_on) {              // warp 2 stores the tile: no math warp waits for the TMA engine
          fence_proxy_async_smem();
          mbar_arrive(&stg_full[wg]);
          ++stg_uses;
        }
      }
      if (!ok) break;
      g0 += d.iters;
      // end of the pass: the accumulators of this key tile are complete once every MMA has run
      if (!mbar_wait(acc_done, ps & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool live = key < T;
      bf16* krow = p.dk + b * p.dk_bs + (long long)min(key, T - 1) * p.dk_ts + kvh * p.dk_hs;
      bf16* vrow = p.dv + b * p.dv_bs + (long long)min(key, T - 1) * p.dv_ts + kvh * p.dv_hs;
      constexpr int kHalfCols = kD / 2;          // dK / dV columns each warpgroup stores
      if (d.iters > 0) {
        if (p.unrot_cos != nullptr) {
          const int pos = min(key, T - 1);
          store_row_unrot_from_tmem<kD>(tmem_base + lane_sel + kColDK, krow, half * (kD / 4), kD / 4,
                                        p.unrot_cos + pos, p.unrot_sin + pos, p.unrot_ld, live);
        } else {
          store_row_from_tmem(tmem_base + lane_sel + kColDK, krow, half * kHalfCols, (half + 1) * kHalfCols, live);
        }
        store_row_from_tmem(tmem_base + lane_sel + kColDV, vrow, half * kHalfCols, (half + 1) * kHalfCols, live);
      } else if (live) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int c = half * kHalfCols; c < (half + 1) * kHalfCols; c += 8) {
          *reinterpret_cast<uint4*>(krow + c) = z;
          *reinterpret_cast<uint4*>(vrow + c) = z;
        }
      }
      tc_fence_before();
      mbar_arrive(acc_free);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, int(*abort_flag)) == 0) p.status[1] = 311;
  }
}

// =================================================================== dK, dV with 128-query iterations
// The same work with a different schedule (head_dim 128). A tcgen05.mma of 64 columns costs about 62 clocks
// where its arithmetic needs 32, one of 128 columns about 78 for 64 (measured with back-to-back instructions),
// so the score products want N = 128. S^T and dP^T of a 128-query tile then take 128 tensor-memory columns
// each, which with the two 128-column accumulators is all there is: nothing is double-buffered. Instead the
// five products of consecutive iterations are interleaved so that the tensor pipe always has one to run while
// the math warps work on another:
//     tensor pipe:   dV(i)   S^T(i+1)   | dK(i)    dP^T(i+1) | dV(i+1) ...
//     math warps :   dS^T(i)            | P^T(i+1)           | dS^T(i+1) ...
// P^T(i) overwrites S^T(i) in place and is consumed by dV(i) before S^T(i+1) is written (the pipe runs the
// products in issue order); dS^T(i) overwrites dP^T(i) and is consumed by dK(i) before dP^T(i+1). Both math
// warpgroups work on every iteration, warpgroup w on query columns [64 w, 64 w + 64) of the tile: a thread owns
// one key row, computes P for its 64 columns, keeps it (packed bf16) in registers and forms dS from it when dP^T
// is there. Its packed columns go to the first 32 columns of its own 64 (columns [0, 32) and [64, 96) of the
// tile hold P^T: every k-step of the gradient products names its A address, so the gap does not matter).
constexpr int FKW_BQ = 128;                      // query rows per iteration
constexpr int FKW_TILE = FKW_BQ * FB_D * 2;      // 32 KiB
struct FdkwSmem {
  static constexpr int kK = 0, kV = FB_TILE, kQ = 2 * FB_TILE;             // stage s: Q_i (32 KiB), dO_i (32 KiB)
  static constexpr int kStage = kQ + 2 * 2 * FKW_TILE;                      // [2] dS^T staging tiles (one per warpgroup)
  static constexpr int kStats = kStage + 2 * FKV_STG;                       // stage s: lse2[128], delta * scale [128]
  static constexpr int kBar = kStats + 2 * 2 * FKW_BQ * 4;
  // kv_full, q_full[2], q_empty[2], st_full[2], s_full, dp_full, p_ready, ds_ready, acc_done, acc_free,
  // stg_full[2], stg_free[2] = 17
  static constexpr int kUsed = kBar + 17 * 8 + 16;
  // All the shared memory of an SM: the tiles leave less than the 1 KiB a worst-case alignment of the base would
  // take, so the kernel checks that what it needs fits behind the aligned base and reports an error otherwise.
  static constexpr int kTotal = 232448;
};
static_assert(FdkwSmem::kUsed <= FdkwSmem::kTotal, "dK/dV kernel: shared memory");

struct DkwPass {
  int n0, i_first, n_qt, iters;
};
__device__ __forceinline__ DkwPass dkw_pass(int ntile, int T, int R, int vlen) {
  DkwPass d;
  d.n0 = ntile * 128;
  d.i_first = ntile;                                          // first 128-query tile at / below the diagonal
  d.n_qt = (T + FKW_BQ - 1) / FKW_BQ - d.i_first;
  d.iters = (d.n0 < vlen) ? R * d.n_qt : 0;
  return d;
}

// P^T for 16 query columns of one key row, packed to bf16 pairs; lse2 points at the 16 per-query values.
template <bool kMask>
__device__ __forceinline__ void fb_p_chunk(const uint32_t (&rs)[16], uint32_t (&pk)[8], float sl2, const float* lse2,
                                           int q_base, int key, bool key_dead) {
#pragma unroll
  for (int e = 0; e < 16; e += 4) {
    const float4 l4 = *reinterpret_cast<const float4*>(lse2 + e);
    const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
    float pv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float pe = exp2f(fmaf(__uint_as_float(rs[e + u]), sl2, -lv[u]));
      if (kMask) {
        if (key_dead || key > q_base + e + u) pe = 0.f;
      }
      pv[u] = pe;
    }
#pragma unroll
    for (int u = 0; u < 4; u += 2) {
      const bf162 t0 = __floats2bfloat162_rn(pv[u], pv[u + 1]);
      pk[(e + u) >> 1] = *reinterpret_cast<const uint32_t*>(&t0);
    }
  }
}

// dS^T = P^T * (dP^T * scale - delta * scale) for the same 16 columns, from the packed P^T.
__device__ __forceinline__ void fb_ds_from_p_chunk(const uint32_t (&rp)[16], const uint32_t (&pk)[8], uint32_t (&dk)[8],
                                                   float scale, const float* dlt_s) {
#pragma unroll
  for (int e = 0; e < 16; e += 4) {
    const float4 d4 = *reinterpret_cast<const float4*>(dlt_s + e);
    const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
    for (int u = 0; u < 4; u += 2) {
      const float2 pf = __bfloat1622float2(*reinterpret_cast<const bf162*>(&pk[(e + u) >> 1]));
      const float d0 = pf.x * fmaf(__uint_as_float(rp[e + u]), scale, -dl[u]);
      const float d1 = pf.y * fmaf(__uint_as_float(rp[e + u + 1]), scale, -dl[u + 1]);
      const bf162 t1 = __floats2bfloat162_rn(d0, d1);
      dk[(e + u) >> 1] = *reinterpret_cast<const uint32_t*>(&t1);
    }
  }
}

__global__ void __launch_bounds__(FBT_THREADS, 1)
flash_bwd_dkv_wide_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                          const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                          const __grid_constant__ CUtensorMap tmDS, const FlashBwdTcParams p) {
  constexpr int kD = FB_D;
  extern __shared__ uint8_t fb_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fb_smem_raw) + 1023) & ~uintptr_t(1023));
  if (smem + FdkwSmem::kUsed > fb_smem_raw + FdkwSmem::kTotal) {      // the same for every thread of every CTA
    if (threadIdx.x == 0 && p.status != nullptr && atomicCAS(p.status, 0, int(ERR_BAD_ARGUMENT)) == 0) p.status[1] = 313;
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FdkwSmem::kBar);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;                    // [2]
  uint64_t* q_empty = q_full + 2;                 // [2]
  uint64_t* st_full = q_empty + 2;                // [2] statistics staged
  uint64_t* s_full = st_full + 2;                 // S^T of the iteration is in tensor memory
  uint64_t* dp_full = s_full + 1;                 // dP^T of the iteration is in tensor memory
  uint64_t* p_ready = dp_full + 1;                // every math thread has written its P^T columns
  uint64_t* ds_ready = p_ready + 1;               // ... its dS^T columns
  uint64_t* acc_done = ds_ready + 1;              // every MMA of a pass has completed
  uint64_t* acc_free = acc_done + 1;              // the dK / dV accumulators of a pass have been stored
  uint64_t* stg_full = acc_free + 1;              // [2]
  uint64_t* stg_free = stg_full + 2;              // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stg_free + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int pair, kvh, b;                               // grid mapping as in flash_bwd_dkv_tc_kernel
  {
    const int n_pairs = p.pairing ? (p.n_tiles + 1) / 2 : p.n_tiles;
    const int per_chunk = n_pairs * p.KVH * p.bchunk;
    const int chunk = int(blockIdx.x) / per_chunk, r = int(blockIdx.x) - chunk * per_chunk;
    const int hb = p.KVH * min(p.bchunk, p.B - chunk * p.bchunk);
    pair = r / hb;
    kvh = (r % hb) % p.KVH;
    b = chunk * p.bchunk + (r % hb) / p.KVH;
  }
  const int T = p.T;
  const int R = p.QH / p.KVH;
  const int vlen = p.valid_len ? checked_index(p.valid_len[b], T, p.status, 302) : T;
  const int tile_of_pass[2] = {pair, p.pairing ? p.n_tiles - 1 - pair : pair};
  const int n_pass = tile_of_pass[0] == tile_of_pass[1] ? 1 : 2;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); mbar_init(&st_full[s], 32); }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_ready, 256);
    mbar_init(ds_ready, 256);
    mbar_init(acc_done, 1);
    mbar_init(acc_free, 256);
    for (int s = 0; s < 2; ++s) { mbar_init(&stg_full[s], 128); mbar_init(&stg_free[s], 1); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmDO); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDS);
  }
  if (warp == 2) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColST = 0, kColDPT = 128, kColDV = 256, kColDK = 384;

  if (warp == 0) {
    if (lane == 0) {
      int g = 0;
      bool ok = true;
      for (int ps = 0; ps < n_pass && ok; ++ps) {
        const DkwPass d = dkw_pass(tile_of_pass[ps], T, R, vlen);
        if (d.iters == 0) continue;
        if (ps > 0) {             // K / V of the previous pass are read by its MMAs until they have all completed
          if (!mbar_wait(acc_done, (ps - 1) & 1, abort_flag)) break;
        }
        mbar_expect_tx(kv_full, 2 * FB_TILE);
        tma_load_4d(smem + FdkwSmem::kK, &tmK, kv_full, 0, kvh, d.n0, b);
        tma_load_4d(smem + FdkwSmem::kK + 16384, &tmK, kv_full, 64, kvh, d.n0, b);
        tma_load_4d(smem + FdkwSmem::kV, &tmV, kv_full, 0, kvh, d.n0, b);
        tma_load_4d(smem + FdkwSmem::kV + 16384, &tmV, kv_full, 64, kvh, d.n0, b);
        for (int it = 0; it < d.iters; ++it, ++g) {
          const int s = g & 1;
          const int h = kvh * R + it / d.n_qt;
          const int m0 = (d.i_first + it % d.n_qt) * FKW_BQ;
          if (!mbar_wait(&q_empty[s], ((g >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sQ = smem + FdkwSmem::kQ + s * 2 * FKW_TILE;
          uint8_t* sDO = sQ + FKW_TILE;
          mbar_expect_tx(&q_full[s], 2 * FKW_TILE);
          tma_load_4d(sQ, &tmQ, &q_full[s], 0, h, m0, b);
          tma_load_4d(sQ + 16384, &tmQ, &q_full[s], 64, h, m0, b);
          tma_load_4d(sDO, &tmDO, &q_full[s], 0, h, m0, b);
          tma_load_4d(sDO + 16384, &tmDO, &q_full[s], 64, h, m0, b);
        }
      }
    }
  } else if (warp == 3) {
    // stages the per-query statistics (lse in log2 units, delta * scale) of each query tile in shared memory
    int g = 0;
    bool ok = true;
    for (int ps = 0; ps < n_pass && ok; ++ps) {
      const DkwPass d = dkw_pass(tile_of_pass[ps], T, R, vlen);
      for (int it = 0; it < d.iters; ++it, ++g) {
        const int s = g & 1;
        const int h = kvh * R + it / d.n_qt;
        const int m0 = (d.i_first + it % d.n_qt) * FKW_BQ;
        if (!mbar_wait(&q_empty[s], ((g >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
        float* st = reinterpret_cast<float*>(smem + FdkwSmem::kStats + s * 2 * FKW_BQ * 4);
        // all eight loads in flight before the first store: one after the other (a store to shared memory may not
        // pass a later global load the compiler cannot tell apart from it) they cost four round trips to L2 per
        // iteration, which made this warp the slowest part of the kernel
        float lv[FKW_BQ / 32], dv[FKW_BQ / 32];
#pragma unroll
        for (int j = 0; j < FKW_BQ / 32; ++j) {
          const int row = m0 + lane + 32 * j;
          const size_t idx = (size_t(b) * p.QH + h) * T + min(row, T - 1);
          lv[j] = __ldg(p.lse + idx);
          dv[j] = __ldg(p.delta + idx);
        }
#pragma unroll
        for (int j = 0; j < FKW_BQ / 32; ++j) {
          const int r = lane + 32 * j;
          st[r] = (m0 + r < T) ? lv[j] * kFbLog2e : INFINITY;       // +inf => P = 0 for rows past T
          st[FKW_BQ + r] = (m0 + r < T) ? dv[j] * p.scale : 0.f;
        }
        mbar_arrive(&st_full[s]);
      }
    }
  } else if (warp == 2) {
    // stores the dS^T staging tiles of both warpgroups (a math warp that did this itself spent a quarter of
    // every iteration waiting for its warpgroup and for the TMA engine, and held the next P^T back)
    if (lane == 0 && p.ds != nullptr) {
      uint32_t uses = 0;
      bool ok = true;
      for (int ps = 0; ps < n_pass && ok; ++ps) {
        const DkwPass d = dkw_pass(tile_of_pass[ps], T, R, vlen);
        for (int it = 0; it < d.iters && ok; ++it, ++uses) {
          const int m0 = (d.i_first + it % d.n_qt) * FKW_BQ;
          for (int w = 0; w < 2; ++w) {
            if (!mbar_wait(&stg_full[w], uses & 1, abort_flag)) { ok = false; break; }
            tma_store_4d_ds(&tmDS, smem + FdkwSmem::kStage + w * FKV_STG, m0 + w * 64, kvh * R + it / d.n_qt, d.n0, b);
            tma_store_commit();
          }
          if (!ok) break;
          tma_store_wait_read<0>();
          mbar_arrive(&stg_free[0]);
          mbar_arrive(&stg_free[1]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, FKW_BQ, 0, 0);   // [128 keys x 128 q], K-major operands
      constexpr uint32_t idesc_g = umma_idesc_bf16(128, kD, 0, 1);       // [128 keys x d], B MN-major
      const uint32_t aK = smem_u32(smem + FdkwSmem::kK), aV = smem_u32(smem + FdkwSmem::kV);
      auto stage_q = [&](int g) { return smem_u32(smem + FdkwSmem::kQ + (g & 1) * 2 * FKW_TILE); };
      auto issue_s = [&](int g) {
        const uint32_t aQ = stage_q(g);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;       // 128-row tiles, 64-column halves
          umma_bf16_ss(tmem_base + kColST, umma_smem_desc(aK + off, 16, 1024), umma_smem_desc(aQ + off, 16, 1024),
                       idesc_s, kk != 0);
        }
        umma_commit(s_full);
      };
      auto issue_dp = [&](int g) {
        const uint32_t aDO = stage_q(g) + FKW_TILE;
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16_ss(tmem_base + kColDPT, umma_smem_desc(aV + off, 16, 1024), umma_smem_desc(aDO + off, 16, 1024),
                       idesc_s, kk != 0);
        }
        umma_commit(dp_full);
      };
      bool ok = true;
      int g0 = 0, kv_loads = 0;
      for (int ps = 0; ps < n_pass && ok; ++ps) {
        const DkwPass d = dkw_pass(tile_of_pass[ps], T, R, vlen);
        if (d.iters > 0) {
          if (!mbar_wait(kv_full, kv_loads & 1, abort_flag)) { ok = false; break; }
          ++kv_loads;
          if (!mbar_wait(&q_full[g0 & 1], (g0 >> 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_s(g0);
          issue_dp(g0);
          if (ps > 0) {           // the accumulators still hold the previous pass until its rows are stored
            if (!mbar_wait(acc_free, (ps - 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
          }
        }
        for (int it = 0; it < d.iters && ok; ++it) {
          const int g = g0 + it;
          const uint32_t aQ = stage_q(g), aDO = aQ + FKW_TILE;
          // dV += P^T dO: A = the packed P^T columns (k-step kk: 16 queries = 8 columns; queries 64.. sit at column
          // 64), B = dO read MN-major (16 query rows per k-step, 64-d halves 16 KiB apart)
          if (!mbar_wait(p_ready, g & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < FKW_BQ / 16; ++kk) {
            const uint32_t acol = kk < 4 ? kk * 8 : 64 + (kk - 4) * 8;
            umma_bf16_ts(tmem_base + kColDV, tmem_base + kColST + acol, umma_smem_desc(aDO + kk * 2048, 16384, 1024),
                         idesc_g, (it | kk) != 0);
          }
          if (it + 1 < d.iters) {   // S^T of the next tile may overwrite P^T once dV has read it: issue order
            if (!mbar_wait(&q_full[(g + 1) & 1], ((g + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            issue_s(g + 1);
          }
          if (!mbar_wait(ds_ready, g & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < FKW_BQ / 16; ++kk) {
            const uint32_t acol = kk < 4 ? kk * 8 : 64 + (kk - 4) * 8;
            umma_bf16_ts(tmem_base + kColDK, tmem_base + kColDPT + acol, umma_smem_desc(aQ + kk * 2048, 16384, 1024),
                         idesc_g, (it | kk) != 0);
          }
          umma_commit(&q_empty[g & 1]);
          if (it + 1 < d.iters) issue_dp(g + 1);
        }
        if (ok && d.iters == 0 && ps > 0) {
          if (!mbar_wait(acc_free, (ps - 1) & 1, abort_flag)) { ok = false; break; }
        }
        if (ok) umma_commit(acc_done);
        g0 += d.iters;
      }
    }
  } else if (warp >= 4) {
    const int q = warp & 3;
    const int wg = (warp - 4) >> 2;           // query columns [64 wg, 64 wg + 64) of every tile
    const int half = wg;                      // dK / dV columns this warpgroup stores at the end of a pass
    const uint32_t lane_sel = uint32_t(q * 32) << 16;
    const float sl2 = p.scale * kFbLog2e;
    uint8_t* stg_row = smem + FdkwSmem::kStage + wg * FKV_STG + (q * 32 + lane) * 128;
    const uint32_t swz = uint32_t(lane & 7);
    const bool ds_on = p.ds != nullptr;
    const uint32_t tS = tmem_base + lane_sel + kColST + wg * 64, tP = tmem_base + lane_sel + kColDPT + wg * 64;
    uint32_t stg_uses = 0;
    bool ok = true;
    int g0 = 0;
    for (int ps = 0; ps < n_pass && ok; ++ps) {
      const DkwPass d = dkw_pass(tile_of_pass[ps], T, R, vlen);
      const int n0 = d.n0;
      const int key = n0 + q * 32 + lane;
      const bool key_dead = key >= vlen;
      for (int it = 0; it < d.iters && ok; ++it) {
        const int g = g0 + it, s2 = g & 1;
        const int m0 = (d.i_first + it % d.n_qt) * FKW_BQ;
        const int qb = m0 + wg * 64;                                     // first query column of this warpgroup
        const float* st = reinterpret_cast<const float*>(smem + FdkwSmem::kStats + s2 * 2 * FKW_BQ * 4) + wg * 64;
        const bool need_mask = (m0 < n0 + 128) || (n0 + 128 > vlen);     // the diagonal tile or the padded tail
        uint32_t pk[4][8];                                               // this thread's P^T, 64 columns packed
        uint32_t ra[16], rb[16];
        if (!mbar_wait(&st_full[s2], (g >> 1) & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait(s_full, g & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        auto p_chunk = [&](const uint32_t (&rs)[16], int c) {
          if (need_mask) fb_p_chunk<true>(rs, pk[c], sl2, st + c * 16, qb + c * 16, key, key_dead);
          else fb_p_chunk<false>(rs, pk[c], sl2, st + c * 16, 0, 0, false);
          tmem_st_32x32b_x8(tS + c * 8, pk[c]);
        };
        tmem_ld_32x32b_x16(tS, ra);
        tmem_ld_wait();
        tmem_ld_32x32b_x16(tS + 16, rb);
        p_chunk(ra, 0);
        tmem_ld_wait();
        tmem_ld_32x32b_x16(tS + 32, ra);
        p_chunk(rb, 1);
        tmem_ld_wait();
        tmem_ld_32x32b_x16(tS + 48, rb);
        p_chunk(ra, 2);
        tmem_ld_wait();
        p_chunk(rb, 3);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(p_ready);
        // ---- dS^T from dP^T and the kept P^T
        if (!mbar_wait(dp_full, g & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (ds_on) {              // the store of this warpgroup's previous tile must have read the staging tile
          if (!mbar_wait(&stg_free[wg], (stg_uses & 1) ^ 1, abort_flag)) { ok = false; break; }
        }
        auto ds_chunk = [&](const uint32_t (&rp)[16], int c) {
          uint32_t dk_[8];
          fb_ds_from_p_chunk(rp, pk[c], dk_, p.scale, st + FKW_BQ + c * 16);
          tmem_st_32x32b_x8(tP + c * 8, dk_);
          if (ds_on) {            // 16 queries = two 16-byte chunks of this key's 128-byte staging row
            *reinterpret_cast<uint4*>(stg_row + ((uint32_t(2 * c) ^ swz) << 4)) = make_uint4(dk_[0], dk_[1], dk_[2], dk_[3]);
            *reinterpret_cast<uint4*>(stg_row + ((uint32_t(2 * c + 1) ^ swz) << 4)) = make_uint4(dk_[4], dk_[5], dk_[6], dk_[7]);
          }
        };
        tmem_ld_32x32b_x16(tP, ra);
        tmem_ld_wait();
        tmem_ld_32x32b_x16(tP + 16, rb);
        ds_chunk(ra, 0);
        tmem_ld_wait();
        tmem_ld_32x32b_x16(tP + 32, ra);
        ds_chunk(rb, 1);
        tmem_ld_wait();
        tmem_ld_32x32b_x16(tP + 48, rb);
        ds_chunk(ra, 2);
        tmem_ld_wait();
        ds_chunk(rb, 3);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(ds_ready);
        if (ds_on) {              // warp 2 stores the tile: no math warp waits for the TMA engine
          fence_proxy_async_smem();
          mbar_arrive(&stg_full[wg]);
          ++stg_uses;
        }
      }
      if (!ok) break;
      g0 += d.iters;
      // end of the pass: the accumulators of this key tile are complete once every MMA has run
      if (!mbar_wait(acc_done, ps & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool live = key < T;
      bf16* krow = p.dk + b * p.dk_bs + (long long)min(key, T - 1) * p.dk_ts + kvh * p.dk_hs;
      bf16* vrow = p.dv + b * p.dv_bs + (long long)min(key, T - 1) * p.dv_ts + kvh * p.dv_hs;
      constexpr int kHalfCols = kD / 2;          // dK / dV columns each warpgroup stores
      if (d.iters > 0) {
        if (p.unrot_cos != nullptr) {
          const int pos = min(key, T - 1);
          store_row_unrot_from_tmem<kD>(tmem_base + lane_sel + kColDK, krow, half * (kD / 4), kD / 4,
                                        p.unrot_cos + pos, p.unrot_sin + pos, p.unrot_ld, live);
        } else {
          store_row_from_tmem(tmem_base + lane_sel + kColDK, krow, half * kHalfCols, (half + 1) * kHalfCols, live);
        }
        store_row_from_tmem(tmem_base + lane_sel + kColDV, vrow, half * kHalfCols, (half + 1) * kHalfCols, live);
      } else if (live) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int c = half * kHalfCols; c < (half + 1) * kHalfCols; c += 8) {
          *reinterpret_cast<uint4*>(krow + c) = z;
          *reinterpret_cast<uint4*>(vrow + c) = z;
        }
      }
      tc_fence_before();
      mbar_arrive(acc_free);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, int(*abort_flag)) == 0) p.status[1] = 314;
  }
}

// One helper stream (and the two events that tie it to the caller's stream) per device.
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};
static SideStream* side_stream() {
  static std::mutex mu;
  static SideStream per_dev[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  SideStream& s = per_dev[dev];
  if (s.stream == nullptr) {
    if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess) return nullptr;
  }
  return &s;
}

int flash_bwd_dq_from_ds(const void* ds, const void* k, void* dq, const void* valid_len, const long long* ks,
                         const long long* dqs, int B, int T, int QH, int KVH, int D, int bchunk,
                         const float* unrot_cos, const float* unrot_sin, int unrot_ld, cudaStream_t st);

static int g_dkv_wide = 1;

// The wide dK/dV kernel needs all but 872 bytes of an SM's shared memory, so it only fits when the dynamic
// shared memory of a kernel starts within that many bytes of a 1 KiB boundary. That offset is a property of the
// platform (it was 0 on every B200 seen): it is measured once per device with a one-warp kernel, and where it
// does not fit head_dim 128 stays on the 64-query kernel.
__global__ void smem_base_probe_kernel(int* out) {
  extern __shared__ uint8_t probe_raw[];
  if (threadIdx.x == 0) *out = int(reinterpret_cast<uintptr_t>(probe_raw) & 1023);
}
static bool dkv_wide_fits() {
  static std::mutex mu;
  static int fits[64];            // 0 unknown, 1 yes, -1 no
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (fits[dev] == 0) {
    int* d = nullptr;
    int off = -1;
    if (cudaMalloc(&d, sizeof(int)) == cudaSuccess) {
      smem_base_probe_kernel<<<1, 32, 1024>>>(d);
      if (cudaMemcpy(&off, d, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) off = -1;
      cudaFree(d);
    }
    const int pad = off < 0 ? 1024 : (1024 - off) & 1023;        // bytes lost to the round-up of the base
    fits[dev] = (FdkwSmem::kUsed + pad <= FdkwSmem::kTotal) ? 1 : -1;
  }
  return fits[dev] > 0;
}
static int g_dkv_pairing = -1;      // -1: by the number of key tiles per SM; 0 / 1: forced (A/B runs)

}  // namespace b200

using namespace b200;

// Gradients w.r.t. (already rotated) q, k and v. delta [B,QH,T] = sum_d dO*O must have been
// computed (b200_flash_delta). strides: q, k, v, dout, dq, dk, dv (3 each: batch, token, head).
// With a workspace `ds_ws` of B * QH * Tp * Tp bf16 (Tp = T rounded up to 128) the dK/dV kernel also
// writes dS^T there and dQ is computed from it by a GEMM kernel (flash_attn_bwd_dq.cu) instead of the
// kernel that recomputes S and dP. With `unrot_cos` / `unrot_sin` (fp32 tables of the rotary embedding,
// transposed: [D / 2][unrot_ld], unrot_ld >= T) dq and dk are written with the inverse rotation applied, i.e.
// as gradients of the un-rotated q and k.
B200_API int b200_flash_bwd_tc(const void* q, const void* k, const void* v, const void* dout, const void* lse,
                               const void* delta, void* dq, void* dk, void* dv, const void* valid_len,
                               const long long* s, int B, int T, int QH, int KVH, int D, float scale, void* ds_ws,
                               const void* unrot_cos, const void* unrot_sin, int unrot_ld, cudaStream_t st) {
  if (B <= 0 || T <= 0) return 0;
  // head_dim 64 exists only in the form with a dS workspace (dK/dV kernel + dQ GEMM)
  if ((D != FB_D && D != 64) || QH % KVH != 0) return static_cast<int>(cudaErrorInvalidValue);
  if (D == 64 && ds_ws == nullptr) return static_cast<int>(cudaErrorInvalidValue);
  for (int i = 0; i < 21; ++i)
    if (s[i] % 8 != 0) return static_cast<int>(cudaErrorInvalidValue);
  const CUtensorMap* tq128 = get_tensor_map_bthd(q, B, T, QH, D, s[0], s[1], s[2], 128, 64);
  const CUtensorMap* tdo128 = get_tensor_map_bthd(dout, B, T, QH, D, s[9], s[10], s[11], 128, 64);
  const CUtensorMap* tq64 = get_tensor_map_bthd(q, B, T, QH, D, s[0], s[1], s[2], 64, 64);
  const CUtensorMap* tdo64 = get_tensor_map_bthd(dout, B, T, QH, D, s[9], s[10], s[11], 64, 64);
  const CUtensorMap* tk = get_tensor_map_bthd(k, B, T, KVH, D, s[3], s[4], s[5], 128, 64);
  const CUtensorMap* tv = get_tensor_map_bthd(v, B, T, KVH, D, s[6], s[7], s[8], 128, 64);
  if (!tq128 || !tdo128 || !tq64 || !tdo64 || !tk || !tv) return static_cast<int>(cudaErrorInvalidValue);
  FlashBwdTcParams p;
  p.dq = static_cast<bf16*>(dq); p.dk = static_cast<bf16*>(dk); p.dv = static_cast<bf16*>(dv);
  p.lse = static_cast<const float*>(lse); p.delta = static_cast<const float*>(delta);
  p.valid_len = static_cast<const int*>(valid_len);
  p.dq_bs = s[12]; p.dq_ts = s[13]; p.dq_hs = s[14];
  p.dk_bs = s[15]; p.dk_ts = s[16]; p.dk_hs = s[17];
  p.dv_bs = s[18]; p.dv_ts = s[19]; p.dv_hs = s[20];
  p.B = B; p.T = T; p.QH = QH; p.KVH = KVH; p.scale = scale; p.status = status_ptr();
  static bool configured = false;
  if (!configured) {
    B200_CHECK(cudaFuncSetAttribute(flash_bwd_dq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    FdqSmem::kTotal));
    B200_CHECK(cudaFuncSetAttribute(flash_bwd_dkv_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    FdkvSmem::kTotal));
    B200_CHECK(cudaFuncSetAttribute(flash_bwd_dkv_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    FdkvSmem::kTotal));
    B200_CHECK(cudaFuncSetAttribute(flash_bwd_dkv_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    FdkwSmem::kTotal));
    configured = true;
  }
  const int nt = (T + 127) / 128;
  p.n_tiles = nt;
  {
    // Q and dO of one batch element (bf16) plus its K and V; about two thirds of the L2 is budgeted
    const double per_batch = 2.0 * T * D * (2.0 * QH + 2.0 * KVH);
    int bc = int(80.0e6 / per_batch);
    p.bchunk = bc < 1 ? 1 : (bc > B ? B : bc);
  }
  // The two kernels are independent (both only read delta). dK/dV has few, long CTAs and, when they
  // number only a few per SM, ends in a ragged tail; dQ has many short ones. Running dQ on a second
  // stream then lets its CTAs take the SMs the dK/dV kernel leaves idle while its last CTAs finish.
  // With many dK/dV CTAs per SM there is no tail worth filling and the kernels run back to back.
  p.ds = static_cast<bf16*>(ds_ws);
  p.ds_tp = (long long)nt * 128;
  p.unrot_cos = static_cast<const float*>(unrot_cos);
  p.unrot_sin = unrot_cos != nullptr ? static_cast<const float*>(unrot_sin) : nullptr;
  p.unrot_ld = unrot_ld;
  if (p.unrot_cos != nullptr && (p.unrot_sin == nullptr || unrot_ld < T)) return static_cast<int>(cudaErrorInvalidValue);
  const CUtensorMap* tds = tk;           // placeholder when no workspace is given (never dereferenced then)
  if (ds_ws != nullptr) {
    const unsigned long long Tp = (unsigned long long)nt * 128;
    tds = get_tensor_map_bthd(ds_ws, B, Tp, QH, Tp, (unsigned long long)QH * Tp * Tp, Tp, Tp * Tp, 128, 64);
    if (!tds) return static_cast<int>(cudaErrorInvalidValue);
  }
  // Between one and three key tiles per SM: pair a long and a short one per CTA (equal work, one balanced wave:
  // 0.32 against 0.38 ms at 256 tiles). Fewer tiles than SMs: one per CTA, every tile gets an SM of its own (0.13
  // against 0.15 ms at 128 tiles); many tiles per SM: one per CTA, longest first.
  const int n_key_tiles = nt * KVH * B;
  p.pairing = g_dkv_pairing >= 0 ? g_dkv_pairing : ((n_key_tiles > num_sms() && n_key_tiles < 3 * num_sms()) ? 1 : 0);
  const int dkv_ctas = (p.pairing ? (nt + 1) / 2 : nt) * KVH * B;
  if (D == 128 && g_dkv_wide && dkv_wide_fits())
    flash_bwd_dkv_wide_kernel<<<dkv_ctas, FBT_THREADS, FdkwSmem::kTotal, st>>>(*tq128, *tdo128, *tk, *tv, *tds, p);
  else if (D == 128)
    flash_bwd_dkv_tc_kernel<128><<<dkv_ctas, FBT_THREADS, FdkvSmem::kTotal, st>>>(*tq64, *tdo64, *tk, *tv, *tds, p);
  else
    flash_bwd_dkv_tc_kernel<64><<<dkv_ctas, FBT_THREADS, FdkvSmem::kTotal, st>>>(*tq64, *tdo64, *tk, *tv, *tds, p);
  B200_CHECK(cudaGetLastError());
  if (ds_ws != nullptr) return flash_bwd_dq_from_ds(ds_ws, k, dq, valid_len, s + 3, s + 12, B, T, QH, KVH, D, p.bchunk,
                                                      p.unrot_cos, p.unrot_sin, p.unrot_ld, st);
  if (dkv_ctas >= 3 * num_sms()) {
    flash_bwd_dq_tc_kernel<<<nt * QH * B, FBT_THREADS, FdqSmem::kTotal, st>>>(*tq128, *tdo128, *tk, *tv, p);
    return static_cast<int>(cudaGetLastError());
  }
  SideStream* side = side_stream();
  if (side == nullptr) return static_cast<int>(cudaErrorUnknown);
  B200_CHECK(cudaEventRecord(side->fork, st));
  B200_CHECK(cudaStreamWaitEvent(side->stream, side->fork, 0));
  flash_bwd_dq_tc_kernel<<<nt * QH * B, FBT_THREADS, FdqSmem::kTotal, side->stream>>>(*tq128, *tdo128, *tk, *tv, p);
  B200_CHECK(cudaGetLastError());
  B200_CHECK(cudaEventRecord(side->join, side->stream));
  B200_CHECK(cudaStreamWaitEvent(st, side->join, 0));
  return 0;
}

// 1 (default): head_dim 128 runs the dK/dV kernel with 128-query iterations (flash_bwd_dkv_wide_kernel); 0: the
// kernel with double-buffered 64-query iterations. Returns the previous setting; a negative argument only reads it.
B200_API int b200_flash_bwd_wide(int on) {
  const int old = g_dkv_wide;
  if (on >= 0) g_dkv_wide = on != 0;
  return old;
}

// Key-tile pairing of the dK/dV kernels: -1 chooses by the number of key tiles per SM (the default), 0 gives every
// CTA one key tile (grid ordered longest first), 1 gives every CTA tiles i and n - 1 - i. Returns the previous value.
B200_API int b200_flash_bwd_pairing(int mode) {
  const int old = g_dkv_pairing;
  if (mode >= -1 && mode <= 1) g_dkv_pairing = mode;
  return old;
}

// 1 when head_dim 128 runs the 128-query dK/dV kernel on the current device (switched on and its shared memory fits).
B200_API int b200_flash_bwd_wide_active() { return (g_dkv_wide && dkv_wide_fits()) ? 1 : 0; }
