// dQ of causal GQA flash attention as a plain tcgen05 GEMM over stored dS (head_dim 128).
//
// The dK/dV kernel (flash_attn_bwd_tc.cu) has every dS^T tile in registers as packed bf16 anyway; when
// it is given a workspace it also writes them to global memory as dS^T[b][h][key][query] (query
// contiguous, row pitch Tp = T rounded up to 128). dQ[q, :] = sum over keys of dS[q, key] * K[key, :]
// is then a GEMM whose A operand is that matrix read MN-major (M = query) and whose B operand is the
// K tile read MN-major (N = d): no scores, no exponentials, no row statistics are recomputed, which
// the dQ kernel that works from Q, K, V and dO has to do (3 MMAs and a softmax-gradient pass per
// tile instead of this kernel's one MMA).
//
// One CTA per (128-query tile, head, batch element): warp 0 streams dS^T and K of the keys at or below the
// diagonal, 64 keys at a time, through a 3-stage TMA ring (32 KiB per stage), warp 1 issues the MMAs into
// a 128 x 128 fp32 accumulator in tensor memory, warps 2..5 convert and store the tile. With 96 KiB of
// shared memory and 128 tensor-memory columns two CTAs share an SM: one streams while the other is in its
// prologue or stores its tile (with one 192 KiB CTA per SM those phases - about a third of a CTA's life
// at T = 2048 - left the memory system idle). The kernel is bound by reading dS (T^2 / 2 bf16 per head)
// from HBM. Every wait is bounded (see ptx.cuh).
#include "common.cuh"
#include "ptx.cuh"
#include "flash_rope_epilogue.cuh"

namespace b200 {

constexpr int DQG_THREADS = 192;
constexpr int DQG_STAGES = 3;
constexpr int DQG_KEYS = 64;                            // keys per stage
constexpr int DQG_TILE = DQG_KEYS * 128 * 2;            // 16 KiB: 64 keys x 128 queries of dS^T, 64 keys x 128 d of K
constexpr int DQG_BOX = DQG_KEYS * 64 * 2;              // 8 KiB: one TMA box, 64 keys x 64 contiguous elements
constexpr int DQG_STAGE_BYTES = 2 * DQG_TILE;

struct DqGemmParams {
  bf16* dq;
  const int* valid_len;
  long long dq_bs, dq_ts, dq_hs;
  int B, T, QH, KVH;
  int n_tiles;           // 128-row tiles per sequence
  int bchunk;            // batch elements whose K stays in L2 together
  const float* unrot_cos;   // optional fp32 rotary tables, transposed [kD / 2][unrot_ld]: dQ leaves with the
  const float* unrot_sin;   // inverse rotation applied
  int unrot_ld;
  int* status;
};

struct DqGemmSmem {
  static constexpr int kBar = DQG_STAGES * DQG_STAGE_BYTES;
  // full[3], empty[3], done = 7 barriers
  static constexpr int kTotal = kBar + 7 * 8 + 16 + 1024;
};

// kD: head dimension (128, or 64: one 64-column box of K per key tile, N = 64, 64 output columns).
template <int kD>
__global__ void __launch_bounds__(DQG_THREADS, 2)
flash_bwd_dq_gemm_kernel(const __grid_constant__ CUtensorMap tmDS, const __grid_constant__ CUtensorMap tmK,
                         const DqGemmParams p) {
  extern __shared__ uint8_t dqg_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dqg_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + DqGemmSmem::kBar);
  uint64_t* empty = full + DQG_STAGES;
  uint64_t* done = empty + DQG_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 1-D grid over chunks of p.bchunk batch elements; inside a chunk the longest rows come first
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
  const int vlen = p.valid_len ? checked_index(p.valid_len[b], T, p.status, 303) : T;
  // 64-key steps: everything up to the end of the diagonal tile, cut at the valid length
  const int n_tiles = min(2 * (mtile + 1), (max(vlen, 1) + DQG_KEYS - 1) / DQG_KEYS);

  if (threadIdx.x == 0) {
    for (int s = 0; s < DQG_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmDS);
    tma_prefetch_desc(&tmK);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % DQG_STAGES;
        if (!mbar_wait(&empty[s], ((j / DQG_STAGES) & 1) ^ 1, abort_flag)) break;
        uint8_t* sA = smem + s * DQG_STAGE_BYTES;
        uint8_t* sK = sA + DQG_TILE;
        mbar_expect_tx(&full[s], DQG_TILE + DQG_KEYS * kD * 2);
        // dS^T: key rows j * 64 .., query columns m0 .. (two boxes of 64 queries); K: the same key rows
        tma_load_4d(sA, &tmDS, &full[s], m0, h, j * DQG_KEYS, b);
        tma_load_4d(sA + DQG_BOX, &tmDS, &full[s], m0 + 64, h, j * DQG_KEYS, b);
        tma_load_4d(sK, &tmK, &full[s], 0, kvh, j * DQG_KEYS, b);
        if (kD == 128) tma_load_4d(sK + DQG_BOX, &tmK, &full[s], 64, kvh, j * DQG_KEYS, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // A = dS^T [64 keys (k) x 128 queries (m)], B = K [64 keys (k) x 128 d (n)]: both MN-major, 64-element
      // chunks of the contiguous dimension one box (8 KiB) apart, 16 key rows per k-step (2 KiB)
      constexpr uint32_t idesc = umma_idesc_bf16(128, kD, 1, 1);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % DQG_STAGES;
        if (!mbar_wait(&full[s], (j / DQG_STAGES) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t aA = smem_u32(smem + s * DQG_STAGE_BYTES), aK = aA + DQG_TILE;
#pragma unroll
        for (int kk = 0; kk < DQG_KEYS / 16; ++kk)
          umma_bf16_ss(tmem_base, umma_smem_desc(aA + kk * 2048, DQG_BOX, 1024),
                       umma_smem_desc(aK + kk * 2048, DQG_BOX, 1024), idesc, (j | kk) != 0);
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(done);
    }
  } else {
    const int q = warp & 3;
    const int row = m0 + q * 32 + lane;
    const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16);
    if (mbar_wait(done, 0, abort_flag)) {
      tc_fence_after();
      const int pos = min(row, T - 1);
      bf16* grow = p.dq + b * p.dq_bs + (long long)pos * p.dq_ts + h * p.dq_hs;
      if (p.unrot_cos != nullptr) {
        store_row_unrot_from_tmem<kD>(taddr, grow, 0, kD / 2, p.unrot_cos + pos, p.unrot_sin + pos, p.unrot_ld, row < T);
      } else {
#pragma unroll 1
      for (int c = 0; c < kD; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c, r);     // warp-collective: every lane takes part, rows past T do not store
        tmem_ld_wait();
        if (row < T) {
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
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, int(*abort_flag)) == 0) p.status[1] = 312;
  }
}

// dq <- dS (as written by the dK/dV kernel into `ds`, [B][QH][Tp][Tp] bf16 with Tp = T rounded up to
// 128) times K. Strides in elements: k (batch, token, head), dq (batch, token, head).
int flash_bwd_dq_from_ds(const void* ds, const void* k, void* dq, const void* valid_len, const long long* ks,
                         const long long* dqs, int B, int T, int QH, int KVH, int D, int bchunk,
                         const float* unrot_cos, const float* unrot_sin, int unrot_ld, cudaStream_t st) {
  if (D != 128 && D != 64) return static_cast<int>(cudaErrorInvalidValue);
  const int nt = (T + 127) / 128;
  const unsigned long long Tp = (unsigned long long)nt * 128;
  const CUtensorMap* tds =
      get_tensor_map_bthd(ds, B, Tp, QH, Tp, (unsigned long long)QH * Tp * Tp, Tp, Tp * Tp, DQG_KEYS, 64);
  const CUtensorMap* tk = get_tensor_map_bthd(k, B, T, KVH, D, ks[0], ks[1], ks[2], DQG_KEYS, 64);
  if (!tds || !tk) return static_cast<int>(cudaErrorInvalidValue);
  DqGemmParams p;
  p.dq = static_cast<bf16*>(dq);
  p.valid_len = static_cast<const int*>(valid_len);
  p.dq_bs = dqs[0]; p.dq_ts = dqs[1]; p.dq_hs = dqs[2];
  p.B = B; p.T = T; p.QH = QH; p.KVH = KVH; p.n_tiles = nt; p.bchunk = bchunk < 1 ? 1 : bchunk;
  p.unrot_cos = unrot_cos; p.unrot_sin = unrot_sin; p.unrot_ld = unrot_ld;
  p.status = status_ptr();
  static bool configured = false;
  if (!configured) {
    B200_CHECK(cudaFuncSetAttribute(flash_bwd_dq_gemm_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    DqGemmSmem::kTotal));
    B200_CHECK(cudaFuncSetAttribute(flash_bwd_dq_gemm_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    DqGemmSmem::kTotal));
    configured = true;
  }
  if (D == 128)
    flash_bwd_dq_gemm_kernel<128><<<nt * QH * B, DQG_THREADS, DqGemmSmem::kTotal, st>>>(*tds, *tk, p);
  else
    flash_bwd_dq_gemm_kernel<64><<<nt * QH * B, DQG_THREADS, DqGemmSmem::kTotal, st>>>(*tds, *tk, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace b200
