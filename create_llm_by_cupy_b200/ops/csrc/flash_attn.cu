// Causal grouped-query flash attention, forward and backward, with the rotary embedding fused
// into the tile loads (Q and K are rotated on their way from global to shared memory; dQ and dK
// are un-rotated in registers before they are stored). No [T, T] tensor is ever materialised
// and the log-sum-exp is the only thing the forward pass keeps besides O.
//
// Layout: Q/K/V/O are addressed as base + b*batch_stride + t*token_stride + h*head_stride + d,
// so the kernels read Q, K and V straight out of the packed [M, K|Q|V] projection buffer.
// Query head h uses KV head h / (QH / KVH).
//
// The backward pass is split into two kernels, each shaped like the forward one:
//   flash_bwd_dkv : one CTA per 64-key tile, loops over the query tiles at or below the diagonal
//                   for every query head of the group, accumulating dK and dV in registers;
//   flash_bwd_dq  : one CTA per 128-query tile, loops over key tiles, accumulating dQ.
// Neither needs atomics or an fp32 dQ scratch buffer; the price is recomputing S and dP twice.
//
// Reference counterparts: cupy_flash_gqa_forward / backward (model/flash_attention.py:51-176),
// the Triton forward (model/flash_attention.py:195-282) and apply_rotary_pos_emb_inplace
// (model/fast_layers.py:27-61). Tensor-core path: mma.sync m16n8k16 (bf16, fp32 accumulate).
#include "common.cuh"

namespace b200 {

struct FlashParams {
  const bf16* q; const bf16* k; const bf16* v;
  bf16* o;
  const bf16* dout;     // bwd
  bf16* dq; bf16* dk; bf16* dv;
  float* lse;           // [B, QH, T]
  float* delta;         // [B, QH, T]  sum_d dO*O (bwd)
  const int* valid_len; // [B] or null: keys >= valid_len[b] are masked
  const float* rcos; const float* rsin;   // [T, D/2] or null when RoPE is off
  long long q_bs, q_ts, q_hs;
  long long k_bs, k_ts, k_hs;
  long long v_bs, v_ts, v_hs;
  long long o_bs, o_ts, o_hs;
  long long do_bs, do_ts, do_hs;
  long long dq_bs, dq_ts, dq_hs;
  long long dk_bs, dk_ts, dk_hs;
  long long dv_bs, dv_ts, dv_hs;
  int B, T, QH, KVH;
  float scale;
};

__device__ __forceinline__ uint32_t smem_u32_generic(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mma / ldmatrix helpers
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  bf162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

// Shared-memory tile of ROWS x D bf16, rows of D/8 16-byte chunks, chunk index XOR-swizzled so
// that the 8 rows one ldmatrix phase touches fall into distinct bank groups.
template <int D>
__device__ __forceinline__ int swz(int row, int chunk) {
  return (D >= 64) ? (chunk ^ (row & 7)) : (chunk ^ ((row >> 1) & 3));
}
template <int D>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
  return base + uint32_t(row * (D * 2) + swz<D>(row, chunk) * 16);
}

// A-operand fragments (16 rows x 16 k) of a row-major tile: rows r0.., k chunk pair kc (16 k = 2 chunks).
template <int D>
__device__ __forceinline__ void lds_a(uint32_t (&a)[4], uint32_t base, int r0, int kstep, int lane) {
  const int row = r0 + (lane & 7) + ((lane >> 3) & 1) * 8;
  const int chunk = kstep * 2 + (lane >> 4);
  ldsm_x4(a, tile_addr<D>(base, row, chunk));
}
// B-operand fragments for C = A * Tile^T: tile rows are the n index (16 of them from n0), k along
// the row. r[0],r[1] = (b0,b1) of n-tile n0..n0+7 ; r[2],r[3] = (b0,b1) of n-tile n0+8..n0+15.
template <int D>
__device__ __forceinline__ void lds_b_nt(uint32_t (&r)[4], uint32_t base, int n0, int kstep, int lane) {
  const int i = lane >> 3;
  const int row = n0 + (lane & 7) + (i >> 1) * 8;
  const int chunk = kstep * 2 + (i & 1);
  ldsm_x4(r, tile_addr<D>(base, row, chunk));
}
// B-operand fragments for C = A * Tile: tile rows are the k index (16 of them from k0), n along
// the row (16 of them from chunk pair nc). r[0],r[1] = (b0,b1) of n-tile 2*nc ; r[2],r[3] of 2*nc+1.
template <int D>
__device__ __forceinline__ void lds_b_nn(uint32_t (&r)[4], uint32_t base, int k0, int nc, int lane) {
  const int i = lane >> 3;
  const int row = k0 + (lane & 7) + (i & 1) * 8;
  const int chunk = nc * 2 + (i >> 1);
  ldsm_x4_t(r, tile_addr<D>(base, row, chunk));
}
// ---------------------------------------------------------------- tile loads (global -> regs -> smem)
// A tile of ROWS x D is split into items (row, jc): the 16-byte chunk jc of the first half of the
// head dim and its rotary partner jc + D/16. NI = items per thread.
template <int ROWS, int D, int THREADS>
struct TileLoader {
  static constexpr int kHalfChunks = D / 16;
  static constexpr int kItems = ROWS * kHalfChunks;
  static constexpr int NI = (kItems + THREADS - 1) / THREADS;
  uint4 lo[NI], hi[NI];

  __device__ __forceinline__ void load(const bf16* base, long long row_stride, int row0, int row_limit, int tid) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int it = tid + i * THREADS;
      const int row = it / kHalfChunks, jc = it % kHalfChunks;
      if (it < kItems && row0 + row < row_limit) {
        const bf16* p = base + (long long)(row0 + row) * row_stride + jc * 8;
        lo[i] = *reinterpret_cast<const uint4*>(p);
        hi[i] = *reinterpret_cast<const uint4*>(p + D / 2);
      } else {
        lo[i] = make_uint4(0, 0, 0, 0);
        hi[i] = make_uint4(0, 0, 0, 0);
      }
    }
  }
  // sign = +1 rotates (forward), -1 un-rotates.
  template <bool ROPE>
  __device__ __forceinline__ void store(uint32_t smem_base, const float* rcos, const float* rsin, int row0, int T,
                                        int tid) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int it = tid + i * THREADS;
      if (it >= kItems) continue;
      const int row = it / kHalfChunks, jc = it % kHalfChunks;
      uint4 a = lo[i], b = hi[i];
      if (ROPE) {
        const int pos = min(row0 + row, T - 1);
        const float4* c4 = reinterpret_cast<const float4*>(rcos + size_t(pos) * (D / 2) + jc * 8);
        const float4* s4 = reinterpret_cast<const float4*>(rsin + size_t(pos) * (D / 2) + jc * 8);
        const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
        const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        bf162* pa = reinterpret_cast<bf162*>(&a);
        bf162* pb = reinterpret_cast<bf162*>(&b);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x1 = __bfloat1622float2(pa[e]);
          const float2 x2 = __bfloat1622float2(pb[e]);
          pa[e] = __floats2bfloat162_rn(x1.x * cs[2 * e] - x2.x * sn[2 * e], x1.y * cs[2 * e + 1] - x2.y * sn[2 * e + 1]);
          pb[e] = __floats2bfloat162_rn(x2.x * cs[2 * e] + x1.x * sn[2 * e], x2.y * cs[2 * e + 1] + x1.y * sn[2 * e + 1]);
        }
      }
      asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(tile_addr<D>(smem_base, row, jc)), "r"(a.x), "r"(a.y),
                   "r"(a.z), "r"(a.w));
      asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(tile_addr<D>(smem_base, row, jc + kHalfChunks)),
                   "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w));
    }
  }
};

// Un-rotate (inverse RoPE) an accumulator held in the mma C layout: acc[nt][0..1] = (row g, cols
// nt*8 + 2t, +1), acc[nt][2..3] = (row g+8, same cols). Pair (j, j + D/2) = n-tiles nt and nt + D/16.
template <int D>
__device__ __forceinline__ void unrotate_acc(float (&acc)[D / 8][4], const float* rcos, const float* rsin, int pos_lo,
                                             int pos_hi, int T, int lane) {
  const int t = lane & 3;
  const int pl = min(pos_lo, T - 1), ph = min(pos_hi, T - 1);
#pragma unroll
  for (int nt = 0; nt < D / 16; ++nt) {
    const int j = nt * 8 + 2 * t;
    const float2 cl = *reinterpret_cast<const float2*>(rcos + size_t(pl) * (D / 2) + j);
    const float2 sl = *reinterpret_cast<const float2*>(rsin + size_t(pl) * (D / 2) + j);
    const float2 ch = *reinterpret_cast<const float2*>(rcos + size_t(ph) * (D / 2) + j);
    const float2 sh = *reinterpret_cast<const float2*>(rsin + size_t(ph) * (D / 2) + j);
    float* a = acc[nt];
    float* b = acc[nt + D / 16];
    // forward: y1 = x1 c - x2 s ; y2 = x2 c + x1 s.  gradient / inverse: x1 = y1 c + y2 s ; x2 = y2 c - y1 s
    float y1, y2;
    y1 = a[0]; y2 = b[0]; a[0] = y1 * cl.x + y2 * sl.x; b[0] = y2 * cl.x - y1 * sl.x;
    y1 = a[1]; y2 = b[1]; a[1] = y1 * cl.y + y2 * sl.y; b[1] = y2 * cl.y - y1 * sl.y;
    y1 = a[2]; y2 = b[2]; a[2] = y1 * ch.x + y2 * sh.x; b[2] = y2 * ch.x - y1 * sh.x;
    y1 = a[3]; y2 = b[3]; a[3] = y1 * ch.y + y2 * sh.y; b[3] = y2 * ch.y - y1 * sh.y;
  }
}

// Store a 16-row x D accumulator (C layout) of one warp as bf16 through a warp-private staging
// area (row-major, D*2 bytes per row, swizzled) so that global stores are 16 bytes wide.
template <int D>
__device__ __forceinline__ void store_acc_rows(const float (&acc)[D / 8][4], uint32_t stage_base, uint8_t* stage_ptr,
                                               bf16* gbase, long long row_stride, int row0, int row_limit, int lane,
                                               float mul_lo, float mul_hi) {
  const int g = lane >> 2, t = lane & 3;
  __syncwarp();
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    const uint32_t v0 = pack_bf16(acc[nt][0] * mul_lo, acc[nt][1] * mul_lo);
    const uint32_t v1 = pack_bf16(acc[nt][2] * mul_hi, acc[nt][3] * mul_hi);
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(tile_addr<D>(stage_base, g, nt) + t * 4), "r"(v0));
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(tile_addr<D>(stage_base, g + 8, nt) + t * 4), "r"(v1));
  }
  __syncwarp();
  constexpr int kChunks = D / 8;
  for (int it = lane; it < 16 * kChunks; it += 32) {
    const int row = it / kChunks, c = it % kChunks;
    if (row0 + row < row_limit) {
      const uint4 val = *reinterpret_cast<const uint4*>(stage_ptr + row * (D * 2) + swz<D>(row, c) * 16);
      *reinterpret_cast<uint4*>(gbase + (long long)(row0 + row) * row_stride + c * 8) = val;
    }
  }
  __syncwarp();
}

constexpr int FA_BM = 128;     // query rows per CTA (8 warps x 16)
constexpr int FA_BN = 64;      // keys per iteration
constexpr int FA_THREADS = 256;
constexpr float kLog2e = 1.4426950408889634f;

// ================================================================= forward
template <int D, bool ROPE>
__global__ void __launch_bounds__(FA_THREADS, 1) flash_fwd_kernel(const FlashParams p) {
  extern __shared__ __align__(128) uint8_t fa_smem[];
  uint8_t* sQ = fa_smem;                               // FA_BM x D  (re-used as the O staging area)
  uint8_t* sK = sQ + FA_BM * D * 2;                    // FA_BN x D
  uint8_t* sV = sK + FA_BN * D * 2;                    // FA_BN x D
  const uint32_t aQ = smem_u32_generic(sQ), aK = smem_u32_generic(sK), aV = smem_u32_generic(sV);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int mtile = gridDim.x - 1 - blockIdx.x;        // heavy (late) tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.QH / p.KVH);
  const int m0 = mtile * FA_BM;
  const int T = p.T;
  const int vlen = p.valid_len ? min(p.valid_len[b], T) : T;

  const bf16* qb = p.q + b * p.q_bs + h * p.q_hs;
  const bf16* kb = p.k + b * p.k_bs + kvh * p.k_hs;
  const bf16* vb = p.v + b * p.v_bs + kvh * p.v_hs;

  {
    TileLoader<FA_BM, D, FA_THREADS> lq;
    lq.load(qb, p.q_ts, m0, T, tid);
    lq.template store<ROPE>(aQ, p.rcos, p.rsin, m0, T, tid);
  }
  TileLoader<FA_BN, D, FA_THREADS> lk, lv;
  const int n_tiles = (min(m0 + FA_BM, T) + FA_BN - 1) / FA_BN;
  lk.load(kb, p.k_ts, 0, T, tid);
  lv.load(vb, p.v_ts, 0, T, tid);
  lk.template store<ROPE>(aK, p.rcos, p.rsin, 0, T, tid);
  lv.template store<false>(aV, nullptr, nullptr, 0, T, tid);
  __syncthreads();

  uint32_t qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) lds_a<D>(qf[ks], aQ, warp * 16, ks, lane);

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  const float sl2 = p.scale * kLog2e;
  const int qrow_lo = m0 + warp * 16 + g, qrow_hi = qrow_lo + 8;

  for (int j = 0; j < n_tiles; ++j) {
    const int n0 = j * FA_BN;
    if (j + 1 < n_tiles) {
      lk.load(kb, p.k_ts, n0 + FA_BN, T, tid);
      lv.load(vb, p.v_ts, n0 + FA_BN, T, tid);
    }
    float s[FA_BN / 8][4];
#pragma unroll
    for (int i = 0; i < FA_BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < FA_BN / 16; ++np) {
        uint32_t r[4];
        lds_b_nt<D>(r, aK, np * 16, ks, lane);
        mma_bf16(s[2 * np], qf[ks], r[0], r[1]);
        mma_bf16(s[2 * np + 1], qf[ks], r[2], r[3]);
      }
    }
    // mask (only tiles that touch the diagonal or the valid-length edge)
    const bool need_mask = (n0 + FA_BN - 1 > m0 + warp * 16) || (n0 + FA_BN > vlen);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < FA_BN / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[i][e] * sl2;
        if (need_mask) {
          const int key = n0 + i * 8 + 2 * t4 + (e & 1);
          const int qr = (e < 2) ? qrow_lo : qrow_hi;
          if (key > qr || key >= vlen) v = -INFINITY;
        }
        s[i][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float mnew = fmaxf(mrow[r], mx[r]);
      msafe[r] = (mnew == -INFINITY) ? 0.f : mnew;
      corr[r] = exp2f(mrow[r] - msafe[r]);
      mrow[r] = mnew;
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pf[FA_BN / 16][4];
#pragma unroll
    for (int i = 0; i < FA_BN / 8; ++i) {
      const float p0 = exp2f(s[i][0] - msafe[0]), p1 = exp2f(s[i][1] - msafe[0]);
      const float p2 = exp2f(s[i][2] - msafe[1]), p3 = exp2f(s[i][3] - msafe[1]);
      rs[0] += p0 + p1;
      rs[1] += p2 + p3;
      pf[i >> 1][(i & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) lrow[r] = lrow[r] * corr[r] + rs[r];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0];
      o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < FA_BN / 16; ++kk) {
#pragma unroll
      for (int nc = 0; nc < D / 16; ++nc) {
        uint32_t r[4];
        lds_b_nn<D>(r, aV, kk * 16, nc, lane);
        mma_bf16(o[2 * nc], pf[kk], r[0], r[1]);
        mma_bf16(o[2 * nc + 1], pf[kk], r[2], r[3]);
      }
    }
    __syncthreads();
    if (j + 1 < n_tiles) {
      lk.template store<ROPE>(aK, p.rcos, p.rsin, n0 + FA_BN, T, tid);
      lv.template store<false>(aV, nullptr, nullptr, n0 + FA_BN, T, tid);
    }
    __syncthreads();
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
  }
  const float inv0 = lrow[0] > 0.f ? 1.f / lrow[0] : 0.f;
  const float inv1 = lrow[1] > 0.f ? 1.f / lrow[1] : 0.f;
  if (t4 == 0) {
    float* lse = p.lse + (size_t(b) * p.QH + h) * T;
    if (qrow_lo < T) lse[qrow_lo] = (lrow[0] > 0.f) ? mrow[0] * 0.6931471805599453f + logf(lrow[0]) : -INFINITY;
    if (qrow_hi < T) lse[qrow_hi] = (lrow[1] > 0.f) ? mrow[1] * 0.6931471805599453f + logf(lrow[1]) : -INFINITY;
  }
  // all warps are past their last read of sQ (fragments are in registers since before the loop)
  bf16* ob = p.o + b * p.o_bs + h * p.o_hs;
  store_acc_rows<D>(o, aQ + warp * 16 * D * 2, sQ + warp * 16 * D * 2, ob, p.o_ts, m0 + warp * 16, T, lane, inv0, inv1);
}

// ================================================================= backward: delta = sum_d dO * O
__global__ void flash_delta_kernel(const FlashParams p, int D) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int total = p.B * p.QH * p.T;
  if (warp >= total) return;
  const int t = warp % p.T, h = (warp / p.T) % p.QH, b = warp / (p.T * p.QH);
  const bf16* o = p.o + b * p.o_bs + (long long)t * p.o_ts + h * p.o_hs;
  const bf16* d = p.dout + b * p.do_bs + (long long)t * p.do_ts + h * p.do_hs;
  float s = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const bf162*>(o + i));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const bf162*>(d + i));
    s += a.x * c.x + a.y * c.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) p.delta[(size_t(b) * p.QH + h) * p.T + t] = s;
}

// The same with 16-byte loads: LPR = D / 8 lanes share a row, a warp covers 32 / LPR rows at a time and
// every thread keeps U rows in flight. Needs 16-byte aligned rows (strides that are multiples of 8).
// Rows are numbered with the head fastest, (b, t, h): in the packed [B, T, heads, D] layout consecutive
// rows are then consecutive in memory, so a warp's loads cover whole contiguous lines (numbered with the
// token fastest every 256-byte row sat one token pitch apart, and the pass ran at a third of the bandwidth).
template <int LPR, int U>
__global__ void __launch_bounds__(256) flash_delta_vec_kernel(const FlashParams p) {
  constexpr int RPW = 32 / LPR;                      // rows per warp and step
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPR, li = lane % LPR;
  const long long total = (long long)p.B * p.QH * p.T;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r0 = warp0 * RPW * U; r0 < total; r0 += nwarps * RPW * U) {
    uint4 a[U], c[U];
    long long row[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      row[u] = r0 + u * RPW + sub;
      if (row[u] < total) {
        const int h = int(row[u] % p.QH), t = int((row[u] / p.QH) % p.T), b = int(row[u] / ((long long)p.T * p.QH));
        a[u] = *reinterpret_cast<const uint4*>(p.o + b * p.o_bs + (long long)t * p.o_ts + h * p.o_hs + li * 8);
        c[u] = *reinterpret_cast<const uint4*>(p.dout + b * p.do_bs + (long long)t * p.do_ts + h * p.do_hs + li * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float s = 0.f;
      if (row[u] < total) {
        const bf162* a2 = reinterpret_cast<const bf162*>(&a[u]);
        const bf162* c2 = reinterpret_cast<const bf162*>(&c[u]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = __bfloat1622float2(a2[e]), y = __bfloat1622float2(c2[e]);
          s += x.x * y.x + x.y * y.y;
        }
      }
#pragma unroll
      for (int off = LPR / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
      if (li == 0 && row[u] < total) {
        const int h = int(row[u] % p.QH), t = int((row[u] / p.QH) % p.T), b = int(row[u] / ((long long)p.T * p.QH));
        p.delta[(size_t(b) * p.QH + h) * p.T + t] = s;
      }
    }
  }
}

static bool launch_delta_vec(const FlashParams& p, int D, cudaStream_t st) {
  const long long strides[6] = {p.o_bs, p.o_ts, p.o_hs, p.do_bs, p.do_ts, p.do_hs};
  for (long long v : strides)
    if (v % 8 != 0) return false;
  if (((reinterpret_cast<uintptr_t>(p.o) | reinterpret_cast<uintptr_t>(p.dout)) & 15) != 0) return false;
  const long long total = (long long)p.B * p.QH * p.T;
  constexpr int U = 4;
  auto grid_for_rows = [&](int rpw) {
    const long long warps = (total + rpw * U - 1) / (rpw * U);
    const long long blocks = (warps + 7) / 8;
    const long long cap = (long long)num_sms() * 8;
    return int(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
  };
  if (D == 128) flash_delta_vec_kernel<16, U><<<grid_for_rows(2), 256, 0, st>>>(p);
  else if (D == 64) flash_delta_vec_kernel<8, U><<<grid_for_rows(4), 256, 0, st>>>(p);
  else if (D == 32) flash_delta_vec_kernel<4, U><<<grid_for_rows(8), 256, 0, st>>>(p);
  else return false;
  return true;
}

// ================================================================= backward: dK, dV
// CTA = 64 keys (4 warps x 16 keys). Works on S^T = K Q^T so that every warp owns key rows.
constexpr int FB_BN = 64;       // keys per CTA
constexpr int FB_BM = 64;       // query rows per iteration
constexpr int FB_THREADS = 128;

template <int D, bool ROPE>
__global__ void __launch_bounds__(FB_THREADS, 1) flash_bwd_dkv_kernel(const FlashParams p) {
  extern __shared__ __align__(128) uint8_t fa_smem[];
  uint8_t* sK = fa_smem;                       // FB_BN x D (rotated)   -> dK staging at the end
  uint8_t* sV = sK + FB_BN * D * 2;            // FB_BN x D             -> dV staging at the end
  uint8_t* sQ = sV + FB_BN * D * 2;            // FB_BM x D (rotated)
  uint8_t* sDO = sQ + FB_BM * D * 2;           // FB_BM x D
  float* sLse = reinterpret_cast<float*>(sDO + FB_BM * D * 2);   // FB_BM
  float* sDelta = sLse + FB_BM;                                   // FB_BM
  const uint32_t aK = smem_u32_generic(sK), aV = smem_u32_generic(sV), aQ = smem_u32_generic(sQ),
                 aDO = smem_u32_generic(sDO);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int ntile = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int n0 = ntile * FB_BN;
  const int T = p.T;
  const int R = p.QH / p.KVH;
  const int vlen = p.valid_len ? min(p.valid_len[b], T) : T;

  {
    TileLoader<FB_BN, D, FB_THREADS> lk;
    lk.load(p.k + b * p.k_bs + kvh * p.k_hs, p.k_ts, n0, T, tid);
    lk.template store<ROPE>(aK, p.rcos, p.rsin, n0, T, tid);
    lk.load(p.v + b * p.v_bs + kvh * p.v_hs, p.v_ts, n0, T, tid);
    lk.template store<false>(aV, nullptr, nullptr, n0, T, tid);
  }

  float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
    dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
  }
  const float sl2 = p.scale * kLog2e;
  const int key_lo = n0 + warp * 16 + g, key_hi = key_lo + 8;
  const int m_first = (n0 / FB_BM) * FB_BM;     // first query tile that can see these keys
  const int n_mtiles = (T - m_first + FB_BM - 1) / FB_BM;
  const int total_iters = (n0 < vlen) ? R * n_mtiles : 0;   // keys past valid_len get zero gradients

  TileLoader<FB_BM, D, FB_THREADS> lq, ldo;
  float lse_r = 0.f, delta_r = 0.f;
  auto issue_loads = [&](int it) {
    const int r = it / n_mtiles, mt = it % n_mtiles;
    const int h = kvh * R + r;
    const int m0 = m_first + mt * FB_BM;
    lq.load(p.q + b * p.q_bs + h * p.q_hs, p.q_ts, m0, T, tid);
    ldo.load(p.dout + b * p.do_bs + h * p.do_hs, p.do_ts, m0, T, tid);
    if (tid < FB_BM) {
      const int row = m0 + tid;
      const size_t idx = (size_t(b) * p.QH + h) * T + min(row, T - 1);
      lse_r = (row < T) ? p.lse[idx] : INFINITY;   // +inf => P = 0 for rows past T
      delta_r = (row < T) ? p.delta[idx] : 0.f;
    }
  };
  auto commit_loads = [&](int it) {
    const int mt = it % n_mtiles;
    const int m0 = m_first + mt * FB_BM;
    lq.template store<ROPE>(aQ, p.rcos, p.rsin, m0, T, tid);
    ldo.template store<false>(aDO, nullptr, nullptr, m0, T, tid);
    if (tid < FB_BM) {
      sLse[tid] = lse_r * kLog2e;
      sDelta[tid] = delta_r;
    }
  };

  if (total_iters > 0) {
    issue_loads(0);
    commit_loads(0);
  }
  __syncthreads();

  for (int it = 0; it < total_iters; ++it) {
    const int mt = it % n_mtiles;
    const int m0 = m_first + mt * FB_BM;
    if (it + 1 < total_iters) issue_loads(it + 1);

#pragma unroll
    for (int half = 0; half < FB_BM / 32; ++half) {
      const int q0 = half * 32;     // 32 query columns at a time to bound register use
      // S^T[key][q] = K[key][:] . Q[q][:]
      float st[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) st[i][0] = st[i][1] = st[i][2] = st[i][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t kf[4];
        lds_a<D>(kf, aK, warp * 16, ks, lane);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t r[4];
          lds_b_nt<D>(r, aQ, q0 + np * 16, ks, lane);
          mma_bf16(st[2 * np], kf, r[0], r[1]);
          mma_bf16(st[2 * np + 1], kf, r[2], r[3]);
        }
      }
      // dP^T[key][q] = V[key][:] . dO[q][:]
      float dpt[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) dpt[i][0] = dpt[i][1] = dpt[i][2] = dpt[i][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t vf[4];
        lds_a<D>(vf, aV, warp * 16, ks, lane);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t r[4];
          lds_b_nt<D>(r, aDO, q0 + np * 16, ks, lane);
          mma_bf16(dpt[2 * np], vf, r[0], r[1]);
          mma_bf16(dpt[2 * np + 1], vf, r[2], r[3]);
        }
      }
      // P^T and dS^T as A-operand fragments (k = query index)
      uint32_t pf[2][4], dsf[2][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float pv[4], dsv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int qc = q0 + i * 8 + 2 * t4 + (e & 1);
          const int qrow = m0 + qc;
          const int key = (e < 2) ? key_lo : key_hi;
          float pe = exp2f(st[i][e] * sl2 - sLse[qc]);
          if (key > qrow || key >= vlen) pe = 0.f;
          pv[e] = pe;
          dsv[e] = pe * (dpt[i][e] - sDelta[qc]) * p.scale;
        }
        pf[i >> 1][(i & 1) * 2 + 0] = pack_bf16(pv[0], pv[1]);
        pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(pv[2], pv[3]);
        dsf[i >> 1][(i & 1) * 2 + 0] = pack_bf16(dsv[0], dsv[1]);
        dsf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(dsv[2], dsv[3]);
      }
      // dV[key][d] += P^T[key][q] dO[q][d] ;  dK[key][d] += dS^T[key][q] Q[q][d]
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
        for (int nc = 0; nc < D / 16; ++nc) {
          uint32_t r[4];
          lds_b_nn<D>(r, aDO, q0 + kk * 16, nc, lane);
          mma_bf16(dv[2 * nc], pf[kk], r[0], r[1]);
          mma_bf16(dv[2 * nc + 1], pf[kk], r[2], r[3]);
          lds_b_nn<D>(r, aQ, q0 + kk * 16, nc, lane);
          mma_bf16(dk[2 * nc], dsf[kk], r[0], r[1]);
          mma_bf16(dk[2 * nc + 1], dsf[kk], r[2], r[3]);
        }
      }
    }
    __syncthreads();
    if (it + 1 < total_iters) commit_loads(it + 1);
    __syncthreads();
  }

  if (ROPE) unrotate_acc<D>(dk, p.rcos, p.rsin, key_lo, key_hi, T, lane);
  __syncthreads();   // every warp is done with sK / sV before they become staging areas
  bf16* dkb = p.dk + b * p.dk_bs + kvh * p.dk_hs;
  bf16* dvb = p.dv + b * p.dv_bs + kvh * p.dv_hs;
  store_acc_rows<D>(dk, aK + warp * 16 * D * 2, sK + warp * 16 * D * 2, dkb, p.dk_ts, n0 + warp * 16, T, lane, 1.f, 1.f);
  store_acc_rows<D>(dv, aV + warp * 16 * D * 2, sV + warp * 16 * D * 2, dvb, p.dv_ts, n0 + warp * 16, T, lane, 1.f, 1.f);
}

// ================================================================= backward: dQ
template <int D, bool ROPE>
__global__ void __launch_bounds__(FA_THREADS, 1) flash_bwd_dq_kernel(const FlashParams p) {
  extern __shared__ __align__(128) uint8_t fa_smem[];
  uint8_t* sQ = fa_smem;                               // FA_BM x D (rotated) -> dQ staging at the end
  uint8_t* sDO = sQ + FA_BM * D * 2;                   // FA_BM x D
  uint8_t* sK = sDO + FA_BM * D * 2;                   // FA_BN x D (rotated)
  uint8_t* sV = sK + FA_BN * D * 2;                    // FA_BN x D
  const uint32_t aQ = smem_u32_generic(sQ), aDO = smem_u32_generic(sDO), aK = smem_u32_generic(sK),
                 aV = smem_u32_generic(sV);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int mtile = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.QH / p.KVH);
  const int m0 = mtile * FA_BM;
  const int T = p.T;
  const int vlen = p.valid_len ? min(p.valid_len[b], T) : T;

  const bf16* kb = p.k + b * p.k_bs + kvh * p.k_hs;
  const bf16* vb = p.v + b * p.v_bs + kvh * p.v_hs;
  {
    TileLoader<FA_BM, D, FA_THREADS> lq;
    lq.load(p.q + b * p.q_bs + h * p.q_hs, p.q_ts, m0, T, tid);
    lq.template store<ROPE>(aQ, p.rcos, p.rsin, m0, T, tid);
    lq.load(p.dout + b * p.do_bs + h * p.do_hs, p.do_ts, m0, T, tid);
    lq.template store<false>(aDO, nullptr, nullptr, m0, T, tid);
  }
  TileLoader<FA_BN, D, FA_THREADS> lk, lv;
  const int n_tiles = (min(m0 + FA_BM, T) + FA_BN - 1) / FA_BN;
  lk.load(kb, p.k_ts, 0, T, tid);
  lv.load(vb, p.v_ts, 0, T, tid);
  lk.template store<ROPE>(aK, p.rcos, p.rsin, 0, T, tid);
  lv.template store<false>(aV, nullptr, nullptr, 0, T, tid);
  __syncthreads();

  const int qrow_lo = m0 + warp * 16 + g, qrow_hi = qrow_lo + 8;
  const size_t sbase = (size_t(b) * p.QH + h) * T;
  const float lse_lo = (qrow_lo < T) ? p.lse[sbase + qrow_lo] * kLog2e : INFINITY;
  const float lse_hi = (qrow_hi < T) ? p.lse[sbase + qrow_hi] * kLog2e : INFINITY;
  const float dl_lo = (qrow_lo < T) ? p.delta[sbase + qrow_lo] : 0.f;
  const float dl_hi = (qrow_hi < T) ? p.delta[sbase + qrow_hi] : 0.f;

  float dq[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;
  const float sl2 = p.scale * kLog2e;

  for (int j = 0; j < n_tiles; ++j) {
    const int n0 = j * FA_BN;
    if (j + 1 < n_tiles) {
      lk.load(kb, p.k_ts, n0 + FA_BN, T, tid);
      lv.load(vb, p.v_ts, n0 + FA_BN, T, tid);
    }
    float s[FA_BN / 8][4], dp[FA_BN / 8][4];
#pragma unroll
    for (int i = 0; i < FA_BN / 8; ++i) {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t qf[4], df[4];
      lds_a<D>(qf, aQ, warp * 16, ks, lane);
      lds_a<D>(df, aDO, warp * 16, ks, lane);
#pragma unroll
      for (int np = 0; np < FA_BN / 16; ++np) {
        uint32_t r[4];
        lds_b_nt<D>(r, aK, np * 16, ks, lane);
        mma_bf16(s[2 * np], qf, r[0], r[1]);
        mma_bf16(s[2 * np + 1], qf, r[2], r[3]);
        lds_b_nt<D>(r, aV, np * 16, ks, lane);
        mma_bf16(dp[2 * np], df, r[0], r[1]);
        mma_bf16(dp[2 * np + 1], df, r[2], r[3]);
      }
    }
    uint32_t dsf[FA_BN / 16][4];
#pragma unroll
    for (int i = 0; i < FA_BN / 8; ++i) {
      float dsv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = n0 + i * 8 + 2 * t4 + (e & 1);
        const int qr = (e < 2) ? qrow_lo : qrow_hi;
        float pe = exp2f(s[i][e] * sl2 - ((e < 2) ? lse_lo : lse_hi));
        if (key > qr || key >= vlen) pe = 0.f;
        dsv[e] = pe * (dp[i][e] - ((e < 2) ? dl_lo : dl_hi)) * p.scale;
      }
      dsf[i >> 1][(i & 1) * 2 + 0] = pack_bf16(dsv[0], dsv[1]);
      dsf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(dsv[2], dsv[3]);
    }
#pragma unroll
    for (int kk = 0; kk < FA_BN / 16; ++kk) {
#pragma unroll
      for (int nc = 0; nc < D / 16; ++nc) {
        uint32_t r[4];
        lds_b_nn<D>(r, aK, kk * 16, nc, lane);
        mma_bf16(dq[2 * nc], dsf[kk], r[0], r[1]);
        mma_bf16(dq[2 * nc + 1], dsf[kk], r[2], r[3]);
      }
    }
    __syncthreads();
    if (j + 1 < n_tiles) {
      lk.template store<ROPE>(aK, p.rcos, p.rsin, n0 + FA_BN, T, tid);
      lv.template store<false>(aV, nullptr, nullptr, n0 + FA_BN, T, tid);
    }
    __syncthreads();
  }
  if (ROPE) unrotate_acc<D>(dq, p.rcos, p.rsin, qrow_lo, qrow_hi, T, lane);
  bf16* dqb = p.dq + b * p.dq_bs + h * p.dq_hs;
  // the loop ended with __syncthreads: no warp still reads sQ
  store_acc_rows<D>(dq, aQ + warp * 16 * D * 2, sQ + warp * 16 * D * 2, dqb, p.dq_ts, m0 + warp * 16, T, lane, 1.f, 1.f);
}

// ================================================================= decode (one new token, KV cache)
// q [B, QH, D]; cache K/V [B, KVH, Tmax, D] (K already rotated); len[b] keys are valid.
// One warp per (b, head): keys strided over lanes is wasteful for D-wide dot products, so every
// lane owns D/32.. elements of the head dim and the warp walks the keys; 4 warps split the keys.
template <int D>
__global__ void __launch_bounds__(128) decode_attn_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc,
                                                          const bf16* __restrict__ vc, bf16* __restrict__ out,
                                                          const int* __restrict__ lens, int QH, int KVH, int Tmax,
                                                          float scale) {
  constexpr int EPL = (D + 31) / 32;        // elements per lane
  __shared__ float s_m[4], s_l[4];
  __shared__ float s_o[4][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const int kvh = h / (QH / KVH);
  const int len = min(lens[b], Tmax);
  float qv[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int d = lane + e * 32;
    qv[e] = (d < D) ? __bfloat162float(q[(size_t(b) * QH + h) * D + d]) * scale : 0.f;
  }
  const bf16* kb = kc + (size_t(b) * KVH + kvh) * Tmax * D;
  const bf16* vb = vc + (size_t(b) * KVH + kvh) * Tmax * D;
  float m = -INFINITY, l = 0.f, acc[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
  for (int t = warp; t < len; t += 4) {
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int d = lane + e * 32;
      if (d < D) dot += qv[e] * __bfloat162float(kb[size_t(t) * D + d]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    const float mn = fmaxf(m, dot);
    const float c = __expf(m - mn), pe = __expf(dot - mn);
    l = l * c + pe;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int d = lane + e * 32;
      if (d < D) acc[e] = acc[e] * c + pe * __bfloat162float(vb[size_t(t) * D + d]);
    }
    m = mn;
  }
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int d = lane + e * 32;
    if (d < D) s_o[warp][d] = acc[e];
  }
  __syncthreads();
  if (warp == 0) {
    float M = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
    float L = 0.f;
    float w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[i] = (s_m[i] == -INFINITY) ? 0.f : __expf(s_m[i] - M);
      L += s_l[i] * w[i];
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int d = lane + e * 32;
      if (d < D) {
        const float v = s_o[0][d] * w[0] + s_o[1][d] * w[1] + s_o[2][d] * w[2] + s_o[3][d] * w[3];
        out[(size_t(b) * QH + h) * D + d] = __float2bfloat16(v * inv);
      }
    }
  }
}

template <typename K>
static int set_smem(K kern, int bytes) {
  return static_cast<int>(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}

template <int D>
static int launch_fwd(const FlashParams& p, bool rope, cudaStream_t st) {
  const int smem = (FA_BM + 2 * FA_BN) * D * 2;
  dim3 grid((p.T + FA_BM - 1) / FA_BM, p.QH, p.B);
  if (rope) {
    static bool done = false;
    if (!done) { int e = set_smem(flash_fwd_kernel<D, true>, smem); if (e) return e; done = true; }
    flash_fwd_kernel<D, true><<<grid, FA_THREADS, smem, st>>>(p);
  } else {
    static bool done = false;
    if (!done) { int e = set_smem(flash_fwd_kernel<D, false>, smem); if (e) return e; done = true; }
    flash_fwd_kernel<D, false><<<grid, FA_THREADS, smem, st>>>(p);
  }
  return static_cast<int>(cudaGetLastError());
}

template <int D>
static int launch_bwd(const FlashParams& p, bool rope, cudaStream_t st) {
  if (!launch_delta_vec(p, D, st)) {
    const int total_warps = p.B * p.QH * p.T;
    flash_delta_kernel<<<(total_warps + 7) / 8, 256, 0, st>>>(p, D);
  }
  const int smem_kv = (2 * FB_BN + 2 * FB_BM) * D * 2 + 2 * FB_BM * 4;
  const int smem_q = (2 * FA_BM + 2 * FA_BN) * D * 2;
  dim3 grid_kv((p.T + FB_BN - 1) / FB_BN, p.KVH, p.B);
  dim3 grid_q((p.T + FA_BM - 1) / FA_BM, p.QH, p.B);
  if (rope) {
    static bool done = false;
    if (!done) {
      int e = set_smem(flash_bwd_dkv_kernel<D, true>, smem_kv); if (e) return e;
      e = set_smem(flash_bwd_dq_kernel<D, true>, smem_q); if (e) return e;
      done = true;
    }
    flash_bwd_dkv_kernel<D, true><<<grid_kv, FB_THREADS, smem_kv, st>>>(p);
    flash_bwd_dq_kernel<D, true><<<grid_q, FA_THREADS, smem_q, st>>>(p);
  } else {
    static bool done = false;
    if (!done) {
      int e = set_smem(flash_bwd_dkv_kernel<D, false>, smem_kv); if (e) return e;
      e = set_smem(flash_bwd_dq_kernel<D, false>, smem_q); if (e) return e;
      done = true;
    }
    flash_bwd_dkv_kernel<D, false><<<grid_kv, FB_THREADS, smem_kv, st>>>(p);
    flash_bwd_dq_kernel<D, false><<<grid_q, FA_THREADS, smem_q, st>>>(p);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace b200

using namespace b200;

// strides: 8 groups of (batch, token, head) element strides in the order q, k, v, o, dout, dq, dk, dv.
static void fill_strides(FlashParams& p, const long long* s) {
  p.q_bs = s[0]; p.q_ts = s[1]; p.q_hs = s[2];
  p.k_bs = s[3]; p.k_ts = s[4]; p.k_hs = s[5];
  p.v_bs = s[6]; p.v_ts = s[7]; p.v_hs = s[8];
  p.o_bs = s[9]; p.o_ts = s[10]; p.o_hs = s[11];
  p.do_bs = s[12]; p.do_ts = s[13]; p.do_hs = s[14];
  p.dq_bs = s[15]; p.dq_ts = s[16]; p.dq_hs = s[17];
  p.dk_bs = s[18]; p.dk_ts = s[19]; p.dk_hs = s[20];
  p.dv_bs = s[21]; p.dv_ts = s[22]; p.dv_hs = s[23];
}

static bool strides_ok(const long long* s, int n, const void* const* ptrs, int nptr) {
  for (int i = 0; i < n; ++i)
    if (s[i] % 8 != 0) return false;            // 16-byte vector access on every row
  for (int i = 0; i < nptr; ++i)
    if (ptrs[i] && (reinterpret_cast<uintptr_t>(ptrs[i]) & 15)) return false;
  return true;
}

B200_API int b200_flash_fwd(const void* q, const void* k, const void* v, void* o, void* lse, const void* valid_len,
                            const void* rcos, const void* rsin, const long long* strides, int B, int T, int QH,
                            int KVH, int D, float scale, cudaStream_t st) {
  if (B <= 0 || T <= 0) return 0;
  const void* ptrs[4] = {q, k, v, o};
  if (!strides_ok(strides, 12, ptrs, 4) || QH % KVH != 0) return static_cast<int>(cudaErrorInvalidValue);
  FlashParams p = {};
  p.q = static_cast<const bf16*>(q); p.k = static_cast<const bf16*>(k); p.v = static_cast<const bf16*>(v);
  p.o = static_cast<bf16*>(o); p.lse = static_cast<float*>(lse);
  p.valid_len = static_cast<const int*>(valid_len);
  p.rcos = static_cast<const float*>(rcos); p.rsin = static_cast<const float*>(rsin);
  fill_strides(p, strides);
  p.B = B; p.T = T; p.QH = QH; p.KVH = KVH; p.scale = scale;
  const bool rope = rcos != nullptr;
  switch (D) {
    case 32: return launch_fwd<32>(p, rope, st);
    case 64: return launch_fwd<64>(p, rope, st);
    case 128: return launch_fwd<128>(p, rope, st);
    default: return static_cast<int>(cudaErrorInvalidValue);
  }
}

B200_API int b200_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                            const void* lse, void* delta, void* dq, void* dk, void* dv, const void* valid_len,
                            const void* rcos, const void* rsin, const long long* strides, int B, int T, int QH,
                            int KVH, int D, float scale, cudaStream_t st) {
  if (B <= 0 || T <= 0) return 0;
  const void* ptrs[8] = {q, k, v, o, dout, dq, dk, dv};
  if (!strides_ok(strides, 24, ptrs, 8) || QH % KVH != 0) return static_cast<int>(cudaErrorInvalidValue);
  FlashParams p = {};
  p.q = static_cast<const bf16*>(q); p.k = static_cast<const bf16*>(k); p.v = static_cast<const bf16*>(v);
  p.o = const_cast<bf16*>(static_cast<const bf16*>(o)); p.dout = static_cast<const bf16*>(dout);
  p.lse = const_cast<float*>(static_cast<const float*>(lse)); p.delta = static_cast<float*>(delta);
  p.dq = static_cast<bf16*>(dq); p.dk = static_cast<bf16*>(dk); p.dv = static_cast<bf16*>(dv);
  p.valid_len = static_cast<const int*>(valid_len);
  p.rcos = static_cast<const float*>(rcos); p.rsin = static_cast<const float*>(rsin);
  fill_strides(p, strides);
  p.B = B; p.T = T; p.QH = QH; p.KVH = KVH; p.scale = scale;
  const bool rope = rcos != nullptr;
  switch (D) {
    case 32: return launch_bwd<32>(p, rope, st);
    case 64: return launch_bwd<64>(p, rope, st);
    case 128: return launch_bwd<128>(p, rope, st);
    default: return static_cast<int>(cudaErrorInvalidValue);
  }
}

B200_API int b200_decode_attn(const void* q, const void* kcache, const void* vcache, void* out, const void* lens,
                              int B, int QH, int KVH, int Tmax, int D, float scale, cudaStream_t st) {
  if (B <= 0) return 0;
  dim3 grid(QH, B);
#define B200_DEC(DD)                                                                                             \
  decode_attn_kernel<DD><<<grid, 128, 0, st>>>(static_cast<const bf16*>(q), static_cast<const bf16*>(kcache),    \
                                               static_cast<const bf16*>(vcache), static_cast<bf16*>(out),        \
                                               static_cast<const int*>(lens), QH, KVH, Tmax, scale)
  switch (D) {
    case 32: B200_DEC(32); break;
    case 64: B200_DEC(64); break;
    case 128: B200_DEC(128); break;
    default: return static_cast<int>(cudaErrorInvalidValue);
  }
#undef B200_DEC
  return static_cast<int>(cudaGetLastError());
}

// delta[b, h, t] = sum_d dO * O (fp32), the row term of the softmax gradient. strides: o (3), dout (3).
B200_API int b200_flash_delta(const void* o, const void* dout, void* delta, const long long* strides, int B, int T,
                              int QH, int D, cudaStream_t st) {
  if (B <= 0 || T <= 0) return 0;
  FlashParams p = {};
  p.o = const_cast<bf16*>(static_cast<const bf16*>(o));
  p.dout = static_cast<const bf16*>(dout);
  p.delta = static_cast<float*>(delta);
  p.o_bs = strides[0]; p.o_ts = strides[1]; p.o_hs = strides[2];
  p.do_bs = strides[3]; p.do_ts = strides[4]; p.do_hs = strides[5];
  p.B = B; p.T = T; p.QH = QH;
  if (!launch_delta_vec(p, D, st)) {
    const int total_warps = B * QH * T;
    flash_delta_kernel<<<(total_warps + 7) / 8, 256, 0, st>>>(p, D);
  }
  return static_cast<int>(cudaGetLastError());
}
