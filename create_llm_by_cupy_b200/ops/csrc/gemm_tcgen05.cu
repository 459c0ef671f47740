// bf16 GEMM on the 5th-generation tensor cores: D[M,N] = alpha * op(A) * op(B) (+ C).
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer   global -> 128B-swizzled shared-memory stages (cp.async.bulk.tensor)
//   warp 1      MMA issuer     one elected thread issues tcgen05.mma (128 x BN x 16) into TMEM
//   warps 2..5  epilogue       tcgen05.ld the fp32 accumulator, scale / add C / convert, store
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of tile i overlaps
// the main loop of tile i+1. Operands may be K-major (row-major [MN, K]) or MN-major (row-major
// [K, MN]); both are fed to the tensor core straight from the TMA-written tiles, so the three
// forms a training step needs (x*W, dy*W^T, x^T*dy) run without a transpose pass.
//
// This file is the replacement for every cuBLAS call site of the reference
// (model/fast_layers.py:217,341,420-458,736-815,1328-1471).
#include "common.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;

enum GemmFlags : int {
  GEMM_OUT_F32 = 1,   // D (and C) are fp32 instead of bf16
  GEMM_ADD_C = 2,     // D = alpha * A*B + C
};

// All-gather fused into the GEMM (one kernel does both): the first `n_copy` CTAs of the grid do no
// math; they pull every rank's slice of a ZeRO unit out of peer memory into the local unit buffer
// with bulk TMA copies (peer -> shared -> local global, a ring of 32 KiB buffers per CTA) and
// publish progress in 1 MiB segment counters. The GEMM CTAs' producer warps wait (bounded) on the
// segments that hold the rows of the B operand (a weight matrix inside that unit buffer) before
// they issue the TMA loads for them, so the tensor cores start on the first rows of the weight
// while later rows - and the rest of the unit - are still crossing NVLink. When the kernel ends
// the whole unit is local. TMA loads never use cluster multicast.
constexpr int AG_MAX_W = 8;
constexpr int AG_CHUNK = 32 * 1024;            // bytes per bulk copy
constexpr int AG_SEG_SHIFT = 20;               // 1 MiB progress segments
constexpr int AG_NBUF = 6;

struct AgFusion {
  const void* src[AG_MAX_W];     // rank q's slice of the unit (peer pointers; src[rank] is local)
  void* dst;                     // local unit buffer, W * slice_bytes
  unsigned long long* seg;       // progress counters, one per MiB of dst, monotonically increasing
  unsigned long long slice_bytes;
  unsigned long long b_off;      // byte offset of the B matrix inside dst
  unsigned long long b_row_bytes;
  unsigned long long first_byte; // copy order starts at the chunk holding this byte (B's first row)
  unsigned int epoch;            // counters of a complete segment read epoch * segment_bytes
  int W, n_copy;
  // The part of the unit this kernel copies: n_chunks chunks starting at the one that holds
  // first_byte, i.e. bytes [r_lo, r_hi) of dst. The whole unit, or only the chunks that hold B
  // (the rest of the unit is then pulled by a separate kernel on the communication stream).
  long long n_chunks;
  unsigned long long r_lo, r_hi;
};

// Chunk grid of the copy: every rank's slice is cut into AG_CHUNK pieces (the last one short).
struct AgRegion { unsigned long long r_lo, r_hi; long long n_chunks; };
static AgRegion ag_region(unsigned long long slice_bytes, int W, unsigned long long b_off, unsigned long long b_bytes,
                          bool only_b) {
  const unsigned long long cps = (slice_bytes + AG_CHUNK - 1) / AG_CHUNK;
  if (!only_b || b_bytes == 0) return AgRegion{0ull, slice_bytes * W, (long long)(cps * W)};
  const unsigned long long last = b_off + b_bytes - 1;
  const unsigned long long q0 = b_off / slice_bytes, c0 = (b_off % slice_bytes) / AG_CHUNK;
  const unsigned long long q1 = last / slice_bytes, c1 = (last % slice_bytes) / AG_CHUNK;
  AgRegion r;
  r.r_lo = q0 * slice_bytes + c0 * AG_CHUNK;
  const unsigned long long end1 = q1 * slice_bytes + (c1 + 1) * AG_CHUNK;
  r.r_hi = end1 < (q1 + 1) * slice_bytes ? end1 : (q1 + 1) * slice_bytes;
  r.n_chunks = (long long)((q1 * cps + c1) - (q0 * cps + c0) + 1);
  return r;
}

struct GemmParams {
  void* D;
  const void* C;
  int M, N, K;
  int ldd, ldc;
  int flags;
  float alpha;
  int* status;
  AgFusion ag;
};

template <int BN>
struct GemmSmem {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = GEMM_BM * GEMM_BK * 2;
  static constexpr int kBBytes = BN * GEMM_BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  // full[kStages], empty[kStages], tmem_full[2], tmem_empty[2], tmem base, abort flag
  static constexpr int kTotal = kBarOffset + (2 * kStages + 4) * 8 + 16 + 1024 /* alignment slack */;
};

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& mb, int& nb) {
  constexpr int GROUP_M = 16;
  const int per_group = GROUP_M * num_n;
  const int g = t / per_group;
  const int first_m = g * GROUP_M;
  const int gsz = min(num_m - first_m, GROUP_M);
  const int r = t - g * per_group;
  mb = first_m + (r % gsz);
  nb = r / gsz;
}

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long ag_seg_bytes(const AgFusion& ag, unsigned long long seg) {
  // bytes of this segment that THIS kernel copies and credits
  const unsigned long long lo = max(seg << AG_SEG_SHIFT, ag.r_lo);
  const unsigned long long hi = min(ag.r_hi, (seg + 1) << AG_SEG_SHIFT);
  return hi > lo ? hi - lo : 0ull;
}

// Credit a finished chunk [pos, pos + bytes) of the unit buffer to the segment counters.
__device__ __forceinline__ void ag_publish(const AgFusion& ag, unsigned long long pos, unsigned long long bytes) {
  fence_proxy_async_all();
  __threadfence();
  while (bytes > 0) {
    const unsigned long long seg = pos >> AG_SEG_SHIFT;
    const unsigned long long room = ((seg + 1) << AG_SEG_SHIFT) - pos;
    const unsigned long long part = bytes < room ? bytes : room;
    atomicAdd(ag.seg + seg, part);
    pos += part;
    bytes -= part;
  }
}

// Copy role of one CTA (thread 0 drives it): chunks cta, cta + n_copy, ... in rotated order.
__device__ void ag_copy_role(const AgFusion& ag, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int* status) {
  const unsigned long long cps = (ag.slice_bytes + AG_CHUNK - 1) / AG_CHUNK;     // chunks per slice
  const long long total = (long long)cps * ag.W;
  const long long j0 = (long long)(ag.first_byte / ag.slice_bytes) * cps + (ag.first_byte % ag.slice_bytes) / AG_CHUNK;
  const long long mine = (ag.n_chunks - blockIdx.x + ag.n_copy - 1) / ag.n_copy;
  auto chunk_of = [&](long long i, const void*& src, unsigned long long& pos, uint32_t& bytes) {
    const long long j = (j0 + blockIdx.x + i * ag.n_copy) % total;
    const int q = int(j / (long long)cps);
    const unsigned long long c = (unsigned long long)(j % (long long)cps) * AG_CHUNK;
    const unsigned long long left = ag.slice_bytes - c;
    bytes = uint32_t(left < AG_CHUNK ? left : AG_CHUNK);
    src = static_cast<const uint8_t*>(ag.src[q]) + c;
    pos = (unsigned long long)q * ag.slice_bytes + c;
  };
  // Software pipeline driven by one thread: loads run AG_NBUF - 2 chunks ahead of the stores; a
  // buffer is re-filled once the store that used it has finished READING shared memory; chunks are
  // credited to the segment counters in batches of 8, after their stores have fully completed.
  auto issue_load = [&](long long i) {
    const void* src; unsigned long long pos; uint32_t bytes;
    chunk_of(i, src, pos, bytes);
    const int buf = int(i % AG_NBUF);
    mbar_expect_tx(&bars[buf], bytes);
    bulk_g2s(smem + buf * AG_CHUNK, src, bytes, &bars[buf]);
  };
  auto publish_upto = [&](long long from, long long to) {   // chunks [from, to)
    if (to <= from) return;
    fence_proxy_async_all();
    __threadfence();
    for (long long i = from; i < to; ++i) {
      const void* src; unsigned long long pos; uint32_t bytes;
      chunk_of(i, src, pos, bytes);
      unsigned long long left = bytes;
      while (left > 0) {
        const unsigned long long seg = pos >> AG_SEG_SHIFT;
        const unsigned long long room = ((seg + 1) << AG_SEG_SHIFT) - pos;
        const unsigned long long part = left < room ? left : room;
        atomicAdd(ag.seg + seg, part);
        pos += part;
        left -= part;
      }
    }
  };
  constexpr int kAhead = AG_NBUF - 2;
  bool ok = true;
  long long published = 0;
  for (long long i = 0; i < mine && i < kAhead; ++i) issue_load(i);
  for (long long i = 0; i < mine; ++i) {
    const int buf = int(i % AG_NBUF);
    if (!mbar_wait(&bars[buf], uint32_t((i / AG_NBUF) & 1), abort_flag)) { ok = false; break; }
    const void* src; unsigned long long pos; uint32_t bytes;
    chunk_of(i, src, pos, bytes);
    bulk_s2g(static_cast<uint8_t*>(ag.dst) + pos, smem + buf * AG_CHUNK, bytes);
    tma_store_commit();
    tma_store_wait_read<1>();                 // stores up to chunk i - 1 no longer read their buffers
    if (i + kAhead < mine) issue_load(i + kAhead);   // re-fills the buffer chunk i - 2 used
    if ((i & 7) == 7) {
      tma_store_wait<2>();                    // stores up to chunk i - 2 are complete
      publish_upto(published, i - 1);
      published = i - 1;
    }
  }
  tma_store_wait<0>();
  if (ok) {
    publish_upto(published, mine);
  } else if (status != nullptr && atomicCAS(status, 0, int(*abort_flag)) == 0) {
    status[1] = 110;
  }
}

// Producer-side wait for the segments that cover bytes [lo, hi) of the unit buffer. `have_lo`,
// `have_hi` remember the contiguous range of segments already seen complete.
__device__ __forceinline__ bool ag_wait_bytes(const AgFusion& ag, unsigned long long lo, unsigned long long hi,
                                              long long& have_lo, long long& have_hi, volatile int* abort_flag) {
  const long long s_lo = (long long)(lo >> AG_SEG_SHIFT), s_hi = (long long)((hi - 1) >> AG_SEG_SHIFT);
  if (s_lo >= have_lo && s_hi <= have_hi) return true;
  for (long long s = s_lo; s <= s_hi; ++s) {
    if (s >= have_lo && s <= have_hi) continue;
    const unsigned long long want = (unsigned long long)ag.epoch * ag_seg_bytes(ag, (unsigned long long)s);
    const uint64_t deadline = globaltimer_ns() + B200_WAIT_NS;
    uint32_t spins = 0;
    while (ld_acquire_gpu_u64(ag.seg + s) < want) {
      if ((++spins & 31) == 0) {
        if (*abort_flag) return false;
        if (globaltimer_ns() > deadline) { *abort_flag = ERR_PEER_TIMEOUT; return false; }
      }
    }
  }
  if (have_hi < have_lo || s_lo > have_hi + 1 || s_hi < have_lo - 1) { have_lo = s_lo; have_hi = s_hi; }
  else { have_lo = min(have_lo, s_lo); have_hi = max(have_hi, s_hi); }
  fence_proxy_async_all();
  return true;
}

template <int BN, bool A_MN, bool B_MN, bool AG>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmParams p) {
  using S = GemmSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int cta0 = AG ? p.ag.n_copy : 0;             // first GEMM CTA
  const int gemm_ctas = int(gridDim.x) - cta0;
  if (AG && int(blockIdx.x) < cta0) {
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AG_NBUF * AG_CHUNK);
    volatile int* aflag = reinterpret_cast<volatile int*>(bars + AG_NBUF);
    if (threadIdx.x == 0) {
      for (int i = 0; i < AG_NBUF; ++i) mbar_init(&bars[i], 1);
      *aflag = 0;
      mbar_fence_init();
      fence_proxy_async_smem();
      ag_copy_role(p.ag, smem, bars, aflag, p.status);
    }
    return;
  }
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty = full + S::kStages;
  uint64_t* tfull = empty + S::kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + GEMM_BM - 1) / GEMM_BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + GEMM_BK - 1) / GEMM_BK;
  constexpr uint32_t kTmemCols = 2 * BN;   // 256 or 512, a power of two

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) tmem_alloc(tmem_base_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long have_lo = 0, have_hi = -1;
      for (int t = int(blockIdx.x) - cta0; t < num_tiles && ok; t += gemm_ctas) {
        int mb, nb;
        tile_coords(t, num_m, num_n, mb, nb);
        const int m0 = mb * GEMM_BM, n0 = nb * BN;
        if (AG && !B_MN) {   // B rows are the n index: this tile needs rows n0 .. n0 + BN
          const unsigned long long r1 = (unsigned long long)min(n0 + BN, p.N);
          if (!ag_wait_bytes(p.ag, p.ag.b_off + (unsigned long long)n0 * p.ag.b_row_bytes,
                             p.ag.b_off + r1 * p.ag.b_row_bytes, have_lo, have_hi, abort_flag)) { ok = false; break; }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (AG && B_MN) {  // B rows are the k index: this k-block needs rows k0 .. k0 + 64
            const unsigned long long r0 = (unsigned long long)kb * GEMM_BK;
            const unsigned long long r1 = (unsigned long long)min((kb + 1) * GEMM_BK, p.K);
            if (!ag_wait_bytes(p.ag, p.ag.b_off + r0 * p.ag.b_row_bytes, p.ag.b_off + r1 * p.ag.b_row_bytes,
                               have_lo, have_hi, abort_flag)) { ok = false; break; }
          }
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sA = smem + stage * S::kStageBytes;
          uint8_t* sB = sA + S::kABytes;
          mbar_expect_tx(&full[stage], S::kStageBytes);
          const int k0 = kb * GEMM_BK;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < GEMM_BM / 64; ++c) tma_load_2d(sA + c * 8192, &tmA, &full[stage], m0 + c * 64, k0);
          } else {
            tma_load_2d(sA, &tmA, &full[stage], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sB + c * 8192, &tmB, &full[stage], n0 + c * 64, k0);
          } else {
            tma_load_2d(sB, &tmB, &full[stage], k0, n0);
          }
          if (++stage == S::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(GEMM_BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = int(blockIdx.x) - cta0; t < num_tiles && ok; t += gemm_ctas) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sB = sA + S::kABytes;
#pragma unroll
          for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
            const uint64_t adesc = A_MN ? umma_smem_desc(sA + kk * 2048, 8192, 1024)
                                        : umma_smem_desc(sA + kk * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc(sB + kk * 2048, 8192, 1024)
                                        : umma_smem_desc(sB + kk * 32, 16, 1024);
            umma_bf16_ss(tmem_d, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);   // frees the smem stage once these MMAs have read it
          if (++stage == S::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);       // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool out_f32 = (p.flags & GEMM_OUT_F32) != 0;
    const bool add_c = (p.flags & GEMM_ADD_C) != 0;
    const bool vec_ok = out_f32 ? ((p.ldd & 3) == 0 && (reinterpret_cast<uintptr_t>(p.D) & 15) == 0 &&
                                   (!add_c || ((p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0)))
                                : ((p.ldd & 7) == 0 && (reinterpret_cast<uintptr_t>(p.D) & 15) == 0 &&
                                   (!add_c || ((p.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0)));
    bool ok = true;
    for (int t = int(blockIdx.x) - cta0; t < num_tiles && ok; t += gemm_ctas) {
      int mb, nb;
      tile_coords(t, num_m, num_n, mb, nb);
      const int row = mb * GEMM_BM + q * 32 + lane;
      const int n0 = nb * BN;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
          const bool full_chunk = vec_ok && (col0 + 32 <= p.N);
          if (out_f32) {
            float* drow = static_cast<float*>(p.D) + size_t(row) * p.ldd + col0;
            const float* crow = add_c ? static_cast<const float*>(p.C) + size_t(row) * p.ldc + col0 : nullptr;
            if (full_chunk) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                if (add_c) {
                  const float4 cc = *reinterpret_cast<const float4*>(crow + j);
                  o.x += cc.x; o.y += cc.y; o.z += cc.z; o.w += cc.w;
                }
                *reinterpret_cast<float4*>(drow + j) = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) drow[j] = v[j] + (add_c ? crow[j] : 0.f);
            }
          } else {
            bf16* drow = static_cast<bf16*>(p.D) + size_t(row) * p.ldd + col0;
            const bf16* crow = add_c ? static_cast<const bf16*>(p.C) + size_t(row) * p.ldc + col0 : nullptr;
            if (full_chunk) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (add_c) {
                  const uint4 cc = *reinterpret_cast<const uint4*>(crow + j);
                  const bf162* c2 = reinterpret_cast<const bf162*>(&cc);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(c2[e]);
                    v[j + 2 * e] += f.x;
                    v[j + 2 * e + 1] += f.y;
                  }
                }
                uint4 o;
                bf162* o2 = reinterpret_cast<bf162*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(v[j + 2 * e], v[j + 2 * e + 1]);
                *reinterpret_cast<uint4*>(drow + j) = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
                const float cv = add_c ? __bfloat162float(crow[j]) : 0.f;
                drow[j] = __float2bfloat16(v[j] + cv);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, int(*abort_flag)) == 0) p.status[1] = 100 + BN / 128;
  }
}

// Fallback for shapes the TMA path cannot take (pitch or base not 16-byte aligned): a plain
// shared-memory tiled GEMM on the CUDA cores. Correct for any shape and stride; slow.
template <bool A_MN, bool B_MN>
__global__ void gemm_fallback_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B, int lda, int ldb,
                                     const GemmParams p) {
  __shared__ float sA[16][17];
  __shared__ float sB[16][17];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int row = blockIdx.y * 16 + ty, col = blockIdx.x * 16 + tx;
  float acc = 0.f;
  for (int k0 = 0; k0 < p.K; k0 += 16) {
    const int ka = k0 + tx, kb = k0 + ty;
    float a = 0.f, b = 0.f;
    if (row < p.M && ka < p.K) a = __bfloat162float(A_MN ? A[size_t(ka) * lda + row] : A[size_t(row) * lda + ka]);
    if (col < p.N && kb < p.K) b = __bfloat162float(B_MN ? B[size_t(kb) * ldb + col] : B[size_t(col) * ldb + kb]);
    sA[ty][tx] = a;
    sB[ty][tx] = b;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) acc += sA[ty][k] * sB[k][tx];
    __syncthreads();
  }
  if (row < p.M && col < p.N) {
    float v = acc * p.alpha;
    if (p.flags & GEMM_OUT_F32) {
      if (p.flags & GEMM_ADD_C) v += static_cast<const float*>(p.C)[size_t(row) * p.ldc + col];
      static_cast<float*>(p.D)[size_t(row) * p.ldd + col] = v;
    } else {
      if (p.flags & GEMM_ADD_C) v += __bfloat162float(static_cast<const bf16*>(p.C)[size_t(row) * p.ldc + col]);
      static_cast<bf16*>(p.D)[size_t(row) * p.ldd + col] = __float2bfloat16(v);
    }
  }
}

template <int BN, bool A_MN, bool B_MN, bool AG = false>
static int launch_tc(const CUtensorMap* tA, const CUtensorMap* tB, const GemmParams& p, cudaStream_t stream,
                     int max_ctas) {
  using S = GemmSmem<BN>;
  auto kern = gemm_bf16_tc_kernel<BN, A_MN, B_MN, AG>;
  static bool configured = false;   // per template instantiation; one device per process
  if (!configured) {
    B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
    configured = true;
  }
  const int num_tiles = ((p.M + GEMM_BM - 1) / GEMM_BM) * ((p.N + BN - 1) / BN);
  int grid = num_sms();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (AG) {
    // copy CTAs + GEMM CTAs, all resident at once (one CTA per SM)
    const int gemm_ctas = grid - p.ag.n_copy < num_tiles ? grid - p.ag.n_copy : num_tiles;
    grid = gemm_ctas + p.ag.n_copy;
  } else if (num_tiles < grid) {
    grid = num_tiles;
  }
  kern<<<grid, GEMM_THREADS, S::kTotal, stream>>>(*tA, *tB, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace b200

using namespace b200;

// D[M,N] = alpha * op(A) op(B) (+ C).
//   a_mn_major = 0: A is row-major [M, K] (pitch lda);  1: A is row-major [K, M]  (i.e. A^T given)
//   b_mn_major = 0: B is row-major [N, K] (pitch ldb);  1: B is row-major [K, N]
//   flags: GEMM_OUT_F32 | GEMM_ADD_C. C may alias D. bn = 0 picks the tile width automatically.
//   max_ctas > 0 limits the persistent grid (used to leave SMs free for a concurrent copy kernel).
B200_API int b200_gemm_bf16(const void* A, const void* B, void* D, const void* C, int M, int N, int K, int lda,
                            int ldb, int ldd, int ldc, int a_mn_major, int b_mn_major, int flags, float alpha,
                            int bn, int max_ctas, int force_fallback, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return static_cast<int>(cudaErrorInvalidValue);
  GemmParams p;
  p.D = D; p.C = C; p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.ldc = ldc; p.flags = flags; p.alpha = alpha;
  p.status = status_ptr();
  p.ag = AgFusion{};

  const bool aligned = ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0 &&
                       (lda % 8) == 0 && (ldb % 8) == 0;
  if (!aligned || force_fallback) {
    dim3 block(16, 16), grid((N + 15) / 16, (M + 15) / 16);
    const bf16* a = static_cast<const bf16*>(A);
    const bf16* b = static_cast<const bf16*>(B);
    if (a_mn_major && b_mn_major) gemm_fallback_kernel<true, true><<<grid, block, 0, stream>>>(a, b, lda, ldb, p);
    else if (a_mn_major) gemm_fallback_kernel<true, false><<<grid, block, 0, stream>>>(a, b, lda, ldb, p);
    else if (b_mn_major) gemm_fallback_kernel<false, true><<<grid, block, 0, stream>>>(a, b, lda, ldb, p);
    else gemm_fallback_kernel<false, false><<<grid, block, 0, stream>>>(a, b, lda, ldb, p);
    return static_cast<int>(cudaGetLastError());
  }

  if (bn == 0) {
    // 256-wide tiles halve the A re-reads; 128-wide tiles quantise better on small problems.
    const long t256 = long((M + 127) / 128) * ((N + 255) / 256);
    const long t128 = long((M + 127) / 128) * ((N + 127) / 128);
    const int sms = num_sms();
    const double eff256 = double(t256) / double(((t256 + sms - 1) / sms) * sms);
    const double eff128 = double(t128) / double(((t128 + sms - 1) / sms) * sms);
    bn = (N <= 128 || eff128 > eff256 * 1.15) ? 128 : 256;
  }

  // K-major operand: matrix [MN, K], box 64 (K) x tile rows. MN-major: matrix [K, MN], box 64 x 64.
  const CUtensorMap* tA = a_mn_major ? get_tensor_map_2d(A, K, M, lda, 64, 64, 2, SWIZZLE_128B_)
                                     : get_tensor_map_2d(A, M, K, lda, GEMM_BM, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tB = b_mn_major ? get_tensor_map_2d(B, K, N, ldb, 64, 64, 2, SWIZZLE_128B_)
                                     : get_tensor_map_2d(B, N, K, ldb, bn, 64, 2, SWIZZLE_128B_);
  if (!tA || !tB) return static_cast<int>(cudaErrorInvalidValue);

#define B200_DISPATCH(BN_)                                                                          \
  if (a_mn_major && b_mn_major) return launch_tc<BN_, true, true>(tA, tB, p, stream, max_ctas);     \
  if (a_mn_major) return launch_tc<BN_, true, false>(tA, tB, p, stream, max_ctas);                  \
  if (b_mn_major) return launch_tc<BN_, false, true>(tA, tB, p, stream, max_ctas);                  \
  return launch_tc<BN_, false, false>(tA, tB, p, stream, max_ctas);
  if (bn == 128) { B200_DISPATCH(128) }
  B200_DISPATCH(256)
#undef B200_DISPATCH
}

// The byte range [out[0], out[1]) of the unit buffer that b200_gemm_bf16_allgather copies itself when
// called with only_b != 0 for a B matrix of b_bytes at b_off; out[2] = number of chunks.
B200_API int b200_ag_region(unsigned long long slice_bytes, int W, unsigned long long b_off, unsigned long long b_bytes,
                            unsigned long long* out) {
  if (W < 1 || W > AG_MAX_W || slice_bytes == 0 || out == nullptr) return static_cast<int>(cudaErrorInvalidValue);
  const AgRegion r = ag_region(slice_bytes, W, b_off, b_bytes, true);
  out[0] = r.r_lo; out[1] = r.r_hi; out[2] = (unsigned long long)r.n_chunks;
  return 0;
}

// GEMM with the all-gather of a ZeRO unit fused in (see AgFusion). only_b: copy just the chunks that
// hold B (the caller pulls the rest of the unit with b200_symm_all_gather in its skip mode). B must be a weight matrix that
// lives at byte offset b_off inside the local unit buffer `ag_dst` (row pitch b_row_bytes); the
// unit's W slices are read from `ag_src[q]` (peer pointers). seg = zero-initialised counters, one
// per MiB of the unit buffer; epoch = 1, 2, ... per use of that buffer. Returns when launched;
// when the kernel completes the whole unit buffer is filled.
B200_API int b200_gemm_bf16_allgather(const void* A, void* D, const void* C, int M, int N, int K, int lda, int ldd,
                                      int ldc, int a_mn_major, int b_mn_major, int flags, float alpha,
                                      const void* const* ag_src, void* ag_dst, void* seg,
                                      unsigned long long slice_bytes, unsigned long long b_off, int W, int n_copy,
                                      unsigned int epoch, int only_b, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || W < 1 || W > AG_MAX_W || n_copy < 1) return static_cast<int>(cudaErrorInvalidValue);
  if (slice_bytes % 16 != 0 || b_off % 16 != 0) return static_cast<int>(cudaErrorInvalidValue);
  GemmParams p;
  p.D = D; p.C = C; p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.ldc = ldc; p.flags = flags; p.alpha = alpha;
  p.status = status_ptr();
  p.ag = AgFusion{};
  for (int q = 0; q < W; ++q) p.ag.src[q] = ag_src[q];
  p.ag.dst = ag_dst;
  p.ag.seg = static_cast<unsigned long long*>(seg);
  p.ag.slice_bytes = slice_bytes;
  p.ag.b_off = b_off;
  const int ldb = b_mn_major ? N : K;
  p.ag.b_row_bytes = (unsigned long long)ldb * 2;
  p.ag.first_byte = b_off;
  p.ag.epoch = epoch;
  p.ag.W = W;
  p.ag.n_copy = n_copy;
  {
    const unsigned long long b_rows = b_mn_major ? (unsigned long long)K : (unsigned long long)N;
    const AgRegion r = ag_region(slice_bytes, W, b_off, b_rows * p.ag.b_row_bytes, only_b != 0);
    p.ag.r_lo = r.r_lo; p.ag.r_hi = r.r_hi; p.ag.n_chunks = r.n_chunks;
  }
  const void* B = static_cast<const uint8_t*>(ag_dst) + b_off;
  if ((reinterpret_cast<uintptr_t>(A) & 15) != 0 || (lda % 8) != 0 || (ldb % 8) != 0)
    return static_cast<int>(cudaErrorInvalidValue);
  const int bn = 256;
  const CUtensorMap* tA = a_mn_major ? get_tensor_map_2d(A, K, M, lda, 64, 64, 2, SWIZZLE_128B_)
                                     : get_tensor_map_2d(A, M, K, lda, GEMM_BM, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tB = b_mn_major ? get_tensor_map_2d(B, K, N, ldb, 64, 64, 2, SWIZZLE_128B_)
                                     : get_tensor_map_2d(B, N, K, ldb, bn, 64, 2, SWIZZLE_128B_);
  if (!tA || !tB) return static_cast<int>(cudaErrorInvalidValue);
  if (a_mn_major && b_mn_major) return launch_tc<256, true, true, true>(tA, tB, p, stream, 0);
  if (a_mn_major) return launch_tc<256, true, false, true>(tA, tB, p, stream, 0);
  if (b_mn_major) return launch_tc<256, false, true, true>(tA, tB, p, stream, 0);
  return launch_tc<256, false, false, true>(tA, tB, p, stream, 0);
}
