// bf16 GEMM on tcgen05 with CTA pairs (cta_group::2): D[M,N] = alpha * op(A) * op(B) (+ C).
//
// Two CTAs of a cluster (two SMs) cooperate on one 256 x 256 output tile. Each CTA stages its own
// 128 rows of A and HALF of the B tile (128 of the 256 columns) in shared memory; one thread of
// the leader CTA issues tcgen05.mma.cta_group::2, which reads A and B from both CTAs' shared
// memory and accumulates each CTA's 128 x 256 half of D in that CTA's TMEM. Compared with the
// single-CTA kernel every SM pulls 32 KiB instead of 48 KiB per 64-deep k-block from L2 and the
// ring is 6 stages deep instead of 4, which is what it takes to keep the tensor pipe fed.
//
// Synchronisation (all mbarriers live at the same offsets in both CTAs):
//   full[s]       leader only. The leader's producer arms it with the bytes of BOTH CTAs; the
//                 follower's TMA loads complete on it too (cp.async.bulk.tensor ... cta_group::2
//                 with the leader's barrier address). No cluster multicast is used by any load.
//   empty[s]      one per CTA; the leader's tcgen05.commit arrives on both (multicast commit).
//   tmem_full[a]  one per CTA; multicast commit after the last k-block of a tile.
//   tmem_empty[a] leader only, 8 arrivals: the 4 epilogue warps of each CTA (the follower's
//                 arrive remotely through the cluster shared-memory window).
//   sched_full[i] one per CTA; sched_empty[i] leader only (see "Tile scheduler").
// Waits are bounded exactly as in the single-CTA kernel.
//
// Tile scheduler. Every pair starts on the tile of its own index; all further tiles are handed
// out dynamically: the leader's producer thread takes the next tile index from a global counter
// (one tile ahead of the one it is loading), writes it into a
// 4-slot ring that exists in both CTAs' shared memory and signals sched_full[slot] in both. The
// follower's producer, the MMA thread and the eight epilogue warps read the ring and each arrive
// on the leader's sched_empty[slot] (10 arrivals) before the slot is reused. An index beyond the
// last tile is the stop mark; every pair draws exactly one, and the pair that draws the last one
// puts the counter back to zero for the launch that reuses it. A pair that starts late (its SMs
// were still busy with the previous kernel, or with a kernel of another stream) simply draws
// fewer tiles, which a fixed tile-to-pair assignment cannot do.
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int G2_BM = 128;          // rows per CTA (256 per pair)
constexpr int G2_BN = 256;          // columns per pair; each CTA stages 128 of them
constexpr int G2_BK = 64;
constexpr int G2_THREADS = 192;
constexpr int G2_STAGES = 6;
constexpr int G2_A_BYTES = G2_BM * G2_BK * 2;          // 16 KiB
constexpr int G2_B_BYTES = (G2_BN / 2) * G2_BK * 2;    // 16 KiB
constexpr int G2_STAGE_BYTES = G2_A_BYTES + G2_B_BYTES;
constexpr int G2_SCHED = 4;         // slots of the tile-index ring
constexpr int G2_STG_BYTES = 128 * 128;                 // epilogue staging tile: 128 rows x 128 bytes
constexpr int G2_STG_OFF = G2_STAGES * G2_STAGE_BYTES;  // two staging tiles follow the operand ring
constexpr int G2_BAR_OFF2 = G2_STG_OFF + 2 * G2_STG_BYTES;
constexpr int G2_SMEM = G2_BAR_OFF2 + (2 * G2_STAGES + 4 + 2 * G2_SCHED + 2) * 8 + 16 + G2_SCHED * 4 + 1024;
constexpr int G2_SCHED_SLOTS = 1024;   // {next tile, finished pairs} counter pairs, used round-robin by launches

// G2_WHOLE_TILES (caller): never halve tiles - set for GEMMs that run beside a GEMM of another stream,
// whose CTAs fill the SMs a part-filled last round leaves idle anyway.
enum Gemm2Flags : int { G2_OUT_F32 = 1, G2_ADD_C = 2, G2_TMA_OUT = 4, G2_WHOLE_TILES = 8 };

// What the epilogue does with the accumulator (a template parameter: the plain instantiations keep their
// register count).
//   EPI_ROPE       rotary embedding on the leading columns (K|Q|V projection)
//   EPI_SWIGLU     B = [gate | value]; a work item holds 128 gate columns beside the 128 value columns of the
//                  same index and leaves silu(gate) * value (and, on request, the raw projection)
//   EPI_CE_STATS   LM head: nothing is stored but per-row (max, sum of exp, target logit) of the tile's columns
//   EPI_CE_DLOGITS LM head again: (exp(logit - lse) - onehot) * coef leaves as bf16
//   EPI_SWIGLU_BWD D = A B^T is d(activation); the epilogue fetches the stored gate / value tiles by TMA and
//                  leaves d(gate), d(value) (the backward of silu(gate) * value), d(activation) is never stored
//   EPI_DELTA      D = A B^T is d(attention output) [tokens, heads x head_dim]; the epilogue also fetches the forward's
//                  output tile by TMA and leaves delta[b, head, t] = sum_d dO O, which the attention backward needs
enum Gemm2Epi : int {
  EPI_PLAIN = 0, EPI_ROPE = 1, EPI_SWIGLU = 2, EPI_CE_STATS = 3, EPI_CE_DLOGITS = 4, EPI_SWIGLU_BWD = 5, EPI_DELTA = 6
};

struct Gemm2Params {
  void* D;
  const void* C;
  int M, N, K;
  int ldd, ldc;
  int flags;
  float alpha;
  int* status;
  int* sched;      // [0] next tile index, [1] pairs that have drawn their stop mark; both 0 between launches
  // Work items: the first t_full are whole 256 x 256 tiles; every tile after that is cut into two
  // 256 x 128 halves (items t_full + 2 i and t_full + 2 i + 1). The launcher halves the tiles of a last,
  // less than half filled round of CTA pairs, which then takes about half a tile time instead of a whole one.
  int t_full, n_items;
  // Rotary embedding in the epilogue (bf16 output through TMA only): the columns below rope_cols are heads of
  // width rope_dim (128 or 64) whose pairs (j, j + rope_dim / 2) are rotated by the angle of position
  // row % rope_T. The tables are fp32 and TRANSPOSED, [rope_dim / 2][rope_ld]: a thread owns one row, so the 32
  // lanes of a warp (consecutive positions) then read consecutive words. Null rope_cos: off.
  const float* rope_cos;
  const float* rope_sin;
  int rope_T, rope_cols, rope_dim, rope_ld;
  // EPI_SWIGLU: N = 2 * sw_I. The leader CTA stages gate columns [g0, g0 + 128), the follower value columns
  // [sw_I + g0, sw_I + g0 + 128); the activation goes out through the map in the tmBh slot (no half tiles in this
  // mode), the raw gate / value halves through tmD / tmC when sw_store_gv is set.
  int sw_I, sw_store_gv;
  // EPI_CE_*: rows are tokens, column j is vocabulary id ce_col0 + j. Targets outside [0, vocabulary) match no column.
  const int* ce_targets;     // [M]
  float* ce_pmax;            // [tile columns][M] row maximum over one 256-column tile (EPI_CE_STATS)
  float* ce_psum;            // [tile columns][M] sum of exp(logit - that maximum)
  float* ce_tlogit;          // [M] logit of the target, written by the tile that holds it
  const float* ce_lse;       // [M] log-sum-exp of the whole row (EPI_CE_DLOGITS)
  const float* ce_coef;      // [M] valid * gradient scale / number of valid rows
  int ce_col0, ce_nt0;       // vocabulary id of column 0; tile-column index of this call's first tile in pmax / psum
  int ce_vocab;              // size of the whole vocabulary when the caller knows it (debug build: targets are checked)
  // EPI_DELTA: row = b * dl_T + t, column = head * dl_dim + d (dl_dim 128 or 64); the forward output O is read through
  // the map in the tmC slot; dl_out [batch][dl_heads][dl_T] fp32.
  float* dl_out;
  int dl_T, dl_heads, dl_dim;
};

// A work item: tile coordinates, first column and width.
struct G2Item {
  int mb, nb, n0, bn;
};

static __device__ int g_tile_sched[2 * G2_SCHED_SLOTS];

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t smem_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion is counted on a barrier that may live in the peer CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_out, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_out)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this offset in BOTH CTAs once the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}

// Write one word into the peer CTA's shared memory and count its 4 bytes on the peer's mbarrier;
// the word is visible to whoever sees that barrier phase complete. Nothing here waits.
__device__ __forceinline__ void st_async_u32(uint32_t cluster_addr, uint32_t v, uint32_t cluster_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.u32 [%0], %1, [%2];"
               ::"r"(cluster_addr), "r"(v), "r"(cluster_bar)
               : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster_relaxed(uint32_t cluster_bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.relaxed.cluster.shared::cluster.b64 _, [%0], %1;"
               ::"r"(cluster_bar), "r"(bytes)
               : "memory");
}
// "This slot has been read": a relaxed arrive, issued only once `value` (what was read from the
// slot) has reached its register. A release here would make the caller wait for everything it
// has in flight, which for the MMA thread is the whole queue of tensor-core work.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed_after(uint32_t cluster_addr, int value) {
  asm volatile(
      "{\n\t.reg .b32 dep;\n\t"
      "mov.b32 dep, %1;\n\t"
      "mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];\n\t}"
      ::"r"(cluster_addr), "r"(value)
      : "memory");
}

// Consumer side of the tile-index ring (one instance per consuming thread or warp).
struct TileRingReader {
  int slot = 0;
  uint32_t phase = 0;
  // Returns the next tile index, or -1 when the wait was abandoned. `arrive` is true for the one
  // lane that reports the slot as read.
  __device__ __forceinline__ int next(uint64_t* sched_full, uint64_t* sched_empty, volatile int* ring,
                                      volatile int* abort_flag, bool whole_warp, bool arrive, bool remote_writer) {
    // In the leader the index is an ordinary shared-memory store before an arrive; in the follower
    // it arrives as an asynchronous store counted on the barrier. Either way a plain wait sees it.
    (void)remote_writer;
    if (!mbar_wait(&sched_full[slot], phase, abort_flag)) return -1;
    const int t = ring[slot];
    if (whole_warp) __syncwarp();
    if (arrive) mbar_arrive_cluster_relaxed_after(mapa_u32(smem_u32(&sched_empty[slot]), 0), t);
    if (++slot == G2_SCHED) { slot = 0; phase ^= 1; }
    return t;
  }
};

__device__ __forceinline__ void named_bar_sync_128(int id) {
  asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory");
}

__device__ __forceinline__ void tile_coords2(int t, int num_m, int num_n, int& mb, int& nb);
__device__ __forceinline__ G2Item g2_item(int t, int t_full, int num_m, int num_n) {
  G2Item it;
  int tile = t, half = -1;
  if (t >= t_full) {
    tile = t_full + ((t - t_full) >> 1);
    half = (t - t_full) & 1;
  }
  tile_coords2(tile, num_m, num_n, it.mb, it.nb);
  it.bn = half < 0 ? 256 : 128;
  it.n0 = it.nb * 256 + (half == 1 ? 128 : 0);
  return it;
}

__device__ __forceinline__ void tile_coords2(int t, int num_m, int num_n, int& mb, int& nb) {
  constexpr int GROUP_M = 8;
  const int per_group = GROUP_M * num_n;
  const int g = t / per_group;
  const int first_m = g * GROUP_M;
  const int gsz = min(num_m - first_m, GROUP_M);
  const int r = t - g * per_group;
  mb = first_m + (r % gsz);
  nb = r / gsz;
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2_THREADS, 1)
gemm_bf16_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmD,
                     const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmE,
                     const Gemm2Params p) {
  // The SwiGLU-backward epilogue works on two fetched tiles per group and prefetches the next pair: it trades
  // one stage of the operand ring for two more staging tiles (5 x 32 KiB + 4 x 16 KiB instead of 6 + 2).
  constexpr int kStages = EPI == EPI_SWIGLU_BWD ? G2_STAGES - 1 : G2_STAGES;
  constexpr int kStg = EPI == EPI_SWIGLU_BWD ? 4 : 2;
  constexpr int kStgOff = kStages * G2_STAGE_BYTES;
  static_assert(kStgOff + kStg * G2_STG_BYTES == G2_BAR_OFF2 && 2 * kStages + kStg == 2 * G2_STAGES + 2, "smem layout");
  extern __shared__ uint8_t smem_raw2[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw2) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + G2_BAR_OFF2);
  uint64_t* empty = full + kStages;
  uint64_t* tfull = empty + kStages;
  uint64_t* tempty = tfull + 2;
  uint64_t* sched_full = tempty + 2;
  uint64_t* sched_empty = sched_full + G2_SCHED;
  uint64_t* stage_ready = sched_empty + G2_SCHED;      // [kStg]: epilogue staging tile holds its input (or is simply free)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stage_ready + kStg);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* tile_ring = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();            // 0 = leader of the pair
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_m = (p.M + 2 * G2_BM - 1) / (2 * G2_BM);
  constexpr bool kRope = EPI == EPI_ROPE;
  // SwiGLU: one tile column per 128 activation columns (its accumulator is 128 gate + 128 value columns)
  const int num_n = EPI == EPI_SWIGLU ? (p.sw_I + G2_BN / 2 - 1) / (G2_BN / 2) : (p.N + G2_BN - 1) / G2_BN;
  const int num_tiles = p.n_items;          // work items (whole tiles and half tiles)
  const int num_kb = (p.K + G2_BK - 1) / G2_BK;
  const bool dyn = p.sched != nullptr;      // null: tile t + k * num_pairs goes to pair t (fixed assignment)

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);
    }
    for (int i = 0; i < G2_SCHED; ++i) {
      mbar_init(&sched_full[i], 1);
      mbar_init(&sched_empty[i], 10);
    }
    for (int i = 0; i < kStg; ++i) mbar_init(&stage_ready[i], 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                  // both CTAs' barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int wslot = 0;                 // leader: ring write position
      uint32_t wphase = 0;
      TileRingReader rd;             // follower: ring read position
      // Leader: hand tile `tile` to every consumer of the pair.
      auto publish = [&](int tile) -> bool {
        if (!mbar_wait(&sched_empty[wslot], wphase ^ 1, abort_flag)) return false;
        tile_ring[wslot] = tile;
        mbar_arrive(&sched_full[wslot]);                                  // this CTA's readers
        const uint32_t peer_bar = mapa_u32(smem_u32(&sched_full[wslot]), 1);
        mbar_expect_tx_cluster_relaxed(peer_bar, 4);                      // the follower's readers
        st_async_u32(mapa_u32(smem_u32(const_cast<int*>(&tile_ring[wslot])), 1), uint32_t(tile), peer_bar);
        if (++wslot == G2_SCHED) { wslot = 0; wphase ^= 1; }
        return true;
      };
      int t = pair, t_next = 0;      // the first tile needs no hand-out
      const int publish_kb = num_kb > 8 ? 8 : num_kb - 1;
      while (ok && t < num_tiles) {
        // the draw is in flight while this tile's first loads are issued
        if (!dyn) t_next = t + num_pairs;
        else if (rank == 0) t_next = num_pairs + atomicAdd(&p.sched[0], 1);
        const G2Item wi = g2_item(t, p.t_full, num_m, num_n);
        const int m0 = wi.mb * 2 * G2_BM + int(rank) * G2_BM;
        const int n0 = EPI == EPI_SWIGLU ? wi.nb * (G2_BN / 2) + int(rank) * p.sw_I : wi.n0 + int(rank) * (wi.bn / 2);
        const uint32_t stage_tx = 2 * (G2_A_BYTES + (wi.bn / 2) * G2_BK * 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sA = smem + stage * G2_STAGE_BYTES;
          uint8_t* sB = sA + G2_A_BYTES;
          if (rank == 0) mbar_expect_tx(&full[stage], stage_tx);             // bytes of both CTAs
          const uint32_t bar = mapa_u32(smem_u32(&full[stage]), 0);           // the leader's barrier
          const int k0 = kb * G2_BK;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < G2_BM / 64; ++c) tma_load_2d_pair(sA + c * 8192, &tmA, bar, m0 + c * 64, k0);
          } else {
            tma_load_2d_pair(sA, &tmA, bar, k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < (G2_BN / 2) / 64; ++c)
              if (c * 64 < wi.bn / 2) tma_load_2d_pair(sB + c * 8192, &tmB, bar, n0 + c * 64, k0);
          } else {
            tma_load_2d_pair(sB, wi.bn == G2_BN ? &tmB : &tmBh, bar, k0, n0);      // 128 or 64 rows of B
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
          if (dyn && rank == 0 && kb == publish_kb && !publish(t_next)) { ok = false; break; }
        }
        if (!ok) break;
        if (rank == 0 || !dyn) {
          t = t_next;
        } else {
          t = rd.next(sched_full, sched_empty, tile_ring, abort_flag, false, true, rank != 0);
          ok = t >= 0;
        }
      }
      if (dyn && rank == 0 && ok) {
        // this pair has drawn its stop mark; the last pair to do so rewinds the counters
        __threadfence();
        if (atomicAdd(&p.sched[1], 1) == num_pairs - 1) {
          p.sched[0] = 0;
          p.sched[1] = 0;
          __threadfence();
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc_full = umma_idesc_bf16(2 * G2_BM, G2_BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t idesc_half = umma_idesc_bf16(2 * G2_BM, G2_BN / 2, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      TileRingReader rd;
      for (int t = pair; ok && t >= 0 && t < num_tiles;
           t = dyn ? rd.next(sched_full, sched_empty, tile_ring, abort_flag, false, true, rank != 0) : t + num_pairs) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * G2_BN;
        const uint32_t idesc = t < p.t_full ? idesc_full : idesc_half;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * G2_STAGE_BYTES);
          const uint32_t sB = sA + G2_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < G2_BK / 16; ++kk) {
            const uint64_t adesc = A_MN ? umma_smem_desc(sA + kk * 2048, 8192, 1024)
                                        : umma_smem_desc(sA + kk * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc(sB + kk * 2048, 8192, 1024)
                                        : umma_smem_desc(sB + kk * 32, 16, 1024);
            umma_bf16_ss_pair(tmem_d, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&tfull[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool out_f32 = (p.flags & G2_OUT_F32) != 0;
    const bool add_c = (p.flags & G2_ADD_C) != 0;
    const bool vec_ok = out_f32 ? ((p.ldd & 3) == 0 && (reinterpret_cast<uintptr_t>(p.D) & 15) == 0 &&
                                   (!add_c || ((p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0)))
                                : ((p.ldd & 7) == 0 && (reinterpret_cast<uintptr_t>(p.D) & 15) == 0 &&
                                   (!add_c || ((p.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0)));
    bool ok = true;
    TileRingReader rd;
    if constexpr (EPI == EPI_CE_STATS) {
      // LM-head logits that never leave the SM: every thread folds its row of the accumulator into
      // (max, sum of exp, target logit) over the tile's valid columns and writes three floats.
      const int r = q * 32 + lane;
      for (int t = pair; ok && t >= 0 && t < num_tiles;
           t = dyn ? rd.next(sched_full, sched_empty, tile_ring, abort_flag, true, lane == 0, rank != 0)
                   : t + num_pairs) {
        const G2Item wi = g2_item(t, p.t_full, num_m, num_n);
        const int row = wi.mb * 2 * G2_BM + int(rank) * G2_BM + r;
        const int ncols = min(wi.bn, p.N - wi.n0);                       // valid columns of this tile
        int tcol = -1;
        if (row < p.M) {
          int tgt = __ldg(p.ce_targets + row);
#ifdef B200_BOUNDS_CHECK
          // a target beyond the vocabulary would silently count as "no target logit": the debug build reports it
          if (p.ce_vocab > 0 && tgt >= 0) tgt = checked_index(tgt, p.ce_vocab - 1, p.status, 304);
#endif
          tcol = tgt - p.ce_col0 - wi.n0;
        }
        if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * G2_BN;
        float mx = -INFINITY, sum = 0.f, tl = 0.f;
#pragma unroll 1
        for (int c = 0; c < wi.bn / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + c * 32, v);
          tmem_ld_wait();
          if (c == wi.bn / 32 - 1) {                     // accumulator fully read: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty[acc]), 0));
          }
          const int left = ncols - c * 32;
          if (left > 0) {
            float cm = -INFINITY;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < left) cm = fmaxf(cm, __uint_as_float(v[j]));
            const float nm = fmaxf(mx, cm);
            float part = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < left) part += __expf(__uint_as_float(v[j]) - nm);
              if (c * 32 + j == tcol) tl = __uint_as_float(v[j]);
            }
            sum = sum * __expf(mx - nm) + part;
            mx = nm;
          }
        }
        if (row < p.M) {
          const size_t at = size_t(p.ce_nt0 + wi.nb) * size_t(p.M) + size_t(row);
          p.ce_pmax[at] = mx;
          p.ce_psum[at] = sum;
          if (tcol >= 0 && tcol < ncols) p.ce_tlogit[row] = tl;
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    } else if constexpr (EPI == EPI_SWIGLU) {
      // 256 rows x 128 activation columns per item: accumulator columns [0, 128) are the gate, [128, 256)
      // the value. Per 64-column group the thread's row leaves as up to three 128-byte staging rows (raw
      // gate, raw value, activation), each stored by TMA; two staging tiles alternate as in the plain path.
      uint8_t* stg = smem + kStgOff;
      const int r = q * 32 + lane;
      const uint32_t swz = uint32_t(r & 7);
      const bool elected = (warp == 2 && lane == 0);
      uint32_t gcount = 0;
      // One group: this thread's 64 fp32 values -> bf16 -> staging row; one thread stores the tile. `more`: another
      // group of the same item follows (its staging tile is released here; an item's first one at the item's start).
      auto put = [&](const uint32_t (&v)[64], const CUtensorMap* map, int x, int y, bool more) -> bool {
        const uint32_t b = gcount & 1;
        if (!mbar_wait(&stage_ready[b], (gcount >> 1) & 1, abort_flag)) return false;
        uint8_t* rowp = stg + b * G2_STG_BYTES + r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint4 o;
          bf162* o2 = reinterpret_cast<bf162*>(&o);
#pragma unroll
          for (int e = 0; e < 4; ++e)
            o2[e] = __floats2bfloat162_rn(__uint_as_float(v[8 * c + 2 * e]), __uint_as_float(v[8 * c + 2 * e + 1]));
          *reinterpret_cast<uint4*>(rowp + ((uint32_t(c) ^ swz) << 4)) = o;
        }
        fence_proxy_async_smem();
        named_bar_sync_128(1);
        if (elected) {
          if (x < p.sw_I) tma_store_2d(map, stg + b * G2_STG_BYTES, x, y);      // a group wholly past the edge is dropped
          tma_store_commit();
          if (more) {
            tma_store_wait_read<1>();
            mbar_arrive(&stage_ready[(gcount + 1) & 1]);
          }
        }
        ++gcount;
        return true;
      };
      for (int t = pair; ok && t >= 0 && t < num_tiles;
           t = dyn ? rd.next(sched_full, sched_empty, tile_ring, abort_flag, true, lane == 0, rank != 0)
                   : t + num_pairs) {
        const G2Item wi = g2_item(t, p.t_full, num_m, num_n);
        const int row0 = wi.mb * 2 * G2_BM + int(rank) * G2_BM;
        const int g0 = wi.nb * (G2_BN / 2);
        if (elected) {
          tma_store_wait_read<1>();                      // the store that last used this staging tile has read it
          mbar_arrive(&stage_ready[gcount & 1]);
        }
        if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * G2_BN;
#pragma unroll 1
        for (int g = 0; g < 2 && ok; ++g) {
          uint32_t ga[64], va[64];
          tmem_ld_32x32b_x32(taddr + g * 64, *reinterpret_cast<uint32_t(*)[32]>(&ga[0]));
          tmem_ld_32x32b_x32(taddr + g * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&ga[32]));
          tmem_ld_32x32b_x32(taddr + G2_BN / 2 + g * 64, *reinterpret_cast<uint32_t(*)[32]>(&va[0]));
          tmem_ld_32x32b_x32(taddr + G2_BN / 2 + g * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&va[32]));
          tmem_ld_wait();
          if (g == 1) {                                  // accumulator fully read: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty[acc]), 0));
          }
          const int x = g0 + g * 64;
          if (p.sw_store_gv) {
            if (!put(ga, &tmD, x, row0, true)) { ok = false; break; }
            if (!put(va, &tmC, x, row0, true)) { ok = false; break; }
          }
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            const float gt = __uint_as_float(ga[j]);
            ga[j] = __float_as_uint(gt / (1.f + __expf(-gt)) * __uint_as_float(va[j]));
          }
          if (!put(ga, &tmBh, x, row0, g == 0)) { ok = false; break; }
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (elected) tma_store_wait<0>();
    } else if constexpr (EPI == EPI_SWIGLU_BWD) {
      // The accumulator is d(act) for 256 rows x 256 columns. Per 64-column group the stored gate and value tiles
      // (bf16, the two halves of the forward projection; maps tmBh / tmE) are fetched by TMA into a pair of staging
      // tiles, turned in place into d(gate) and d(value) and stored (maps tmD / tmC). Two pairs alternate: the next
      // group's pair is fetched while this one is computed.
      uint8_t* stg = smem + kStgOff;
      const int r = q * 32 + lane;
      const uint32_t swz = uint32_t(r & 7);
      const bool elected = (warp == 2 && lane == 0);
      uint32_t ucount = 0;                               // groups handled so far; pair = ucount & 1
      auto fetch = [&](uint32_t uc, int x, int y) {      // by the elected thread: fill pair uc & 1 for a group
        const uint32_t b = (uc & 1) * 2;
        if (x < p.sw_I) {
          mbar_expect_tx(&stage_ready[b], G2_STG_BYTES);
          tma_load_2d(stg + b * G2_STG_BYTES, &tmBh, &stage_ready[b], x, y);
          mbar_expect_tx(&stage_ready[b + 1], G2_STG_BYTES);
          tma_load_2d(stg + (b + 1) * G2_STG_BYTES, &tmE, &stage_ready[b + 1], x, y);
        } else {                                         // wholly past the edge: nothing to fetch, nothing is stored
          mbar_arrive(&stage_ready[b]);
          mbar_arrive(&stage_ready[b + 1]);
        }
      };
      for (int t = pair; ok && t >= 0 && t < num_tiles;
           t = dyn ? rd.next(sched_full, sched_empty, tile_ring, abort_flag, true, lane == 0, rank != 0)
                   : t + num_pairs) {
        const G2Item wi = g2_item(t, p.t_full, num_m, num_n);
        const int row0 = wi.mb * 2 * G2_BM + int(rank) * G2_BM;
        const int n0 = wi.n0;
        const int ngroups = wi.bn / 64;
        if (elected) {
          tma_store_wait_read<1>();                      // the stores that last used this pair have read it
          fetch(ucount, n0, row0);
        }
        if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * G2_BN;
#pragma unroll 1
        for (int g = 0; g < ngroups; ++g) {
          const uint32_t b = (ucount & 1) * 2;
          if (elected && g + 1 < ngroups) {              // prefetch the next group's pair
            tma_store_wait_read<0>();                    // the other pair's stores (previous group) have read it
            fetch(ucount + 1, n0 + (g + 1) * 64, row0);
          }
          uint32_t v[64];
          tmem_ld_32x32b_x32(taddr + g * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
          tmem_ld_32x32b_x32(taddr + g * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
          tmem_ld_wait();
          if (g == ngroups - 1) {                        // accumulator fully read: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty[acc]), 0));
          }
          const uint32_t ph = (ucount >> 1) & 1;
          if (!mbar_wait(&stage_ready[b], ph, abort_flag) || !mbar_wait(&stage_ready[b + 1], ph, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* grow = stg + b * G2_STG_BYTES + r * 128;
          uint8_t* vrow = grow + G2_STG_BYTES;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint4* gp = reinterpret_cast<uint4*>(grow + ((uint32_t(c) ^ swz) << 4));
            uint4* vp = reinterpret_cast<uint4*>(vrow + ((uint32_t(c) ^ swz) << 4));
            uint4 gq = *gp, vq = *vp;
            bf162* g2 = reinterpret_cast<bf162*>(&gq);
            bf162* v2 = reinterpret_cast<bf162*>(&vq);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 gf = __bfloat1622float2(g2[e]), vf = __bfloat1622float2(v2[e]);
              const float d0 = __uint_as_float(v[8 * c + 2 * e]), d1 = __uint_as_float(v[8 * c + 2 * e + 1]);
              const float s0 = 1.f / (1.f + __expf(-gf.x)), s1 = 1.f / (1.f + __expf(-gf.y));
              g2[e] = __floats2bfloat162_rn(d0 * vf.x * s0 * (1.f + gf.x * (1.f - s0)),
                                            d1 * vf.y * s1 * (1.f + gf.y * (1.f - s1)));
              v2[e] = __floats2bfloat162_rn(d0 * gf.x * s0, d1 * gf.y * s1);
            }
            *gp = gq;
            *vp = vq;
          }
          fence_proxy_async_smem();
          named_bar_sync_128(1);
          if (elected) {
            const int x = n0 + g * 64;
            if (x < p.sw_I) {
              tma_store_2d(&tmD, stg + b * G2_STG_BYTES, x, row0);
              tma_store_2d(&tmC, stg + (b + 1) * G2_STG_BYTES, x, row0);
            }
            tma_store_commit();
          }
          ++ucount;
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (elected) tma_store_wait<0>();
    } else
    if (p.flags & G2_TMA_OUT) {
      // Output through shared memory and TMA. A tile leaves in groups of 128 bytes per row (64 bf16
      // or 32 fp32 columns): every thread converts its accumulator row and writes it into a
      // 128-row staging tile in the 128-byte swizzle, one thread stores the tile with
      // cp.async.bulk.tensor (full 128-byte lines to L2, clipped at the matrix edge). With `add`
      // the same staging tile is first filled with the C tile by a TMA load. Two staging tiles
      // alternate, so the store of one group overlaps the conversion of the next.
      const int gcols = out_f32 ? 32 : 64;
      uint8_t* stg = smem + kStgOff;
      const int r = q * 32 + lane;
      const uint32_t swz = uint32_t(r & 7);
      const bool elected = (warp == 2 && lane == 0);
      uint32_t gcount = 0;
      auto arm = [&](uint32_t gc, int x, int y) {       // make staging tile gc & 1 ready for group gc
        const uint32_t b = gc & 1;
        if (add_c || EPI == EPI_DELTA) {
          mbar_expect_tx(&stage_ready[b], G2_STG_BYTES);
          tma_load_2d(stg + b * G2_STG_BYTES, &tmC, &stage_ready[b], x, y);
        } else {
          mbar_arrive(&stage_ready[b]);
        }
      };
      for (int t = pair; ok && t >= 0 && t < num_tiles;
           t = dyn ? rd.next(sched_full, sched_empty, tile_ring, abort_flag, true, lane == 0, rank != 0)
                   : t + num_pairs) {
        const G2Item wi = g2_item(t, p.t_full, num_m, num_n);
        const int row0 = wi.mb * 2 * G2_BM + int(rank) * G2_BM;
        const int n0 = wi.n0;
        const int ngroups = wi.bn / gcols;
        const bool rope_on = kRope && !out_f32 && n0 < p.rope_cols;
        const float* cs_row = nullptr;      // element j of this row's tables is at [j * rope_ld]
        const float* sn_row = nullptr;
        if (rope_on) {
          const int pos = min(row0 + r, p.M - 1) % p.rope_T;
          cs_row = p.rope_cos + pos;
          sn_row = p.rope_sin + pos;
        }
        float ce_lse = 0.f, ce_coef = 0.f;
        int ce_t = -1;                          // target as a column of this call (vocabulary id - ce_col0)
        if constexpr (EPI == EPI_CE_DLOGITS) {
          const int row = min(row0 + r, p.M - 1);
          ce_lse = __ldg(p.ce_lse + row);
          ce_coef = __ldg(p.ce_coef + row);
          ce_t = __ldg(p.ce_targets + row) - p.ce_col0;
        }
        float dl_sum = 0.f;                     // EPI_DELTA: dO . O over the head's columns seen so far
        if (elected) {
          tma_store_wait_read<1>();                      // the store that last used this staging tile has read it
          arm(gcount, n0, row0);
        }
        if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * G2_BN;
#pragma unroll 1
        for (int g = 0; g < ngroups; ++g) {
          const uint32_t b = gcount & 1;
          if (!mbar_wait(&stage_ready[b], (gcount >> 1) & 1, abort_flag)) { ok = false; break; }
          uint8_t* rowp = stg + b * G2_STG_BYTES + r * 128;
          if (out_f32) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(taddr + g * 32, v);
            tmem_ld_wait();
            if (g == ngroups - 1) {                      // accumulator fully read: hand it back to the MMA warp
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty[acc]), 0));
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              float4* dst = reinterpret_cast<float4*>(rowp + ((uint32_t(c) ^ swz) << 4));
              float4 o = make_float4(__uint_as_float(v[4 * c]) * p.alpha, __uint_as_float(v[4 * c + 1]) * p.alpha,
                                     __uint_as_float(v[4 * c + 2]) * p.alpha, __uint_as_float(v[4 * c + 3]) * p.alpha);
              if (add_c) {
                const float4 cc = *dst;
                o.x += cc.x; o.y += cc.y; o.z += cc.z; o.w += cc.w;
              }
              *dst = o;
            }
          } else {
            uint32_t v[64];
            tmem_ld_32x32b_x32(taddr + g * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
            tmem_ld_32x32b_x32(taddr + g * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
            const bool rope_g = kRope && rope_on && n0 + g * 64 < p.rope_cols;
            if (rope_g && p.rope_dim == 128) {
              // this group is one half of a 128-wide head; the other half is the neighbouring group
              uint32_t w[64];
              tmem_ld_32x32b_x32(taddr + (g ^ 1) * 64, *reinterpret_cast<uint32_t(*)[32]>(&w[0]));
              tmem_ld_32x32b_x32(taddr + (g ^ 1) * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&w[32]));
              tmem_ld_wait();
              const float sgn = (g & 1) ? 1.f : -1.f;      // first half: x1 c - x2 s; second half: x2 c + x1 s
#pragma unroll
              for (int j = 0; j < 64; ++j) {
                const float c = __ldg(cs_row + size_t(j) * p.rope_ld), sn = __ldg(sn_row + size_t(j) * p.rope_ld);
                v[j] = __float_as_uint(fmaf(__uint_as_float(v[j]), c, sgn * __uint_as_float(w[j]) * sn));
              }
            } else {
              tmem_ld_wait();
              if constexpr (EPI == EPI_CE_DLOGITS) {
                // logits -> (softmax - onehot) * coef with the row's log-sum-exp from the forward pass
                const int tcol = ce_t - (n0 + g * 64);
#pragma unroll
                for (int j = 0; j < 64; ++j) {
                  float x = __expf(__uint_as_float(v[j]) - ce_lse);
                  if (j == tcol) x -= 1.f;
                  v[j] = __float_as_uint(x * ce_coef);
                }
              }
              if (rope_g) {                                  // 64-wide head: both halves are in this group
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const float c = __ldg(cs_row + size_t(j) * p.rope_ld), sn = __ldg(sn_row + size_t(j) * p.rope_ld);
                  const float x1 = __uint_as_float(v[j]), x2 = __uint_as_float(v[j + 32]);
                  v[j] = __float_as_uint(fmaf(x1, c, -x2 * sn));
                  v[j + 32] = __float_as_uint(fmaf(x2, c, x1 * sn));
                }
              }
            }
            if (g == ngroups - 1) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty[acc]), 0));
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              uint4* dst = reinterpret_cast<uint4*>(rowp + ((uint32_t(c) ^ swz) << 4));
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[8 * c + e]) * p.alpha;
              if (add_c) {
                const uint4 cc = *dst;
                const bf162* c2 = reinterpret_cast<const bf162*>(&cc);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 ff = __bfloat1622float2(c2[e]);
                  f[2 * e] += ff.x;
                  f[2 * e + 1] += ff.y;
                }
              }
              uint4 o;
              bf162* o2 = reinterpret_cast<bf162*>(&o);
#pragma unroll
              for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
              if constexpr (EPI == EPI_DELTA) {
                // the staging tile holds the forward output; the product uses dO as it is stored (rounded)
                const uint4 cc = *dst;
                const bf162* c2 = reinterpret_cast<const bf162*>(&cc);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 of = __bfloat1622float2(c2[e]), df = __bfloat1622float2(o2[e]);
                  dl_sum = fmaf(df.x, of.x, fmaf(df.y, of.y, dl_sum));
                }
              }
              *dst = o;
            }
            if constexpr (EPI == EPI_DELTA) {
              const int col_end = n0 + (g + 1) * 64;
              if (col_end % p.dl_dim == 0) {                 // the head is complete
                const int row = row0 + r;
                const int head = col_end / p.dl_dim - 1;
                if (row < p.M && head < p.dl_heads) {
                  const int bi = row / p.dl_T;
                  p.dl_out[(size_t(bi) * p.dl_heads + head) * size_t(p.dl_T) + size_t(row - bi * p.dl_T)] = dl_sum;
                }
                dl_sum = 0.f;
              }
            }
          }
          fence_proxy_async_smem();
          named_bar_sync_128(1);
          if (elected) {
            tma_store_2d(&tmD, stg + b * G2_STG_BYTES, n0 + g * gcols, row0);
            tma_store_commit();
            if (g + 1 < ngroups) {
              tma_store_wait_read<1>();
              arm(gcount + 1, n0 + (g + 1) * gcols, row0);
            }
          }
          ++gcount;
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (elected) tma_store_wait<0>();
    } else
    for (int t = pair; ok && t >= 0 && t < num_tiles;
         t = dyn ? rd.next(sched_full, sched_empty, tile_ring, abort_flag, true, lane == 0, rank != 0) : t + num_pairs) {
      const G2Item wi = g2_item(t, p.t_full, num_m, num_n);
      const int row = wi.mb * 2 * G2_BM + int(rank) * G2_BM + q * 32 + lane;
      const int n0 = wi.n0;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * G2_BN;
#pragma unroll 1
      for (int c = 0; c < wi.bn / 32; ++c) {
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
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty[acc]), 0));   // the leader's barrier
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // the leader's MMAs read the follower's shared memory until here
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, int(*abort_flag)) == 0) p.status[1] = 120;
  }
}

static int g_dynamic_tiles = 1;
static int g_half_tiles = 1;

// Counter pair for one launch. Kernels of different streams may run at the same time, so launches
// take the slots round-robin; a slot is back to zero when its kernel has finished.
static int* next_sched_slot() {
  static std::mutex mu;
  static int* base[64] = {};
  static unsigned next = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (base[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_tile_sched) != cudaSuccess) return nullptr;
    base[dev] = static_cast<int*>(ptr);
  }
  return base[dev] + 2 * (next++ % G2_SCHED_SLOTS);
}

template <bool A_MN, bool B_MN, int EPI = EPI_PLAIN>
static int launch_tc2(const CUtensorMap* tA, const CUtensorMap* tB, const CUtensorMap* tBh, const CUtensorMap* tD,
                      const CUtensorMap* tC, const Gemm2Params& p, cudaStream_t stream, const CUtensorMap* tE = nullptr) {
  auto kern = gemm_bf16_tc2_kernel<A_MN, B_MN, EPI>;
  static bool configured = false;
  if (!configured) {
    B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM));
    configured = true;
  }
  const int tile_cols = EPI == EPI_SWIGLU ? (p.sw_I + G2_BN / 2 - 1) / (G2_BN / 2) : (p.N + G2_BN - 1) / G2_BN;
  const int whole = ((p.M + 2 * G2_BM - 1) / (2 * G2_BM)) * tile_cols;
  const int all_pairs = num_sms() / 2;
  // a last round that fills less than half of the pairs is run on half tiles (plain and rotary epilogues only)
  int halved = 0;
  if (g_half_tiles && (EPI <= EPI_ROPE || EPI == EPI_DELTA) && !(p.flags & G2_WHOLE_TILES) && whole > all_pairs) {
    const int rem = whole % all_pairs;
    if (rem > 0 && 2 * rem <= all_pairs) halved = rem;
  }
  const int num_tiles = whole + halved;
  int pairs = all_pairs;
  if (num_tiles < pairs) pairs = num_tiles;
  Gemm2Params q = p;
  q.t_full = whole - halved;
  q.n_items = num_tiles;
  q.sched = nullptr;
  if (g_dynamic_tiles && num_tiles > pairs) {
    q.sched = next_sched_slot();
    if (q.sched == nullptr) return static_cast<int>(cudaErrorInvalidValue);
  }
  kern<<<2 * pairs, G2_THREADS, G2_SMEM, stream>>>(*tA, *tB, *tBh, *tD, *tC, tE ? *tE : *tA, q);
  return static_cast<int>(cudaGetLastError());
}

static Gemm2Params base_params(void* D, const void* C, int M, int N, int K, int ldd, int ldc, int flags, float alpha) {
  Gemm2Params p = {};
  p.D = D; p.C = C; p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.ldc = ldc; p.flags = flags; p.alpha = alpha;
  p.status = status_ptr();
  return p;
}

}  // namespace b200

using namespace b200;

// 1: tiles beyond each pair's first are handed out from a counter; 0: fixed round-robin assignment.
B200_API int b200_gemm_2cta_dynamic_tiles(int on) {
  const int old = g_dynamic_tiles;
  if (on >= 0) g_dynamic_tiles = on != 0;
  return old;
}

// 1: the tiles of a last round that fills less than half of the CTA pairs are split into 256 x 128 halves.
B200_API int b200_gemm_2cta_half_tiles(int on) {
  const int old = g_half_tiles;
  if (on >= 0) g_half_tiles = on != 0;
  return old;
}

static int gemm_2cta_run(const void* A, const void* B, void* D, const void* C, int M, int N, int K, int lda, int ldb,
                         int ldd, int ldc, int a_mn_major, int b_mn_major, int flags, float alpha,
                         const float* rope_cos, const float* rope_sin, int rope_T, int rope_ld, int rope_cols,
                         int rope_dim, cudaStream_t stream);

// Same contract as b200_gemm_bf16 (TMA-legal operands only: 16-byte aligned bases and pitches).
B200_API int b200_gemm_bf16_2cta(const void* A, const void* B, void* D, const void* C, int M, int N, int K, int lda,
                                 int ldb, int ldd, int ldc, int a_mn_major, int b_mn_major, int flags, float alpha,
                                 cudaStream_t stream) {
  return gemm_2cta_run(A, B, D, C, M, N, K, lda, ldb, ldd, ldc, a_mn_major, b_mn_major, flags, alpha, nullptr, nullptr,
                       0, 0, 0, 0, stream);
}

// D = rope(A B): the first `rope_cols` columns of the bf16 result are heads of width `rope_dim` (128 or 64,
// rope_cols a multiple of it) that leave the epilogue rotated by the angle of position row % rope_T (fp32 tables,
// transposed: [rope_dim / 2][rope_ld], rope_ld >= rope_T). No C operand; D must be TMA-addressable (16-byte
// aligned base and pitch).
B200_API int b200_gemm_bf16_2cta_rope(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb,
                                      int ldd, int a_mn_major, int b_mn_major, int flags, const void* rope_cos,
                                      const void* rope_sin, int rope_T, int rope_ld, int rope_cols, int rope_dim,
                                      cudaStream_t stream) {
  if ((rope_dim != 128 && rope_dim != 64) || rope_T <= 0 || rope_ld < rope_T || rope_cols <= 0 ||
      rope_cols % rope_dim != 0 || rope_cols > N || rope_cos == nullptr || rope_sin == nullptr ||
      (flags & (G2_OUT_F32 | G2_ADD_C)) != 0 || (reinterpret_cast<uintptr_t>(D) & 15) != 0 || (ldd % 8) != 0)
    return static_cast<int>(cudaErrorInvalidValue);
  return gemm_2cta_run(A, B, D, nullptr, M, N, K, lda, ldb, ldd, 0, a_mn_major, b_mn_major, flags, 1.0f,
                       static_cast<const float*>(rope_cos), static_cast<const float*>(rope_sin), rope_T, rope_ld,
                       rope_cols, rope_dim, stream);
}

static int gemm_2cta_run(const void* A, const void* B, void* D, const void* C, int M, int N, int K, int lda, int ldb,
                         int ldd, int ldc, int a_mn_major, int b_mn_major, int flags, float alpha,
                         const float* rope_cos, const float* rope_sin, int rope_T, int rope_ld, int rope_cols,
                         int rope_dim, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return static_cast<int>(cudaErrorInvalidValue);
  if (((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) != 0 || (lda % 8) != 0 || (ldb % 8) != 0)
    return static_cast<int>(cudaErrorInvalidValue);
  Gemm2Params p = base_params(D, C, M, N, K, ldd, ldc, flags, alpha);
  p.rope_cos = rope_cos; p.rope_sin = rope_sin; p.rope_T = rope_T; p.rope_cols = rope_cols; p.rope_dim = rope_dim;
  p.rope_ld = rope_ld;
  const CUtensorMap* tA = a_mn_major ? get_tensor_map_2d(A, K, M, lda, 64, 64, 2, SWIZZLE_128B_)
                                     : get_tensor_map_2d(A, M, K, lda, G2_BM, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tB = b_mn_major ? get_tensor_map_2d(B, K, N, ldb, 64, 64, 2, SWIZZLE_128B_)
                                     : get_tensor_map_2d(B, N, K, ldb, G2_BN / 2, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tBh = b_mn_major ? tB : get_tensor_map_2d(B, N, K, ldb, G2_BN / 4, 64, 2, SWIZZLE_128B_);
  if (!tA || !tB || !tBh) return static_cast<int>(cudaErrorInvalidValue);
  // Output (and C) through TMA when their bases and pitches are 16-byte aligned; otherwise the
  // epilogue stores straight from registers.
  const int eb = (flags & G2_OUT_F32) ? 4 : 2;
  const bool add = (flags & G2_ADD_C) != 0;
  const CUtensorMap* tD = tA;
  const CUtensorMap* tC = tA;
  if ((reinterpret_cast<uintptr_t>(D) & 15) == 0 && (size_t(ldd) * eb) % 16 == 0 &&
      (!add || ((reinterpret_cast<uintptr_t>(C) & 15) == 0 && (size_t(ldc) * eb) % 16 == 0))) {
    const CUtensorMap* d = get_tensor_map_2d(D, M, N, ldd, 128, 128 / eb, eb, SWIZZLE_128B_);
    const CUtensorMap* c = add ? get_tensor_map_2d(C, M, N, ldc, 128, 128 / eb, eb, SWIZZLE_128B_) : d;
    if (d && c) {
      tD = d;
      tC = c;
      p.flags |= G2_TMA_OUT;
    }
  }
  if (p.rope_cos != nullptr) {       // the rotating epilogue exists for row-major A (x W) and TMA output
    if (!(p.flags & G2_TMA_OUT) || a_mn_major) return static_cast<int>(cudaErrorInvalidValue);
    if (b_mn_major) return launch_tc2<false, true, EPI_ROPE>(tA, tB, tBh, tD, tC, p, stream);
    return launch_tc2<false, false, EPI_ROPE>(tA, tB, tBh, tD, tC, p, stream);
  }
  if (a_mn_major && b_mn_major) return launch_tc2<true, true>(tA, tB, tBh, tD, tC, p, stream);
  if (a_mn_major) return launch_tc2<true, false>(tA, tB, tBh, tD, tC, p, stream);
  if (b_mn_major) return launch_tc2<false, true>(tA, tB, tBh, tD, tC, p, stream);
  return launch_tc2<false, false>(tA, tB, tBh, tD, tC, p, stream);
}

// act[M, I] = silu(A W_gate) * (A W_value) for B = [W_gate | W_value] ([K, 2 I] row-major), A [M, K] row-major,
// in the epilogue of ONE GEMM: a work item's accumulator holds 128 gate columns (the leader CTA's half of B)
// beside the 128 value columns of the same index (the follower's half). GV ([M, 2 I], pitch ldgv), when not null,
// also receives the raw projection (the backward needs it). I must be a multiple of 8 (16-byte column offset of
// the value half); every base 16-byte aligned, every pitch a multiple of 8 elements.
B200_API int b200_gemm_bf16_2cta_swiglu(const void* A, const void* B, void* GV, void* ACT, int M, int I, int K, int lda,
                                        int ldb, int ldgv, int ldact, int flags, cudaStream_t stream) {
  if (M <= 0 || I <= 0) return 0;
  if (K <= 0 || (I % 8) != 0 || ACT == nullptr) return static_cast<int>(cudaErrorInvalidValue);
  const uintptr_t all = reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(GV) |
                        reinterpret_cast<uintptr_t>(ACT);
  if ((all & 15) != 0 || (lda % 8) != 0 || (ldb % 8) != 0 || (ldact % 8) != 0 || (GV != nullptr && (ldgv % 8) != 0))
    return static_cast<int>(cudaErrorInvalidValue);
  Gemm2Params p = base_params(ACT, nullptr, M, 2 * I, K, ldact, 0, (flags & G2_WHOLE_TILES) | G2_TMA_OUT, 1.0f);
  p.sw_I = I;
  p.sw_store_gv = GV != nullptr;
  const CUtensorMap* tA = get_tensor_map_2d(A, M, K, lda, G2_BM, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tB = get_tensor_map_2d(B, K, 2 * I, ldb, 64, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tAct = get_tensor_map_2d(ACT, M, I, ldact, 128, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tG = tA;
  const CUtensorMap* tV = tA;
  if (GV != nullptr) {
    tG = get_tensor_map_2d(GV, M, I, ldgv, 128, 64, 2, SWIZZLE_128B_);
    tV = get_tensor_map_2d(static_cast<const bf16*>(GV) + I, M, I, ldgv, 128, 64, 2, SWIZZLE_128B_);
  }
  if (!tA || !tB || !tAct || !tG || !tV) return static_cast<int>(cudaErrorInvalidValue);
  return launch_tc2<false, true, EPI_SWIGLU>(tA, tB, tAct, tG, tV, p, stream);
}

// LM-head forward without logits in memory: for A [M, K] (tokens) and B [N, K] (vocabulary rows col0 .. col0 + N,
// K-major) every 256-column tile leaves, per row, the maximum and the sum of exp(logit - maximum) of its valid
// columns in pmax / psum ([tile columns][M], this call's first tile column at index nt0) and the tile that holds
// the row's target writes that logit to tlogit[row]. A merge over the tile columns gives the row's log-sum-exp.
B200_API int b200_gemm_bf16_2cta_ce_stats(const void* A, const void* B, int M, int N, int K, int lda, int ldb,
                                          const void* targets, void* pmax, void* psum, void* tlogit, int col0, int nt0,
                                          int vocab, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) != 0 || (lda % 8) != 0 ||
      (ldb % 8) != 0 || !targets || !pmax || !psum || !tlogit)
    return static_cast<int>(cudaErrorInvalidValue);
  Gemm2Params p = base_params(nullptr, nullptr, M, N, K, 0, 0, G2_WHOLE_TILES, 1.0f);
  p.ce_targets = static_cast<const int*>(targets);
  p.ce_pmax = static_cast<float*>(pmax);
  p.ce_psum = static_cast<float*>(psum);
  p.ce_tlogit = static_cast<float*>(tlogit);
  p.ce_col0 = col0;
  p.ce_nt0 = nt0;
  p.ce_vocab = vocab;
  const CUtensorMap* tA = get_tensor_map_2d(A, M, K, lda, G2_BM, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tB = get_tensor_map_2d(B, N, K, ldb, G2_BN / 2, 64, 2, SWIZZLE_128B_);
  if (!tA || !tB) return static_cast<int>(cudaErrorInvalidValue);
  return launch_tc2<false, false, EPI_CE_STATS>(tA, tB, tB, tA, tA, p, stream);
}

// LM-head backward, first GEMM: D[M, N] (bf16) = (exp(A B^T - lse[row]) - [column == target]) * coef[row], the
// gradient of the mean cross-entropy w.r.t. the logits of vocabulary rows col0 .. col0 + N, formed on the
// accumulator (the logits themselves are never stored). D must be TMA-addressable.
B200_API int b200_gemm_bf16_2cta_ce_dlogits(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb,
                                            int ldd, const void* targets, const void* lse, const void* coef, int col0,
                                            cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  const uintptr_t all = reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(D);
  if (K <= 0 || (all & 15) != 0 || (lda % 8) != 0 || (ldb % 8) != 0 || (ldd % 8) != 0 || !targets || !lse || !coef)
    return static_cast<int>(cudaErrorInvalidValue);
  Gemm2Params p = base_params(D, nullptr, M, N, K, ldd, 0, G2_WHOLE_TILES | G2_TMA_OUT, 1.0f);
  p.ce_targets = static_cast<const int*>(targets);
  p.ce_lse = static_cast<const float*>(lse);
  p.ce_coef = static_cast<const float*>(coef);
  p.ce_col0 = col0;
  const CUtensorMap* tA = get_tensor_map_2d(A, M, K, lda, G2_BM, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tB = get_tensor_map_2d(B, N, K, ldb, G2_BN / 2, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tD = get_tensor_map_2d(D, M, N, ldd, 128, 64, 2, SWIZZLE_128B_);
  if (!tA || !tB || !tD) return static_cast<int>(cudaErrorInvalidValue);
  return launch_tc2<false, false, EPI_CE_DLOGITS>(tA, tB, tB, tD, tD, p, stream);
}

// Backward of the fused SwiGLU: d(act) = DOUT W_out^T (DOUT [M, K] row-major, W_out [I, K] K-major) is formed in
// tensor memory and never stored; the epilogue reads the forward's projection GV = [gate | value] ([M, 2 I]) tile by
// tile through TMA and writes DGV = [d gate | d value] with
//   d gate = d act * value * s * (1 + gate (1 - s)),  d value = d act * gate * s,  s = sigmoid(gate).
// I a multiple of 8; every base 16-byte aligned, every pitch a multiple of 8 elements. GV and DGV may not alias.
B200_API int b200_gemm_bf16_2cta_swiglu_bwd(const void* DOUT, const void* WOUT, const void* GV, void* DGV, int M, int I,
                                            int K, int lda, int ldb, int ldgv, int lddgv, int flags,
                                            cudaStream_t stream) {
  if (M <= 0 || I <= 0) return 0;
  const uintptr_t all = reinterpret_cast<uintptr_t>(DOUT) | reinterpret_cast<uintptr_t>(WOUT) |
                        reinterpret_cast<uintptr_t>(GV) | reinterpret_cast<uintptr_t>(DGV);
  if (K <= 0 || (I % 8) != 0 || GV == nullptr || DGV == nullptr || GV == DGV || (all & 15) != 0 || (lda % 8) != 0 ||
      (ldb % 8) != 0 || (ldgv % 8) != 0 || (lddgv % 8) != 0)
    return static_cast<int>(cudaErrorInvalidValue);
  Gemm2Params p = base_params(DGV, nullptr, M, I, K, lddgv, 0, G2_WHOLE_TILES | G2_TMA_OUT, 1.0f);
  p.sw_I = I;
  const CUtensorMap* tA = get_tensor_map_2d(DOUT, M, K, lda, G2_BM, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tB = get_tensor_map_2d(WOUT, I, K, ldb, G2_BN / 2, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tG = get_tensor_map_2d(GV, M, I, ldgv, 128, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tV = get_tensor_map_2d(static_cast<const bf16*>(GV) + I, M, I, ldgv, 128, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tDG = get_tensor_map_2d(DGV, M, I, lddgv, 128, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tDV = get_tensor_map_2d(static_cast<bf16*>(DGV) + I, M, I, lddgv, 128, 64, 2, SWIZZLE_128B_);
  if (!tA || !tB || !tG || !tV || !tDG || !tDV) return static_cast<int>(cudaErrorInvalidValue);
  return launch_tc2<false, false, EPI_SWIGLU_BWD>(tA, tB, tG, tDG, tDV, p, stream, tV);
}

// d(attention output) and delta in one pass: DO[M, N] (bf16) = DY W_O^T for DY [M, K] row-major and W_O [N, K] K-major,
// where row = b * T + t and column = head * head_dim + d; the epilogue reads the forward's attention output O
// ([M, N], pitch ldo) tile by tile through TMA and also leaves DELTA[b][head][t] = sum_d DO O (fp32, computed from DO as
// it is stored). head_dim 128 or 64, N = heads * head_dim, M a multiple of T; every base 16-byte aligned, every pitch
// a multiple of 8 elements. O and DO may not alias.
B200_API int b200_gemm_bf16_2cta_delta(const void* DY, const void* WO, void* DO, const void* O, void* DELTA, int M, int N,
                                       int K, int lda, int ldb, int lddo, int ldo, int T, int head_dim, int flags,
                                       cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  const uintptr_t all = reinterpret_cast<uintptr_t>(DY) | reinterpret_cast<uintptr_t>(WO) |
                        reinterpret_cast<uintptr_t>(DO) | reinterpret_cast<uintptr_t>(O);
  if (K <= 0 || T <= 0 || (M % T) != 0 || (head_dim != 128 && head_dim != 64) || (N % head_dim) != 0 || DO == nullptr ||
      O == nullptr || DELTA == nullptr || DO == O || (all & 15) != 0 || (lda % 8) != 0 || (ldb % 8) != 0 ||
      (lddo % 8) != 0 || (ldo % 8) != 0)
    return static_cast<int>(cudaErrorInvalidValue);
  Gemm2Params p = base_params(DO, O, M, N, K, lddo, ldo, (flags & G2_WHOLE_TILES) | G2_TMA_OUT, 1.0f);
  p.dl_out = static_cast<float*>(DELTA);
  p.dl_T = T;
  p.dl_heads = N / head_dim;
  p.dl_dim = head_dim;
  const CUtensorMap* tA = get_tensor_map_2d(DY, M, K, lda, G2_BM, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tB = get_tensor_map_2d(WO, N, K, ldb, G2_BN / 2, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tBh = get_tensor_map_2d(WO, N, K, ldb, G2_BN / 4, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tD = get_tensor_map_2d(DO, M, N, lddo, 128, 64, 2, SWIZZLE_128B_);
  const CUtensorMap* tO = get_tensor_map_2d(O, M, N, ldo, 128, 64, 2, SWIZZLE_128B_);
  if (!tA || !tB || !tBh || !tD || !tO) return static_cast<int>(cudaErrorInvalidValue);
  return launch_tc2<false, false, EPI_DELTA>(tA, tB, tBh, tD, tO, p, stream);
}
