// Symmetric-memory runtime and the fused gradient path over NVLink / NVSwitch peer memory.
//
// Every rank owns one heap (cudaMalloc) whose IPC handle is exchanged once; after that each rank
// holds a table of W device pointers, one per peer heap, and buffers are addressed as
// (heap base + offset) with the same offset on every rank. The first 64 KiB of a heap is its
// signal pad: 32-bit epoch flags that peers write with st.release.sys and the owner polls with
// ld.acquire.sys. Every poll loop has a wall-clock deadline; when it runs out the kernel records
// ERR_PEER_TIMEOUT in the status word and returns (no trap, no endless spin).
//
// rs_reduce_kernel is the reduce-scatter of one gradient bucket fused with what follows it:
//   start barrier (all ranks finished writing the bucket)  ->  each rank pulls ITS slice of all W
//   peer buckets with 16-byte P2P loads, sums in fp32       ->  one of
//       STORE      : write the reduced slice (bf16 or fp32) into the gradient shard
//       ACCUMULATE : add it into the fp32 gradient shard (gradient accumulation)
//       ADAM       : scale and apply AdamW directly (fp32 master/m/v, bf16 parameter shard)
//   plus, fused in the same pass, the sum of squares / non-finite flag that the global-norm clip
//   needs                                                   ->  end barrier (all ranks finished
//   reading, so the bucket may be overwritten and updated parameters are visible).
// It replaces ncclReduceScatter + cast + accumulate + grad_stats (+ AdamW) — the reference's
// reduce(root=owner) + `grad_shard += tmp` + grad_stats_f16_kernel + adam_update_kernel
// (model/ZeRO3.py:1362-1450, 746-796; model/optimizer.py:112-151).
//
// ag_pull_kernel is the matching all-gather by P2P pulls (used for units whose gather is not
// fused into a GEMM). Blocks of one launch may stand for several "virtual ranks" (gridDim.y) so
// that the multi-rank protocol can be exercised as ONE kernel on a single GPU.
#include <string.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int SYMM_MAX_W = 8;
constexpr int SYMM_PAD_BYTES = 64 * 1024;
constexpr int SYMM_MAX_BLOCKS = 256;          // blocks (per virtual rank) that take part in a barrier
// signal pad layout (uint32 index): channel c, block b, source rank r -> ((c * MAX_BLOCKS) + b) * MAX_W + r
constexpr int SYMM_CHANNELS = 8;
static_assert(SYMM_CHANNELS * SYMM_MAX_BLOCKS * SYMM_MAX_W * 4 <= SYMM_PAD_BYTES, "signal pad too small");

struct SymmTable {
  void* base[SYMM_MAX_W];      // heap base of every rank, as mapped into THIS process
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Barrier among the same-numbered blocks of all W ranks. Thread p < W signals rank p and waits
// for rank p's signal. Returns false (for the whole block) when a wait ran out of time.
__device__ bool peer_block_barrier(const SymmTable& tab, int rank, int W, int channel, uint32_t epoch,
                                   unsigned long long wait_ns, int* status, int kernel_id) {
  int fail = 0;          // combined over the block with a barrier-reduction: no shared memory is used
  if (threadIdx.x < W) {
    const int p = threadIdx.x;
    const int slot = (channel * SYMM_MAX_BLOCKS + int(blockIdx.x)) * SYMM_MAX_W;
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(tab.base[p]) + slot + rank, epoch);
    const uint32_t* mine = static_cast<const uint32_t*>(tab.base[rank]) + slot + p;
    const uint64_t deadline = globaltimer_ns() + wait_ns;
    uint32_t spins = 0;
    while (int32_t(ld_acquire_sys(mine) - epoch) < 0) {
      __nanosleep(spins < 64 ? 100 : 1000);     // back off: the SM is shared with compute kernels
      if ((++spins & 63) == 0 && globaltimer_ns() > deadline) {
        fail = 1;
        if (status != nullptr && atomicCAS(status, 0, ERR_PEER_TIMEOUT) == 0) {
          status[1] = kernel_id;
          status[2] = p;
        }
        break;
      }
    }
  }
  return __syncthreads_or(fail) == 0;
}

enum RsMode : int { RS_STORE = 0, RS_ACCUMULATE = 1, RS_ADAM = 2 };

struct RsAdam {
  float* m; float* v; float* master; bf16* param;
  float lr, beta1, beta2, eps, weight_decay, m_corr, v_corr, grad_scale;
};

struct RsParams {
  SymmTable tab[SYMM_MAX_W];     // tab[v]: peer table as seen by virtual rank v (production: only tab[0])
  void* dst[SYMM_MAX_W];         // reduced slice destination of virtual rank v
  float* stats[SYMM_MAX_W];      // [sum of squares, non-finite flag] or null
  RsAdam adam[SYMM_MAX_W];
  unsigned long long bucket_off; // byte offset of the bucket inside every heap
  long long n_slice;             // elements per rank slice (multiple of 8)
  // Part of the BUCKET to reduce, [range_lo, range_hi) in elements (multiples of 8): every rank handles the
  // intersection with its own slice, possibly nothing. The whole bucket is [0, W * n_slice).
  long long range_lo, range_hi;
  int rank0, W, mode, dst_fp32, do_stats;
  uint32_t epoch;
  unsigned long long wait_ns;
  int* status;
  // Staged form (one real rank per launch): the peers' parts of this rank's slice have already been copied into
  // LOCAL memory by the copy engines, peer (rank + 1 + q) % W at stage + q * stage_stride elements, element 0 of a
  // part being element stage_first of the slice. The kernel then touches no peer memory and has no barrier.
  const bf16* stage;
  long long stage_stride, stage_first;
};

__device__ __forceinline__ void adam_apply(float g, float& m, float& v, float& w, const RsAdam& a) {
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  if (a.weight_decay > 0.f) w *= (1.f - a.lr * a.weight_decay);
  w -= a.lr * (m * a.m_corr) / (sqrtf(v * a.v_corr) + a.eps);
}

// What happens to one reduced vector (8 gradients in fp32): AdamW, store or accumulate, plus the
// statistics of the global-norm clip.
__device__ __forceinline__ void rs_consume(const RsParams& p, int vr, long long i, float (&acc)[8], float& ss,
                                           int& bad) {
  if (p.mode == RS_ADAM) {
    const RsAdam& a = p.adam[vr];
    float4* m4 = reinterpret_cast<float4*>(a.m) + 2 * i;
    float4* v4 = reinterpret_cast<float4*>(a.v) + 2 * i;
    float4* w4 = reinterpret_cast<float4*>(a.master) + 2 * i;
    float mm[8], vv[8], ww[8];
    *reinterpret_cast<float4*>(mm) = m4[0]; *reinterpret_cast<float4*>(mm + 4) = m4[1];
    *reinterpret_cast<float4*>(vv) = v4[0]; *reinterpret_cast<float4*>(vv + 4) = v4[1];
    *reinterpret_cast<float4*>(ww) = w4[0]; *reinterpret_cast<float4*>(ww + 4) = w4[1];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (!isfinite(acc[e])) bad = 1;
      ss += acc[e] * acc[e];
      adam_apply(acc[e] * a.grad_scale, mm[e], vv[e], ww[e], a);
    }
    m4[0] = *reinterpret_cast<float4*>(mm); m4[1] = *reinterpret_cast<float4*>(mm + 4);
    v4[0] = *reinterpret_cast<float4*>(vv); v4[1] = *reinterpret_cast<float4*>(vv + 4);
    w4[0] = *reinterpret_cast<float4*>(ww); w4[1] = *reinterpret_cast<float4*>(ww + 4);
    uint4 o;
    bf162* o2 = reinterpret_cast<bf162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(ww[2 * e], ww[2 * e + 1]);
    reinterpret_cast<uint4*>(a.param)[i] = o;
  } else if (p.dst_fp32) {
    float4* d4 = reinterpret_cast<float4*>(p.dst[vr]) + 2 * i;
    if (p.mode == RS_ACCUMULATE) {
      const float4 o0 = d4[0], o1 = d4[1];
      acc[0] += o0.x; acc[1] += o0.y; acc[2] += o0.z; acc[3] += o0.w;
      acc[4] += o1.x; acc[5] += o1.y; acc[6] += o1.z; acc[7] += o1.w;
    }
    d4[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    d4[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if (p.do_stats) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (!isfinite(acc[e])) bad = 1; else ss += acc[e] * acc[e];
      }
    }
  } else {
    uint4 o;
    bf162* o2 = reinterpret_cast<bf162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    reinterpret_cast<uint4*>(p.dst[vr])[i] = o;
    if (p.do_stats) {
      // statistics of what is stored (the bf16-rounded value), as the separate pass would see it
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(o2[e]);
        if (!isfinite(f.x) || !isfinite(f.y)) bad = 1; else ss += f.x * f.x + f.y * f.y;
      }
    }
  }
}

// The pull-and-sum loop. Every thread keeps W x U = 8 16-byte peer loads in flight (an NVLink round
// trip is a few microseconds, so bandwidth is bought with outstanding loads, not with threads).
template <int WT, int U>
__device__ __forceinline__ void rs_loop(const RsParams& p, int vr, const uint4* const (&src)[SYMM_MAX_W], long long v_lo,
                                        long long v_hi, float& ss, int& bad) {
  constexpr int WM = WT > 0 ? WT : SYMM_MAX_W;
  const int W = WT > 0 ? WT : p.W;
  const long long stride = (long long)gridDim.x * blockDim.x;
  // vectors [v_lo, v_hi) of this rank's slice (8 gradients each)
  for (long long i0 = v_lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < v_hi; i0 += stride * U) {
    uint4 raw[U][WM];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < v_hi) {
#pragma unroll
        for (int q = 0; q < WM; ++q)
          if (q < W) raw[u][q] = src[q][i];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= v_hi) break;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int q = 0; q < WM; ++q) {
        if (q < W) {
          const bf162* h = reinterpret_cast<const bf162*>(&raw[u][q]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            acc[2 * e] += f.x;
            acc[2 * e + 1] += f.y;
          }
        }
      }
      rs_consume(p, vr, i, acc, ss, bad);
    }
  }
}

__global__ void __launch_bounds__(256, 2) rs_reduce_kernel(const RsParams p) {
  const int vr = blockIdx.y;
  const int rank = p.rank0 + vr;
  const SymmTable& tab = p.tab[vr];
  const int W = p.W;
  const bool staged = p.stage != nullptr;
  if (!staged && !peer_block_barrier(tab, rank, W, 0, 2 * p.epoch - 1, p.wait_ns, p.status, 201)) return;

  const uint4* src[SYMM_MAX_W];
#pragma unroll
  for (int q = 0; q < SYMM_MAX_W; ++q) {
    // start with the next rank so that at any moment the ranks pull from different peers
    const int peer = (rank + 1 + q) % W;
    src[q] = reinterpret_cast<const uint4*>(static_cast<const char*>(tab.base[q < W ? peer : rank]) + p.bucket_off) +
             size_t(rank) * (p.n_slice / 8);
    // staged: the same summation order, but the peers' parts are read from the local staging buffer (indexed like
    // the slice: the pointer is moved back by the part's first element)
    if (staged && q < W - 1)
      src[q] = reinterpret_cast<const uint4*>(p.stage + size_t(q) * size_t(p.stage_stride)) - p.stage_first / 8;
  }
  float ss = 0.f;
  int bad = 0;
  // this rank's share of the requested bucket range, as vectors of its slice
  const long long s0 = (long long)rank * p.n_slice;
  const long long lo = min(max(p.range_lo - s0, 0ll), p.n_slice), hi = min(max(p.range_hi - s0, 0ll), p.n_slice);
  const long long v_lo = lo / 8, v_hi = hi / 8;
  switch (W) {
    case 2: rs_loop<2, 4>(p, vr, src, v_lo, v_hi, ss, bad); break;
    case 4: rs_loop<4, 2>(p, vr, src, v_lo, v_hi, ss, bad); break;
    case 8: rs_loop<8, 1>(p, vr, src, v_lo, v_hi, ss, bad); break;
    default: rs_loop<0, 1>(p, vr, src, v_lo, v_hi, ss, bad); break;
  }
  if (p.do_stats && p.stats[vr] != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ss += __shfl_xor_sync(0xffffffffu, ss, o);
      bad |= __shfl_xor_sync(0xffffffffu, bad, o);
    }
    if ((threadIdx.x & 31) == 0) {
      if (ss != 0.f) atomicAdd(&p.stats[vr][0], ss);
      if (bad) p.stats[vr][1] = 1.f;
    }
  }
  // all of this block's reads (and parameter writes) are done before peers are told so
  if (!staged) peer_block_barrier(tab, rank, W, 0, 2 * p.epoch, p.wait_ns, p.status, 202);
}

struct AgParams {
  SymmTable tab[SYMM_MAX_W];
  void* out[SYMM_MAX_W];          // local gather buffer of virtual rank v (W * n_slice elements)
  unsigned long long shard_off;   // byte offset of the unit's slice inside every heap
  long long n_slice;              // elements per rank slice (multiple of 8)
  int rank0, W;
  // range of the gather buffer in 16-byte vectors and what to do with it:
  // 0 copy everything, 1 leave [range_lo, range_hi) out (another kernel fills it), 2 copy only that range
  long long range_lo, range_hi;
  int range_mode;
};

// Plain all-gather by pulls: out[q * n_slice + i] = peer q's slice[i]. No barrier inside: parameter
// shards only change in the optimizer step, which is fenced by symm_barrier_kernel.
__global__ void __launch_bounds__(512) ag_pull_kernel(const AgParams p) {
  const int vr = blockIdx.y;
  const int rank = p.rank0 + vr;
  const long long nvec = p.n_slice / 8;
  uint4* out = static_cast<uint4*>(p.out[vr]);
  constexpr int U = 4;     // independent 16-byte loads in flight per thread (NVLink latency is ~2 us)
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int q = 0; q < p.W; ++q) {
    const int peer = (rank + q) % p.W;     // own slice first, then peers in ring order
    const uint4* s = reinterpret_cast<const uint4*>(static_cast<const char*>(p.tab[vr].base[peer]) + p.shard_off);
    uint4* d = out + (long long)peer * nvec;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride * U) {
      uint4 v[U];
      bool take[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long k = i + u * stride;
        const long long g = (long long)peer * nvec + k;      // position in the gather buffer
        const bool inside = g >= p.range_lo && g < p.range_hi;
        take[u] = k < nvec && (p.range_mode == 0 || (p.range_mode == 1 ? !inside : inside));
        if (take[u]) v[u] = s[k];
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (take[u]) d[i + u * stride] = v[u];
    }
  }
}

struct BarrierParams {
  SymmTable tab[SYMM_MAX_W];
  int rank0, W, channel;
  uint32_t epoch;
  unsigned long long wait_ns;
  int* status;
};

__global__ void symm_barrier_kernel(const BarrierParams p) {
  peer_block_barrier(p.tab[blockIdx.y], p.rank0 + blockIdx.y, p.W, p.channel, p.epoch, p.wait_ns, p.status, 203);
}

// Waits on a flag nobody sets: exercises the time-out path (returns an error status, stays usable).
__global__ void symm_wait_probe_kernel(const uint32_t* flag, uint32_t want, unsigned long long wait_ns, int* status) {
  const uint64_t deadline = globaltimer_ns() + wait_ns;
  uint32_t spins = 0;
  while (int32_t(ld_acquire_sys(flag) - want) < 0) {
    if ((++spins & 63) == 0 && globaltimer_ns() > deadline) {
      if (status != nullptr && atomicCAS(status, 0, ERR_PEER_TIMEOUT) == 0) status[1] = 204;
      return;
    }
  }
}

}  // namespace b200

using namespace b200;

// ---------------------------------------------------------------- heap + IPC
B200_API int b200_symm_alloc(unsigned long long bytes, void** out) {
  void* p = nullptr;
  B200_CHECK(cudaMalloc(&p, bytes));
  B200_CHECK(cudaMemset(p, 0, bytes));
  *out = p;
  return 0;
}
B200_API int b200_symm_free(void* p) { return static_cast<int>(cudaFree(p)); }
B200_API int b200_symm_export(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  B200_CHECK(cudaIpcGetMemHandle(&h, p));
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
B200_API int b200_symm_import(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  B200_CHECK(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
B200_API int b200_symm_unimport(void* p) { return static_cast<int>(cudaIpcCloseMemHandle(p)); }
B200_API int b200_symm_pad_bytes() { return SYMM_PAD_BYTES; }

// Peer copies of one collective, each on a helper stream of its own so that several copy engines (and several
// NVLink paths through the switch) work at once: `st` forks into the helper streams with one event and joins them
// with one event per copy. Two sets of helper streams per device - set 0 for parameter gathers, set 1 for
// gradient reductions - so that a gather issued on one caller stream never queues behind the copies of a
// reduction issued on another. The events are reused by every call: a stream wait refers to the record that
// precedes it in host order, and all calls of a device come from one host thread at a time (the mutex covers
// the creation).
struct CopyFan {
  cudaStream_t s[SYMM_MAX_W] = {};
  cudaEvent_t fork = nullptr;
  cudaEvent_t join[SYMM_MAX_W] = {};
  bool ready = false;
};
static int g_parallel_copies = 0;

static CopyFan* copy_fan(int set) {
  static std::mutex mu;
  static CopyFan fans[64][2];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || set < 0 || set > 1) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  CopyFan& f = fans[dev][set];
  if (!f.ready) {
    if (cudaEventCreateWithFlags(&f.fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    for (int i = 0; i < SYMM_MAX_W; ++i) {
      if (cudaStreamCreateWithFlags(&f.s[i], cudaStreamNonBlocking) != cudaSuccess) return nullptr;
      if (cudaEventCreateWithFlags(&f.join[i], cudaEventDisableTiming) != cudaSuccess) return nullptr;
    }
    f.ready = true;
  }
  return &f;
}

struct PeerCopy {
  void* dst;
  const void* src;
  size_t bytes;
};

static int fan_copies(int set, const PeerCopy* c, int n, cudaStream_t st) {
  if (n <= 0) return 0;
  CopyFan* f = (g_parallel_copies && n > 1) ? copy_fan(set) : nullptr;
  if (f == nullptr) {
    for (int i = 0; i < n; ++i) B200_CHECK(cudaMemcpyAsync(c[i].dst, c[i].src, c[i].bytes, cudaMemcpyDeviceToDevice, st));
    return 0;
  }
  B200_CHECK(cudaEventRecord(f->fork, st));
  for (int i = 0; i < n && i < SYMM_MAX_W; ++i) {
    B200_CHECK(cudaStreamWaitEvent(f->s[i], f->fork, 0));
    B200_CHECK(cudaMemcpyAsync(c[i].dst, c[i].src, c[i].bytes, cudaMemcpyDeviceToDevice, f->s[i]));
    B200_CHECK(cudaEventRecord(f->join[i], f->s[i]));
    B200_CHECK(cudaStreamWaitEvent(st, f->join[i], 0));
  }
  return 0;
}

// 1: the peer copies of a copy-engine gather / reduce-scatter run on helper streams side by side; 0 (default): one
// after the other on the caller's stream. Measured at 4 GPUs on one 88.6 MB unit: the gather gains little (126 against
// 132 us) and the staged reduce-scatter loses (237 against 189 us: the fork and join events sit between the barrier
// kernels and the copies); the 1.3 B step is the same within its noise. Returns the previous setting; a negative
// argument only reads it.
B200_API int b200_symm_parallel_copies(int on) {
  const int old = g_parallel_copies;
  if (on >= 0) g_parallel_copies = on != 0;
  return old;
}

static int fill_tables(SymmTable* dst, const void* const* bases, int W, int vranks) {
  // bases: vranks x W pointers (row v = table of virtual rank v)
  for (int v = 0; v < vranks; ++v)
    for (int r = 0; r < SYMM_MAX_W; ++r) dst[v].base[r] = r < W ? const_cast<void*>(bases[v * W + r]) : nullptr;
  return 0;
}

// mode: 0 store, 1 accumulate (fp32 dst), 2 adam. adam_ptrs: vranks x 4 pointers (m, v, master, param);
// adam_f: lr, beta1, beta2, eps, weight_decay, m_corr, v_corr, grad_scale.
static int symm_reduce_scatter_impl(const void* const* bases, int W, int rank0, int vranks,
                                    unsigned long long bucket_off, long long n_slice, long long range_lo,
                                    long long range_hi, void* const* dst, int dst_fp32, int mode, void* const* stats,
                                    int do_stats, void* const* adam_ptrs, const float* adam_f, unsigned int epoch,
                                    unsigned long long wait_ns, int blocks, cudaStream_t st,
                                    const void* stage = nullptr, long long stage_stride = 0, long long stage_first = 0) {
  if (W < 1 || W > SYMM_MAX_W || vranks < 1 || vranks > SYMM_MAX_W || (n_slice % 8) != 0 || range_lo < 0 ||
      range_hi > (long long)W * n_slice || range_lo > range_hi || ((range_lo | range_hi) % 8) != 0)
    return static_cast<int>(cudaErrorInvalidValue);
  if (n_slice == 0) return 0;
  RsParams p = {};
  fill_tables(p.tab, bases, W, vranks);
  for (int v = 0; v < vranks; ++v) {
    p.dst[v] = dst ? dst[v] : nullptr;
    p.stats[v] = stats ? static_cast<float*>(stats[v]) : nullptr;
    if (mode == RS_ADAM) {
      p.adam[v] = RsAdam{static_cast<float*>(adam_ptrs[4 * v]), static_cast<float*>(adam_ptrs[4 * v + 1]),
                         static_cast<float*>(adam_ptrs[4 * v + 2]), static_cast<bf16*>(adam_ptrs[4 * v + 3]),
                         adam_f[0], adam_f[1], adam_f[2], adam_f[3], adam_f[4], adam_f[5], adam_f[6], adam_f[7]};
    }
  }
  p.bucket_off = bucket_off; p.n_slice = n_slice; p.rank0 = rank0; p.W = W; p.mode = mode; p.dst_fp32 = dst_fp32;
  p.range_lo = range_lo; p.range_hi = range_hi;
  p.do_stats = do_stats; p.epoch = epoch; p.wait_ns = wait_ns; p.status = status_ptr();
  p.stage = static_cast<const bf16*>(stage); p.stage_stride = stage_stride; p.stage_first = stage_first;
  if (blocks < 1) blocks = 1;
  if (blocks > SYMM_MAX_BLOCKS && stage == nullptr) blocks = SYMM_MAX_BLOCKS;     // barrier slots; none when staged
  B200_PREFER_MAX_SMEM(rs_reduce_kernel);
  rs_reduce_kernel<<<dim3(blocks, vranks), 256, 0, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// mode: 0 store, 1 accumulate (fp32 dst), 2 adam. adam_ptrs: vranks x 4 pointers (m, v, master, param);
// adam_f: lr, beta1, beta2, eps, weight_decay, m_corr, v_corr, grad_scale.
B200_API int b200_symm_reduce_scatter(const void* const* bases, int W, int rank0, int vranks,
                                      unsigned long long bucket_off, long long n_slice, void* const* dst, int dst_fp32,
                                      int mode, void* const* stats, int do_stats, void* const* adam_ptrs,
                                      const float* adam_f, unsigned int epoch, unsigned long long wait_ns, int blocks,
                                      cudaStream_t st) {
  return symm_reduce_scatter_impl(bases, W, rank0, vranks, bucket_off, n_slice, 0, (long long)W * n_slice, dst,
                                  dst_fp32, mode, stats, do_stats, adam_ptrs, adam_f, epoch, wait_ns, blocks, st);
}

// The same restricted to the elements [range_lo, range_hi) of the bucket (multiples of 8): a gradient bucket
// is reduced in parts as soon as each part is complete (sub-buckets), every rank taking what falls into its slice.
// dst still points at the START of the rank's reduced slice.
B200_API int b200_symm_reduce_scatter_range(const void* const* bases, int W, int rank0, int vranks,
                                            unsigned long long bucket_off, long long n_slice, long long range_lo,
                                            long long range_hi, void* const* dst, int dst_fp32, int mode,
                                            void* const* stats, int do_stats, void* const* adam_ptrs,
                                            const float* adam_f, unsigned int epoch, unsigned long long wait_ns,
                                            int blocks, cudaStream_t st) {
  return symm_reduce_scatter_impl(bases, W, rank0, vranks, bucket_off, n_slice, range_lo, range_hi, dst, dst_fp32,
                                  mode, stats, do_stats, adam_ptrs, adam_f, epoch, wait_ns, blocks, st);
}

B200_API int b200_symm_barrier(const void* const* bases, int W, int rank0, int vranks, int channel, unsigned int epoch,
                               unsigned long long wait_ns, cudaStream_t st);

// Reduce-scatter with the copy engines doing the moving: (1) barrier - every rank's bucket is complete; (2) one
// cudaMemcpyAsync per peer brings that peer's part of THIS rank's slice into the local staging buffer; (3) barrier -
// every rank has read what it needs, the buckets may be rewritten; (4) a local kernel sums the staged parts and the
// rank's own part in the order of the pull kernel (bit-identical result) and stores / accumulates / applies AdamW,
// with the statistics. No SM waits on a peer or on NVLink: the kernel of step 4 runs at HBM speed. `stage` holds
// W - 1 parts of `stage_stride` elements (>= the rank's share of [range_lo, range_hi), a multiple of 8). `barriers`
// 0 leaves steps 1 and 3 out (single-GPU tests that run the ranks one after the other). Channel `channel` (>= 1) with
// epochs 2 * epoch - 1 and 2 * epoch.
B200_API int b200_symm_reduce_scatter_staged(const void* const* bases, int W, int rank, unsigned long long bucket_off,
                                             long long n_slice, long long range_lo, long long range_hi, void* dst,
                                             int dst_fp32, int mode, void* stats, int do_stats, void* const* adam_ptrs,
                                             const float* adam_f, void* stage, long long stage_stride, int barriers,
                                             int channel, unsigned int epoch, unsigned long long wait_ns, int blocks,
                                             cudaStream_t st) {
  if (W < 1 || W > SYMM_MAX_W || rank < 0 || rank >= W || (n_slice % 8) != 0 || range_lo < 0 ||
      range_hi > (long long)W * n_slice || range_lo > range_hi || ((range_lo | range_hi) % 8) != 0 || stage == nullptr ||
      (stage_stride % 8) != 0)
    return static_cast<int>(cudaErrorInvalidValue);
  if (n_slice == 0) return 0;
  const long long s0 = (long long)rank * n_slice;
  const long long lo = std::min(std::max(range_lo - s0, 0ll), n_slice), hi = std::min(std::max(range_hi - s0, 0ll), n_slice);
  if (hi - lo > stage_stride) return static_cast<int>(cudaErrorInvalidValue);
  if (barriers) {
    const int rc = b200_symm_barrier(bases, W, rank, 1, channel, 2 * epoch - 1, wait_ns, st);
    if (rc != 0) return rc;
  }
  if (hi > lo) {
    PeerCopy c[SYMM_MAX_W];
    for (int q = 0; q < W - 1; ++q) {
      const int peer = (rank + 1 + q) % W;
      c[q].src = static_cast<const char*>(bases[peer]) + bucket_off + size_t(s0 + lo) * 2;
      c[q].dst = static_cast<char*>(stage) + size_t(q) * size_t(stage_stride) * 2;
      c[q].bytes = size_t(hi - lo) * 2;
    }
    const int rc = fan_copies(1, c, W - 1, st);
    if (rc != 0) return rc;
  }
  if (barriers) {
    const int rc = b200_symm_barrier(bases, W, rank, 1, channel, 2 * epoch, wait_ns, st);
    if (rc != 0) return rc;
  }
  if (hi <= lo) return 0;
  void* dsts[1] = {dst};
  void* sts[1] = {stats};
  return symm_reduce_scatter_impl(bases, W, rank, 1, bucket_off, n_slice, range_lo, range_hi, dsts, dst_fp32, mode, sts,
                                  do_stats, adam_ptrs, adam_f, 0, wait_ns, blocks, st, stage, stage_stride, lo);
}

static int symm_all_gather_impl(const void* const* bases, int W, int rank0, int vranks, unsigned long long shard_off,
                                long long n_slice, void* const* out, int blocks, unsigned long long range_lo_bytes,
                                unsigned long long range_hi_bytes, int range_mode, cudaStream_t st) {
  if (W < 1 || W > SYMM_MAX_W || vranks < 1 || vranks > SYMM_MAX_W || (n_slice % 8) != 0)
    return static_cast<int>(cudaErrorInvalidValue);
  if (n_slice == 0) return 0;
  AgParams p = {};
  fill_tables(p.tab, bases, W, vranks);
  for (int v = 0; v < vranks; ++v) p.out[v] = out[v];
  p.shard_off = shard_off; p.n_slice = n_slice; p.rank0 = rank0; p.W = W;
  if (range_mode < 0 || range_mode > 2 || (range_lo_bytes | range_hi_bytes) % 16 != 0)
    return static_cast<int>(cudaErrorInvalidValue);
  p.range_lo = (long long)(range_lo_bytes / 16); p.range_hi = (long long)(range_hi_bytes / 16); p.range_mode = range_mode;
  if (blocks < 1) blocks = 1;
  B200_PREFER_MAX_SMEM(ag_pull_kernel);
  ag_pull_kernel<<<dim3(blocks, vranks), 512, 0, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_symm_all_gather(const void* const* bases, int W, int rank0, int vranks, unsigned long long shard_off,
                                  long long n_slice, void* const* out, int blocks, cudaStream_t st) {
  return symm_all_gather_impl(bases, W, rank0, vranks, shard_off, n_slice, out, blocks, 0, 0, 0, st);
}

// As b200_symm_all_gather, restricted by a byte range of the gather buffer: mode 1 leaves the range
// out (it is filled by the GEMM that consumes it), mode 2 copies only the range.
B200_API int b200_symm_all_gather_range(const void* const* bases, int W, int rank0, int vranks,
                                        unsigned long long shard_off, long long n_slice, void* const* out, int blocks,
                                        unsigned long long range_lo_bytes, unsigned long long range_hi_bytes,
                                        int range_mode, cudaStream_t st) {
  return symm_all_gather_impl(bases, W, rank0, vranks, shard_off, n_slice, out, blocks, range_lo_bytes,
                              range_hi_bytes, range_mode, st);
}

// All-gather by the copy engines: one cudaMemcpyAsync per rank slice (peer heap -> local gather buffer) on
// `st`, peers taken in ring order starting after this rank so that at any moment the ranks read from
// different sources. No SM takes part, which is the point: the parameter prefetch of a ZeRO unit runs beside
// persistent GEMMs that are tuned for all SMs. `out` may contain the local slice itself (an in-place gather
// of a replicated buffer): the copy of a slice onto itself is skipped. Ordering against the owners' updates
// is the caller's (stream events plus symm_barrier_kernel), exactly as for ag_pull_kernel.
B200_API int b200_symm_all_gather_copy(const void* const* bases, int W, int rank, unsigned long long shard_off,
                                       long long n_slice, int elem_bytes, void* out, cudaStream_t st) {
  if (W < 1 || W > SYMM_MAX_W || rank < 0 || rank >= W || n_slice < 0 || elem_bytes < 1)
    return static_cast<int>(cudaErrorInvalidValue);
  const size_t bytes = size_t(n_slice) * size_t(elem_bytes);
  if (bytes == 0) return 0;
  PeerCopy c[SYMM_MAX_W];
  int n = 0;
  for (int q = 1; q <= W; ++q) {
    const int peer = (rank + q) % W;          // the local slice comes last
    const char* src = static_cast<const char*>(bases[peer]) + shard_off;
    char* dst = static_cast<char*>(out) + size_t(peer) * bytes;
    if (src == dst) continue;
    c[n].src = src; c[n].dst = dst; c[n].bytes = bytes;
    ++n;
  }
  return fan_copies(0, c, n, st);
}

// The copy-engine gather without the byte range [lo, hi) of the gather buffer (the consuming GEMM fills that part
// itself while it runs): per peer slice the bytes before and after the range, at most two copies.
B200_API int b200_symm_all_gather_copy_skip(const void* const* bases, int W, int rank, unsigned long long shard_off,
                                            long long n_slice, int elem_bytes, void* out, unsigned long long lo,
                                            unsigned long long hi, cudaStream_t st) {
  if (W < 1 || W > SYMM_MAX_W || rank < 0 || rank >= W || n_slice < 0 || elem_bytes < 1 || lo > hi)
    return static_cast<int>(cudaErrorInvalidValue);
  const size_t bytes = size_t(n_slice) * size_t(elem_bytes);
  if (bytes == 0) return 0;
  for (int q = 1; q <= W; ++q) {
    const int peer = (rank + q) % W;
    const size_t a = size_t(peer) * bytes, b = a + bytes;
    const char* src = static_cast<const char*>(bases[peer]) + shard_off;
    char* dst = static_cast<char*>(out);
    const size_t cuts[2][2] = {{a, std::min<size_t>(b, lo)}, {std::max<size_t>(a, hi), b}};
    for (int c = 0; c < 2; ++c) {
      if (cuts[c][1] <= cuts[c][0]) continue;
      if (src + (cuts[c][0] - a) == dst + cuts[c][0]) continue;
      B200_CHECK(cudaMemcpyAsync(dst + cuts[c][0], src + (cuts[c][0] - a), cuts[c][1] - cuts[c][0],
                                 cudaMemcpyDeviceToDevice, st));
    }
  }
  return 0;
}

B200_API int b200_symm_barrier(const void* const* bases, int W, int rank0, int vranks, int channel, unsigned int epoch,
                               unsigned long long wait_ns, cudaStream_t st) {
  if (W < 1 || W > SYMM_MAX_W || channel < 1 || channel >= SYMM_CHANNELS) return static_cast<int>(cudaErrorInvalidValue);
  BarrierParams p = {};
  fill_tables(p.tab, bases, W, vranks);
  p.rank0 = rank0; p.W = W; p.channel = channel; p.epoch = epoch; p.wait_ns = wait_ns; p.status = status_ptr();
  B200_PREFER_MAX_SMEM(symm_barrier_kernel);
  symm_barrier_kernel<<<dim3(1, vranks), 32, 0, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_symm_wait_probe(const void* flag, unsigned int want, unsigned long long wait_ns, cudaStream_t st) {
  symm_wait_probe_kernel<<<1, 1, 0, st>>>(static_cast<const uint32_t*>(flag), want, wait_ns, status_ptr());
  return static_cast<int>(cudaGetLastError());
}
