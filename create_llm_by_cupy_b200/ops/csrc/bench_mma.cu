// Micro-benchmark behind the shape choices of the attention kernels: what one tcgen05.mma costs when instructions
// are issued back to back (one CTA per SM, M = 128, K = 16, bf16), by N, by where A comes from (shared or tensor
// memory) and with or without other warps loading and storing tensor memory at the same time. Operands are zeros:
// only the timing matters. Every wait is bounded.
#include "common.cuh"
#include "ptx.cuh"

namespace b200 {

// MODE 0: A and B from shared memory, both K-major; MODE 1: A from tensor memory, B from shared memory MN-major.
// traffic: 0 none; 1 eight warps loop over tcgen05.ld; 2 the same with a tcgen05.st per round.
template <int N, int MODE>
__global__ void __launch_bounds__(384, 1) bench_mma_kernel(long long* out, int reps, int depth, int traffic) {
  extern __shared__ uint8_t bm_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(bm_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  __shared__ int stop;
  volatile __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    stop = 0;
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < (96 << 10) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  const int warp = threadIdx.x >> 5;
  if (warp == 2) tmem_alloc(&slot, 512);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = slot;
  if (threadIdx.x == 32) {
    constexpr uint32_t idesc = MODE == 0 ? umma_idesc_bf16(128, N, 0, 0) : umma_idesc_bf16(128, N, 0, 1);
    const uint32_t aA = smem_u32(smem), aB = aA + (32 << 10);
    const long long t0 = clock64();
    uint32_t phase = 0;
    for (int r = 0; r < reps; ++r) {
      for (int j = 0; j < depth; ++j) {
        const int kk = j & 3;
        if (MODE == 0)
          umma_bf16_ss(tb + 256, umma_smem_desc(aA + kk * 32, 16, 1024), umma_smem_desc(aB + kk * 32, 16, 1024), idesc,
                       j != 0);
        else
          umma_bf16_ts(tb + 256, tb + 128 + kk * 8, umma_smem_desc(aB + kk * 2048, 8192, 1024), idesc, j != 0);
      }
      umma_commit(&bar);
      if (!mbar_wait(&bar, phase, &abort_flag)) break;
      phase ^= 1;
    }
    const long long t1 = clock64();
    if (blockIdx.x == 0) out[0] = t1 - t0;
    *reinterpret_cast<volatile int*>(&stop) = 1;
  } else if (warp >= 4 && traffic != 0) {
    const uint32_t t = tb + (uint32_t((warp & 3) * 32) << 16) + ((warp >= 8) ? 64 : 0);
    uint32_t acc = 0;
    long long n = 0;
    const long long t0 = clock64();
    while (*reinterpret_cast<volatile int*>(&stop) == 0 && n < 2000000) {
      uint32_t a[16], b[16];
      tmem_ld_32x32b_x16(t, a);
      tmem_ld_32x32b_x16(t + 16, b);
      tmem_ld_wait();
      acc += a[3] ^ b[5];
      if (traffic == 2) {
        uint32_t pk[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) pk[i] = a[i] + b[i];
        tmem_st_32x32b_x8(t + 32, pk);
        tmem_st_wait();
      }
      ++n;
    }
    const long long t1 = clock64();
    if (blockIdx.x == 0 && threadIdx.x == 128) {
      out[1] = n > 0 ? (t1 - t0) / n : 0;       // clocks per round of two 16-column loads
      out[2] = acc;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tb, 512);
  }
}

template <int N, int MODE>
static int bench_mma_run(int traffic, int reps, int depth, long long* out3) {
  auto k = bench_mma_kernel<N, MODE>;
  B200_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 << 10));
  long long* d = nullptr;
  B200_CHECK(cudaMalloc(&d, 32));
  B200_CHECK(cudaMemset(d, 0, 32));
  k<<<num_sms(), 384, 100 << 10>>>(d, 2, depth, traffic);          // warm-up
  B200_CHECK(cudaDeviceSynchronize());
  k<<<num_sms(), 384, 100 << 10>>>(d, reps, depth, traffic);
  const cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) cudaMemcpy(out3, d, 24, cudaMemcpyDeviceToHost);
  cudaFree(d);
  return static_cast<int>(e);
}

}  // namespace b200

using namespace b200;

// out3: [clocks for reps * depth instructions, clocks per load round of the traffic warps, checksum].
// n in {64, 128, 256}; a_in_tmem 0 / 1 (N = 256 only from shared memory).
B200_API int b200_bench_mma(int n, int a_in_tmem, int traffic, int reps, int depth, long long* out3) {
  if (reps < 1 || depth < 1 || depth > 64 || traffic < 0 || traffic > 2) return static_cast<int>(cudaErrorInvalidValue);
  if (!a_in_tmem) {
    if (n == 64) return bench_mma_run<64, 0>(traffic, reps, depth, out3);
    if (n == 128) return bench_mma_run<128, 0>(traffic, reps, depth, out3);
    if (n == 256) return bench_mma_run<256, 0>(traffic, reps, depth, out3);
  } else {
    if (n == 64) return bench_mma_run<64, 1>(traffic, reps, depth, out3);
    if (n == 128) return bench_mma_run<128, 1>(traffic, reps, depth, out3);
  }
  return static_cast<int>(cudaErrorInvalidValue);
}
