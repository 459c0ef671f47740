// Host-side helpers shared by every translation unit of the native library:
//   * the exported-symbol macro and launch-error convention (every entry point returns a
//     cudaError_t-compatible int, 0 = success);
//   * the device status word kernels use to report a bounded wait that ran out;
//   * a cache of TMA tensor maps (cuTensorMapEncodeTiled is looked up through the runtime so the
//     library does not link against libcuda).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define B200_API extern "C" __attribute__((visibility("default")))

#define B200_CHECK(expr)                                                                      \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    if (_e != cudaSuccess) {                                                                  \
      fprintf(stderr, "[b200] %s failed at %s:%d: %s\n", #expr, __FILE__, __LINE__,           \
              cudaGetErrorString(_e));                                                        \
      return static_cast<int>(_e);                                                            \
    }                                                                                         \
  } while (0)

// Kernels that are meant to run BESIDE the persistent GEMM / attention CTAs (collectives, AdamW pipelined with
// the next forward) ask for the same shared-memory carve-out as those CTAs, the maximum. An SM holds one
// carve-out configuration at a time: a small kernel left on the driver's default (a small shared-memory
// partition) and a 225 KiB GEMM CTA cannot be resident on one SM together, so each waits for the other to
// drain - and a persistent GEMM cannot finish before every one of its CTAs has had its turn.
#define B200_PREFER_MAX_SMEM(kernel)                                                                            \
  do {                                                                                                          \
    static bool _done = false;                                                                                  \
    if (!_done) {                                                                                               \
      cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared); \
      _done = true;                                                                                             \
    }                                                                                                           \
  } while (0)

namespace b200 {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

// Device pointer to a 4-int status block owned by the Python side:
// [0] first error code, [1] kernel id that raised it, [2..3] free for detail.
int* status_ptr();

enum SwizzleMode { SWIZZLE_NONE_ = 0, SWIZZLE_128B_ = 3 };

// Returns a pointer to a cached 2D tensor map for a row-major matrix of `rows` x `cols` elements
// of `elem_bytes` bytes with a row pitch of `ld` elements. The box is box_cols x box_rows.
// Returns nullptr (and prints why) when the matrix breaks a TMA rule (16-byte base / pitch).
const CUtensorMap* get_tensor_map_2d(const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                                     uint32_t box_rows, uint32_t box_cols, int elem_bytes, int swizzle);

const CUtensorMap* get_tensor_map_bthd(const void* base, uint64_t B, uint64_t T, uint64_t heads, uint64_t D,
                                       uint64_t bs, uint64_t ts, uint64_t hs, uint32_t box_t, uint32_t box_d);

int num_sms();

#ifdef __CUDACC__
// A length or index that a kernel reads from device memory (valid key lengths, target ids) and then uses to bound
// its loops or to pick a column. Every build clamps it into [0, hi]; the debug build (-DB200_BOUNDS_CHECK=1, made by
// ``B200_BOUNDS_CHECK=1 python -m create_llm_by_cupy_b200.ops.build``) also reports a value outside that range through
// the status word (error 4, the kernel id, the offending value) - the stand-in for a memory checker on arguments
// that only exist on the device.
__device__ __forceinline__ int checked_index(int v, int hi, int* status, int kernel_id) {
#ifdef B200_BOUNDS_CHECK
  if ((v < 0 || v > hi) && status != nullptr && atomicCAS(status, 0, 4) == 0) {
    status[1] = kernel_id;
    status[2] = v;
  }
#else
  (void)status;
  (void)kernel_id;
#endif
  return v < 0 ? 0 : (v > hi ? hi : v);
}
#endif

}  // namespace b200
