// Process-wide state of the native library: status word, SM count, TMA tensor-map cache.
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace b200 {

static int* g_status = nullptr;
int* status_ptr() { return g_status; }

int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

struct MapKey {
  uint64_t base, rows, cols, ld;
  uint32_t box_rows, box_cols;
  int elem_bytes, swizzle;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
           box_cols == o.box_cols && elem_bytes == o.elem_bytes && swizzle == o.swizzle;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = k.base * 0x9E3779B97F4A7C15ull;
    h ^= (k.rows + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.cols + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.ld + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= ((uint64_t(k.box_rows) << 32 | k.box_cols) + (h << 6) + (h >> 2));
    h ^= ((uint64_t(k.elem_bytes) << 8 | uint64_t(k.swizzle)) + (h << 6) + (h >> 2));
    return static_cast<size_t>(h);
  }
};

const CUtensorMap* get_tensor_map_2d(const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                                     uint32_t box_cols, int elem_bytes, int swizzle) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap*, MapKeyHash> cache;
  MapKey key{reinterpret_cast<uint64_t>(base), rows, cols, ld, box_rows, box_cols, elem_bytes, swizzle};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;

  if ((key.base & 15) != 0 || ((ld * elem_bytes) & 15) != 0) {
    fprintf(stderr, "[b200] tensor map: base %p or pitch %llu B is not 16-byte aligned\n", base,
            (unsigned long long)(ld * elem_bytes));
    return nullptr;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    fprintf(stderr, "[b200] cuTensorMapEncodeTiled is not available from this driver\n");
    return nullptr;
  }
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap* m = new CUtensorMap;
  CUresult r = fn(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle == SWIZZLE_128B_ ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[b200] cuTensorMapEncodeTiled failed (%d): rows=%llu cols=%llu ld=%llu box=%ux%u\n", (int)r,
            (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld, box_rows, box_cols);
    delete m;
    return nullptr;
  }
  if (cache.size() > 65536) {  // unbounded growth guard for callers that churn addresses
    for (auto& kv : cache) delete kv.second;
    cache.clear();
  }
  cache.emplace(key, m);
  return m;
}

// 4-D map over a [B, T, heads, D] tensor addressed with element strides (batch, token, head; D
// contiguous). Dimension order for the copy coordinates is (d, head, t, b); the box is
// box_d x 1 x box_t x 1 with 128-byte swizzle. Not cached by address alone: keyed on everything.
const CUtensorMap* get_tensor_map_bthd(const void* base, uint64_t B, uint64_t T, uint64_t heads, uint64_t D,
                                       uint64_t bs, uint64_t ts, uint64_t hs, uint32_t box_t, uint32_t box_d) {
  static std::mutex mu;
  struct K4 { uint64_t v[10]; bool operator==(const K4& o) const { return memcmp(v, o.v, sizeof(v)) == 0; } };
  struct H4 { size_t operator()(const K4& k) const { uint64_t h = 1469598103934665603ull; for (uint64_t x : k.v) { h ^= x; h *= 1099511628211ull; } return size_t(h); } };
  static std::unordered_map<K4, CUtensorMap*, H4> cache;
  K4 key{{reinterpret_cast<uint64_t>(base), B, T, heads, D, bs, ts, hs, box_t, box_d}};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  if ((key.v[0] & 15) != 0 || ((bs * 2) & 15) || ((ts * 2) & 15) || ((hs * 2) & 15)) {
    fprintf(stderr, "[b200] 4-D tensor map: base or a stride is not 16-byte aligned\n");
    return nullptr;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return nullptr;
  cuuint64_t dims[4] = {D, heads, T, B};
  cuuint64_t strides[3] = {hs * 2, ts * 2, bs * 2};
  cuuint32_t box[4] = {box_d, 1, box_t, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMap* m = new CUtensorMap;
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[b200] cuTensorMapEncodeTiled (4-D) failed (%d)\n", (int)r);
    delete m;
    return nullptr;
  }
  if (cache.size() > 65536) { for (auto& kv : cache) delete kv.second; cache.clear(); }
  cache.emplace(key, m);
  return m;
}

}  // namespace b200

// Register the device status block (4 ints, zero-initialised by the caller).
B200_API int b200_set_status_ptr(void* p) {
  b200::g_status = static_cast<int*>(p);
  return 0;
}

B200_API int b200_num_sms() { return b200::num_sms(); }

B200_API int b200_abi_version() { return 1; }
