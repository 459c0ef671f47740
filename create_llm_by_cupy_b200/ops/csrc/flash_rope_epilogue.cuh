// Epilogue shared by the tcgen05 attention-backward kernels (head_dim 128 or 64): store one fp32 accumulator
// row from tensor memory as bf16, applying the inverse rotary embedding on the way.
//
// The kernels work on rotated Q and K, so their dQ and dK are gradients of the rotated tensors. The
// gradient of the un-rotated one is the inverse rotation of the same row (pairs (j, j + D/2), angle of
// the row's position): y1 = x1 c + x2 s, y2 = x2 c - x1 s. Doing it here, on the fp32 accumulator a
// thread already holds, removes the separate in-place pass over the [dK | dQ] columns.
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace b200 {

// Pairs j in [j0, j0 + nj) (nj a multiple of 16) of the row at TMEM address `taddr` (column 0 of the
// kD-wide accumulator). The tables are fp32 and TRANSPOSED, [kD / 2][ld]: cs_row / sn_row point at this row's
// position in line 0 and element j is at [j * ld], so the lanes of a warp (consecutive positions) read
// consecutive words. The TMEM loads are warp-collective: every lane calls this, `active` only predicates
// the global stores.
template <int kD>
__device__ __forceinline__ void store_row_unrot_from_tmem(uint32_t taddr, bf16* grow, int j0, int nj,
                                                          const float* __restrict__ cs_row,
                                                          const float* __restrict__ sn_row, int ld, bool active) {
#pragma unroll 1
  constexpr int kHalf = kD / 2;
  for (int j = j0; j < j0 + nj; j += 16) {
    uint32_t a[16], b[16];
    tmem_ld_32x32b_x16(taddr + j, a);
    tmem_ld_32x32b_x16(taddr + kHalf + j, b);
    tmem_ld_wait();
    if (!active) continue;
    uint32_t y1[8], y2[8];
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
      float cc[4], ss[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        cc[e] = __ldg(cs_row + size_t(j + i + e) * ld);
        ss[e] = __ldg(sn_row + size_t(j + i + e) * ld);
      }
      float o1[4], o2[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x1 = __uint_as_float(a[i + e]), x2 = __uint_as_float(b[i + e]);
        o1[e] = fmaf(x1, cc[e], x2 * ss[e]);
        o2[e] = fmaf(x2, cc[e], -x1 * ss[e]);
      }
#pragma unroll
      for (int e = 0; e < 4; e += 2) {
        const bf162 t1 = __floats2bfloat162_rn(o1[e], o1[e + 1]);
        const bf162 t2 = __floats2bfloat162_rn(o2[e], o2[e + 1]);
        y1[(i + e) >> 1] = *reinterpret_cast<const uint32_t*>(&t1);
        y2[(i + e) >> 1] = *reinterpret_cast<const uint32_t*>(&t2);
      }
    }
    *reinterpret_cast<uint4*>(grow + j) = make_uint4(y1[0], y1[1], y1[2], y1[3]);
    *reinterpret_cast<uint4*>(grow + j + 8) = make_uint4(y1[4], y1[5], y1[6], y1[7]);
    *reinterpret_cast<uint4*>(grow + kHalf + j) = make_uint4(y2[0], y2[1], y2[2], y2[3]);
    *reinterpret_cast<uint4*>(grow + kHalf + j + 8) = make_uint4(y2[4], y2[5], y2[6], y2[7]);
  }
}

}  // namespace b200
