// Epilogue shared by the dense GEMM kernels: drain one warp's 32 TMEM lanes (32 rows of the
// accumulator, `kColumns` fp32 columns) to C.
//
// Each 32-column chunk is read with tcgen05.ld (lane = row), transposed through a per-warp
// 32x32 shared-memory block whose 16-byte pieces are XOR-swizzled by the row (conflict-free
// both ways), and written so that 8 lanes cover one 128-byte row segment: coalesced 128-bit
// stores, four rows per warp instruction. Rows >= m and columns >= n are predicated off, which
// is the clipped store of the hc kernel (examples/amdgpu_gfx11_wmma_matmul.py:284-298). When C's
// base or pitch is not 16-byte aligned the same data goes out as 32-bit stores, one 128-byte row
// segment per instruction.
#pragma once

#include "sm100_ptx.cuh"

namespace hc {
namespace sm100 {

// `release_bar`: mbarrier (cluster-window address when `release_remote`) that receives one
// arrival from this warp as soon as the accumulator has been read completely.
template <int kColumns>
__device__ __forceinline__ void drain_accumulator_rows(uint32_t taddr, float *stage, float *__restrict__ c,
                                                       long long ldc, int m, int n, int row_base,
                                                       int col_base, bool vec_ok, int lane,
                                                       uint32_t release_bar, bool release_remote) {
#pragma unroll 1
  for (int chunk = 0; chunk < kColumns / 32; ++chunk) {
    uint32_t r[32];
    tmem_load_32x32b_x32(taddr + chunk * 32, r);
    tmem_load_wait();
    if (chunk == kColumns / 32 - 1) {
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (release_remote)
          mbar_arrive_cluster(release_bar);
        else
          mbar_arrive(release_bar);
      }
    }
    const int col0 = col_base + chunk * 32;
    if (col0 >= n)
      continue;  // warp-uniform
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 v = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                   __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
      *reinterpret_cast<float4 *>(stage + lane * 32 + ((q ^ (lane & 7)) << 2)) = v;
    }
    __syncwarp();
    if (vec_ok) {
      const int piece = lane & 7;
      const int col = col0 + piece * 4;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = i * 4 + (lane >> 3);
        const int row = row_base + rr;
        const float4 v = *reinterpret_cast<const float4 *>(stage + rr * 32 + ((piece ^ (rr & 7)) << 2));
        if (row < m) {
          float *dst = c + static_cast<long long>(row) * ldc + col;
          if (col + 3 < n) {
            __stcs(reinterpret_cast<float4 *>(dst), v);
          } else {
            if (col < n) __stcs(dst, v.x);
            if (col + 1 < n) __stcs(dst + 1, v.y);
            if (col + 2 < n) __stcs(dst + 2, v.z);
          }
        }
      }
    } else {
      const int col = col0 + lane;
#pragma unroll 4
      for (int rr = 0; rr < 32; ++rr) {
        const int row = row_base + rr;
        const float v = stage[rr * 32 + ((((lane >> 2) ^ (rr & 7)) << 2) | (lane & 3))];
        if (row < m && col < n)
          __stcs(c + static_cast<long long>(row) * ldc + col, v);
      }
    }
    __syncwarp();
  }
}

} // namespace sm100
} // namespace hc
