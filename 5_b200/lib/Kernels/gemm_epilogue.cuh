// Epilogue shared by the dense GEMM kernels: drain one warp's 32 TMEM lanes (32 rows of the
// accumulator, `kColumns` fp32 columns) to C.
//
// Each 32-column chunk is read with tcgen05.ld (lane = row), transposed through a per-warp
// 32x32 shared-memory block whose 16-byte pieces are XOR-swizzled by the row (conflict-free
// both ways), and written so that 8 lanes cover one 128-byte row segment: coalesced 128-bit
// stores, four rows per warp instruction. Rows >= m and columns >= n are predicated off, which
// is the clipped store of the hc kernel (examples/amdgpu_gfx11_wmma_matmul.py:284-298). When C's
// base or pitch is not 16-byte aligned the rows are still written with aligned 128-bit stores, one row
// segment per instruction, after a per-row peel to the next 16-byte boundary.
#pragma once

#include "sm100_ptx.cuh"

namespace hc {
namespace sm100 {

// Writes one 32-column chunk (already in registers, lane = row) of this warp's 32 rows to C.
__device__ __forceinline__ void write_chunk(const uint32_t (&r)[32], int chunk, float *stage,
                                            float *__restrict__ c, long long ldc, int m, int n,
                                            int row_base, int col_base, bool vec_ok, int lane) {
  const int col0 = col_base + chunk * 32;
  if (col0 >= n)
    return;  // warp-uniform
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
    // C's rows do not start on 16-byte boundaries (odd pitch or base). Each row segment is
    // still written mostly with aligned 128-bit stores: `shift` elements bring the address
    // to a 16-byte boundary, then up to 8 aligned float4, and the few elements left over at
    // both ends go out as 32-bit stores. 8 lanes serve one row, 4 rows per instruction.
    const int piece = lane & 7;
    // Phase (in elements, mod 4) of the address of C[row_base, col0]; it advances by ldc mod 4
    // per row.
    const unsigned phase0 = (static_cast<unsigned>(reinterpret_cast<uintptr_t>(c) >> 2) +
                             static_cast<unsigned>(row_base) * static_cast<unsigned>(ldc & 3) +
                             static_cast<unsigned>(col0)) & 3u;
    const unsigned phase_step = static_cast<unsigned>(ldc & 3);
    float *tile_dst = c + static_cast<long long>(row_base) * ldc + col0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = i * 4 + (lane >> 3);
      const int shift = static_cast<int>((4u - ((phase0 + static_cast<unsigned>(rr) * phase_step) & 3u)) & 3u);
      const float *src = stage + rr * 32;
      const int swz = rr & 7;
      if (row_base + rr < m) {
        float *dst = tile_dst + static_cast<long long>(rr) * ldc;
        const int e0 = shift + piece * 4;
        if (e0 + 3 < 32) {
          auto elem = [&](int e) { return src[(((e >> 2) ^ swz) << 2) | (e & 3)]; };
          const float4 v = make_float4(elem(e0), elem(e0 + 1), elem(e0 + 2), elem(e0 + 3));
          if (col0 + e0 + 3 < n) {
            __stcs(reinterpret_cast<float4 *>(dst + e0), v);
          } else {
            if (col0 + e0 < n) __stcs(dst + e0, v.x);
            if (col0 + e0 + 1 < n) __stcs(dst + e0 + 1, v.y);
            if (col0 + e0 + 2 < n) __stcs(dst + e0 + 2, v.z);
          }
        }
        if (shift != 0 && piece < 4) {
          // Elements [0, shift) before the first aligned group and [28 + shift, 32) after the last.
          const int e = piece < shift ? piece : 28 + piece;
          if (col0 + e < n)
            __stcs(dst + e, src[(((e >> 2) ^ swz) << 2) | (e & 3)]);
        }
      }
    }
  }
  __syncwarp();
}

// `release_bar`: mbarrier (cluster-window address when `release_remote`) that receives one
// arrival from this warp as soon as the accumulator has been read completely.
//
// The TMEM load of the next chunk is in flight while the current chunk is transposed and
// stored (two register sets alternate), so the TMEM latency is hidden behind the stores.
template <int kColumns>
__device__ __forceinline__ void drain_accumulator_rows(uint32_t taddr, float *stage, float *__restrict__ c,
                                                       long long ldc, int m, int n, int row_base,
                                                       int col_base, bool vec_ok, int lane,
                                                       uint32_t release_bar, bool release_remote) {
  constexpr int kChunks = kColumns / 32;
  static_assert(kChunks % 2 == 0, "chunks are processed in pairs");
  uint32_t ra[32], rb[32];
  tmem_load_32x32b_x32(taddr, ra);
#pragma unroll 1
  for (int chunk = 0; chunk < kChunks; chunk += 2) {
    tmem_load_wait_for(ra);
    tmem_load_32x32b_x32(taddr + (chunk + 1) * 32, rb);
    write_chunk(ra, chunk, stage, c, ldc, m, n, row_base, col_base, vec_ok, lane);
    tmem_load_wait_for(rb);
    if (chunk + 2 < kChunks) {
      tmem_load_32x32b_x32(taddr + (chunk + 2) * 32, ra);
    } else {
      // Accumulator fully read: hand it back to the MMA issuer.
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (release_remote)
          mbar_arrive_cluster(release_bar);
        else
          mbar_arrive(release_bar);
      }
    }
    write_chunk(rb, chunk + 1, stage, c, ldc, m, n, row_base, col_base, vec_ok, lane);
  }
}

} // namespace sm100
} // namespace hc
