// Epilogue shared by the dense GEMM kernels: drain one warp's 32 TMEM lanes (32 rows of the
// accumulator, `kColumns` fp32 columns) to C.
//
// Each 32-column chunk is read with tcgen05.ld (lane = row), transposed through a per-warp
// 32x32 shared-memory block whose 16-byte pieces are XOR-swizzled by the row (conflict-free
// both ways), and written so that 8 lanes cover one 128-byte row segment: coalesced 128-bit
// stores, four rows per warp instruction. Rows >= m and columns >= n are predicated off, which
// is the clipped store of the hc kernel (examples/amdgpu_gfx11_wmma_matmul.py:284-298). When C's
// base or pitch is not 16-byte aligned the rows are still written with aligned 128-bit stores:
// each row is rotated to its own 16-byte phase while it is staged.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_launch.h"
#include "sm100_ptx.cuh"

namespace hc {
namespace sm100 {

// ---------------------------------------------------------------- 16-bit C ----------
// Two float32 values rounded to nearest even and packed (first value in the low half).
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi, int c_dtype) {
  if (c_dtype == kCTypeF16) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
  }
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&h);
}

__device__ __forceinline__ uint16_t round_to_16(float v, int c_dtype) {
  if (c_dtype == kCTypeF16)
    return __half_as_ushort(__float2half_rn(v));
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// maximum / minimum as NumPy (and so the reference simulator) define them: a NaN operand gives
// NaN, where fmaxf/fminf would return the other operand.
__device__ __forceinline__ float max_nan(float a, float b) {
  float d;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}
__device__ __forceinline__ float min_nan(float a, float b) {
  float d;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}

// One element of C of whatever type, at element index `index`.
__device__ __forceinline__ void store_c_element(void *c, long long index, float v, int c_dtype) {
  if (c_dtype == kCTypeF32)
    __stcs(static_cast<float *>(c) + index, v);
  else
    static_cast<uint16_t *>(c)[index] = round_to_16(v, c_dtype);
}

// The fused element-wise work on one value that is about to be stored at `dst` (column `col`).
__device__ __forceinline__ float finish_value(float v, const float *dst, int col, const Epilogue &ep) {
  if (ep.accumulate)
    v += __ldcs(dst);
#pragma unroll
  for (int i = 0; i < kMaxEpilogueOps; ++i) {
    if (i < ep.op_count) {
      const int kind = ep.op_kind[i];
      const float x = kind == kEpilogueBiasColumn ? __ldg(ep.bias + col) : ep.op_value[i];
      v = kind == kEpilogueScale ? v * x
        : kind == kEpilogueMax   ? max_nan(v, x)
        : kind == kEpilogueMin   ? min_nan(v, x)
                                 : v + x;
    }
  }
  return v;
}

// The operations on the eight groups a lane stores per chunk. The kind of each operation is the
// same for the whole grid, so it is branched on once per chunk and the work inside is one
// instruction per value. `bias_of(i)` gives the four bias values of group i.
template <typename BiasFn>
__device__ __forceinline__ void apply_ops_to_groups(float4 (&v)[8], const Epilogue &ep, BiasFn bias_of) {
#pragma unroll
  for (int op = 0; op < kMaxEpilogueOps; ++op) {
    if (op >= ep.op_count)
      break;
    const int kind = ep.op_kind[op];
    const float x = ep.op_value[op];
    if (kind == kEpilogueScale) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i].x *= x; v[i].y *= x; v[i].z *= x; v[i].w *= x;
      }
    } else if (kind == kEpilogueAdd) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i].x += x; v[i].y += x; v[i].z += x; v[i].w += x;
      }
    } else if (kind == kEpilogueMax) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i].x = max_nan(v[i].x, x); v[i].y = max_nan(v[i].y, x); v[i].z = max_nan(v[i].z, x); v[i].w = max_nan(v[i].w, x);
      }
    } else if (kind == kEpilogueMin) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i].x = min_nan(v[i].x, x); v[i].y = min_nan(v[i].y, x); v[i].z = min_nan(v[i].z, x); v[i].w = min_nan(v[i].w, x);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 b = bias_of(i);
        v[i].x += b.x; v[i].y += b.y; v[i].z += b.z; v[i].w += b.w;
      }
    }
  }
}

// With an accumulating kernel the epilogue reads C before it writes it. Each lane asks for the
// lines of its row of the tile to be brought into L2 while the tile's products are still being
// accumulated, so that those reads do not wait on DRAM.
__device__ __forceinline__ void prefetch_c_tile_row(const float *c, long long ldc, int m, int n, int row,
                                                    int col_base, int columns) {
  if (row >= m)
    return;
  const float *p = c + static_cast<long long>(row) * ldc;
  for (int col = col_base; col < col_base + columns && col < n; col += 32)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p + col));
}

// The operations on N values of one column (all take the same bias), the kind of each operation
// branched on once for the lot.
template <int N>
__device__ __forceinline__ void apply_ops_to_column(float (&v)[N], float bias, const Epilogue &ep) {
#pragma unroll
  for (int op = 0; op < kMaxEpilogueOps; ++op) {
    if (op >= ep.op_count)
      break;
    const int kind = ep.op_kind[op];
    const float x = kind == kEpilogueBiasColumn ? bias : ep.op_value[op];
    if (kind == kEpilogueScale) {
#pragma unroll
      for (int j = 0; j < N; ++j)
        v[j] *= x;
    } else if (kind == kEpilogueMax) {
#pragma unroll
      for (int j = 0; j < N; ++j)
        v[j] = max_nan(v[j], x);
    } else if (kind == kEpilogueMin) {
#pragma unroll
      for (int j = 0; j < N; ++j)
        v[j] = min_nan(v[j], x);
    } else {
#pragma unroll
      for (int j = 0; j < N; ++j)
        v[j] += x;
    }
  }
}

// The operations on a chunk that is still in its tensor-memory layout (lane = row, r[j] = column
// col0 + j): one instruction per value and operation, the kind branched on once per chunk. Used
// whenever C's previous contents are not needed, so that the chunk can then leave like a plain one
// (TMA store, or the coalesced writers for an odd pitch).
__device__ __forceinline__ void apply_ops_lane_row(uint32_t (&r)[32], int col0, int n, int lane, const Epilogue &ep) {
  float bias_lane = 0.0f;
  if (ep.bias != nullptr && col0 + lane < n)
    bias_lane = __ldg(ep.bias + col0 + lane);
#pragma unroll
  for (int op = 0; op < kMaxEpilogueOps; ++op) {
    if (op >= ep.op_count)
      break;
    const int kind = ep.op_kind[op];
    const float x = ep.op_value[op];
    if (kind == kEpilogueScale) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        r[j] = __float_as_uint(__uint_as_float(r[j]) * x);
    } else if (kind == kEpilogueAdd) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        r[j] = __float_as_uint(__uint_as_float(r[j]) + x);
    } else if (kind == kEpilogueMax) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        r[j] = __float_as_uint(max_nan(__uint_as_float(r[j]), x));
    } else if (kind == kEpilogueMin) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        r[j] = __float_as_uint(min_nan(__uint_as_float(r[j]), x));
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        r[j] = __float_as_uint(__uint_as_float(r[j]) + __shfl_sync(0xffffffffu, bias_lane, j));
    }
  }
}

// Stages this lane's 32 values with the row rotated left by kShift elements, so that the
// 16-byte groups of the row *in memory* (which start kShift elements into the chunk) land on
// 16-byte pieces of the staging block.
template <int kShift>
__device__ __forceinline__ void stage_row_shifted(const uint32_t (&r)[32], float *buf, int lane) {
#pragma unroll
  for (int q = 0; q < (kShift == 0 ? 8 : 7); ++q) {
    const float4 v = make_float4(__uint_as_float(r[4 * q + kShift]), __uint_as_float(r[4 * q + kShift + 1]),
                                 __uint_as_float(r[4 * q + kShift + 2]), __uint_as_float(r[4 * q + kShift + 3]));
    *reinterpret_cast<float4 *>(buf + lane * 32 + ((q ^ (lane & 7)) << 2)) = v;
  }
}

// v + previous (the element's old value, when accumulating), then the operations; `bias`: of the element's column.
__device__ __forceinline__ float finish_loaded(float v, float previous, float bias, const Epilogue &ep) {
  v += previous;
#pragma unroll
  for (int i = 0; i < kMaxEpilogueOps; ++i) {
    if (i < ep.op_count) {
      const int kind = ep.op_kind[i];
      const float x = kind == kEpilogueBiasColumn ? bias : ep.op_value[i];
      v = kind == kEpilogueScale ? v * x
        : kind == kEpilogueMax   ? max_nan(v, x)
        : kind == kEpilogueMin   ? min_nan(v, x)
                                 : v + x;
    }
  }
  return v;
}

// Previous contents of four consecutive elements of C starting at column `col` (zeros past n);
// `src` is 16-byte aligned, so a group that lies inside C is one 128-bit load.
__device__ __forceinline__ float4 load_previous(const float *src, int col, int n) {
  if (col + 3 < n)
    return __ldcs(reinterpret_cast<const float4 *>(src));
  float4 old = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  if (col < n) old.x = __ldcs(src);
  if (col + 1 < n) old.y = __ldcs(src + 1);
  if (col + 2 < n) old.z = __ldcs(src + 2);
  return old;
}

// One 32-column chunk of an accumulating launch whose stores cannot do the addition (C's base or
// pitch rules out TMA, push targets, or operations after the sum in a launch split over k): C's
// previous contents are read here and the operations run here, after that addition.
// The accesses are those of the plain writer below -- 8 lanes x 128 bits per row segment, each
// row rotated to its own 16-byte phase when C's rows are not aligned -- and every read of the
// chunk (the staged groups, the group that straddles the previous chunk, the single elements at
// the ends of a tile row) is issued before its first store: a load cannot move above a store that
// might alias it, so reads placed between the stores would each cost a full memory latency. The
// tile's rows were prefetched into L2 during the k-loop.
__device__ __forceinline__ void write_chunk_reading_c(const uint32_t (&r)[32], int chunk, bool last_chunk,
                                                      float *buf, float *__restrict__ c, long long ldc, int m,
                                                      int n, int row_base, int col_base, bool vec_ok, int lane,
                                                      float (&carry)[6], const Epilogue &ep) {
  const int col0 = col_base + chunk * 32;
  if (col0 >= n)
    return;  // warp-uniform
  const int piece = lane & 7;
  const bool acc = ep.accumulate != 0;
  // One bias value per lane (column col0 + lane); groups fetch theirs by shuffle.
  float bias_lane = 0.0f;
  if (ep.bias != nullptr && col0 + lane < n)
    bias_lane = __ldg(ep.bias + col0 + lane);
  float4 previous[8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
    previous[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  if (vec_ok) {
    const int col = col0 + piece * 4;
    if (acc) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = row_base + i * 4 + (lane >> 3);
        if (row < m)
          previous[i] = load_previous(c + static_cast<long long>(row) * ldc + col, col, n);
      }
    }
    const float4 bias =
        make_float4(__shfl_sync(0xffffffffu, bias_lane, piece * 4), __shfl_sync(0xffffffffu, bias_lane, piece * 4 + 1),
                    __shfl_sync(0xffffffffu, bias_lane, piece * 4 + 2), __shfl_sync(0xffffffffu, bias_lane, piece * 4 + 3));
    stage_row_shifted<0>(r, buf, lane);
    __syncwarp();
    float4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = i * 4 + (lane >> 3);
      v[i] = *reinterpret_cast<const float4 *>(buf + rr * 32 + ((piece ^ (rr & 7)) << 2));
      v[i].x += previous[i].x; v[i].y += previous[i].y; v[i].z += previous[i].z; v[i].w += previous[i].w;
    }
    apply_ops_to_groups(v, ep, [&](int) { return bias; });
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = row_base + i * 4 + (lane >> 3);
      if (row < m) {
        const long long offset = static_cast<long long>(row) * ldc + col;
        float *dst = c + offset;
        if (col + 3 < n) {
          __stcs(reinterpret_cast<float4 *>(dst), v[i]);
          for (int t = 0; t < ep.push_count; ++t)  // the peers' copies of C
            __stcs(reinterpret_cast<float4 *>(ep.push[t] + offset), v[i]);
        } else {
          for (int t = -1; t < ep.push_count; ++t) {
            float *edge = t < 0 ? dst : ep.push[t] + offset;
            if (col < n) __stcs(edge, v[i].x);
            if (col + 1 < n) __stcs(edge + 1, v[i].y);
            if (col + 2 < n) __stcs(edge + 2, v[i].z);
          }
        }
      }
    }
    __syncwarp();
    return;
  }
  // Rows that do not start on 16-byte boundaries: see write_chunk for the layout.
  const unsigned phase0 = (static_cast<unsigned>(reinterpret_cast<uintptr_t>(c) >> 2) +
                           static_cast<unsigned>(row_base) * static_cast<unsigned>(ldc & 3) +
                           static_cast<unsigned>(col0)) & 3u;
  const unsigned phase_step = static_cast<unsigned>(ldc & 3);
  auto shift_of = [&](int rr) {
    return static_cast<int>((4u - ((phase0 + static_cast<unsigned>(rr) * phase_step) & 3u)) & 3u);
  };
  float *tile_dst = c + static_cast<long long>(row_base) * ldc + col0;
  // -- every read of the chunk --
  // Row rr = 4 i + (lane >> 3) of the staged groups: its phase does not depend on i (four pitches are
  // a multiple of 16 bytes), so a lane's groups start at the same element e0 of every row it serves.
  const int e0 = shift_of(lane >> 3) + piece * 4;
  if (acc && e0 + 3 < 32) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = i * 4 + (lane >> 3);
      if (row_base + rr < m)
        previous[i] = load_previous(tile_dst + static_cast<long long>(rr) * ldc + e0, col0 + e0, n);
    }
  }
  const int shift = shift_of(lane);
  float *dst = tile_dst + static_cast<long long>(lane) * ldc;
  const bool own = shift != 0 && row_base + lane < m;  // this lane writes the ragged ends of its row itself
  const bool tail_now = last_chunk || col0 + 32 >= n;
  // lead: old values of the group that straddles the previous chunk (chunk > 0) or of the elements
  // before the first aligned group (chunk 0); tail: of the elements after the last aligned group.
  float4 lead = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float tail[3] = {0.0f, 0.0f, 0.0f};
  if (acc && own) {
    if (chunk == 0) {
      if (col0 < n) lead.x = __ldcs(dst);
      if (shift >= 2 && col0 + 1 < n) lead.y = __ldcs(dst + 1);
      if (shift == 3 && col0 + 2 < n) lead.z = __ldcs(dst + 2);
    } else {
      lead = load_previous(dst + shift - 4, col0 + shift - 4, n);
    }
    if (tail_now) {
#pragma unroll
      for (int e = 29; e < 32; ++e)
        if (e >= 28 + shift && col0 + e < n)
          tail[e - 29] = __ldcs(dst + e);
    }
  }
  // Bias values of the columns at the two ends of the chunk, for the elements a lane finishes itself
  // (those of the previous chunk's last three columns travel in `carry`).
  const float b0 = __shfl_sync(0xffffffffu, bias_lane, 0), b1 = __shfl_sync(0xffffffffu, bias_lane, 1),
              b2 = __shfl_sync(0xffffffffu, bias_lane, 2);
  const float b29 = __shfl_sync(0xffffffffu, bias_lane, 29), b30 = __shfl_sync(0xffffffffu, bias_lane, 30),
              b31 = __shfl_sync(0xffffffffu, bias_lane, 31);
  // -- stage, then the stores --
  if (shift == 0)
    stage_row_shifted<0>(r, buf, lane);
  else if (shift == 1)
    stage_row_shifted<1>(r, buf, lane);
  else if (shift == 2)
    stage_row_shifted<2>(r, buf, lane);
  else
    stage_row_shifted<3>(r, buf, lane);
  if (own) {
    const float f0 = __uint_as_float(r[0]), f1 = __uint_as_float(r[1]), f2 = __uint_as_float(r[2]);
    if (chunk == 0) {
      if (col0 < n) __stcs(dst, finish_loaded(f0, lead.x, b0, ep));
      if (shift >= 2 && col0 + 1 < n) __stcs(dst + 1, finish_loaded(f1, lead.y, b1, ep));
      if (shift == 3 && col0 + 2 < n) __stcs(dst + 2, finish_loaded(f2, lead.z, b2, ep));
    } else {
      // The straddling group: its first 4 - shift elements were kept from the previous chunk.
      const float4 v = shift == 1 ? make_float4(carry[0], carry[1], carry[2], f0)
                     : shift == 2 ? make_float4(carry[1], carry[2], f0, f1)
                                  : make_float4(carry[2], f0, f1, f2);
      const float4 vb = shift == 1 ? make_float4(carry[3], carry[4], carry[5], b0)
                      : shift == 2 ? make_float4(carry[4], carry[5], b0, b1)
                                   : make_float4(carry[5], b0, b1, b2);
      float *group = dst + shift - 4;
      const int group_col = col0 + shift - 4;
      float4 out;  // (elements at or past column n are computed from zeros and not stored)
      out.x = finish_loaded(v.x, lead.x, vb.x, ep);
      out.y = finish_loaded(v.y, lead.y, vb.y, ep);
      out.z = finish_loaded(v.z, lead.z, vb.z, ep);
      out.w = finish_loaded(v.w, lead.w, vb.w, ep);
      if (group_col + 3 < n) {
        __stcs(reinterpret_cast<float4 *>(group), out);
      } else {
        __stcs(group, out.x);
        if (group_col + 1 < n) __stcs(group + 1, out.y);
        if (group_col + 2 < n) __stcs(group + 2, out.z);
      }
    }
    if (tail_now) {
#pragma unroll
      for (int e = 29; e < 32; ++e)
        if (e >= 28 + shift && col0 + e < n)
          __stcs(dst + e, finish_loaded(__uint_as_float(r[e]), tail[e - 29], e == 29 ? b29 : (e == 30 ? b30 : b31), ep));
    }
  }
  carry[0] = __uint_as_float(r[29]);
  carry[1] = __uint_as_float(r[30]);
  carry[2] = __uint_as_float(r[31]);
  carry[3] = b29;
  carry[4] = b30;
  carry[5] = b31;
  __syncwarp();
  float4 v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = i * 4 + (lane >> 3);
    v[i] = *reinterpret_cast<const float4 *>(buf + rr * 32 + ((piece ^ (rr & 7)) << 2));
    v[i].x += previous[i].x; v[i].y += previous[i].y; v[i].z += previous[i].z; v[i].w += previous[i].w;
  }
  // (e0 + j) & 31: lanes whose groups are skipped below still take part in the shuffles.
  const float4 bias =
      make_float4(__shfl_sync(0xffffffffu, bias_lane, e0 & 31), __shfl_sync(0xffffffffu, bias_lane, (e0 + 1) & 31),
                  __shfl_sync(0xffffffffu, bias_lane, (e0 + 2) & 31), __shfl_sync(0xffffffffu, bias_lane, (e0 + 3) & 31));
  apply_ops_to_groups(v, ep, [&](int) { return bias; });
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = i * 4 + (lane >> 3);
    if (row_base + rr < m && e0 + 3 < 32) {
      float *group = tile_dst + static_cast<long long>(rr) * ldc + e0;
      if (col0 + e0 + 3 < n) {
        __stcs(reinterpret_cast<float4 *>(group), v[i]);
      } else {
        if (col0 + e0 < n) __stcs(group, v[i].x);
        if (col0 + e0 + 1 < n) __stcs(group + 1, v[i].y);
        if (col0 + e0 + 2 < n) __stcs(group + 2, v[i].z);
      }
    }
  }
  __syncwarp();
}

// Writes one 32-column chunk (already in registers, lane = row, operations applied) of this warp's
// 32 rows to C. `carry` holds the last three values of this lane's row from the previous chunk
// (odd-pitch path only); `last_chunk` says that no further chunk of the tile follows.
__device__ __forceinline__ void write_chunk(const uint32_t (&r)[32], int chunk, bool last_chunk, float *buf,
                                            float *__restrict__ c, long long ldc, int m, int n,
                                            int row_base, int col_base, bool vec_ok, int lane,
                                            float (&carry)[6], const Epilogue &ep) {
  const int col0 = col_base + chunk * 32;
  if (col0 >= n)
    return;  // warp-uniform
  const int piece = lane & 7;
  if (vec_ok) {
    const int col = col0 + piece * 4;
    stage_row_shifted<0>(r, buf, lane);
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = i * 4 + (lane >> 3);
      const float4 value = *reinterpret_cast<const float4 *>(buf + rr * 32 + ((piece ^ (rr & 7)) << 2));
      const int row = row_base + rr;
      if (row < m) {
        const long long offset = static_cast<long long>(row) * ldc + col;
        float *dst = c + offset;
        if (col + 3 < n) {
          __stcs(reinterpret_cast<float4 *>(dst), value);
          // The same 128-byte row segments go to every push target (peer GPUs' copies of C).
          for (int t = 0; t < ep.push_count; ++t)
            __stcs(reinterpret_cast<float4 *>(ep.push[t] + offset), value);
        } else {
          for (int t = -1; t < ep.push_count; ++t) {
            float *edge = t < 0 ? dst : ep.push[t] + offset;
            if (col < n) __stcs(edge, value.x);
            if (col + 1 < n) __stcs(edge + 1, value.y);
            if (col + 2 < n) __stcs(edge + 2, value.z);
          }
        }
      }
    }
  } else {
    // C's rows do not start on 16-byte boundaries (odd pitch or base). For row r, `shift(r)`
    // elements separate C[r, col0] from the next 16-byte boundary. The lane that owns the row
    // stages it rotated by that shift (so memory-aligned groups become staging pieces); the one
    // group that straddles two chunks it writes itself, joining the end of the previous chunk
    // with the start of this one, and only at the two ends of the tile row do single elements
    // go out as 32-bit stores. The staged groups then leave exactly as on the aligned path:
    // 8 lanes x 128-bit per row, four rows per instruction.
    const unsigned phase0 = (static_cast<unsigned>(reinterpret_cast<uintptr_t>(c) >> 2) +
                             static_cast<unsigned>(row_base) * static_cast<unsigned>(ldc & 3) +
                             static_cast<unsigned>(col0)) & 3u;
    const unsigned phase_step = static_cast<unsigned>(ldc & 3);
    auto shift_of = [&](int rr) {
      return static_cast<int>((4u - ((phase0 + static_cast<unsigned>(rr) * phase_step) & 3u)) & 3u);
    };
    float *tile_dst = c + static_cast<long long>(row_base) * ldc + col0;
    {
      const int shift = shift_of(lane);
      float *dst = tile_dst + static_cast<long long>(lane) * ldc;
      const bool row_ok = row_base + lane < m;
      if (shift == 0)
        stage_row_shifted<0>(r, buf, lane);
      else if (shift == 1)
        stage_row_shifted<1>(r, buf, lane);
      else if (shift == 2)
        stage_row_shifted<2>(r, buf, lane);
      else
        stage_row_shifted<3>(r, buf, lane);
      if (shift != 0 && row_ok) {
        const float f0 = __uint_as_float(r[0]), f1 = __uint_as_float(r[1]), f2 = __uint_as_float(r[2]);
        if (chunk == 0) {
          // Elements before the first aligned group of the tile row.
          if (col0 < n) __stcs(dst, f0);
          if (shift >= 2 && col0 + 1 < n) __stcs(dst + 1, f1);
          if (shift == 3 && col0 + 2 < n) __stcs(dst + 2, f2);
        } else {
          // The group that straddles the previous chunk and this one: its first 4 - shift
          // elements were kept from the previous chunk in `carry`.
          const float4 v = shift == 1 ? make_float4(carry[0], carry[1], carry[2], f0)
                         : shift == 2 ? make_float4(carry[1], carry[2], f0, f1)
                                      : make_float4(carry[2], f0, f1, f2);
          float *group = dst + shift - 4;
          const int group_col = col0 + shift - 4;
          if (group_col + 3 < n) {
            __stcs(reinterpret_cast<float4 *>(group), v);
          } else {
            // Only the elements left of column n exist (the previous chunk's are always inside).
            __stcs(group, v.x);
            if (group_col + 1 < n) __stcs(group + 1, v.y);
            if (group_col + 2 < n) __stcs(group + 2, v.z);
          }
        }
        if (last_chunk || col0 + 32 >= n) {
          // No next chunk will complete the trailing group: write its elements singly.
          for (int e = 28 + shift; e < 32; ++e)
            if (col0 + e < n)
              __stcs(dst + e, __uint_as_float(e == 29 ? r[29] : (e == 30 ? r[30] : r[31])));
        }
      }
      carry[0] = __uint_as_float(r[29]);
      carry[1] = __uint_as_float(r[30]);
      carry[2] = __uint_as_float(r[31]);
    }
    __syncwarp();
    // Row rr = 4 i + (lane >> 3): its phase does not depend on i (four pitches are a multiple of 16
    // bytes), so a lane's groups start at the same element e0 of every row it serves.
    const int e0 = shift_of(lane >> 3) + piece * 4;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = i * 4 + (lane >> 3);
      const float4 value = *reinterpret_cast<const float4 *>(buf + rr * 32 + ((piece ^ (rr & 7)) << 2));
      if (row_base + rr < m && e0 + 3 < 32) {
        float *dst = tile_dst + static_cast<long long>(rr) * ldc + e0;
        if (col0 + e0 + 3 < n) {
          __stcs(reinterpret_cast<float4 *>(dst), value);
        } else {
          if (col0 + e0 < n) __stcs(dst, value.x);
          if (col0 + e0 + 1 < n) __stcs(dst + 1, value.y);
          if (col0 + e0 + 2 < n) __stcs(dst + 2, value.z);
        }
      }
    }
  }
  __syncwarp();
}

// The chunk leaves through the TMA store engine: staged exactly as for the coalesced stores (the
// XOR of the 16-byte piece with the row is the 128-byte swizzle of the tensor map), then one
// elected lane issues a 32x32 box store. Rows >= m and columns >= n are clipped by the tensor map.
// Needs C's base and pitch 16-byte aligned; `buf` is 1024-byte aligned.
// `add`: the box is added to C (TMA reduction) instead of replacing it.
// `push`: the same box also goes to every push target (the peers' copies of C), one more TMA store
// per target from the same staged block.
__device__ __forceinline__ void store_chunk_tma(const uint32_t (&r)[32], int chunk, float *buf,
                                                const CUtensorMap *tmap_c, int m, int n, int row_base,
                                                int col_base, int lane, bool add = false,
                                                const PushMaps *push = nullptr) {
  const int col0 = col_base + chunk * 32;
  if (col0 >= n || row_base >= m)
    return;  // warp-uniform
  if (lane == 0)
    tma_store_wait_read();  // the previous chunk's store has read the buffer
  __syncwarp();
  stage_row_shifted<0>(r, buf, lane);
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    if (add)
      tma_reduce_add_2d(tmap_c, smem_u32(buf), col0, row_base);
    else
      tma_store_2d(tmap_c, smem_u32(buf), col0, row_base);
    if (push != nullptr)
      for (int t = 0; t < push->count; ++t)
        tma_store_2d(&push->map[t], smem_u32(buf), col0, row_base);
    tma_store_commit();
  }
}

// An accumulating launch with operations after the sum, C addressable by TMA: the chunk's previous
// contents are loaded into the staging block by TMA (`bar`: this warp's mbarrier, `phase` its
// parity, kept across chunks), each lane adds its row to its registers, the operations run, and
// the chunk is staged again and stored by TMA. Returns false when the wait for the load gave up.
__device__ __forceinline__ bool accumulate_chunk_tma(uint32_t (&r)[32], int chunk, float *buf,
                                                     const CUtensorMap *tmap_c, int m, int n, int row_base,
                                                     int col_base, int lane, uint32_t bar, uint32_t &phase,
                                                     volatile uint32_t *abort_flag, const Epilogue &ep) {
  const int col0 = col_base + chunk * 32;
  if (col0 >= n || row_base >= m)
    return true;  // warp-uniform
  if (lane == 0) {
    tma_store_wait_read();  // the previous chunk's store has read the block
    mbar_arrive_expect_tx(bar, 32 * 32 * 4);
    tma_load_2d(smem_u32(buf), tmap_c, bar, col0, row_base);  // rows >= m, columns >= n arrive as zeros
  }
  const bool arrived = mbar_wait(bar, phase, abort_flag);
  phase ^= 1u;
  if (!__all_sync(0xffffffffu, arrived))
    return false;
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const float4 old = *reinterpret_cast<const float4 *>(buf + lane * 32 + ((q ^ (lane & 7)) << 2));
    r[4 * q] = __float_as_uint(__uint_as_float(r[4 * q]) + old.x);
    r[4 * q + 1] = __float_as_uint(__uint_as_float(r[4 * q + 1]) + old.y);
    r[4 * q + 2] = __float_as_uint(__uint_as_float(r[4 * q + 2]) + old.z);
    r[4 * q + 3] = __float_as_uint(__uint_as_float(r[4 * q + 3]) + old.w);
  }
  apply_ops_lane_row(r, col0, n, lane, ep);
  __syncwarp();  // every lane has read its row before any lane overwrites the block
  stage_row_shifted<0>(r, buf, lane);
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(tmap_c, smem_u32(buf), col0, row_base);
    tma_store_commit();
  }
  return true;
}

// 16-bit C, 64 columns at a time: `w` holds this lane's row as 32 packed pairs (columns col0 ..
// col0 + 63). Staged like a float32 chunk (the rows are 128 bytes either way) and stored by TMA
// through a 16-bit tensor map with a 64 x 32 box.
__device__ __forceinline__ void store_block16_tma(const uint32_t (&w)[32], int col0, float *buf,
                                                  const CUtensorMap *tmap_c, int m, int n, int row_base, int lane) {
  if (col0 >= n || row_base >= m)
    return;  // warp-uniform
  if (lane == 0)
    tma_store_wait_read();
  __syncwarp();
  stage_row_shifted<0>(w, buf, lane);
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(tmap_c, smem_u32(buf), col0, row_base);
    tma_store_commit();
  }
}

// 16-bit C whose base or pitch rules out TMA: the block is staged the same way and written row by
// row, each lane storing elements `lane` and `lane + 32` of the row (64 contiguous bytes per
// instruction), predicated at the edges. `columns`: 64, or 32 when only the low half of `w` is set.
__device__ __forceinline__ void store_block16_plain(const uint32_t (&w)[32], int col0, int columns, float *buf,
                                                    uint16_t *__restrict__ c, long long ldc, int m, int n,
                                                    int row_base, int lane) {
  if (col0 >= n || row_base >= m)
    return;  // warp-uniform
  stage_row_shifted<0>(w, buf, lane);
  __syncwarp();
  const uint16_t *halves = reinterpret_cast<const uint16_t *>(buf);
#pragma unroll 4
  for (int rr = 0; rr < 32; ++rr) {
    if (row_base + rr >= m)
      break;
    uint16_t *dst = c + static_cast<long long>(row_base + rr) * ldc + col0;
    for (int e = lane; e < columns; e += 32) {
      // Element e of the row sits in 16-byte piece e / 8, which was stored at piece ^ (row & 7).
      const int piece = (e >> 3) ^ (rr & 7);
      if (col0 + e < n)
        dst[e] = halves[rr * 64 + piece * 8 + (e & 7)];
    }
  }
  __syncwarp();
}

// The accumulator drain for a 16-bit C: two 32-column chunks make one 64-column block of packed
// pairs; element-wise operations run on the float32 values first.
template <int kColumns>
__device__ __forceinline__ void drain_accumulator_rows16(uint32_t taddr, float *stage, void *c, long long ldc, int m,
                                                         int n, int row_base, int col_base, int lane,
                                                         uint32_t release_bar, bool release_remote,
                                                         const Epilogue &ep, const CUtensorMap *tmap_c) {
  constexpr int kChunks = kColumns / 32;
  static_assert(kChunks % 2 == 0, "chunks are processed in pairs");
  uint32_t ra[32], rb[32], w[32];
  const bool ops = ep.op_count != 0;
  tmem_load_32x32b_x32(taddr, ra);
#pragma unroll 1
  for (int chunk = 0; chunk < kChunks; chunk += 2) {
    const int col0 = col_base + chunk * 32;
    tmem_load_wait_for(ra);
    tmem_load_32x32b_x32(taddr + (chunk + 1) * 32, rb);
    if (ops && col0 < n)
      apply_ops_lane_row(ra, col0, n, lane, ep);
#pragma unroll
    for (int j = 0; j < 16; ++j)
      w[j] = pack_pair(__uint_as_float(ra[2 * j]), __uint_as_float(ra[2 * j + 1]), ep.c_dtype);
    tmem_load_wait_for(rb);
    if (chunk + 2 < kChunks) {
      tmem_load_32x32b_x32(taddr + (chunk + 2) * 32, ra);
    } else {
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (release_remote)
          mbar_arrive_cluster(release_bar);
        else
          mbar_arrive(release_bar);
      }
    }
    if (ops && col0 + 32 < n)
      apply_ops_lane_row(rb, col0 + 32, n, lane, ep);
#pragma unroll
    for (int j = 0; j < 16; ++j)
      w[16 + j] = pack_pair(__uint_as_float(rb[2 * j]), __uint_as_float(rb[2 * j + 1]), ep.c_dtype);
    if (tmap_c != nullptr)
      store_block16_tma(w, col0, stage, tmap_c, m, n, row_base, lane);
    else
      store_block16_plain(w, col0, 64, stage, static_cast<uint16_t *>(c), ldc, m, n, row_base, lane);
  }
}

// `release_bar`: mbarrier (cluster-window address when `release_remote`) that receives one
// arrival from this warp as soon as the accumulator has been read completely.
//
// The TMEM load of the next chunk is in flight while the current chunk is transposed and
// stored (two register sets alternate), so the TMEM latency is hidden behind the stores.
template <int kColumns, bool kReadsC>
__device__ __forceinline__ void drain_accumulator_rows(uint32_t taddr, float *stage, void *c_any,
                                                       long long ldc, int m, int n, int row_base,
                                                       int col_base, bool vec_ok, int lane,
                                                       uint32_t release_bar, bool release_remote,
                                                       const Epilogue &ep, const CUtensorMap *tmap_c,
                                                       uint32_t c_load_bar = 0, uint32_t *c_load_phase = nullptr,
                                                       volatile uint32_t *abort_flag = nullptr,
                                                       const PushMaps *push_maps = nullptr) {
  constexpr int kChunks = kColumns / 32;
  static_assert(kChunks % 2 == 0, "chunks are processed in pairs");
  if constexpr (!kReadsC) {
    if (ep.c_dtype != kCTypeF32) {  // grid-uniform
      drain_accumulator_rows16<kColumns>(taddr, stage, c_any, ldc, m, n, row_base, col_base, lane, release_bar,
                                         release_remote, ep, tmap_c);
      return;
    }
  }
  float *__restrict__ c = static_cast<float *>(c_any);
  uint32_t ra[32], rb[32];
  float carry[6] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
  // Stores of an aligned C go through TMA (`tmap_c` is null otherwise).
  const bool tma = !kReadsC && tmap_c != nullptr;
  const bool tma_add = ep.accumulate_by_tma != 0;
  const bool tma_load_add = !kReadsC && ep.accumulate_by_tma_load != 0 && c_load_phase != nullptr;
  const bool ops_first = !kReadsC && ep.op_count != 0 && !tma_load_add;  // element-wise work done in registers
  tmem_load_32x32b_x32(taddr, ra);
#pragma unroll 1
  for (int chunk = 0; chunk < kChunks; chunk += 2) {
    tmem_load_wait_for(ra);
    tmem_load_32x32b_x32(taddr + (chunk + 1) * 32, rb);
    if (ops_first && col_base + chunk * 32 < n)
      apply_ops_lane_row(ra, col_base + chunk * 32, n, lane, ep);
    if (tma_load_add)
      accumulate_chunk_tma(ra, chunk, stage, tmap_c, m, n, row_base, col_base, lane, c_load_bar, *c_load_phase,
                           abort_flag, ep);
    else if (tma)
      store_chunk_tma(ra, chunk, stage, tmap_c, m, n, row_base, col_base, lane, tma_add, push_maps);
    else if constexpr (kReadsC)
      write_chunk_reading_c(ra, chunk, false, stage, c, ldc, m, n, row_base, col_base, vec_ok, lane, carry, ep);
    else
      write_chunk(ra, chunk, false, stage, c, ldc, m, n, row_base, col_base, vec_ok, lane, carry, ep);
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
    if (ops_first && col_base + (chunk + 1) * 32 < n)
      apply_ops_lane_row(rb, col_base + (chunk + 1) * 32, n, lane, ep);
    if (tma_load_add)
      accumulate_chunk_tma(rb, chunk + 1, stage, tmap_c, m, n, row_base, col_base, lane, c_load_bar, *c_load_phase,
                           abort_flag, ep);
    else if (tma)
      store_chunk_tma(rb, chunk + 1, stage, tmap_c, m, n, row_base, col_base, lane, tma_add, push_maps);
    else if constexpr (kReadsC)
      write_chunk_reading_c(rb, chunk + 1, chunk + 2 >= kChunks, stage, c, ldc, m, n, row_base, col_base, vec_ok, lane,
                            carry, ep);
    else
      write_chunk(rb, chunk + 1, chunk + 2 >= kChunks, stage, c, ldc, m, n, row_base, col_base, vec_ok, lane, carry,
                  ep);
  }
}

} // namespace sm100
} // namespace hc

namespace hc {
namespace sm100 {

// Split-k, second half, run by the warp whose unit arrived last: the partial tiles of all splits
// are added in split order and the sums leave through the same chunk writers as an unsplit tile.
// `partial_rows`: this warp's first row of split 0's partial tile, at the warp's first column
// (rows are `partial_ld` floats apart, consecutive splits `split_stride` floats). The partial
// tiles are read the way C is written -- 8 lanes per 128-byte row segment -- so every load
// instruction fetches four full lines.
// (Not inlined: it runs once per tile, and kept apart it cannot raise the register demand of the
// chunk loop that every tile goes through.)
template <int kColumns, bool kReadsC>
__device__ __noinline__ void reduce_partials_rows(const float *partial_rows, int partial_ld, size_t split_stride,
                                                  int splits, float *stage, void *c_any, long long ldc,
                                                  int m, int n, int row_base, int col_base, bool vec_ok, int lane,
                                                  const Epilogue &ep, const CUtensorMap *tmap_c) {
  constexpr int kChunks = kColumns / 32;
  float carry[6] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
  float *__restrict__ c = static_cast<float *>(c_any);
  const bool half_out = !kReadsC && ep.c_dtype != kCTypeF32;  // then `tmap_c` (64-column boxes) is not used here
  const bool tma = !kReadsC && tmap_c != nullptr && !half_out;
  const bool ops_first = !kReadsC && ep.op_count != 0;
  const int piece = lane & 7;
  const float *lane_base = partial_rows + static_cast<size_t>(lane >> 3) * partial_ld + piece * 4;
#pragma unroll 1
  for (int chunk = 0; chunk < kChunks; ++chunk) {
    if (col_base + chunk * 32 >= n || row_base >= m)
      break;  // warp-uniform: nothing of this or any later chunk is inside C
    float4 sum[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      sum[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 2
    for (int s = 0; s < splits; ++s) {
      const float *src = lane_base + s * split_stride + chunk * 32;
      float4 part[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        part[i] = __ldcg(reinterpret_cast<const float4 *>(src + static_cast<size_t>(i * 4) * partial_ld));
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sum[i].x += part[i].x; sum[i].y += part[i].y; sum[i].z += part[i].z; sum[i].w += part[i].w;
      }
    }
    if (tma) {
      if (ops_first) {
        // Each lane's groups start at column piece * 4 of the chunk: its four bias values.
        const int col0 = col_base + chunk * 32;
        float bias_lane = 0.0f;
        if (ep.bias != nullptr && col0 + lane < n)
          bias_lane = __ldg(ep.bias + col0 + lane);
        const float4 bias = make_float4(__shfl_sync(0xffffffffu, bias_lane, piece * 4),
                                        __shfl_sync(0xffffffffu, bias_lane, piece * 4 + 1),
                                        __shfl_sync(0xffffffffu, bias_lane, piece * 4 + 2),
                                        __shfl_sync(0xffffffffu, bias_lane, piece * 4 + 3));
        apply_ops_to_groups(sum, ep, [&](int) { return bias; });
      }
      if (lane == 0)
        tma_store_wait_read();  // the previous chunk's store has read the buffer
      __syncwarp();
    }
    // The sums go into the staging block where the coalesced writers would read them ...
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = i * 4 + (lane >> 3);
      *reinterpret_cast<float4 *>(stage + rr * 32 + ((piece ^ (rr & 7)) << 2)) = sum[i];
    }
    if (tma) {
      // ... which is already the layout of a TMA box.
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (ep.accumulate_by_tma != 0)
          tma_reduce_add_2d(tmap_c, smem_u32(stage), col_base + chunk * 32, row_base);
        else
          tma_store_2d(tmap_c, smem_u32(stage), col_base + chunk * 32, row_base);
        tma_store_commit();
      }
      continue;
    }
    // Otherwise each lane takes its row back into registers and the chunk goes through the
    // ordinary writer (odd pitches, fused work, push targets).
    __syncwarp();
    uint32_t r[32];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 v = *reinterpret_cast<const float4 *>(stage + lane * 32 + ((q ^ (lane & 7)) << 2));
      r[4 * q] = __float_as_uint(v.x);
      r[4 * q + 1] = __float_as_uint(v.y);
      r[4 * q + 2] = __float_as_uint(v.z);
      r[4 * q + 3] = __float_as_uint(v.w);
    }
    if (ops_first)
      apply_ops_lane_row(r, col_base + chunk * 32, n, lane, ep);
    if (half_out) {
      uint32_t w[32];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        w[j] = pack_pair(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]), ep.c_dtype);
        w[16 + j] = 0u;
      }
      store_block16_plain(w, col_base + chunk * 32, 32, stage, static_cast<uint16_t *>(c_any), ldc, m, n, row_base,
                          lane);
      continue;
    }
    if constexpr (kReadsC)
      write_chunk_reading_c(r, chunk, chunk == kChunks - 1, stage, c, ldc, m, n, row_base, col_base, vec_ok, lane, carry,
                            ep);
    else
      write_chunk(r, chunk, chunk == kChunks - 1, stage, c, ldc, m, n, row_base, col_base, vec_ok, lane, carry, ep);
  }
}

// One unit of a dense launch: a whole tile (parts == 1) or one k range of a split tile.
struct DenseUnit {
  int tile;
  int part, parts;
  int split_index;  // of a split unit: its number among the split units (partial tile index)
  int split_tile;   // of a split unit: its tile's number among the split tiles (counter index)
};

__device__ __forceinline__ DenseUnit decode_unit(int unit, const SplitK &split) {
  DenseUnit u;
  if (unit < split.first_split_tile || split.splits == 1) {
    u.tile = unit;
    u.part = 0;
    u.parts = 1;
    u.split_index = 0;
    u.split_tile = 0;
    return u;
  }
  u.split_index = unit - split.first_split_tile;
  u.split_tile = u.split_index / split.splits;
  u.part = u.split_index - u.split_tile * split.splits;
  u.parts = split.splits;
  u.tile = split.first_split_tile + u.split_tile;
  return u;
}

// Counts this warp's partial rows in; true for the warp whose unit completes the tile. The
// partial rows written before the call are visible to that warp after it.
__device__ __forceinline__ bool split_arrive_is_last(unsigned *counter, int splits, int lane) {
  __threadfence();
  __syncwarp();
  unsigned arrived = 0;
  if (lane == 0)
    arrived = atomicAdd(counter, 1u);
  arrived = __shfl_sync(0xffffffffu, arrived, 0);
  if (arrived != static_cast<unsigned>(splits - 1))
    return false;
  __threadfence();
  return true;
}

} // namespace sm100
} // namespace hc
