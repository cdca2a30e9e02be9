// Pairwise distances for sm_100a:  out[i, j] = sqrt(sum_h (x1[i, h] - x2[j, h])^2), float32.
//
// The hc kernel class behind it is the two-dimensional workgroup kernel of the reference's
// simulator tests (tests/test_simulator.py:142-167):
//
//     gid = group.work_offset
//     lhs = group.load(x1[gid[0]:], shape=(group.shape[0], x1.shape[1]))   # rows past the end: inactive
//     rhs = group.load(x2[gid[1]:], shape=(group.shape[1], x2.shape[1]))
//     diff = ((lhs[:, None, :] - rhs[None, :, :]) ** 2).sum(axis=2)
//     group.store(out[gid[0]:, gid[1]:], np.sqrt(diff))                    # only inside out
//
// with work_shape=(W1, W2): every (i, j) below (W1, W2) is computed once and nothing else is
// written. The group shape is not observable, so the launch is re-tiled: a CTA of 256 threads
// computes 32 x 64 outputs, a thread 2 x 4 of them, from rows staged (transposed) in shared memory.
//
// The result is bit-identical to the reference simulator's, which computes in float32 with NumPy:
// one rounding per operation -- the difference, its square (np.power with exponent 2 multiplies), the
// additions -- so nothing here may be contracted into a fused multiply-add (__fsub_rn, __fmul_rn,
// __fadd_rn), and the sum over h runs in the order of NumPy's float32 sum of a contiguous vector
// (hc/_sim_types.py:1100-1102 reduces `payload[active]` with np.sum): a vector of at most 128
// elements is summed into eight interleaved accumulators r[h % 8], combined as
// ((r0 + r1) + (r2 + r3)) + ((r4 + r5) + (r6 + r7)), then the h % 8 tail is added in order; a longer
// vector is split at n / 2 rounded down to a multiple of 8 and its halves are summed that way
// recursively and added. The host lists the leaves of that recursion (start, length, and how many
// pending partial sums to add once the leaf is done); every thread walks the list with the eight
// accumulators per output in registers and the pending partial sums on a small stack.
// Arithmetic: 3 float32 instructions per (i, j, h), none of them fusable; the kernel is bound by the
// float32 issue rate, not by memory (the rows of a tile are re-read from L2 by the tiles beside it).
#include "gemm_launch.h"

#include <cstdint>
#include <cstdlib>

namespace hc {
namespace sm100 {

namespace {

constexpr int kTileCols = 64;     // rows of x2 per CTA (outputs j)
constexpr int kThreads = 256;     // 16 x 16: a thread owns kRowsPerThread rows x 4 columns
constexpr int kChunk = 32;        // h staged per step
constexpr int kColsPitch = kTileCols + 4;  // floats; keeps the 16-byte reads aligned
// Rows of x1 per CTA (outputs i) and the pitch of their staging, for 2 or 4 rows per thread: the
// pitch keeps the 8-byte (16-byte) reads of a thread's rows aligned.
__host__ __device__ constexpr int tile_rows(int rows_per_thread) { return 16 * rows_per_thread; }
__host__ __device__ constexpr int rows_pitch(int rows_per_thread) { return tile_rows(rows_per_thread) + rows_per_thread; }
constexpr int kStackDepth = 24;   // pending partial sums: the recursion halves n down to 128

// The part of a chunk one thread brings in: `kVectors` groups of four consecutive h of one row each
// (vector v of the chunk is row v / 8, h 4 (v % 8) .. + 3). Rows at or past `limit` and h at or past
// `h_end` read as zeros (they are never used for an output that is stored, nor added to a sum).
template <int kVectors>
struct Fetched {
  float4 value[kVectors];
};

template <int kVectors>
__device__ __forceinline__ Fetched<kVectors> fetch_rows(const float *__restrict__ x, long long ld, int row0, int limit,
                                                        int h0, int h_end, bool vector_ok) {
  Fetched<kVectors> f;
#pragma unroll
  for (int i = 0; i < kVectors; ++i) {
    const int v = static_cast<int>(threadIdx.x) + i * kThreads;
    const int row = v / (kChunk / 4), h = (v % (kChunk / 4)) * 4;
    float4 value = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (row0 + row < limit && h0 + h < h_end) {
      const float *src = x + static_cast<long long>(row0 + row) * ld + h0 + h;
      if (vector_ok && h0 + h + 3 < h_end) {
        value = __ldg(reinterpret_cast<const float4 *>(src));
      } else {
        value.x = __ldg(src);
        if (h0 + h + 1 < h_end) value.y = __ldg(src + 1);
        if (h0 + h + 2 < h_end) value.z = __ldg(src + 2);
        if (h0 + h + 3 < h_end) value.w = __ldg(src + 3);
      }
    }
    f.value[i] = value;
  }
  return f;
}

// ... and puts into shared memory transposed: dst[h][row].
template <int kVectors, int kPitch>
__device__ __forceinline__ void stage_rows(float *dst, const Fetched<kVectors> &f) {
#pragma unroll
  for (int i = 0; i < kVectors; ++i) {
    const int v = static_cast<int>(threadIdx.x) + i * kThreads;
    const int row = v / (kChunk / 4), h = (v % (kChunk / 4)) * 4;
    dst[(h + 0) * kPitch + row] = f.value[i].x;
    dst[(h + 1) * kPitch + row] = f.value[i].y;
    dst[(h + 2) * kPitch + row] = f.value[i].z;
    dst[(h + 3) * kPitch + row] = f.value[i].w;
  }
}

// The values of a thread's rows (kR of them, consecutive) and columns (4) at one h.
template <int kR>
__device__ __forceinline__ void load_operands(const float *rows_s, const float *cols_s, int hh, int ty, int tx,
                                              float (&av)[kR], float (&bv)[4]) {
  if constexpr (kR == 2) {
    const float2 a = *reinterpret_cast<const float2 *>(rows_s + hh * rows_pitch(2) + ty * 2);
    av[0] = a.x, av[1] = a.y;
  } else {
    const float4 a = *reinterpret_cast<const float4 *>(rows_s + hh * rows_pitch(4) + ty * 4);
    av[0] = a.x, av[1] = a.y, av[2] = a.z, av[3] = a.w;
  }
  const float4 b = *reinterpret_cast<const float4 *>(cols_s + hh * kColsPitch + tx * 4);
  bv[0] = b.x, bv[1] = b.y, bv[2] = b.z, bv[3] = b.w;
}

// kR: rows per thread (2: 32 x 64 outputs per CTA, two CTAs per SM; 4: 64 x 64, one CTA per SM, half
// the shared-memory loads per arithmetic instruction).
template <int kR, bool kSqrt>
__global__ void __launch_bounds__(kThreads, kR == 2 ? 2 : 1)
pairwise_f32_kernel(const float *__restrict__ x1, long long ld1, const float *__restrict__ x2, long long ld2,
                    float *__restrict__ out, long long ldo, int w1, int w2, int h, const int4 *__restrict__ leaves,
                    int num_leaves, int tiles_j) {
  constexpr int kTileRows = tile_rows(kR), kRowsPitch = rows_pitch(kR), kOutputs = kR * 4;
  constexpr int kRowVectors = kTileRows * (kChunk / 4) / kThreads;  // 1 or 2
  constexpr int kColVectors = kTileCols * (kChunk / 4) / kThreads;  // 2
  static_assert(kRowVectors * kThreads == kTileRows * (kChunk / 4) && kColVectors * kThreads == kTileCols * (kChunk / 4),
                "every thread brings in the same number of vectors");
  __shared__ __align__(16) float rows_s[kChunk * kRowsPitch];
  __shared__ __align__(16) float cols_s[kChunk * kColsPitch];
  const int tile_i = blockIdx.x / tiles_j, tile_j = blockIdx.x - tile_i * tiles_j;
  const int i0 = tile_i * kTileRows, j0 = tile_j * kTileCols;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const bool vec1 = (ld1 & 3) == 0 && (reinterpret_cast<uintptr_t>(x1) & 15) == 0;
  const bool vec2 = (ld2 & 3) == 0 && (reinterpret_cast<uintptr_t>(x2) & 15) == 0;

  float pending[kOutputs][kStackDepth];  // per output: partial sums waiting for their right-hand neighbour
  int depth = 0;
  float acc[kOutputs][8];
  float sum[kOutputs];
  // The chunks of all leaves in order; the next chunk's values are fetched into registers while the
  // current one is being used.
  int leaf = 0;
  int4 entry = num_leaves > 0 ? leaves[0] : make_int4(0, 0, 0, 0);  // x: first h, y: length, z: additions once done
  int c0 = entry.x;
  Fetched<kRowVectors> next_rows;
  Fetched<kColVectors> next_cols;
  if (num_leaves > 0) {
    next_rows = fetch_rows<kRowVectors>(x1, ld1, i0, w1, c0, entry.x + entry.y, vec1);
    next_cols = fetch_rows<kColVectors>(x2, ld2, j0, w2, c0, entry.x + entry.y, vec2);
  }
#pragma unroll 1
  while (leaf < num_leaves) {
    const int begin = entry.x, full = entry.y & ~7, end = entry.x + entry.y;
    __syncthreads();  // the previous chunk has been read
    stage_rows<kRowVectors, kRowsPitch>(rows_s, next_rows);
    stage_rows<kColVectors, kColsPitch>(cols_s, next_cols);
    __syncthreads();
    int following_leaf = leaf, following_c0 = c0 + kChunk;
    int4 following = entry;
    if (following_c0 >= end) {
      following_leaf = leaf + 1;
      if (following_leaf < num_leaves) {
        following = leaves[following_leaf];
        following_c0 = following.x;
      }
    }
    if (following_leaf < num_leaves) {
      next_rows = fetch_rows<kRowVectors>(x1, ld1, i0, w1, following_c0, following.x + following.y, vec1);
      next_cols = fetch_rows<kColVectors>(x2, ld2, j0, w2, following_c0, following.x + following.y, vec2);
    }
    if (c0 == begin) {
#pragma unroll
      for (int o = 0; o < kOutputs; ++o)
#pragma unroll
        for (int j = 0; j < 8; ++j)
          acc[o][j] = 0.0f;  // (0 + s == s exactly: a square is never -0)
    }
    const int groups = min(kChunk, begin + full - c0) / 8;  // whole groups of eight in this chunk (may be <= 0)
#pragma unroll 1
    for (int g = 0; g < groups; ++g) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float av[kR], bv[4];
        load_operands<kR>(rows_s, cols_s, g * 8 + j, ty, tx, av, bv);
#pragma unroll
        for (int r = 0; r < kR; ++r)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float d = __fsub_rn(av[r], bv[c]);
            acc[r * 4 + c][j] = __fadd_rn(acc[r * 4 + c][j], __fmul_rn(d, d));
          }
      }
    }
    if (c0 + kChunk >= end) {
      // The leaf is complete: combine the accumulators, then the tail of fewer than eight values
      // (it lies in this chunk) in order.
#pragma unroll
      for (int o = 0; o < kOutputs; ++o)
        sum[o] = __fadd_rn(__fadd_rn(__fadd_rn(acc[o][0], acc[o][1]), __fadd_rn(acc[o][2], acc[o][3])),
                           __fadd_rn(__fadd_rn(acc[o][4], acc[o][5]), __fadd_rn(acc[o][6], acc[o][7])));
      for (int hh = begin + full - c0; hh < end - c0; ++hh) {
        float av[kR], bv[4];
        load_operands<kR>(rows_s, cols_s, hh, ty, tx, av, bv);
#pragma unroll
        for (int r = 0; r < kR; ++r)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float d = __fsub_rn(av[r], bv[c]);
            sum[r * 4 + c] = __fadd_rn(sum[r * 4 + c], __fmul_rn(d, d));
          }
      }
      // Push, then add the pairs the recursion closes here (left + right).
      if (depth < kStackDepth) {
#pragma unroll
        for (int o = 0; o < kOutputs; ++o)
          pending[o][depth] = sum[o];
        ++depth;
      }
      for (int a = 0; a < entry.z && depth >= 2; ++a) {
        --depth;
#pragma unroll
        for (int o = 0; o < kOutputs; ++o)
          pending[o][depth - 1] = __fadd_rn(pending[o][depth - 1], pending[o][depth]);
      }
    }
    leaf = following_leaf;
    entry = following;
    c0 = following_c0;
  }

#pragma unroll
  for (int r = 0; r < kR; ++r) {
    const int i = i0 + ty * kR + r;
    if (i >= w1)
      continue;
    float v[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float total = num_leaves > 0 ? pending[r * 4 + c][0] : 0.0f;  // an empty sum is 0
      v[c] = kSqrt ? __fsqrt_rn(total) : total;
    }
    const int j = j0 + tx * 4;
    float *dst = out + static_cast<long long>(i) * ldo + j;
    if (j + 3 < w2 && (ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
      __stcs(reinterpret_cast<float4 *>(dst), make_float4(v[0], v[1], v[2], v[3]));
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (j + c < w2)
          __stcs(dst + c, v[c]);
    }
  }
}

void list_leaves(int begin, int n, int4 *out, int *count, int capacity) {
  if (n <= 128) {
    if (*count < capacity)
      out[*count] = make_int4(begin, n, 0, 0);
    ++*count;
    return;
  }
  int left = n / 2;
  left -= left % 8;
  list_leaves(begin, left, out, count, capacity);
  list_leaves(begin + left, n - left, out, count, capacity);
  if (*count - 1 < capacity)
    out[*count - 1].z += 1;  // the right half's last leaf closes this pair
}

} // namespace

int pairwise_schedule(int h, int4 *leaves, int capacity) {
  int count = 0;
  if (h > 0)
    list_leaves(0, h, leaves, &count, capacity);
  return count;
}

int pairwise_max_h() {
  // The stack of pending partial sums holds kStackDepth entries: the recursion halves n until it is
  // at most 128, so h up to 2^20 needs 14.
  return 1 << 20;
}

template <int kR>
cudaError_t launch_pairwise_tiles(const float *x1, long long ld1, const float *x2, long long ld2, float *out,
                                  long long ldo, int w1, int w2, int h, int take_sqrt, const int4 *leaves_dev,
                                  int num_leaves, cudaStream_t stream) {
  const long long tiles_i = (w1 + tile_rows(kR) - 1) / tile_rows(kR), tiles_j = (w2 + kTileCols - 1) / kTileCols;
  if (tiles_i * tiles_j > 0x7fffffffLL)
    return cudaErrorInvalidValue;
  const unsigned grid = static_cast<unsigned>(tiles_i * tiles_j);
  if (take_sqrt)
    pairwise_f32_kernel<kR, true><<<grid, kThreads, 0, stream>>>(x1, ld1, x2, ld2, out, ldo, w1, w2, h, leaves_dev,
                                                                 num_leaves, static_cast<int>(tiles_j));
  else
    pairwise_f32_kernel<kR, false><<<grid, kThreads, 0, stream>>>(x1, ld1, x2, ld2, out, ldo, w1, w2, h, leaves_dev,
                                                                  num_leaves, static_cast<int>(tiles_j));
  return cudaGetLastError();
}

cudaError_t launch_pairwise_f32(const float *x1, long long ld1, const float *x2, long long ld2, float *out,
                                long long ldo, int w1, int w2, int h, int take_sqrt, const int4 *leaves_dev,
                                int num_leaves, cudaStream_t stream) {
  if (w1 <= 0 || w2 <= 0)
    return cudaSuccess;
  if (h < 0 || h > pairwise_max_h() || (h > 0 && (leaves_dev == nullptr || num_leaves < 1)))
    return cudaErrorInvalidValue;
  int rows_per_thread = 2;
  if (const char *forced = std::getenv("HC_CUDA_PAIRWISE_ROWS"))  // tuning aid: 2 or 4 rows per thread
    rows_per_thread = std::atoi(forced);
  if (rows_per_thread == 4)
    return launch_pairwise_tiles<4>(x1, ld1, x2, ld2, out, ldo, w1, w2, h, take_sqrt, leaves_dev, num_leaves, stream);
  return launch_pairwise_tiles<2>(x1, ld1, x2, ld2, out, ldo, w1, w2, h, take_sqrt, leaves_dev, num_leaves, stream);
}

} // namespace sm100
} // namespace hc
