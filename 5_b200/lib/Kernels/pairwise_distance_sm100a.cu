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
// computes 32 x 64 outputs, a thread 2 x 4 of them (as four pairs of neighbouring columns), from rows
// staged (transposed) in shared memory.
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
// Arithmetic: 3 float32 operations per (i, j, h), none of them fusable; the kernel is bound by the
// float32 rate, not by memory (the rows of a tile are re-read from L2 by the tiles beside it). The
// operations are issued two outputs at a time as packed float32x2 instructions (add.rn.f32x2 and,
// for the square, fma.rn.f32x2 with a zero addend: two independent, individually rounded IEEE
// operations per lane), which halves the issue
// slots the arithmetic takes. x1 is staged negated and duplicated, so that d = x2 + (-x1) needs no
// operand shuffling: (b - a)^2 and (a - b)^2 are the same float32 number.
#include "gemm_launch.h"

#include <cstdint>

namespace hc {
namespace sm100 {

namespace {

constexpr int kTileRows = 32;     // of x1 per CTA (outputs i)
constexpr int kTileCols = 64;     // rows of x2 per CTA (outputs j)
constexpr int kThreads = 256;     // 16 x 16: a thread owns 2 rows x 4 columns
constexpr int kChunk = 32;        // h staged per step
constexpr int kRowsPitch = 2 * kTileRows + 4;  // floats: every value of x1 twice; 16-byte reads stay aligned
constexpr int kColsPitch = kTileCols + 4;      // floats; 16-byte reads stay aligned
constexpr int kStackDepth = 24;   // pending partial sums: the recursion halves n down to 128
constexpr int kPairs = 4;         // a thread's outputs as pairs of neighbouring columns: pair 2 r + p

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

// ... and puts into shared memory transposed, dst[h][row]; the rows of x1 negated and twice each,
// dst[h][2 row], dst[h][2 row + 1] = -x1[row][h] (the two lanes of a packed operation).
template <int kVectors, int kPitch, bool kNegatedTwice>
__device__ __forceinline__ void stage_rows(float *dst, const Fetched<kVectors> &f) {
#pragma unroll
  for (int i = 0; i < kVectors; ++i) {
    const int v = static_cast<int>(threadIdx.x) + i * kThreads;
    const int row = v / (kChunk / 4), h = (v % (kChunk / 4)) * 4;
    const float value[4] = {f.value[i].x, f.value[i].y, f.value[i].z, f.value[i].w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if constexpr (kNegatedTwice)
        *reinterpret_cast<float2 *>(dst + (h + q) * kPitch + 2 * row) = make_float2(-value[q], -value[q]);
      else
        dst[(h + q) * kPitch + row] = value[q];
    }
  }
}

// Packed float32x2 addition and multiplication, each lane rounded to nearest on its own. Written as
// PTX with the rounding mode spelled out: an operation with an explicit rounding modifier is never
// contracted with a neighbour into a fused multiply-add (the add2(acc, mul2(d, d)) of the
// CUDA headers was, and came out one unit in the last place away from NumPy on a third of the sums).
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<const unsigned long long *>(&a)), "l"(*reinterpret_cast<const unsigned long long *>(&b)));
  return *reinterpret_cast<float2 *>(&d);
}

// d * d for a packed pair, written as the fused form d * d + (+0): exactly the rounded product (a
// square is never -0, and x + (+0) == x for every other x). ptxas contracts a packed multiply that
// feeds a packed add into one fused multiply-add -- with the rounding modes spelled out, with
// -fmad=false, and when the add is itself written as square * 1 + acc (measured each time: a third
// of the sums one unit in the last place away from NumPy, and equal to the fused model) -- but a
// fused multiply-add with a +0 addend is not a multiply (they differ when the product is -0), so it
// has to stay, and nothing contracts a fused multiply-add with the add that follows.
__device__ __forceinline__ float2 square2(float2 d) {
  const float2 zero = make_float2(0.0f, 0.0f);
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %1, %2;"
      : "=l"(r)
      : "l"(*reinterpret_cast<const unsigned long long *>(&d)), "l"(*reinterpret_cast<const unsigned long long *>(&zero)));
  return *reinterpret_cast<float2 *>(&r);
}

// One h of a thread's 2 x 4 outputs: pair 2 r + p holds columns 2 p, 2 p + 1 of row r.
__device__ __forceinline__ void squared_differences(const float *rows_s, const float *cols_s, int hh, int ty, int tx,
                                                    float2 (&square)[kPairs]) {
  const float4 a = *reinterpret_cast<const float4 *>(rows_s + hh * kRowsPitch + ty * 4);  // -a0, -a0, -a1, -a1
  const float4 b = *reinterpret_cast<const float4 *>(cols_s + hh * kColsPitch + tx * 4);
  const float2 minus_a[2] = {make_float2(a.x, a.y), make_float2(a.z, a.w)};
  const float2 b_pair[2] = {make_float2(b.x, b.y), make_float2(b.z, b.w)};
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      const float2 d = add2(b_pair[p], minus_a[r]);  // b - a, each lane rounded on its own
      square[2 * r + p] = square2(d);
    }
}

template <bool kSqrt>
__global__ void __launch_bounds__(kThreads, 2)
pairwise_f32_kernel(const float *__restrict__ x1, long long ld1, const float *__restrict__ x2, long long ld2,
                    float *__restrict__ out, long long ldo, int w1, int w2, int h, const int4 *__restrict__ leaves,
                    int num_leaves, int tiles_j) {
  constexpr int kRowVectors = kTileRows * (kChunk / 4) / kThreads;  // 1
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

  float2 pending[kPairs][kStackDepth];  // per pair of outputs: partial sums waiting for their right-hand neighbour
  int depth = 0;
  float2 acc[kPairs][8];
  float2 sum[kPairs];
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
    stage_rows<kRowVectors, kRowsPitch, true>(rows_s, next_rows);
    stage_rows<kColVectors, kColsPitch, false>(cols_s, next_cols);
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
      for (int o = 0; o < kPairs; ++o)
#pragma unroll
        for (int j = 0; j < 8; ++j)
          acc[o][j] = make_float2(0.0f, 0.0f);  // (0 + s == s exactly: a square is never -0)
    }
    const int groups = min(kChunk, begin + full - c0) / 8;  // whole groups of eight in this chunk (may be <= 0)
#pragma unroll 4
    for (int g = 0; g < groups; ++g) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float2 square[kPairs];
        squared_differences(rows_s, cols_s, g * 8 + j, ty, tx, square);
#pragma unroll
        for (int o = 0; o < kPairs; ++o)
          acc[o][j] = add2(acc[o][j], square[o]);
      }
    }
    if (c0 + kChunk >= end) {
      // The leaf is complete: combine the accumulators, then the tail of fewer than eight values
      // (it lies in this chunk) in order.
#pragma unroll
      for (int o = 0; o < kPairs; ++o)
        sum[o] = add2(add2(add2(acc[o][0], acc[o][1]), add2(acc[o][2], acc[o][3])),
                            add2(add2(acc[o][4], acc[o][5]), add2(acc[o][6], acc[o][7])));
      for (int hh = begin + full - c0; hh < end - c0; ++hh) {
        float2 square[kPairs];
        squared_differences(rows_s, cols_s, hh, ty, tx, square);
#pragma unroll
        for (int o = 0; o < kPairs; ++o)
          sum[o] = add2(sum[o], square[o]);
      }
      // Push, then add the pairs the recursion closes here (left + right).
      if (depth < kStackDepth) {
#pragma unroll
        for (int o = 0; o < kPairs; ++o)
          pending[o][depth] = sum[o];
        ++depth;
      }
      for (int a = 0; a < entry.z && depth >= 2; ++a) {
        --depth;
#pragma unroll
        for (int o = 0; o < kPairs; ++o)
          pending[o][depth - 1] = add2(pending[o][depth - 1], pending[o][depth]);
      }
    }
    leaf = following_leaf;
    entry = following;
    c0 = following_c0;
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = i0 + ty * 2 + r;
    if (i >= w1)
      continue;
    const float2 zero = make_float2(0.0f, 0.0f);  // an empty sum is 0
    const float2 left = num_leaves > 0 ? pending[2 * r][0] : zero, right = num_leaves > 0 ? pending[2 * r + 1][0] : zero;
    float v[4] = {left.x, left.y, right.x, right.y};
    if (kSqrt) {
#pragma unroll
      for (int c = 0; c < 4; ++c)
        v[c] = __fsqrt_rn(v[c]);
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

cudaError_t launch_pairwise_f32(const float *x1, long long ld1, const float *x2, long long ld2, float *out,
                                long long ldo, int w1, int w2, int h, int take_sqrt, const int4 *leaves_dev,
                                int num_leaves, cudaStream_t stream) {
  if (w1 <= 0 || w2 <= 0)
    return cudaSuccess;
  if (h < 0 || h > pairwise_max_h() || (h > 0 && (leaves_dev == nullptr || num_leaves < 1)))
    return cudaErrorInvalidValue;
  const long long tiles_i = (w1 + kTileRows - 1) / kTileRows, tiles_j = (w2 + kTileCols - 1) / kTileCols;
  if (tiles_i * tiles_j > 0x7fffffffLL)
    return cudaErrorInvalidValue;
  const unsigned grid = static_cast<unsigned>(tiles_i * tiles_j);
  if (take_sqrt)
    pairwise_f32_kernel<true><<<grid, kThreads, 0, stream>>>(x1, ld1, x2, ld2, out, ldo, w1, w2, h, leaves_dev,
                                                             num_leaves, static_cast<int>(tiles_j));
  else
    pairwise_f32_kernel<false><<<grid, kThreads, 0, stream>>>(x1, ld1, x2, ld2, out, ldo, w1, w2, h, leaves_dev,
                                                              num_leaves, static_cast<int>(tiles_j));
  return cudaGetLastError();
}

} // namespace sm100
} // namespace hc
