// Row sums for sm_100a:  out[i] = post(sum_h pre(x[i, h])), float32.
//
// The hc kernel class behind it is the one-dimensional workgroup kernel that reduces the rows it
// loads, the reduction of the reference simulator's value type (hc/_sim_types.py:338-351, 501-518,
// 1050-1102) applied to the load of tests/test_simulator.py:153-154:
//
//     r0 = group.work_offset[0]
//     rows = group.load(x[r0:], shape=(group.shape[0], x.shape[1]))   # rows past the end: inactive
//     group.store(out[r0:], rows.sum(axis=1))                         # only inside out
//
// optionally with the rows squared before the sum (`rows * rows`, `rows ** 2`) and the square root
// of the sum taken after it (row norms). With work_shape=(W,) every row below W is reduced once and
// nothing else is written; the group shape is not observable, so the launch is re-tiled.
//
// The result is bit-identical to the reference simulator's, which reduces the active values of a
// row with np.sum (hc/_sim_types.py:1100-1102): float32 additions, one rounding each, in the order
// of NumPy's sum of a contiguous float32 vector -- a vector of at most 128 values goes into eight
// interleaved accumulators r[h % 8] that start as the first eight values and are combined as
// ((r0 + r1) + (r2 + r3)) + ((r4 + r5) + (r6 + r7)) before the h % 8 tail is added in order; fewer
// than eight values are added in order starting from 0; a longer vector is split at n / 2 rounded
// down to a multiple of 8, its halves are summed that way recursively and added; the result is then
// added to the reduction's initial value +0 (which only turns a -0 sum into +0). The host lists the
// leaves of that recursion (the list the pairwise-distance kernel uses).
//
// Work split: two neighbouring lanes own a row, or one of up to 16 parts of a row. Lane q of the pair
// holds accumulators 4 q .. 4 q + 3 of the current leaf and reads the 16 bytes
// x[i, h + 4 q .. h + 4 q + 3] of each group of eight, so a pair reads one 32-byte sector per step and a
// warp 16 of them; eight steps' loads are issued before their additions. The chains of additions of
// one accumulator never leave their lane, so their order is NumPy's; the two lanes meet in one
// shuffle per leaf. The partial sums that wait for their right-hand neighbour in the recursion sit
// on a small per-thread stack.
// A row of more than 128 values is shared by P = 2, 4, 8 or 16 pairs of one warp: the first log2(P)
// levels of the recursion cut the row into P consecutive ranges of leaves (P as large as the
// recursion allows), each pair sums one range exactly as above, and the P results are added in the
// recursion's own order (neighbours first) with shuffles. All lanes of a warp then walk the same
// number of steps with their loads and additions predicated, since ranges and leaves differ in
// length. Up to 16 leaves a pair has one leaf, so a warp's loads fall into consecutive leaves; beyond
// that the ranges also keep many lanes busy when the rows are few.
// Bytes per launch: 4 W H read once + 4 W written; there is no reuse, the kernel is HBM bound.
#include "gemm_launch.h"

#include <cstdint>

namespace hc {
namespace sm100 {

namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerCta = kThreads / 2;
constexpr int kStackDepth = 24;  // pending partial sums: the recursion halves n down to 128
constexpr int kAhead = 8;        // groups of eight values whose loads are in flight together

template <bool kSquare>
__device__ __forceinline__ float prepared(float v) {
  return kSquare ? __fmul_rn(v, v) : v;
}

// x[h .. h + 3] of a row; 16-byte load when the row allows it.
__device__ __forceinline__ float4 load_four(const float *__restrict__ row, int h, bool vector_ok) {
  if (vector_ok)
    return __ldcs(reinterpret_cast<const float4 *>(row + h));
  return make_float4(__ldcs(row + h), __ldcs(row + h + 1), __ldcs(row + h + 2), __ldcs(row + h + 3));
}

// The ranges of leaves of the parts a row is shared among (one part: the whole list).
struct RowParts {
  int parts;      // 1, 2, 4, 8 or 16
  int max_count;  // the longest range
  int first[16];
  int count[16];
};

template <bool kSquare, bool kSqrt, bool kShared>
__global__ void __launch_bounds__(kThreads)
row_sum_f32_kernel(const float *__restrict__ x, long long ldx, float *__restrict__ out, int w,
                   const int4 *__restrict__ leaves, const RowParts parts) {
  const int pair = static_cast<int>(threadIdx.x >> 1), q = static_cast<int>(threadIdx.x & 1);
  const int part = kShared ? pair % parts.parts : 0;
  const int rows_per_cta = kShared ? kRowsPerCta / parts.parts : kRowsPerCta;
  // Rows past the end are computed on the last row (and not stored), so that every lane of a warp
  // takes part in the shuffles.
  const long long i = static_cast<long long>(blockIdx.x) * rows_per_cta + (kShared ? pair / parts.parts : pair);
  const bool stored = i < w;
  const float *__restrict__ row = x + (stored ? i : static_cast<long long>(w) - 1) * ldx;
  const bool vector_ok = (ldx & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  const int first_leaf = parts.first[part], leaf_count = parts.count[part];

  float pending[kStackDepth];
  int depth = 0;
#pragma unroll 1
  for (int t = 0; t < parts.max_count; ++t) {
    const bool live = !kShared || t < leaf_count;
    // x: first h, y: length, z: additions once the leaf is done
    const int4 entry = live ? leaves[first_leaf + t] : make_int4(0, 0, 0, 0);
    const int begin = entry.x, full = entry.y & ~7, end = entry.x + entry.y;
    float total = 0.0f;
    if (entry.y < 8) {
      // (Only a row of fewer than eight values has such a leaf; it is the only one.)
      for (int hh = begin; hh < end; ++hh)
        total = __fadd_rn(total, prepared<kSquare>(__ldcs(row + hh)));
    }
    // A shared row: every lane walks two batches (a leaf has at most 16 groups of eight); otherwise as
    // many as this leaf, the same for the whole warp, needs.
    const bool wide = entry.y >= 8;
    float r0 = 0.0f, r1 = 0.0f, r2 = 0.0f, r3 = 0.0f;
    if (wide) {
      const float4 head = load_four(row, begin + 4 * q, vector_ok);
      r0 = prepared<kSquare>(head.x), r1 = prepared<kSquare>(head.y), r2 = prepared<kSquare>(head.z),
      r3 = prepared<kSquare>(head.w);
    }
    const int batches = kShared ? 2 : (full - 8 + 8 * kAhead - 1) / (8 * kAhead);
    int hh = begin + 8;
    for (int batch = 0; batch < batches; ++batch, hh += 8 * kAhead) {
      float4 v[kAhead];
#pragma unroll
      for (int u = 0; u < kAhead; ++u)
        if (hh + 8 * u < begin + full)
          v[u] = load_four(row, hh + 8 * u + 4 * q, vector_ok);
#pragma unroll
      for (int u = 0; u < kAhead; ++u)
        if (hh + 8 * u < begin + full) {
          r0 = __fadd_rn(r0, prepared<kSquare>(v[u].x));
          r1 = __fadd_rn(r1, prepared<kSquare>(v[u].y));
          r2 = __fadd_rn(r2, prepared<kSquare>(v[u].z));
          r3 = __fadd_rn(r3, prepared<kSquare>(v[u].w));
        }
    }
    // Lane 0 of the pair: (r0 + r1) + (r2 + r3); lane 1: (r4 + r5) + (r6 + r7); their sum is the
    // same number on both lanes (addition commutes).
    const float half = __fadd_rn(__fadd_rn(r0, r1), __fadd_rn(r2, r3));
    const float other = __shfl_xor_sync(0xffffffffu, half, 1);
    if (wide) {
      total = __fadd_rn(half, other);
      for (hh = begin + full; hh < end; ++hh)
        total = __fadd_rn(total, prepared<kSquare>(__ldcs(row + hh)));
    }
    if (!live)
      continue;
    // Push, then add the pairs the recursion closes here (left + right). The additions that close
    // pairs reaching beyond this part's range find the stack down to one value and are left to the
    // shuffles below.
    if (depth < kStackDepth)
      pending[depth++] = total;
    for (int a = 0; a < entry.z && depth >= 2; ++a) {
      --depth;
      pending[depth - 1] = __fadd_rn(pending[depth - 1], pending[depth]);
    }
  }
  float value = parts.max_count > 0 ? pending[0] : 0.0f;
  if (kShared) {
    // Neighbouring parts first, as the recursion adds its halves.
    for (int step = 1; step < parts.parts; step <<= 1)
      value = __fadd_rn(value, __shfl_xor_sync(0xffffffffu, value, 2 * step));
  }
  if (!stored || q != 0 || part != 0 || parts.max_count < 1)
    return;
  value = __fadd_rn(value, 0.0f);  // the reduction starts from +0: a sum of -0 becomes +0
  if (kSqrt)
    value = __fsqrt_rn(value);
  out[i] = value;
}

int count_leaves(int n) {
  if (n <= 128)
    return 1;
  int left = n / 2;
  left -= left % 8;
  return count_leaves(left) + count_leaves(n - left);
}

// The ranges of leaves of the 2^depth subtrees at `depth` of the recursion over n values, in order;
// false when a subtree above that depth is a leaf already.
bool list_parts(int n, int depth, int first_leaf, RowParts *parts, int *index) {
  if (depth == 0) {
    parts->first[*index] = first_leaf;
    parts->count[*index] = count_leaves(n);
    ++*index;
    return true;
  }
  if (n <= 128)
    return false;
  int left = n / 2;
  left -= left % 8;
  return list_parts(left, depth - 1, first_leaf, parts, index) &&
         list_parts(n - left, depth - 1, first_leaf + count_leaves(left), parts, index);
}

} // namespace

int row_sum_parts(int h) {
  // As many ranges as the recursion has levels to cut at, up to 16. With as many ranges as leaves a
  // warp reads 16 consecutive leaves (8 KB) at a time whatever the row length, and the results meet
  // in shuffles instead of on the stack; with more leaves than that the ranges are what keeps many
  // lanes busy when the rows are few. Measured on 2^19 rows of 512 values: 5.66 TB/s with one pair per
  // row, 6.68 with four; 8192 rows of 32768: 1.98 against 5.19 TB/s with sixteen.
  int parts = 1, depth = 0;
  while (parts < 16) {
    RowParts probe;
    int index = 0;
    if (!list_parts(h, depth + 1, 0, &probe, &index))
      break;
    parts *= 2;
    ++depth;
  }
  return parts;
}

cudaError_t launch_row_sum_f32(const float *x, long long ldx, float *out, int w, int h, int square, int take_sqrt,
                               const int4 *leaves_dev, int num_leaves, cudaStream_t stream) {
  if (w <= 0 || h <= 0)
    return cudaSuccess;  // a row without values is not stored
  if (h > pairwise_max_h() || leaves_dev == nullptr || num_leaves < 1)
    return cudaErrorInvalidValue;
  RowParts parts;
  parts.parts = row_sum_parts(h);
  // Rows that only allow 4-byte loads (a pitch or base off the 16-byte grid) keep one pair each when
  // there are enough of them to fill the GPU: with four times the load instructions the predicated
  // steps of shared rows cost more than the consecutive leaves give (300000 rows of 1031 values:
  // 3.7 TB/s against 2.2).
  const bool vector_ok = (ldx & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  if (!vector_ok && w >= 65536)
    parts.parts = 1;
  int depth = 0, index = 0;
  while ((1 << depth) < parts.parts)
    ++depth;
  if (!list_parts(h, depth, 0, &parts, &index) || index != parts.parts)
    return cudaErrorInvalidValue;
  parts.max_count = 0;
  int total = 0;
  for (int p = 0; p < parts.parts; ++p) {
    parts.max_count = parts.count[p] > parts.max_count ? parts.count[p] : parts.max_count;
    total += parts.count[p];
  }
  for (int p = parts.parts; p < 16; ++p)
    parts.first[p] = parts.count[p] = 0;
  if (total != num_leaves)
    return cudaErrorInvalidValue;  // the list on the device is not the one of h
  const int rows_per_cta = kRowsPerCta / parts.parts;
  const unsigned grid = static_cast<unsigned>((static_cast<long long>(w) + rows_per_cta - 1) / rows_per_cta);
  const bool shared = parts.parts > 1;
#define HC_ROW_SUM_LAUNCH(SQUARE, SQRT)                                                                      \
  do {                                                                                                       \
    if (shared)                                                                                              \
      row_sum_f32_kernel<SQUARE, SQRT, true><<<grid, kThreads, 0, stream>>>(x, ldx, out, w, leaves_dev, parts);  \
    else                                                                                                     \
      row_sum_f32_kernel<SQUARE, SQRT, false><<<grid, kThreads, 0, stream>>>(x, ldx, out, w, leaves_dev, parts); \
  } while (0)
  if (square && take_sqrt)
    HC_ROW_SUM_LAUNCH(true, true);
  else if (square)
    HC_ROW_SUM_LAUNCH(true, false);
  else if (take_sqrt)
    HC_ROW_SUM_LAUNCH(false, true);
  else
    HC_ROW_SUM_LAUNCH(false, false);
#undef HC_ROW_SUM_LAUNCH
  return cudaGetLastError();
}

} // namespace sm100
} // namespace hc
