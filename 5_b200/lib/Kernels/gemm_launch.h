// Host-side launch interface of the sm_100a kernels. The C-ABI layer (lib/CAPI/Cuda.cpp)
// is the only caller; it owns argument validation, tensor-map encoding and scratch memory.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

namespace hc {
namespace sm100 {

// How B is stored: [K, N] row-major (the hc kernel's Buffer[K, N]) or [N, K] row-major (B
// transposed, Buffer[N, K]). The matching tensor map is {n inner, k} with 64x64 boxes, or
// {k inner, n} with a 64 x (CTA's rows of n) box.
constexpr int kBLayoutKN = 0;
constexpr int kBLayoutNK = 1;

constexpr int kDTypeF16 = 0;
constexpr int kDTypeBF16 = 1;
constexpr int kDTypeF8E4M3 = 2;  // float8 e4m3fn
constexpr int kDTypeF8E5M2 = 3;  // float8 e5m2
// 8-bit operands run through tcgen05.mma.kind::f8f6f4 and must be K-major (A as [M, K], B as
// [N, K]); the tiles are the same in bytes, so a ring stage holds twice as many k as for 16 bits.
inline bool dtype_is_8bit(int dtype) { return dtype == kDTypeF8E4M3 || dtype == kDTypeF8E5M2; }
inline int dtype_bytes(int dtype) { return dtype_is_8bit(dtype) ? 1 : 2; }
// The A/B format field of the instruction descriptor (see make_idesc_f16).
inline unsigned dtype_format(int dtype) { return (dtype == kDTypeBF16 || dtype == kDTypeF8E5M2) ? 1u : 0u; }
constexpr int kCTypeF32 = 0;
constexpr int kCTypeF16 = 1;
constexpr int kCTypeBF16 = 2;

// Value a kernel writes to the status word when one of its bounded waits ran out.
constexpr int kStatusDeviceWaitTimeout = 5;
constexpr int kStatusCheckFailed = 6;  // checked build: low byte; the number of the check above it

// Additional destinations of a dense GEMM's output: every tile of C is also stored, at the same
// row/column offsets and with the same pitch, to each of these matrices. Used to push a rank's
// column slab of C straight into its peers' memory over NVLink while later tiles are still being
// computed (plain peer stores; nothing is ever loaded from a peer).
constexpr int kMaxPushTargets = 7;

// The push targets as tensor maps (same extents, pitch and 32 x 32 float32 box as C's own map): with
// them the epilogue hands every staged chunk of a tile to the TMA store engine once per
// destination -- C and each peer's copy -- instead of writing the peers' copies with 16-byte stores
// from the warp. Stores only: nothing is loaded from a peer, and no multicast is involved.
struct PushMaps {
  CUtensorMap map[kMaxPushTargets];
  int count;
};

// Element-wise work fused into the store of C. With `accumulate` the previous contents of C are
// the starting value of the sum (the hc kernel that loads its accumulators from `c` before the
// k-loop); `ops` then run in order on every element, mirroring the element-wise statements an
// hc kernel applies to its accumulators between the k-loop and the store. The value that
// reaches C is also what goes to the push targets.
constexpr int kMaxEpilogueOps = 4;
constexpr int kEpilogueScale = 1;       // v = v * value
constexpr int kEpilogueAdd = 2;         // v = v + value
constexpr int kEpilogueMax = 3;         // v = max(v, value)
constexpr int kEpilogueMin = 4;         // v = min(v, value)
constexpr int kEpilogueBiasColumn = 5;  // v = v + bias[column]
struct Epilogue {
  float *push[kMaxPushTargets];
  int push_count;
  int accumulate;
  int op_count;
  int op_kind[kMaxEpilogueOps];
  float op_value[kMaxEpilogueOps];
  const float *bias;
  // Element type of C: 0 float32, 1 float16, 2 bfloat16 (the float32 value rounded to nearest
  // even). 16-bit output is written by the kernels that do not read C.
  int c_dtype;
  // Set by the dense launchers: accumulate by letting the TMA stores add to C (possible when the
  // stores go through TMA and no operation follows the accumulation), so C is never read.
  int accumulate_by_tma;
  // Set by the dense launchers: an accumulation that operations follow, into a C that TMA can
  // address: each chunk of C's previous contents comes in by a TMA load, is added in registers,
  // the operations run, and the chunk leaves by a TMA store.
  int accumulate_by_tma_load;
};

// Splitting dense tiles over k. Tiles [0, first_split_tile) are computed whole; each later tile
// is computed by `splits` units, each over its own range of k-blocks. That covers both a product
// with too few tiles for the GPU (first_split_tile = 0) and the last, partly filled round of a
// larger one (first_split_tile = the tiles of the full rounds), whose tiles would otherwise keep
// most CTAs waiting for a few. A split unit writes its fp32 partial tile to `partials`
// ([split tile][split][tile rows][tile columns]) and counts itself in on `counters` (one word per
// split tile, CTA of the pair and epilogue warp; zero on entry, zero again on exit). The unit that
// arrives last adds the partial tiles in split order -- so the result does not depend on which
// unit that is -- and stores C through the usual epilogue. No unit waits for another.
// The units write their partial tiles with TMA stores: `tmap_partials` (launch argument) is the
// partials buffer as a 2-D fp32 tensor {256 (inner), split units x tile rows}, box {32, 32},
// 128-byte swizzle.
struct SplitK {
  int splits;            // 1: nothing is split
  int first_split_tile;  // tiles before this one are whole
  float *partials;
  unsigned *counters;
};
// What to split for `tiles` tiles on `slots` CTAs (or CTA pairs) and `num_kb` k-blocks: returns the
// number of splits and sets *first_split_tile.
int dense_choose_splits(long long tiles, int slots, int num_kb, long long *first_split_tile);
size_t dense_partials_bytes(long long split_tiles, int splits, bool pairs);
size_t dense_counters_bytes(long long split_tiles);
int dense_block_k(bool pairs);  // k extent of one ring stage of the chosen dense kernel

struct DenseTileShape {
  int block_m, block_n, block_k, stages;
  unsigned smem_bytes;
};
DenseTileShape dense_tile_shape();

// C[m,n] = A * B through the TMA + tcgen05 persistent kernel.
//   tmap_a: A as a 2-D tensor {k (inner), m}, box {64, 128}, 128-byte swizzle.
//   tmap_b: B as a 2-D tensor {n (inner), k}, box {64, 64},  128-byte swizzle.
//   tmap_c: C as a 2-D tensor {n (inner), m}, 128-byte swizzle -- float32 with box {32, 32}, or for
//           a 16-bit C (ep.c_dtype) its element type with box {64, 32} -- or null. When
//           given (C's base and pitch are 16-byte aligned) and the launch is the plain product
//           without push targets, the tiles of C leave through TMA stores.
cudaError_t launch_gemm_dense(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, void *c,
                              int m, int n, int k, long long ldc, int dtype, int group_n,
                              int max_ctas, int b_layout, const Epilogue &ep, const CUtensorMap *tmap_c,
                              const SplitK &split, const CUtensorMap *tmap_partials, int *status,
                                   cudaStream_t stream, int block_n = 256);
// `block_n`: 256, or 128 (dense_narrow_block_n) for tiles of 128 x 128 -- never split over k; tmap_b of a
// B stored [N, K] then has boxes of 128 rows. dense_uses_narrow: whether the 256-wide tiles (or CTA pairs)
// of an m x n product with a short k would keep at most a quarter of the SMs busy while 128-wide tiles fit
// one round; such a product is not split over k.
int dense_narrow_block_n();
bool dense_uses_narrow(long long m, long long n, long long k, int sm_count, bool pairs);

// Few tiles, long k: every 128x256 tile is shared by `groups` thread-block clusters of `cluster_size`
// CTAs (2, 4, 8 or 16), each CTA a range of the k-blocks; the partial tiles are summed through
// distributed shared memory inside a cluster and, with groups > 1, through `partials`
// (dense_cluster_partials_bytes) and `counters` (dense_cluster_counters_bytes, zeroed once; the
// kernel leaves them zero) between clusters -- always in ascending-k order. Takes launch_gemm_dense's
// tensor maps for A and B and a float32 C that TMA can address; `tmap_c` has boxes of 32 columns x
// dense_cluster_store_rows(cluster_size) rows. No push targets.
cudaError_t launch_gemm_dense_cluster(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, const CUtensorMap &tmap_c,
                                      int m, int n, int k, int dtype, int cluster_size, int groups, float *partials,
                                      unsigned *counters, int b_layout, const Epilogue &ep, int *status,
                                      cudaStream_t stream);
int dense_cluster_store_rows(int cluster_size);
size_t dense_cluster_partials_bytes(long long tiles, int groups);
size_t dense_cluster_counters_bytes(long long tiles);
// Clusters of that size that the current device runs at once (0: the size is not available).
int dense_cluster_capacity(int cluster_size);
// The form planned for a product on a device with `sm_count` SMs, from a model of how many clusters
// of each size such a device runs at once (needs no device); cluster_size 0: do not use clusters.
// `elem_bytes`: 2 or 1.
struct ClusterPlan {
  int cluster_size;
  int groups;
};
ClusterPlan dense_cluster_choose(long long m, long long n, long long k, int elem_bytes, int sm_count);

// Same product on CTA pairs: clusters of two CTAs own 256x256 tiles and issue
// tcgen05.mma.cta_group::2. Takes the same tensor maps as launch_gemm_dense. `max_ctas` is
// rounded down to an even number of CTAs.
cudaError_t launch_gemm_dense_pair(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, void *c,
                                   int m, int n, int k, long long ldc, int dtype, int group_n,
                                   int max_ctas, int b_layout, const Epilogue &ep, const CUtensorMap *tmap_c,
                                   const SplitK &split, const CUtensorMap *tmap_partials, int *status,
                                   cudaStream_t stream, const PushMaps *push_maps = nullptr);

// The pair kernel's big brother: 512x256 tiles per pair (a 256x256 accumulator per CTA, all of its
// tensor memory), a quarter fewer operand bytes per flop, no overlap of epilogue and next k-loop.
// For launches whose epilogue never reads C with ordinary loads (stores, element-wise work, 16-bit
// C, accumulation by TMA additions), without split-k and without push targets.
cudaError_t launch_gemm_dense_wide(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, void *c, int m, int n,
                                   int k, long long ldc, int dtype, int group_n, int max_ctas, int b_layout,
                                   const Epilogue &ep, const CUtensorMap *tmap_c, int *status, cudaStream_t stream);
// Whether a product of this shape is large enough for the 512x256 tiles to pay.
bool dense_uses_wide(long long m, long long n, long long k, int sm_count);
constexpr int kDenseWideTileM = 512;

// Whether the dense variant runs on CTA pairs for this problem.
bool dense_uses_pairs(long long m, long long n, long long k, int sm_count, bool pushes = false);
// (`pushes`: the launch also stores its tiles to peers. Such a product keeps the pairs' tile shape when
// it fits one round of single CTAs too: its split decision, and with it the bits of C, then stay those
// of the product without peers.)

struct SkinnyShape {
  int block_n;     // columns of C per work unit
  int block_k;
  int max_m;       // largest M the skinny kernel accepts
  int stages;
  unsigned smem_bytes;
};
SkinnyShape skinny_shape(int m);

// Number of k-splits the skinny kernel would use for this problem on `sm_count` SMs.
int skinny_choose_splits(int n, int k, int sm_count);

// Ring stages a skinny launch of `grid` CTAs uses on a device with `sm_count` SMs: the deep ring
// (all of an SM's shared memory) when no two CTAs share an SM, the shallow one otherwise.
int skinny_ring_stages(int m, int grid, int sm_count);

// Scratch the skinny kernel needs for `splits` > 1: partial sums then arrival counters.
size_t skinny_partials_bytes(int m, int n, int splits);
size_t skinny_counters_bytes(int n);

// C[m,n] = A * B for m <= 64: streams B once, split over k, partial sums reduced in a
// fixed order by the last work unit to finish each block of columns.
//   tmap_a: A as {k (inner), m}, box {64, padded m}; tmap_b as for the dense kernel.
//   partials / counters: scratch (ignored when splits == 1); counters must be zero on
//   entry and are zero again on exit. `max_ctas` caps the grid (two per SM); `sm_count` decides
//   the ring depth (skinny_ring_stages).
cudaError_t launch_gemm_skinny(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, void *c,
                               int m, int n, int k, long long ldc, int dtype, int splits,
                               float *partials, unsigned *counters, int max_ctas, int sm_count,
                               int b_layout, const Epilogue &ep, int *status, cudaStream_t stream);

// Pairwise distances out[i, j] = [sqrt] sum_h (x1[i, h] - x2[j, h])^2 in float32, the sum in the order
// of NumPy's float32 sum. `leaves_dev`: pairwise_schedule(h, ...) copied to the device.
cudaError_t launch_pairwise_f32(const float *x1, long long ld1, const float *x2, long long ld2, float *out,
                                long long ldo, int w1, int w2, int h, int take_sqrt, const int4 *leaves_dev,
                                int num_leaves, cudaStream_t stream);
// Row sums out[i] = [sqrt] sum_h x[i, h] [squared] in float32, the sum in the order of NumPy's float32
// sum (np.sum of the row, starting from +0). `leaves_dev`: pairwise_schedule(h, ...) on the device.
// A row of more than 128 values is shared among row_sum_parts(h) lane pairs (2 to 16) of one warp.
cudaError_t launch_row_sum_f32(const float *x, long long ldx, float *out, int w, int h, int square, int take_sqrt,
                               const int4 *leaves_dev, int num_leaves, cudaStream_t stream);
int row_sum_parts(int h);
// The leaves of NumPy's pairwise summation of h values: {first, length, additions of pending partial
// sums once the leaf is done, 0}. Returns their number (which may exceed `capacity`; nothing is
// written past it).
int pairwise_schedule(int h, int4 *leaves, int capacity);
int pairwise_max_h();

// Small products on the float32 pipes, one small CTA per 16x16 tile, bit-identical to the reference
// simulator (products and sums rounded one by one, k ascending): any pitch and alignment, 16-bit
// operands, every member of the family except push targets. `tiny_takes`: whether the AUTO variant
// hands a product to it (m, n <= 64 and a k-loop staged in one go).
cudaError_t launch_gemm_tiny(const void *a, long long lda, const void *b, long long ldb, void *c, long long ldc, int m,
                             int n, int k, int dtype, int b_layout, const Epilogue &ep, cudaStream_t stream);
bool tiny_takes(long long m, long long n, long long k, int dtype, int sm_count);
int tiny_tile();

// k == 0 with fused element-wise work: C = ops(accumulate ? C : 0), no product to add.
cudaError_t launch_epilogue_only(void *c, int m, int n, long long ldc, const Epilogue &ep,
                                 cudaStream_t stream);

// Launches one thread that waits `budget_cycles` (clamped to [1e3, 2e8]) on a barrier nobody
// signals and then reports kStatusDeviceWaitTimeout through `status`, like a GEMM kernel whose
// wait ran out.
cudaError_t launch_wait_selftest(long long budget_cycles, int *status, cudaStream_t stream);
// Checked build only: one thread checks an index that is made up to be out of range, does not make
// the access and reports the failed check through `status`. cudaErrorNotSupported otherwise.
cudaError_t launch_check_selftest(int *status, cudaStream_t stream);
bool library_is_checked();

// 8-bit operands: copies a rows x cols matrix of bytes (pitch src_ld) to dst with pitch dst_ld
// (a multiple of 16), transposed when `transpose` is set (dst is then cols x rows). This is how a
// float8 B stored [K, N] becomes the K-major [N, K] operand, and how odd pitches are aligned.
cudaError_t launch_repack_bytes(const void *src, long long src_ld, void *dst, long long dst_ld, int rows,
                                int cols, bool transpose, cudaStream_t stream);

// Copies rows x cols matrices of 16-bit elements into buffers whose row pitch is a multiple of 8
// elements (16 bytes), as TMA requires; columns [cols, round_up(cols, 8)) of a destination are
// zeroed. Two copies in one launch (either may be empty: rows or cols 0).
cudaError_t launch_repack_pitch_two(const void *src0, long long src0_ld, void *dst0, long long dst0_ld,
                                    int rows0, int cols0, const void *src1, long long src1_ld, void *dst1,
                                    long long dst1_ld, int rows1, int cols1, cudaStream_t stream);

// ---- the masked element-wise map (one-dimensional load / compute / store kernels) --------------
// out[i] = ops(x[i] [, y[i]]) for i in [0, n), float32: at most kMaxMapOps operations applied in
// order, each with a float32 constant or with the element of the second input.
constexpr int kMaxMapOps = 8;
constexpr int kMapScale = 1;            // v = v * value
constexpr int kMapAdd = 2;              // v = v + value
constexpr int kMapMax = 3;              // v = maximum(v, value)   (NumPy's: NaN propagates; ties give the second operand)
constexpr int kMapMin = 4;              // v = minimum(v, value)
constexpr int kMapReverseSub = 5;       // v = value - v
constexpr int kMapAddOther = 6;         // v = v + y[i]
constexpr int kMapSubOther = 7;         // v = v - y[i]
constexpr int kMapReverseSubOther = 8;  // v = y[i] - v
constexpr int kMapMulOther = 9;         // v = v * y[i]
constexpr int kMapMaxOther = 10;        // v = maximum(v, y[i])
constexpr int kMapMinOther = 11;        // v = minimum(v, y[i])
// maximum / minimum with the operands the other way round. NumPy returns the second operand when
// neither is greater (two zeros of opposite sign), so the order is observable.
constexpr int kMapReverseMax = 12;       // v = maximum(value, v)
constexpr int kMapReverseMin = 13;       // v = minimum(value, v)
constexpr int kMapReverseMaxOther = 14;  // v = maximum(y[i], v)
constexpr int kMapReverseMinOther = 15;  // v = minimum(y[i], v)
inline bool map_op_uses_other(int kind) {
  return (kind >= kMapAddOther && kind <= kMapMinOther) || kind == kMapReverseMaxOther || kind == kMapReverseMinOther;
}
struct MapOps {
  int count;
  int kind[kMaxMapOps];
  float value[kMaxMapOps];
};
// CTAs of the map kernel for n elements on `sm_count` SMs (a persistent grid, eight CTAs per SM).
int map_grid(long long n, int sm_count);
// y may be null when no operation uses the second input. x, y, out: 4-byte aligned; 16-byte
// alignment of all of them selects the 128-bit path.
cudaError_t launch_map_f32(const float *x, const float *y, float *out, long long n, const MapOps &ops,
                           int sm_count, cudaStream_t stream);

} // namespace sm100
} // namespace hc
