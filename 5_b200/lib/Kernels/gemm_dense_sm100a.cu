// Dense tiled GEMM for sm_100a:  C[M,N] (fp32) = A[M,K] * B[K,N], A and B fp16 or bf16,
// all row-major, fp32 accumulation.
//
// This is the B200 replacement for the work that the hc example kernel
// `tiled_gfx11_wmma_matmul` (examples/amdgpu_gfx11_wmma_matmul.py:301-326) describes as a
// grid of 16x16x16 WMMA tiles: zero-initialised accumulator, k-loop of masked tile loads
// (out-of-range elements read as 0), one multiply-accumulate per k-step, masked store.
// Here one CTA owns a 128x256 tile of C:
//
//   warp 0   : TMA producer. Per k-block of 64 it loads one 128x64 box of A (K-major) and
//              four 64x64 boxes of B (N-major) into a 4-deep ring of 128-byte-swizzled
//              shared-memory stages; out-of-range rows/columns/k are zero-filled by TMA.
//   warp 1   : allocates TMEM and issues tcgen05.mma (128x256x16, fp32 accumulate in
//              TMEM); tcgen05.commit hands each ring slot back to the producer.
//   warps 2..: epilogue (eight warps, two per quarter of the TMEM lanes; four in the
//              instantiation that reads C). tcgen05.ld the finished accumulator (two
//              accumulators of 256 columns alternate, so this overlaps the next tile's main
//              loop), stage it in shared memory and store C by TMA, or, when C's pitch rules
//              that out, with coalesced 128-bit stores predicated on the matrix edge.
//
// The kernel is persistent: CTA b processes tiles b, b+grid, ... in an order that walks
// groups of `group_n` tile columns so that concurrently running CTAs share A and B
// through L2.
#include "gemm_epilogue.cuh"
#include "device_checks.cuh"
#include "gemm_launch.h"
#include "sm100_ptx.cuh"

#include <cstdlib>
#include <type_traits>

namespace hc {
namespace sm100 {

namespace dense {

constexpr int kBlockM = 128;
constexpr int kWideBlockN = 256;    // the tile width the planner counts with
constexpr int kNarrowBlockN = 128;  // for products whose 256-wide tiles would leave most SMs idle
constexpr int kBlockK = 64;  // 64 x 2 bytes = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kStages = 4;  // of the 256-wide tiles; the 128-wide ones have five (see Tile)
// Warp 0 loads, warp 1 issues the MMAs, the rest drain accumulators: eight warps in the plain
// kernel (two per quarter of tensor-memory lanes, each half of the tile's columns), four in the
// one that reads C in its epilogue, which needs more registers per thread.
constexpr int kMaxEpilogueWarps = 8;
template <bool kReadsC>
struct Roles {
  static constexpr int kEpilogueWarps = 8;
  static constexpr int kThreads = 64 + 32 * kEpilogueWarps;
};
constexpr uint32_t kATileBytes = kBlockM * kBlockK * 2;            // 16 KiB
constexpr uint32_t kBChunkBytes = 64 * kBlockK * 2;                // 64 columns x 64 k-rows
constexpr uint32_t kEpilogueWarpBytes = 32 * 32 * 4;               // one 32x32 fp32 block
constexpr uint32_t kBarrierBytes = 256;

// What follows from the tile width: 256 columns -- 48 KiB per stage, four stages, all 512 columns of
// tensor memory for the two accumulators; 128 columns -- 32 KiB per stage, five stages (the
// barriers of a sixth would not fit below the per-warp ones), 256 columns of tensor memory.
template <int kBlockN>
struct Tile {
  static constexpr int kStages = kBlockN == kWideBlockN ? dense::kStages : 5;
  static constexpr int kTmemColumns = 2 * kBlockN;  // two fp32 accumulators
  static constexpr uint32_t kBTileBytes = kBChunkBytes * (kBlockN / 64);
  static constexpr uint32_t kStageBytes = kATileBytes + kBTileBytes;
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + kMaxEpilogueWarps * kEpilogueWarpBytes +
                                         kBarrierBytes + 1024 /* alignment slack */;
  static_assert(8 * (2 * kStages + 4) + 8 <= 128, "ring and accumulator barriers end below the per-warp barriers");
};
constexpr uint32_t kSmemBytes = Tile<kWideBlockN>::kSmemBytes;

struct TileCoord {
  int m_blk;
  int n_blk;
};

// Tiles are numbered so that `group_n` neighbouring tile columns are walked row by row
// before moving on: the CTAs running at any moment then cover a compact rectangle of C.
__device__ __forceinline__ TileCoord tile_coord(int tile, int tiles_m, int tiles_n, int group_n) {
  const int tiles_per_group = group_n * tiles_m;
  const int group = tile / tiles_per_group;
  const int first_n = group * group_n;
  const int width = min(group_n, tiles_n - first_n);
  const int in_group = tile - group * tiles_per_group;
  TileCoord tc;
  tc.m_blk = in_group / width;
  tc.n_blk = first_n + in_group % width;
  return tc;
}

// kReadsC: the epilogue has to read C's previous contents (see gemm_dense_pair_kernel).
template <bool kReadsC, int kBlockN>
__global__ void __launch_bounds__(Roles<kReadsC>::kThreads, 1)
gemm_dense_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_c, int c_tma,
                       const __grid_constant__ CUtensorMap tmap_partials, void *c, int m, int n,
                  int k, long long ldc, uint32_t idesc, int tiles_m, int tiles_n, int group_n,
                  int b_layout, int elem8, Epilogue ep, SplitK split, int *status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;  // swizzled tiles need 1 KiB alignment
  uint8_t *smem_gen = smem_raw + (smem_base - raw_addr);
  constexpr int kStages = Tile<kBlockN>::kStages;
  constexpr int kTmemColumns = Tile<kBlockN>::kTmemColumns;
  constexpr uint32_t kStageBytes = Tile<kBlockN>::kStageBytes;

  const uint32_t epi_base = smem_base + kStages * kStageBytes;
  constexpr int kEpilogueWarps = Roles<kReadsC>::kEpilogueWarps;
  constexpr int kColumnsPerWarp = kBlockN * 4 / kEpilogueWarps;
  const uint32_t bar_base = epi_base + kMaxEpilogueWarps * kEpilogueWarpBytes;
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](uint32_t a) { return bar_base + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](uint32_t a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  const uint32_t misc_off = (bar_base - smem_base) + 8u * (2 * kStages + 4);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + misc_off);
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem_gen + misc_off + 4);

  const int warp = static_cast<int>(threadIdx.x >> 5);
  const int lane = static_cast<int>(threadIdx.x & 31);

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (uint32_t a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), kEpilogueWarps);
    }
    for (uint32_t w = 0; w < kMaxEpilogueWarps; ++w)
      mbar_init(bar_base + 128u + 8u * w, 1);  // per epilogue warp: arrival of a chunk of C loaded by TMA
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_descriptor(&tmap_a);
    tma_prefetch_descriptor(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemColumns);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (k + (kBlockK << elem8) - 1) / (kBlockK << elem8);  // 8-bit: twice the k per stage
  // A unit is one tile, or with split-k one range of a tile's k-blocks; the splits of a tile are
  // consecutive units, so they run on neighbouring CTAs at the same time.
  const int num_units = split.splits == 1 ? num_tiles
                                          : split.first_split_tile + (num_tiles - split.first_split_tile) * split.splits;
  auto first_kb = [&](int part, int parts) { return static_cast<int>(static_cast<long long>(part) * num_kb / parts); };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer ------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; ok && unit < num_units; unit += gridDim.x) {
        const DenseUnit u = decode_unit(unit, split);
        const TileCoord tc = tile_coord(u.tile, tiles_m, tiles_n, group_n);
        const int m0 = tc.m_blk * kBlockM;
        const int n0 = tc.n_blk * kBlockN;
        const int kb_end = first_kb(u.part + 1, u.parts);
        if (!HC_CHECK(status, abort_flag, HC_CHECK_TILE_COORDINATES,
                      tc.m_blk >= 0 && tc.m_blk < tiles_m && tc.n_blk >= 0 && tc.n_blk < tiles_n) ||
            !HC_CHECK(status, abort_flag, HC_CHECK_K_BLOCKS,
                      u.part >= 0 && u.part < u.parts && first_kb(u.part, u.parts) >= 0 && kb_end <= num_kb))
          break;
        for (int kb = first_kb(u.part, u.parts); kb < kb_end; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          if (!HC_CHECK(status, abort_flag, HC_CHECK_RING_STAGE,
                        stage < kStages && smem_base + (stage + 1) * kStageBytes <= epi_base) ||
              !HC_CHECK(status, abort_flag, HC_CHECK_TMA_COORDINATES,
                        m0 >= 0 && n0 >= 0 && kb >= 0 && ((n0 * 2) & 15) == 0 &&
                            ((((kb * kBlockK) << elem8) * (elem8 ? 1 : 2)) & 15) == 0)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kATileBytes;
          mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
          tma_load_2d(a_dst, &tmap_a, full_bar(stage), (kb * kBlockK) << elem8, m0);
          if (b_layout == kBLayoutKN) {
#pragma unroll
            for (int j = 0; j < kBlockN / 64; ++j)
              tma_load_2d(b_dst + j * kBChunkBytes, &tmap_b, full_bar(stage), n0 + j * 64, kb * kBlockK);
          } else {
            // B stored [N, K]: one box of kBlockN rows (n) x 64 k, K-major like A.
            tma_load_2d(b_dst, &tmap_b, full_bar(stage), (kb * kBlockK) << elem8, n0);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer --------
    if (lane == 0) {
      // The instruction kind (16-bit or 8-bit operands) is a template argument of the whole role
      // loop, chosen by one branch here.
      auto mma_role = [&](auto f8) {
        constexpr bool kF8 = decltype(f8)::value;
        uint32_t stage = 0, phase = 0;
        uint32_t iter = 0;
        bool ok = true;
        for (int unit = blockIdx.x; ok && unit < num_units; unit += gridDim.x, ++iter) {
          const DenseUnit u = decode_unit(unit, split);
          const uint32_t acc = iter & 1u;
          const uint32_t acc_phase = (iter >> 1) & 1u;
          if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag))
            break;
          tcgen05_fence_after_sync();
          const uint32_t d_tmem = tmem_base + acc * kBlockN;
          const int kb_begin = first_kb(u.part, u.parts), kb_end = first_kb(u.part + 1, u.parts);
          for (int kb = kb_begin; kb < kb_end; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
              ok = false;
              break;
            }
            tcgen05_fence_after_sync();
            const uint32_t a_addr = smem_base + stage * kStageBytes;
            const uint32_t b_addr = a_addr + kATileBytes;
            // A: K-major, groups of 8 rows are 1024 bytes apart.
            const uint64_t a_desc = make_smem_desc_sw128(a_addr, 16, 1024);
            // B stored [K, N]: N-major, 64-column chunks are kBChunkBytes apart, groups of 8 k-rows
            // 1024. B stored [N, K]: K-major exactly like A.
            const bool b_kn = b_layout == kBLayoutKN;
            const uint64_t b_desc = b_kn ? make_smem_desc_sw128(b_addr, kBChunkBytes, 1024)
                                         : make_smem_desc_sw128(b_addr, 16, 1024);
            const uint64_t b_step = b_kn ? 128 : 2;  // descriptor units (16 bytes) per 16-wide k-step
#pragma unroll
            for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
              // Per 16-wide k-step: A advances 32 bytes inside the swizzle row, B advances
              // two groups of 8 k-rows (2048 bytes); both in 16-byte descriptor units.
              umma_ss<kF8>(d_tmem, a_desc + static_cast<uint64_t>(kk * 2), b_desc + static_cast<uint64_t>(kk) * b_step,
                           idesc, (kb != kb_begin || kk != 0) ? 1u : 0u);
            }
            umma_commit(empty_bar(stage));
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (ok)
            umma_commit(tmem_full_bar(acc));
        }
      };
      if (elem8)
        mma_role(std::true_type{});
      else
        mma_role(std::false_type{});
    }
  } else {
    // ------------------------------------------------------------ epilogue ----------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const int column_part = (warp - 2) >> 2;  // which share of the tile's columns this warp drains
    const uint32_t stage_smem = epi_base + (warp - 2) * kEpilogueWarpBytes;
    float *stage_gen = reinterpret_cast<float *>(smem_gen + (stage_smem - smem_base));
    const bool vec_ok = ((ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
    const uint32_t c_load_bar = bar_base + 128u + 8u * static_cast<uint32_t>(warp - 2);
    uint32_t c_load_phase = 0;
    uint32_t iter = 0;
    for (int unit = blockIdx.x; unit < num_units; unit += gridDim.x, ++iter) {
      const DenseUnit u = decode_unit(unit, split);
      const TileCoord tc = tile_coord(u.tile, tiles_m, tiles_n, group_n);
      const uint32_t acc = iter & 1u;
      const uint32_t acc_phase = (iter >> 1) & 1u;
      const int row_base = tc.m_blk * kBlockM + quarter * 32;
      const int col_base = tc.n_blk * kBlockN + column_part * kColumnsPerWarp;
      if (kReadsC || ep.accumulate_by_tma_load)
        prefetch_c_tile_row(static_cast<const float *>(c), ldc, m, n, row_base + lane, col_base, kColumnsPerWarp);
      const bool ready = mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag);
      if (!__all_sync(0xffffffffu, ready))
        break;
      tcgen05_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kBlockN +
                             column_part * kColumnsPerWarp;
      if (!HC_CHECK(status, abort_flag, HC_CHECK_TMEM_COLUMNS,
                    acc * kBlockN + column_part * kColumnsPerWarp + kColumnsPerWarp <= kTmemColumns) ||
          !HC_CHECK(status, abort_flag, HC_CHECK_OUTPUT_RANGE,
                    row_base >= 0 && row_base < tiles_m * kBlockM && col_base >= 0 && col_base < tiles_n * kBlockN) ||
          !HC_CHECK(status, abort_flag, HC_CHECK_PARTIAL_SLOT,
                    u.parts == 1 || (u.split_index >= 0 && u.split_tile >= 0 && u.split_index < num_units)))
        break;
      if (u.parts == 1) {
        drain_accumulator_rows<kColumnsPerWarp, kReadsC>(taddr, stage_gen, c, ldc, m, n, row_base, col_base, vec_ok,
                                                        lane, tmem_empty_bar(acc), /*release_remote=*/false, ep,
                                                        c_tma ? &tmap_c : nullptr, c_load_bar, &c_load_phase,
                                                        abort_flag);
        continue;
      }
      // Split-k: the partial rows go to this unit's tile of the partials buffer (TMA stores, like
      // C); the warp whose unit completes the tile adds the tiles up.
      constexpr size_t kTileFloats = static_cast<size_t>(kBlockM) * kBlockN;
      const int tile_row = quarter * 32, tile_col = column_part * kColumnsPerWarp;
      drain_accumulator_rows<kColumnsPerWarp, false>(taddr, stage_gen, nullptr, 0, 0x7fffffff, kBlockN,
                                                     u.split_index * kBlockM + tile_row, tile_col, true, lane,
                                                     tmem_empty_bar(acc), /*release_remote=*/false, Epilogue{},
                                                     &tmap_partials);
      if (lane == 0) {
        tma_store_wait_all();  // the partial rows are in memory before the unit counts itself in
        fence_proxy_async_all();
      }
      unsigned *counter = split.counters + static_cast<size_t>(u.split_tile) * (2 * kMaxEpilogueWarps) + (warp - 2);
      if (split_arrive_is_last(counter, u.parts, lane)) {
        reduce_partials_rows<kColumnsPerWarp, kReadsC>(
            split.partials + static_cast<size_t>(u.split_tile) * u.parts * kTileFloats +
                static_cast<size_t>(tile_row) * kBlockN + tile_col,
            kBlockN, kTileFloats, u.parts, stage_gen, c, ldc, m, n, row_base, col_base, vec_ok, lane, ep, c_tma ? &tmap_c : nullptr);
        if (lane == 0)
          *counter = 0u;
      }
    }
    if ((c_tma || split.splits > 1) && lane == 0)
      tma_store_wait_all();  // shared memory must outlive the stores that read it
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  if (*abort_flag != 0) {
    // A wait ran out. Record it, then give copies that may still be in flight time to
    // land before the shared memory and TMEM of this CTA are released.
    if (threadIdx.x == 0)
      atomicCAS(status, 0, kStatusDeviceWaitTimeout);  // (a failed check recorded earlier stays)
    const long long start = clock64();
    while (clock64() - start < 2000000LL) {
    }
    __syncthreads();
  }
  if (warp == 1)
    tmem_dealloc(tmem_base, kTmemColumns);
}

} // namespace dense

cudaError_t launch_gemm_dense(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, void *c,
                              int m, int n, int k, long long ldc, int dtype, int group_n,
                              int max_ctas, int b_layout, const Epilogue &ep, const CUtensorMap *tmap_c,
                              const SplitK &split, const CUtensorMap *tmap_partials, int *status,
                                   cudaStream_t stream, int block_n) {
  using namespace dense;
  if (block_n != kWideBlockN && block_n != kNarrowBlockN)
    return cudaErrorInvalidValue;
  const bool narrow = block_n == kNarrowBlockN;
  if (narrow && split.splits != 1)
    return cudaErrorInvalidValue;  // the partial tiles are laid out for 256-wide tiles
  static thread_local int configured_device = -1;
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess)
    return err;
  if (configured_device != device) {
    err = cudaFuncSetAttribute(gemm_dense_kernel<false, kWideBlockN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(Tile<kWideBlockN>::kSmemBytes));
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(gemm_dense_kernel<true, kWideBlockN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(Tile<kWideBlockN>::kSmemBytes));
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(gemm_dense_kernel<false, kNarrowBlockN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(Tile<kNarrowBlockN>::kSmemBytes));
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(gemm_dense_kernel<true, kNarrowBlockN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(Tile<kNarrowBlockN>::kSmemBytes));
    if (err != cudaSuccess)
      return err;
    configured_device = device;
  }
  const int tiles_m = (m + kBlockM - 1) / kBlockM;
  const int tiles_n = (n + block_n - 1) / block_n;
  const long long num_tiles = static_cast<long long>(tiles_m) * tiles_n;
  if (num_tiles <= 0 || num_tiles > 0x7fffffffLL)
    return cudaErrorInvalidValue;
  if (split.splits < 1 ||
      (split.splits > 1 && (split.partials == nullptr || split.counters == nullptr || tmap_partials == nullptr)))
    return cudaErrorInvalidValue;
  if (split.splits > 1 && (split.first_split_tile < 0 || split.first_split_tile >= num_tiles))
    return cudaErrorInvalidValue;
  const long long num_units =
      split.splits == 1 ? num_tiles : split.first_split_tile + (num_tiles - split.first_split_tile) * split.splits;
  const int grid = static_cast<int>(num_units < max_ctas ? num_units : max_ctas);
  const int elem8 = dtype_is_8bit(dtype) ? 1 : 0;
  if (elem8 && b_layout != kBLayoutNK)
    return cudaErrorInvalidValue;  // 8-bit operands are K-major: the caller transposes a [K, N] B first
  const uint32_t idesc = make_idesc_f16(dtype_format(dtype), /*a_mn_major=*/false,
                                        /*b_mn_major=*/b_layout == kBLayoutKN, kBlockM, block_n);
  if (group_n < 1)
    group_n = 1;
  // C leaves through TMA stores when it is aligned (tmap_c) and goes nowhere else. Element-wise work
  // runs in registers before the store; an accumulation that nothing follows is performed by the
  // stores themselves as additions; one that operations follow loads its chunks of C by TMA. Only
  // what is left (odd pitch, push targets, accumulation with operations in a launch split over k)
  // reads C with ordinary loads, in the other instantiation.
  if (ep.c_dtype != kCTypeF32 && (ep.accumulate != 0 || ep.push_count != 0))
    return cudaErrorInvalidValue;  // rejected with a message by the caller's validation
  Epilogue launch_ep = ep;
  const bool tma_possible = tmap_c != nullptr && ep.push_count == 0;
  launch_ep.accumulate_by_tma = (tma_possible && ep.accumulate != 0 && ep.op_count == 0) ? 1 : 0;
  launch_ep.accumulate_by_tma_load =
      (tma_possible && ep.accumulate != 0 && ep.op_count != 0 && split.splits == 1) ? 1 : 0;
  const bool reads_c =
      ep.accumulate != 0 && launch_ep.accumulate_by_tma == 0 && launch_ep.accumulate_by_tma_load == 0;
  const int c_tma = (tma_possible && !reads_c) ? 1 : 0;
  const CUtensorMap c_map = c_tma ? *tmap_c : tmap_a;  // unused unless c_tma
  const CUtensorMap p_map = split.splits > 1 ? *tmap_partials : tmap_a;  // unused unless split
#define HC_DENSE_LAUNCH(READS_C, BLOCK_N)                                                                       \
  gemm_dense_kernel<READS_C, BLOCK_N><<<grid, Roles<READS_C>::kThreads, Tile<BLOCK_N>::kSmemBytes, stream>>>(      \
      tmap_a, tmap_b, c_map, c_tma, p_map, c, m, n, k, ldc, idesc, tiles_m, tiles_n, group_n, b_layout, elem8,  \
      launch_ep, split, status)
  if (reads_c && narrow)
    HC_DENSE_LAUNCH(true, kNarrowBlockN);
  else if (reads_c)
    HC_DENSE_LAUNCH(true, kWideBlockN);
  else if (narrow)
    HC_DENSE_LAUNCH(false, kNarrowBlockN);
  else
    HC_DENSE_LAUNCH(false, kWideBlockN);
#undef HC_DENSE_LAUNCH
  return cudaGetLastError();
}

int dense_choose_splits(long long tiles, int slots, int num_kb, long long *first_split_tile) {
  *first_split_tile = 0;
  if (tiles < 1 || slots < 1 || num_kb < 16)
    return 1;
  // The tiles that do not fill a round of the persistent CTAs: all of them when there are fewer
  // tiles than CTAs, else the remainder after the full rounds. Splitting them is worth it only when
  // at least half of the CTAs (or pairs) would idle meanwhile; every split keeps at least eight
  // k-blocks, so that the k-loop it shortens outweighs the partial tile it adds.
  const long long full_rounds = tiles / slots;
  const long long rest = tiles - full_rounds * slots;
  if (rest == 0 || rest * 2 > slots)
    return 1;
  // After full rounds the split only shortens the last round, by at most half a tile's k-loop,
  // while its partial tiles cost about 10-15 us (measured): it pays from k of about 8192 on.
  if (full_rounds > 0 && num_kb < 64)
    return 1;
  long long splits = slots / rest;
  if (splits > num_kb / 8)
    splits = num_kb / 8;
  if (splits > 32)
    splits = 32;
  if (splits < 2)
    return 1;
  *first_split_tile = full_rounds * slots;
  return static_cast<int>(splits);
}

size_t dense_partials_bytes(long long split_tiles, int splits, bool pairs) {
  if (splits <= 1)
    return 0;
  const size_t tile_floats = static_cast<size_t>(pairs ? 2 * dense::kBlockM : dense::kBlockM) * dense::kWideBlockN;
  return static_cast<size_t>(split_tiles) * splits * tile_floats * sizeof(float);
}

size_t dense_counters_bytes(long long split_tiles) {
  return static_cast<size_t>(split_tiles) * 2 * dense::kMaxEpilogueWarps * sizeof(unsigned);
}

int dense_narrow_block_n() { return dense::kNarrowBlockN; }

bool dense_uses_narrow(long long m, long long n, long long k, int sm_count, bool pairs) {
  if (const char *forced = std::getenv("HC_CUDA_DENSE_NARROW"))  // tuning aid: "1" always, "0" never
    return std::atoi(forced) != 0;
  if (sm_count < 1)
    return false;
  // Only when the 256-wide tiles (on CTA pairs: their 256 x 256) would keep at most a quarter of the
  // SMs busy, the 128 x 128 tiles fit one round and k is short: twice the CTAs then work for a little
  // over half as long each, and no partial tiles have to be added up (1024^3: 12.3 us against 14.4 on
  // 32 CTAs or split over k; 768^3: 10.8 against 12.3). A 128 x 128 tile needs half as many flops per
  // operand byte again as a 128 x 256 one, and what an SM receives of its operands is bounded (1536^3,
  // 144 tiles: a 32 KiB ring stage per CTA every 0.8 us, 16.3 us in all, against 14.6 us for 72 tiles
  // split in two over k), so larger products stay on the wide tiles (2560^3: 45 against 37 us).
  const long long rows = (m + dense::kBlockM - 1) / dense::kBlockM;
  const long long wide_ctas = pairs ? 2 * ((m + 2 * dense::kBlockM - 1) / (2 * dense::kBlockM)) * ((n + 255) / 256)
                                    : rows * ((n + 255) / 256);
  const long long narrow_tiles = rows * ((n + 127) / 128);
  return 4 * wide_ctas <= sm_count && narrow_tiles <= sm_count && narrow_tiles > wide_ctas && k <= 2048;
}

DenseTileShape dense_tile_shape() {
  DenseTileShape s;
  s.block_m = dense::kBlockM;
  s.block_n = dense::kWideBlockN;
  s.block_k = dense::kBlockK;
  s.stages = dense::kStages;
  s.smem_bytes = dense::kSmemBytes;
  return s;
}

} // namespace sm100
} // namespace hc
