// Dense tiled GEMM for sm_100a on CTA pairs: C[M,N] (fp32) = A[M,K] * B[K,N], fp16/bf16 in.
//
// Same contract as gemm_dense_kernel (the hc kernel of
// examples/amdgpu_gfx11_wmma_matmul.py:301-326), larger unit of work: a cluster of two CTAs on
// neighbouring SMs owns a 256x256 tile of C and drives one tcgen05.mma.cta_group::2
// (256x256x16) together.
//
//   CTA r of the pair loads rows [128 r, 128 r + 128) of the A tile and columns
//   [128 r, 128 r + 128) of the B tile into its own shared memory, holds rows
//   [128 r, 128 r + 128) of the accumulator in its own TMEM and writes those rows of C.
//   The instruction, issued by CTA 0, reads both halves of both operands, so each SM fetches
//   32 KiB per 64 of k for 256x256 outputs instead of 48 KiB for 128x256: a third less
//   L2 and shared-memory traffic per flop than the single-CTA kernel. A ring stage holds 128
//   of k (two swizzle-row-wide sub-blocks): 8 MMAs per barrier round trip measured 2.3 % faster
//   than 4.
//
// Synchronisation (mbarriers at identical shared-memory offsets in both CTAs):
//   full[s]       CTA 0 only. One arrival (CTA 0's producer, with expect_tx for both CTAs'
//                 bytes); both producers' TMA loads count their bytes on it.
//   empty[s]      one per CTA. CTA 0's MMA thread commits to its own and to its partner's when the
//                 MMAs that read ring slot s have finished.
//   tmem_full[a]  one per CTA, committed by CTA 0 after the last k-block of a tile.
//   tmem_empty[a] CTA 0 only; one arrival per epilogue warp of either CTA (8 warps per CTA in the
//                 plain instantiation, 4 in the one that reads C).
// No load uses multicast; every CTA fetches its own operand halves.
//
// The epilogue (gemm_epilogue.cuh) stores C by TMA when its base and pitch allow, applies fused
// element-wise operations, writes a float32 or 16-bit C, and, when tiles are split over k, parks
// partial tiles and lets the last unit of a tile add them up.
#include "gemm_epilogue.cuh"
#include "device_checks.cuh"
#include "gemm_launch.h"
#include "sm100_ptx.cuh"

#include <cstdlib>
#include <cstring>
#include <type_traits>

namespace hc {
namespace sm100 {

namespace dense_pair {

constexpr int kTileM = 256;      // per pair
constexpr int kTileN = 256;      // per pair
constexpr int kCtaM = 128;       // rows of A / C per CTA
constexpr int kCtaN = 128;       // columns of B loaded per CTA
#ifndef HC_PAIR_BLOCK_K
#define HC_PAIR_BLOCK_K 128
#endif
constexpr int kBlockK = HC_PAIR_BLOCK_K;  // k extent of one ring stage: 64 or 128
constexpr int kKSub = kBlockK / 64;       // 64-wide (one swizzle row) sub-blocks per stage
constexpr int kUmmaK = 16;
constexpr int kStages = 6 / kKSub;
// Warp 0 loads, warp 1 issues the MMAs, the rest drain accumulators. The plain kernel has eight
// epilogue warps: two per 32-lane quarter of tensor memory, each taking half of the tile's columns,
// so that every scheduler has two of them to interleave (a lone warp per scheduler exposes every
// latency of its chunk loop, which is what bounds shapes with a short k-loop). The kernel that
// reads C in its epilogue needs more registers per thread and keeps four.
constexpr int kMaxEpilogueWarps = 8;
template <bool kReadsC>
struct Roles {
  static constexpr int kEpilogueWarps = 8;
  static constexpr int kThreads = 64 + 32 * kEpilogueWarps;
};
constexpr int kTmemColumns = 512;  // two accumulators of kTileN fp32 columns

constexpr uint32_t kASubBytes = kCtaM * 64 * 2;                   // 128 rows x 64 k: 16 KiB
constexpr uint32_t kATileBytes = kASubBytes * kKSub;
constexpr uint32_t kBBoxBytes = 64 * 64 * 2;                      // 64 columns x 64 k-rows: 8 KiB
constexpr uint32_t kBChunkBytes = kBBoxBytes * kKSub;             // 64 columns x kBlockK k-rows
constexpr uint32_t kBTileBytes = kBChunkBytes * (kCtaN / 64);
constexpr uint32_t kStageBytes = kATileBytes + kBTileBytes;       // 32 KiB per CTA at kBlockK = 64
constexpr uint32_t kEpilogueWarpBytes = 32 * 32 * 4;
constexpr uint32_t kBarrierBytes = 256;
constexpr uint32_t kSmemBytes = kStages * kStageBytes + kMaxEpilogueWarps * kEpilogueWarpBytes +
                                kBarrierBytes + 1024;
static_assert(kSmemBytes <= 227 * 1024, "dynamic shared memory of one CTA");

struct TileCoord {
  int m_blk;
  int n_blk;
};

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

// kReadsC: the epilogue has to read C's previous contents (an accumulating launch whose stores
// cannot do the addition themselves: operations follow it, C's pitch rules out TMA, or there are
// push targets). Every other launch -- the plain product, element-wise operations, accumulation
// by TMA additions -- runs the other instantiation, which never reads C.
template <bool kReadsC>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Roles<kReadsC>::kThreads, 1)
gemm_dense_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                       const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_c, int c_tma,
                       const __grid_constant__ CUtensorMap tmap_partials,
                       const __grid_constant__ PushMaps push_maps, void *c, int m, int n,
                       int k, long long ldc, uint32_t idesc, int tiles_m, int tiles_n, int group_n,
                       int l2_hints, int b_layout, int elem8, Epilogue ep, SplitK split, int *status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - raw_addr);

  const uint32_t epi_base = smem_base + kStages * kStageBytes;
  constexpr int kEpilogueWarps = Roles<kReadsC>::kEpilogueWarps;
  constexpr int kColumnsPerWarp = kTileN * 4 / kEpilogueWarps;  // 4 quarters of lanes share the warps
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
  const uint32_t cta_rank = cluster_cta_rank();  // 0: issues the MMAs, 1: partner

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (uint32_t a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 2 * kEpilogueWarps);
    }
    for (uint32_t w = 0; w < kMaxEpilogueWarps; ++w)
      mbar_init(bar_base + 128u + 8u * w, 1);  // per epilogue warp: arrival of a chunk of C loaded by TMA
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_descriptor(&tmap_a);
    tma_prefetch_descriptor(&tmap_b);
  }
  // Both CTAs' barriers must exist before either CTA signals across the pair.
  cluster_sync_all();
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemColumns);
    tmem_relinquish_alloc_permit_pair();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (k + (kBlockK << elem8) - 1) / (kBlockK << elem8);  // 8-bit: twice the k per stage
  const int cluster_id = static_cast<int>(blockIdx.x >> 1);
  const int num_clusters = static_cast<int>(gridDim.x >> 1);
  // A unit is one tile, or with split-k one range of a tile's k-blocks; the splits of a tile are
  // consecutive units, so they run on neighbouring clusters at the same time.
  const int num_units = split.splits == 1 ? num_tiles
                                          : split.first_split_tile + (num_tiles - split.first_split_tile) * split.splits;
  auto first_kb = [&](int part, int parts) { return static_cast<int>(static_cast<long long>(part) * num_kb / parts); };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer ------
    if (lane == 0) {
      // L2 policy per operand. Default (3): B evict-last, A normal. The group of B tile
      // columns is what every tile row of the group re-reads, so it should outlive the A rows
      // streaming past it; measured +2 % on 8192^3 against no hints (0), while marking A
      // evict-first (1) or both evict-last (2) was no better or worse.
      const uint64_t pol_a = l2_hints == 1 ? l2_policy_evict_first()
                                           : (l2_hints == 2 ? l2_policy_evict_last() : l2_policy_evict_normal());
      const uint64_t pol_b = l2_hints == 0 ? l2_policy_evict_normal() : l2_policy_evict_last();
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int unit = cluster_id; ok && unit < num_units; unit += num_clusters) {
        const DenseUnit u = decode_unit(unit, split);
        const TileCoord tc = tile_coord(u.tile, tiles_m, tiles_n, group_n);
        const int m0 = tc.m_blk * kTileM + static_cast<int>(cta_rank) * kCtaM;
        const int n0 = tc.n_blk * kTileN + static_cast<int>(cta_rank) * kCtaN;
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
          const uint32_t leader_full = map_to_cta(full_bar(stage), 0);
          if (cta_rank == 0)
            mbar_arrive_expect_tx(full_bar(stage), 2 * kStageBytes);
#pragma unroll
          for (int sub = 0; sub < kKSub; ++sub) {
            const int k0 = (kb * kBlockK + sub * 64) << elem8;
            tma_load_2d_pair_hint(a_dst + sub * kASubBytes, &tmap_a, leader_full, k0, m0, pol_a);
            if (b_layout == kBLayoutKN) {
#pragma unroll
              for (int j = 0; j < kCtaN / 64; ++j)
                tma_load_2d_pair_hint(b_dst + j * kBChunkBytes + sub * kBBoxBytes, &tmap_b, leader_full,
                                      n0 + j * 64, k0, pol_b);
            } else {
              // B stored [N, K]: this CTA's 128 rows (n) x 64 k, K-major like A, one box per sub-block.
              tma_load_2d_pair_hint(b_dst + sub * kASubBytes, &tmap_b, leader_full, k0, n0, pol_b);
            }
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (CTA 0) -
    if (lane == 0 && cta_rank == 0) {
      // The instruction kind (16-bit or 8-bit operands) is a template argument of the whole role
      // loop, chosen by one branch here.
      auto mma_role = [&](auto f8) {
        constexpr bool kF8 = decltype(f8)::value;
        uint32_t stage = 0, phase = 0;
        uint32_t iter = 0;
        bool ok = true;
        for (int unit = cluster_id; ok && unit < num_units; unit += num_clusters, ++iter) {
          const DenseUnit u = decode_unit(unit, split);
          const uint32_t acc = iter & 1u;
          const uint32_t acc_phase = (iter >> 1) & 1u;
          if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag))
            break;
          tcgen05_fence_after_sync();
          const uint32_t d_tmem = tmem_base + acc * kTileN;
          const int kb_begin = first_kb(u.part, u.parts), kb_end = first_kb(u.part + 1, u.parts);
          for (int kb = kb_begin; kb < kb_end; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
              ok = false;
              break;
            }
            tcgen05_fence_after_sync();
            const uint32_t a_addr = smem_base + stage * kStageBytes;
            const uint32_t b_addr = a_addr + kATileBytes;
            const bool b_kn = b_layout == kBLayoutKN;
#pragma unroll
            for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
              // A: one 16 KiB sub-block per 64 k, +32 bytes per 16-wide k-step inside its swizzle
              // row. B stored [K, N]: k-rows are contiguous across the stage, +2 KiB per k-step;
              // B stored [N, K]: laid out and advanced exactly like A.
              const uint64_t a_desc = make_smem_desc_sw128(a_addr + (kk / 4) * kASubBytes, 16, 1024) +
                                      static_cast<uint64_t>((kk % 4) * 2);
              const uint64_t b_desc =
                  b_kn ? make_smem_desc_sw128(b_addr, kBChunkBytes, 1024) + static_cast<uint64_t>(kk * 128)
                       : make_smem_desc_sw128(b_addr + (kk / 4) * kASubBytes, 16, 1024) +
                             static_cast<uint64_t>((kk % 4) * 2);
              umma_ss_pair<kF8>(d_tmem, a_desc, b_desc, idesc, (kb != kb_begin || kk != 0) ? 1u : 0u);
            }
            // Hand ring slot `stage` back to both producers.
            umma_commit_pair(map_to_cta(empty_bar(stage), 0));
            umma_commit_pair(map_to_cta(empty_bar(stage), 1));
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (ok) {
            umma_commit_pair(map_to_cta(tmem_full_bar(acc), 0));
            umma_commit_pair(map_to_cta(tmem_full_bar(acc), 1));
          }
        }
      };
      if (elem8)
        mma_role(std::true_type{});
      else
        mma_role(std::false_type{});
    }
  } else {
    // ------------------------------------------------------------ epilogue ----------
    const int quarter = warp & 3;                // the TMEM lanes a warp may read follow warp % 4
    const int column_part = (warp - 2) >> 2;     // which share of the tile's columns it drains
    float *stage_gen = reinterpret_cast<float *>(smem_gen + (epi_base - smem_base) +
                                                 (warp - 2) * kEpilogueWarpBytes);
    const bool vec_ok = ((ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
    const uint32_t c_load_bar = bar_base + 128u + 8u * static_cast<uint32_t>(warp - 2);
    uint32_t c_load_phase = 0;
    uint32_t iter = 0;
    for (int unit = cluster_id; unit < num_units; unit += num_clusters, ++iter) {
      const DenseUnit u = decode_unit(unit, split);
      const TileCoord tc = tile_coord(u.tile, tiles_m, tiles_n, group_n);
      const uint32_t acc = iter & 1u;
      const uint32_t acc_phase = (iter >> 1) & 1u;
      const int row_base = tc.m_blk * kTileM + static_cast<int>(cta_rank) * kCtaM + quarter * 32;
      const int col_base = tc.n_blk * kTileN + column_part * kColumnsPerWarp;
      if (kReadsC || ep.accumulate_by_tma_load)
        prefetch_c_tile_row(static_cast<const float *>(c), ldc, m, n, row_base + lane, col_base, kColumnsPerWarp);
      const bool ready = mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag);
      if (!__all_sync(0xffffffffu, ready))
        break;
      tcgen05_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kTileN +
                             column_part * kColumnsPerWarp;
      if (!HC_CHECK(status, abort_flag, HC_CHECK_TMEM_COLUMNS,
                    acc * kTileN + column_part * kColumnsPerWarp + kColumnsPerWarp <= kTmemColumns) ||
          !HC_CHECK(status, abort_flag, HC_CHECK_OUTPUT_RANGE,
                    row_base >= 0 && row_base < tiles_m * kTileM && col_base >= 0 && col_base < tiles_n * kTileN) ||
          !HC_CHECK(status, abort_flag, HC_CHECK_PARTIAL_SLOT,
                    u.parts == 1 || (u.split_index >= 0 && u.split_tile >= 0 && u.split_index < num_units)))
        break;
      if (u.parts == 1) {
        drain_accumulator_rows<kColumnsPerWarp, kReadsC>(taddr, stage_gen, c, ldc, m, n, row_base, col_base, vec_ok,
                                                        lane, map_to_cta(tmem_empty_bar(acc), 0),
                                                        /*release_remote=*/true, ep, c_tma ? &tmap_c : nullptr,
                                                        c_load_bar, &c_load_phase, abort_flag,
                                                        (c_tma && push_maps.count > 0) ? &push_maps : nullptr);
        continue;
      }
      // Split-k: the partial rows go to this unit's tile of the partials buffer (TMA stores, like
      // C); the warp whose unit completes the tile adds the tiles up.
      constexpr size_t kTileFloats = static_cast<size_t>(kTileM) * kTileN;
      const int tile_row = static_cast<int>(cta_rank) * kCtaM + quarter * 32, tile_col = column_part * kColumnsPerWarp;
      drain_accumulator_rows<kColumnsPerWarp, false>(taddr, stage_gen, nullptr, 0, 0x7fffffff, kTileN,
                                                     u.split_index * kTileM + tile_row, tile_col, true, lane,
                                                     map_to_cta(tmem_empty_bar(acc), 0), /*release_remote=*/true,
                                                     Epilogue{}, &tmap_partials);
      if (lane == 0) {
        tma_store_wait_all();  // the partial rows are in memory before the unit counts itself in
        fence_proxy_async_all();
      }
      unsigned *counter =
          split.counters + (static_cast<size_t>(u.split_tile) * 2 + cta_rank) * kMaxEpilogueWarps + (warp - 2);
      if (split_arrive_is_last(counter, u.parts, lane)) {
        reduce_partials_rows<kColumnsPerWarp, kReadsC>(
            split.partials + static_cast<size_t>(u.split_tile) * u.parts * kTileFloats +
                static_cast<size_t>(tile_row) * kTileN + tile_col,
            kTileN, kTileFloats, u.parts, stage_gen, c, ldc, m, n, row_base, col_base, vec_ok, lane, ep, c_tma ? &tmap_c : nullptr);
        if (lane == 0)
          *counter = 0u;
      }
    }
    if ((c_tma || split.splits > 1) && lane == 0)
      tma_store_wait_all();  // shared memory must outlive the stores that read it
  }

  // Neither CTA may leave (or free TMEM) while its partner can still read its shared memory,
  // write its TMEM or signal its barriers.
  tcgen05_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    if (threadIdx.x == 0)
      atomicCAS(status, 0, kStatusDeviceWaitTimeout);  // (a failed check recorded earlier stays)
    const long long start = clock64();
    while (clock64() - start < 2000000LL) {
    }
  }
  cluster_sync_all();
  tcgen05_fence_after_sync();
  if (warp == 1)
    tmem_dealloc_pair(tmem_base, kTmemColumns);
}

} // namespace dense_pair

cudaError_t launch_gemm_dense_pair(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, void *c,
                                   int m, int n, int k, long long ldc, int dtype, int group_n,
                                   int max_ctas, int b_layout, const Epilogue &ep, const CUtensorMap *tmap_c,
                                   const SplitK &split, const CUtensorMap *tmap_partials, int *status,
                                   cudaStream_t stream, const PushMaps *push_maps) {
  using namespace dense_pair;
  static thread_local int configured_device = -1;
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess)
    return err;
  if (configured_device != device) {
    err = cudaFuncSetAttribute(gemm_dense_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kSmemBytes));
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(gemm_dense_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kSmemBytes));
    if (err != cudaSuccess)
      return err;
    configured_device = device;
  }
  const int tiles_m = (m + kTileM - 1) / kTileM;
  const int tiles_n = (n + kTileN - 1) / kTileN;
  const long long num_tiles = static_cast<long long>(tiles_m) * tiles_n;
  if (num_tiles <= 0 || num_tiles > 0x3fffffffLL)
    return cudaErrorInvalidValue;
  if (split.splits < 1 ||
      (split.splits > 1 && (split.partials == nullptr || split.counters == nullptr || tmap_partials == nullptr)))
    return cudaErrorInvalidValue;
  if (split.splits > 1 && (split.first_split_tile < 0 || split.first_split_tile >= num_tiles))
    return cudaErrorInvalidValue;
  const long long num_units =
      split.splits == 1 ? num_tiles : split.first_split_tile + (num_tiles - split.first_split_tile) * split.splits;
  long long clusters = max_ctas / 2;
  if (clusters < 1)
    clusters = 1;
  if (num_units < clusters)
    clusters = num_units;
  const int elem8 = dtype_is_8bit(dtype) ? 1 : 0;
  if (elem8 && b_layout != kBLayoutNK)
    return cudaErrorInvalidValue;  // 8-bit operands are K-major: the caller transposes a [K, N] B first
  const uint32_t idesc = make_idesc_f16(dtype_format(dtype), /*a_mn_major=*/false,
                                        /*b_mn_major=*/b_layout == kBLayoutKN, kTileM, kTileN);
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
  // With push targets the tiles leave through TMA stores too when the caller supplies the targets'
  // tensor maps and the launch is the plain or element-wise product on whole tiles (an accumulating
  // or split launch keeps the ordinary peer stores: the value the peers need exists in registers
  // only there).
  const bool tma_push = tmap_c != nullptr && push_maps != nullptr && push_maps->count == ep.push_count &&
                        ep.push_count > 0 && ep.accumulate == 0 && split.splits == 1 && ep.c_dtype == kCTypeF32;
  const bool tma_possible = tmap_c != nullptr && (ep.push_count == 0 || tma_push);
  launch_ep.accumulate_by_tma = (tma_possible && ep.accumulate != 0 && ep.op_count == 0) ? 1 : 0;
  launch_ep.accumulate_by_tma_load =
      (tma_possible && ep.accumulate != 0 && ep.op_count != 0 && split.splits == 1) ? 1 : 0;
  const bool reads_c =
      ep.accumulate != 0 && launch_ep.accumulate_by_tma == 0 && launch_ep.accumulate_by_tma_load == 0;
  const int c_tma = (tma_possible && !reads_c) ? 1 : 0;
  const CUtensorMap c_map = c_tma ? *tmap_c : tmap_a;  // unused unless c_tma
  const CUtensorMap p_map = split.splits > 1 ? *tmap_partials : tmap_a;  // unused unless split
  PushMaps no_push;
  no_push.count = 0;
  const PushMaps &push_arg = tma_push ? *push_maps : no_push;
  int l2_hints = 3;
  if (const char *h = std::getenv("HC_CUDA_L2_HINTS"))  // tuning aid
    l2_hints = std::atoi(h);
  const unsigned grid = static_cast<unsigned>(clusters * 2);
  if (reads_c)
    gemm_dense_pair_kernel<true><<<grid, Roles<true>::kThreads, kSmemBytes, stream>>>(
        tmap_a, tmap_b, c_map, c_tma, p_map, push_arg, c, m, n, k, ldc, idesc, tiles_m, tiles_n, group_n, l2_hints, b_layout, elem8, launch_ep, split, status);
  else
    gemm_dense_pair_kernel<false><<<grid, Roles<false>::kThreads, kSmemBytes, stream>>>(
        tmap_a, tmap_b, c_map, c_tma, p_map, push_arg, c, m, n, k, ldc, idesc, tiles_m, tiles_n, group_n, l2_hints, b_layout, elem8, launch_ep, split, status);
  return cudaGetLastError();
}

int dense_block_k(bool pairs) { return pairs ? dense_pair::kBlockK : dense_tile_shape().block_k; }

bool dense_uses_pairs(long long m, long long n, long long k, int sm_count, bool pushes) {
  // HC_CUDA_DENSE_MODE=single|pair forces a mode (tuning aid).
  if (const char *mode = std::getenv("HC_CUDA_DENSE_MODE")) {
    if (std::strcmp(mode, "single") == 0)
      return false;
    if (std::strcmp(mode, "pair") == 0)
      return true;
  }
  if (m <= 128 || sm_count < 2)
    return false;
  // Compare the number of tile rounds each mode needs; a 256x256 pair tile takes about as long
  // as a 128x256 single tile does on one SM, and moves a third less data per flop.
  const long long single_tiles = ((m + 127) / 128) * ((n + 255) / 256);
  const long long pair_tiles = ((m + 255) / 256) * ((n + 255) / 256);
  // One round of single CTAs with a k-loop of moderate length: a launch of thread-block clusters
  // costs 2-3 us more than one of plain CTAs, which the pairs' smaller operand traffic only earns
  // back over a long k (2048^3: 20.5 us on single CTAs against 22.5 on pairs; 2048 x 2048 x 256: 10.3
  // against 13.3; 512 x 8192 x 8192: 64 against 61).
  const char *forced_wide = std::getenv("HC_CUDA_DENSE_WIDE");  // tuning aid: "1" forces the 512x256 pair tiles
  if (single_tiles <= sm_count && k <= 4096 && !pushes &&
      !(forced_wide != nullptr && std::strcmp(forced_wide, "1") == 0))
    return false;
  const long long single_rounds = (single_tiles + sm_count - 1) / sm_count;
  const long long pair_rounds = (pair_tiles + sm_count / 2 - 1) / (sm_count / 2);
  return pair_rounds * 9 <= single_rounds * 10;
}

} // namespace sm100
} // namespace hc
