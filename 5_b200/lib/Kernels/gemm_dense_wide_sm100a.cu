// Dense tiled GEMM for sm_100a on CTA pairs with 512x256 tiles: C[M,N] = A[M,K] * B[K,N], fp32
// accumulation in tensor memory, for products large enough to fill the GPU with such tiles.
//
// Same contract as the other dense kernels (the hc kernel of
// examples/amdgpu_gfx11_wmma_matmul.py:301-326). What differs from gemm_dense_pair_kernel is how
// much of C a pair owns: 512 rows x 256 columns, i.e. a 256 x 256 accumulator per CTA that fills
// all 512 columns of its tensor memory. Per 64 of k each CTA then fetches two 128-row boxes of A
// and its 128 columns of B, 48 KiB for 2 x (128 x 256 x 64) multiply-accumulates, where the
// 256x256 pair tile fetches 32 KiB for half as many: a quarter fewer bytes through L2 and shared
// memory per flop. On a part whose clocks are set by its power cap the energy of moving operands is
// what limits a large product, so this is worth giving up the overlap of one tile's epilogue with
// the next tile's k-loop (there is no second accumulator to compute into): the MMA issuer of the
// next tile starts on each 256-column half as soon as the epilogue has drained that half, and the
// producer keeps the shared-memory ring full across the tile boundary.
//
//   CTA r of the pair loads rows [128 r, +128) and [256 + 128 r, +128) of the A tile and columns
//   [128 r, +128) of the B tile. Two tcgen05.mma.cta_group::2 (256 x 256 x 16) per 16 of k, issued
//   by CTA 0: half h multiplies the h-th A boxes of both CTAs with the whole B tile into tensor
//   memory columns [256 h, +256) of both CTAs; CTA r ends up with rows [256 h + 128 r, +128).
//
// Barriers as in gemm_dense_pair_kernel (full[s] on CTA 0 with both CTAs' bytes, empty[s] per CTA,
// tmem_full[h] per CTA, tmem_empty[h] on CTA 0 with one arrival per epilogue warp of either CTA),
// here with h = accumulator half instead of accumulator buffer. No load uses multicast. Every wait
// is bounded. The launcher uses this kernel only for launches whose epilogue never reads C with
// ordinary loads and that are neither split over k nor pushed to peers; everything else runs
// gemm_dense_pair_kernel.
#include "gemm_epilogue.cuh"
#include "device_checks.cuh"
#include "gemm_launch.h"
#include "sm100_ptx.cuh"

#include <cstdlib>
#include <cstring>
#include <type_traits>

namespace hc {
namespace sm100 {

namespace dense_wide {

constexpr int kTileM = 512;      // per pair
constexpr int kTileN = 256;      // per pair
constexpr int kHalfM = 256;      // rows of one accumulator half (one MMA) per pair
constexpr int kCtaM = 128;       // rows of one A box / one accumulator half per CTA
constexpr int kCtaN = 128;       // columns of B loaded per CTA
constexpr int kBlockK = 64;      // k extent of one ring stage (one 128-byte swizzle row at 16 bits)
constexpr int kUmmaK = 16;
constexpr int kStages = 4;
constexpr int kEpilogueWarps = 8;  // two per 32-lane quarter of tensor memory
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kTmemColumns = 512;  // two halves of kTileN fp32 columns

constexpr uint32_t kABoxBytes = kCtaM * 64 * 2;                   // 128 rows x 64 k: 16 KiB
constexpr uint32_t kATileBytes = 2 * kABoxBytes;                  // both halves
constexpr uint32_t kBBoxBytes = 64 * 64 * 2;                      // 64 columns x 64 k-rows: 8 KiB
constexpr uint32_t kBTileBytes = kBBoxBytes * (kCtaN / 64);       // 16 KiB
constexpr uint32_t kStageBytes = kATileBytes + kBTileBytes;       // 48 KiB per CTA
constexpr uint32_t kEpilogueWarpBytes = 32 * 32 * 4;
constexpr uint32_t kBarrierBytes = 256;
constexpr uint32_t kSmemBytes = kStages * kStageBytes + kEpilogueWarps * kEpilogueWarpBytes + kBarrierBytes + 1024;
static_assert(kSmemBytes <= 227 * 1024, "dynamic shared memory of one CTA");

struct TileCoord {
  int m_blk;
  int n_blk;
};

// Groups of `group_n` tile columns walked row by row, as in the other dense kernels.
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

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_dense_wide_kernel(const __grid_constant__ CUtensorMap tmap_a,
                       const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_c, int c_tma, void *c, int m, int n,
                       int k, long long ldc, uint32_t idesc, int tiles_m, int tiles_n, int group_n,
                       int l2_hints, int b_layout, int elem8, Epilogue ep, int *status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - raw_addr);

  const uint32_t epi_base = smem_base + kStages * kStageBytes;
  constexpr int kColumnsPerWarp = kTileN * 4 / kEpilogueWarps;  // 128: 4 quarters of lanes share the warps
  const uint32_t bar_base = epi_base + kEpilogueWarps * kEpilogueWarpBytes;
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](uint32_t h) { return bar_base + 8u * (2 * kStages + h); };
  auto tmem_empty_bar = [&](uint32_t h) { return bar_base + 8u * (2 * kStages + 2 + h); };
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
    for (uint32_t h = 0; h < 2; ++h) {
      mbar_init(tmem_full_bar(h), 1);
      mbar_init(tmem_empty_bar(h), 2 * kEpilogueWarps);
    }
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer ------
    if (lane == 0) {
      const uint64_t pol_a = l2_hints == 1 ? l2_policy_evict_first()
                                           : (l2_hints == 2 ? l2_policy_evict_last() : l2_policy_evict_normal());
      const uint64_t pol_b = l2_hints == 0 ? l2_policy_evict_normal() : l2_policy_evict_last();
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters) {
        const TileCoord tc = tile_coord(tile, tiles_m, tiles_n, group_n);
        const int m0 = tc.m_blk * kTileM + static_cast<int>(cta_rank) * kCtaM;
        const int n0 = tc.n_blk * kTileN + static_cast<int>(cta_rank) * kCtaN;
        if (!HC_CHECK(status, abort_flag, HC_CHECK_TILE_COORDINATES,
                      tc.m_blk >= 0 && tc.m_blk < tiles_m && tc.n_blk >= 0 && tc.n_blk < tiles_n))
          break;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          if (!HC_CHECK(status, abort_flag, HC_CHECK_RING_STAGE,
                        stage < kStages && smem_base + (stage + 1) * kStageBytes <= epi_base) ||
              !HC_CHECK(status, abort_flag, HC_CHECK_TMA_COORDINATES,
                        m0 >= 0 && n0 >= 0 && ((n0 * 2) & 15) == 0 &&
                            ((((kb * kBlockK) << elem8) * (elem8 ? 1 : 2)) & 15) == 0)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kATileBytes;
          const uint32_t leader_full = map_to_cta(full_bar(stage), 0);
          if (cta_rank == 0)
            mbar_arrive_expect_tx(full_bar(stage), 2 * kStageBytes);
          const int k0 = (kb * kBlockK) << elem8;
          tma_load_2d_pair_hint(a_dst, &tmap_a, leader_full, k0, m0, pol_a);
          tma_load_2d_pair_hint(a_dst + kABoxBytes, &tmap_a, leader_full, k0, m0 + kHalfM, pol_a);
          if (b_layout == kBLayoutKN) {
#pragma unroll
            for (int j = 0; j < kCtaN / 64; ++j)
              tma_load_2d_pair_hint(b_dst + j * kBBoxBytes, &tmap_b, leader_full, n0 + j * 64, k0, pol_b);
          } else {
            // B stored [N, K]: this CTA's 128 rows (n) x 64 k, K-major like A, one box.
            tma_load_2d_pair_hint(b_dst, &tmap_b, leader_full, k0, n0, pol_b);
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
        const bool b_kn = b_layout == kBLayoutKN;
        for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters, ++iter) {
          const uint32_t acc_phase = iter & 1u;  // each tile uses each half once
          for (int kb = 0; ok && kb < num_kb; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
              ok = false;
              break;
            }
            tcgen05_fence_after_sync();
            const uint32_t a_addr = smem_base + stage * kStageBytes;
            const uint32_t b_addr = a_addr + kATileBytes;
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h) {
              if (kb == 0) {
                // The half must have been drained by the previous tile's epilogue.
                if (!mbar_wait(tmem_empty_bar(h), acc_phase ^ 1u, abort_flag)) {
                  ok = false;
                  break;
                }
                tcgen05_fence_after_sync();
              }
#pragma unroll
              for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
                // A: +32 bytes per k-step inside the swizzle row. B stored [K, N]: 64-column chunks
                // 8 KiB apart, +2 KiB per k-step; stored [N, K]: laid out and advanced like A.
                const uint64_t a_desc =
                    make_smem_desc_sw128(a_addr + h * kABoxBytes, 16, 1024) + static_cast<uint64_t>(kk * 2);
                const uint64_t b_desc = b_kn ? make_smem_desc_sw128(b_addr, kBBoxBytes, 1024) + static_cast<uint64_t>(kk * 128)
                                             : make_smem_desc_sw128(b_addr, 16, 1024) + static_cast<uint64_t>(kk * 2);
                umma_ss_pair<kF8>(tmem_base + h * kTileN, a_desc, b_desc, idesc, (kb != 0 || kk != 0) ? 1u : 0u);
              }
              if (kb == num_kb - 1) {
                umma_commit_pair(map_to_cta(tmem_full_bar(h), 0));
                umma_commit_pair(map_to_cta(tmem_full_bar(h), 1));
              }
            }
            if (!ok)
              break;
            // Hand ring slot `stage` back to both producers.
            umma_commit_pair(map_to_cta(empty_bar(stage), 0));
            umma_commit_pair(map_to_cta(empty_bar(stage), 1));
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
            }
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
    const int column_part = (warp - 2) >> 2;     // which half of the tile's columns it drains
    float *stage_gen = reinterpret_cast<float *>(smem_gen + (epi_base - smem_base) + (warp - 2) * kEpilogueWarpBytes);
    const bool vec_ok = ((ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
    uint32_t iter = 0;
    bool ok = true;
    for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters, ++iter) {
      const TileCoord tc = tile_coord(tile, tiles_m, tiles_n, group_n);
      const uint32_t acc_phase = iter & 1u;
      const int col_base = tc.n_blk * kTileN + column_part * kColumnsPerWarp;
#pragma unroll 1
      for (uint32_t h = 0; h < 2; ++h) {
        const bool ready = mbar_wait(tmem_full_bar(h), acc_phase, abort_flag);
        if (!__all_sync(0xffffffffu, ready)) {
          ok = false;
          break;
        }
        tcgen05_fence_after_sync();
        const int row_base = tc.m_blk * kTileM + static_cast<int>(h) * kHalfM + static_cast<int>(cta_rank) * kCtaM +
                             quarter * 32;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + h * kTileN +
                               column_part * kColumnsPerWarp;
        if (!HC_CHECK(status, abort_flag, HC_CHECK_TMEM_COLUMNS,
                      h * kTileN + column_part * kColumnsPerWarp + kColumnsPerWarp <= kTmemColumns) ||
            !HC_CHECK(status, abort_flag, HC_CHECK_OUTPUT_RANGE,
                      row_base >= 0 && row_base < tiles_m * kTileM && col_base >= 0 && col_base < tiles_n * kTileN)) {
          ok = false;
          break;
        }
        drain_accumulator_rows<kColumnsPerWarp, false>(taddr, stage_gen, c, ldc, m, n, row_base, col_base, vec_ok, lane,
                                                       map_to_cta(tmem_empty_bar(h), 0), /*release_remote=*/true, ep,
                                                       c_tma ? &tmap_c : nullptr);
      }
    }
    if (c_tma && lane == 0)
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

} // namespace dense_wide

bool dense_uses_wide(long long m, long long n, long long k, int sm_count) {
  // HC_CUDA_DENSE_WIDE=0|1 forces the choice (tuning aid).
  if (const char *mode = std::getenv("HC_CUDA_DENSE_WIDE")) {
    if (std::strcmp(mode, "0") == 0)
      return false;
    if (std::strcmp(mode, "1") == 0)
      return m > dense_wide::kHalfM && sm_count >= 2;
  }
  // The epilogue of a tile is not hidden behind the next tile's k-loop here, so the k-loop has to
  // be long for the saved operand traffic to outweigh it.
  if (sm_count < 2 || m < 2 * dense_wide::kTileM || k < 4096)
    return false;
  // Worth it when the 512x256 tiles still fill the GPU for several rounds and the tile
  // quantisation does not cost more rounds' worth of time than the 256x256 tiles would.
  const long long slots = sm_count / 2;
  const long long wide_tiles = ((m + 511) / 512) * ((n + 255) / 256);
  const long long pair_tiles = ((m + 255) / 256) * ((n + 255) / 256);
  const long long wide_rounds = (wide_tiles + slots - 1) / slots;
  const long long pair_rounds = (pair_tiles + slots - 1) / slots;
  return wide_rounds >= 3 && wide_rounds * 2 * 100 <= pair_rounds * 103;
}

cudaError_t launch_gemm_dense_wide(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, void *c, int m, int n,
                                   int k, long long ldc, int dtype, int group_n, int max_ctas, int b_layout,
                                   const Epilogue &ep, const CUtensorMap *tmap_c, int *status, cudaStream_t stream) {
  using namespace dense_wide;
  static thread_local int configured_device = -1;
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess)
    return err;
  if (configured_device != device) {
    err = cudaFuncSetAttribute(gemm_dense_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
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
  // What this kernel's epilogue can do: stores (TMA or ordinary), element-wise work in registers, a
  // 16-bit C, accumulation performed by the TMA stores. Anything that has to read C is the pair
  // kernel's.
  const bool tma_possible = tmap_c != nullptr && ep.push_count == 0;
  if (ep.push_count != 0 || (ep.accumulate != 0 && !(tma_possible && ep.op_count == 0)))
    return cudaErrorInvalidValue;
  if (ep.c_dtype != kCTypeF32 && ep.accumulate != 0)
    return cudaErrorInvalidValue;
  const int elem8 = dtype_is_8bit(dtype) ? 1 : 0;
  if (elem8 && b_layout != kBLayoutNK)
    return cudaErrorInvalidValue;  // 8-bit operands are K-major: the caller transposes a [K, N] B first
  long long clusters = max_ctas / 2;
  if (clusters < 1)
    clusters = 1;
  if (num_tiles < clusters)
    clusters = num_tiles;
  const uint32_t idesc = make_idesc_f16(dtype_format(dtype), /*a_mn_major=*/false,
                                        /*b_mn_major=*/b_layout == kBLayoutKN, kHalfM, kTileN);
  if (group_n < 1)
    group_n = 1;
  Epilogue launch_ep = ep;
  launch_ep.accumulate_by_tma = (tma_possible && ep.accumulate != 0) ? 1 : 0;
  launch_ep.accumulate_by_tma_load = 0;
  const int c_tma = tma_possible ? 1 : 0;
  const CUtensorMap c_map = c_tma ? *tmap_c : tmap_a;  // unused unless c_tma
  int l2_hints = 3;
  if (const char *h = std::getenv("HC_CUDA_L2_HINTS"))  // tuning aid
    l2_hints = std::atoi(h);
  const unsigned grid = static_cast<unsigned>(clusters * 2);
  gemm_dense_wide_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tmap_a, tmap_b, c_map, c_tma, c, m, n, k, ldc, idesc,
                                                                 tiles_m, tiles_n, group_n, l2_hints, b_layout, elem8,
                                                                 launch_ep, status);
  return cudaGetLastError();
}

} // namespace sm100
} // namespace hc
