// Dense GEMM for products with few tiles and a long k: each 128x256 tile of C is shared by the CTAs
// of one or several thread-block clusters, every CTA takes a range of the tile's k-blocks, and the
// partial tiles are added through distributed shared memory.
//
// A product like 256 x 256 x 32768 has two 128x256 tiles: one CTA per tile leaves 146 SMs idle, and
// an SM that streams operands from memory it has not touched before pulls only about 50 GB/s, so
// the k-loop has to be spread over as many SMs as possible. Splitting k over independent CTAs that
// meet through partial tiles in global memory keeps the SMs busy but ends in one unit reading every
// partial tile by itself. Here the S CTAs of a cluster (S = 2, 4, 8 or 16) take consecutive ranges of
// k-blocks; each runs the usual pipeline (TMA producer warp -> ring of swizzled stages ->
// tcgen05.mma into tensor memory) and then
//
//   1. drains its accumulator into its own shared memory, over the ring stages that the finished
//      k-loop no longer needs, as 32 blocks of 32x32 floats in the layout of a swizzled TMA box;
//   2. after a cluster barrier, sums the blocks it owns (block b belongs to CTA b mod S) over all S
//      CTAs in rank order -- which is ascending k, so the result does not depend on timing -- reading
//      the other CTAs' copies with ld.shared::cluster. The sum is element-wise and keeps the layout;
//      the CTA's eight epilogue warps share its blocks by groups of rows;
//   3. applies the element-wise operations in that layout and stores the rows by TMA (or adds them
//      to C by TMA, or loads C's previous contents by TMA first).
//
// The hardware schedules the CTAs of a cluster together, so the barrier between 1 and 2 cannot wait
// for a CTA that is not running. When a tile is shared by G > 1 clusters (more SMs than one cluster
// can hold), each cluster writes its sums to a partial tile in global memory and counts itself in
// per group of rows; the warp that arrives last adds the G partial sums in cluster (= k) order and
// does step 3. That reduction reads G x 128 KiB / S per CTA instead of one CTA reading everything,
// and nothing ever waits for another cluster.
// Needs a float32 C that TMA can address (16-byte aligned base and pitch) and no push targets; the
// caller keeps the counter-based split of the persistent kernels otherwise.
#include "gemm_epilogue.cuh"
#include "device_checks.cuh"
#include "gemm_launch.h"
#include "sm100_ptx.cuh"

#include <cstdio>
#include <cstdlib>
#include <type_traits>

namespace hc {
namespace sm100 {

namespace dense_cluster {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;
constexpr int kUmmaK = 16;
constexpr int kStages = 4;
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kTmemColumns = 256;  // one fp32 accumulator of kBlockN columns
constexpr int kBlocks = (kBlockM / 32) * (kBlockN / 32);  // 32x32 blocks of a tile

constexpr uint32_t kATileBytes = kBlockM * kBlockK * 2;
constexpr uint32_t kBChunkBytes = 64 * kBlockK * 2;
constexpr uint32_t kBTileBytes = kBChunkBytes * (kBlockN / 64);
constexpr uint32_t kStageBytes = kATileBytes + kBTileBytes;  // 48 KiB
constexpr uint32_t kBlockBytes = 32 * 32 * 4;                // one 32x32 fp32 block
constexpr uint32_t kPartialBytes = kBlocks * kBlockBytes;    // 128 KiB, laid over the ring
static_assert(kPartialBytes <= kStages * kStageBytes, "the partial tile reuses the ring stages");
constexpr uint32_t kBarrierBytes = 256;
constexpr uint32_t kSmemBytes = kStages * kStageBytes + kEpilogueWarps * kBlockBytes + kBarrierBytes + 1024;

constexpr int kCountersPerTile = kBlocks * 4;  // one per group of rows a warp can own

struct ReduceArgs {
  uint32_t smem_base;  // of the partial tile (the same address in every CTA of the cluster)
  uint32_t ranks;
  int groups, group;   // clusters that share the tile, and which one this is
  float *partials;     // this tile's `groups` partial tiles in global memory (groups > 1)
  unsigned *counters;  // this tile's arrival counters
  float *stage;        // the warp's staging block
  uint32_t c_load_bar;
  volatile uint32_t *abort_flag;
  int m, n, lane;
};

// One group of 4 * kVectors rows of a 32x32 block: summed over the cluster's CTAs (and over the
// tile's clusters), finished and stored. A lane holds kVectors 16-byte pieces; piece i sits
// 512 i + 16 lane bytes into the rows, which is row 4 i + lane / 8 at stored position lane % 8,
// i.e. columns 4 q .. 4 q + 3 with q = (lane % 8) ^ (row % 8) -- the 128-byte swizzle of a TMA box.
template <int kVectors>
__device__ __forceinline__ void reduce_rows(const ReduceArgs &ra, int block, int first_row, int row_base, int col_base,
                                            uint32_t &c_load_phase, const CUtensorMap &tmap_c, const Epilogue &ep) {
  constexpr int kBatch = 16 / kVectors;  // CTAs read at once: sixteen 16-byte loads in flight per lane
  const int lane = ra.lane;
  const uint32_t offset = static_cast<uint32_t>(block) * kBlockBytes + static_cast<uint32_t>(first_row) * 128u +
                          static_cast<uint32_t>(lane) * 16u;
  float4 sum[kVectors];
#pragma unroll
  for (int i = 0; i < kVectors; ++i)
    sum[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 1
  for (uint32_t s0 = 0; s0 < ra.ranks; s0 += kBatch) {
    float4 part[kBatch][kVectors];
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const uint32_t remote = map_to_cta(ra.smem_base + offset, min(s0 + b, ra.ranks - 1));
#pragma unroll
      for (int i = 0; i < kVectors; ++i)
        part[b][i] = ld_shared_cluster_f4(remote + static_cast<uint32_t>(i) * 512u);
    }
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      if (s0 + b < ra.ranks) {
#pragma unroll
        for (int i = 0; i < kVectors; ++i) {
          sum[i].x += part[b][i].x; sum[i].y += part[b][i].y; sum[i].z += part[b][i].z; sum[i].w += part[b][i].w;
        }
      }
    }
  }
  if (ra.groups > 1) {
    // This cluster's sums go to its partial tile; the warp that completes the count adds all of them.
    constexpr size_t kTileFloats = kPartialBytes / 4;
    const size_t at = offset / 4;
    float *mine = ra.partials + static_cast<size_t>(ra.group) * kTileFloats + at;
#pragma unroll
    for (int i = 0; i < kVectors; ++i)
      __stcg(reinterpret_cast<float4 *>(mine + i * 128), sum[i]);
    unsigned *counter = ra.counters + block * 4 + first_row / 8;
    if (!split_arrive_is_last(counter, ra.groups, lane))
      return;
#pragma unroll
    for (int i = 0; i < kVectors; ++i)
      sum[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 2
    for (int g = 0; g < ra.groups; ++g) {
      const float *theirs = ra.partials + static_cast<size_t>(g) * kTileFloats + at;
      float4 part[kVectors];
#pragma unroll
      for (int i = 0; i < kVectors; ++i)
        part[i] = __ldcg(reinterpret_cast<const float4 *>(theirs + i * 128));
#pragma unroll
      for (int i = 0; i < kVectors; ++i) {
        sum[i].x += part[i].x; sum[i].y += part[i].y; sum[i].z += part[i].z; sum[i].w += part[i].w;
      }
    }
    if (lane == 0)
      *counter = 0u;
  }
  // -- finish: C's previous contents, the operations, the store --
  float4 *staged = reinterpret_cast<float4 *>(ra.stage) + lane;  // piece i at staged[32 i]
  if (lane == 0)
    tma_store_wait_read();  // the previous store has read the staging block
  __syncwarp();
  if (ep.accumulate_by_tma_load != 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(ra.c_load_bar, kVectors * 512u);
      tma_load_2d(smem_u32(ra.stage), &tmap_c, ra.c_load_bar, col_base, row_base);  // outside C: zeros
    }
    const bool arrived = mbar_wait(ra.c_load_bar, c_load_phase, ra.abort_flag);
    c_load_phase ^= 1u;
    if (!__all_sync(0xffffffffu, arrived))
      return;
#pragma unroll
    for (int i = 0; i < kVectors; ++i) {
      const float4 old = staged[32 * i];
      sum[i].x += old.x; sum[i].y += old.y; sum[i].z += old.z; sum[i].w += old.w;
    }
    __syncwarp();
  }
#pragma unroll
  for (int op = 0; op < kMaxEpilogueOps; ++op) {
    if (op >= ep.op_count)
      break;
    const int kind = ep.op_kind[op];
    const float x = ep.op_value[op];
#pragma unroll
    for (int i = 0; i < kVectors; ++i) {
      float4 y = make_float4(x, x, x, x);
      if (kind == kEpilogueBiasColumn) {
        const int col = col_base + 4 * ((lane & 7) ^ ((4 * i + (lane >> 3)) & 7));
        y.x = col < ra.n ? __ldg(ep.bias + col) : 0.0f;
        y.y = col + 1 < ra.n ? __ldg(ep.bias + col + 1) : 0.0f;
        y.z = col + 2 < ra.n ? __ldg(ep.bias + col + 2) : 0.0f;
        y.w = col + 3 < ra.n ? __ldg(ep.bias + col + 3) : 0.0f;
      }
      float4 &v = sum[i];
      if (kind == kEpilogueScale) {
        v.x *= y.x; v.y *= y.y; v.z *= y.z; v.w *= y.w;
      } else if (kind == kEpilogueMax) {
        v.x = max_nan(v.x, y.x); v.y = max_nan(v.y, y.y); v.z = max_nan(v.z, y.z); v.w = max_nan(v.w, y.w);
      } else if (kind == kEpilogueMin) {
        v.x = min_nan(v.x, y.x); v.y = min_nan(v.y, y.y); v.z = min_nan(v.z, y.z); v.w = min_nan(v.w, y.w);
      } else {
        v.x += y.x; v.y += y.y; v.z += y.z; v.w += y.w;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kVectors; ++i)
    staged[32 * i] = sum[i];
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    if (ep.accumulate_by_tma != 0)
      tma_reduce_add_2d(&tmap_c, smem_u32(ra.stage), col_base, row_base);
    else
      tma_store_2d(&tmap_c, smem_u32(ra.stage), col_base, row_base);
    tma_store_commit();
  }
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_dense_cluster_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const __grid_constant__ CUtensorMap tmap_c, int m, int n, int k, uint32_t idesc,
                          int tiles_n, int groups, float *partials, unsigned *counters, int b_layout, int elem8,
                          Epilogue ep, int *status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  // The same offset in every CTA of the cluster (the dynamic shared memory of all CTAs of a kernel
  // starts at the same address), so a block's address can be mapped to any other CTA.
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - raw_addr);

  const uint32_t epi_base = smem_base + kStages * kStageBytes;
  const uint32_t bar_base = epi_base + kEpilogueWarps * kBlockBytes;
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (kStages + s); };
  const uint32_t tmem_full_bar = bar_base + 8u * (2 * kStages);
  const uint32_t misc_off = (bar_base - smem_base) + 8u * (2 * kStages + 2);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + misc_off);
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem_gen + misc_off + 4);

  const int warp = static_cast<int>(threadIdx.x >> 5);
  const int lane = static_cast<int>(threadIdx.x & 31);
  const uint32_t rank = cluster_cta_rank();
  const uint32_t ranks = cluster_cta_count();
  const int tile = static_cast<int>(cluster_id_x()) / groups;
  const int group = static_cast<int>(cluster_id_x()) - tile * groups;  // which of the tile's clusters

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tmem_full_bar, 1);
    for (uint32_t w = 0; w < kEpilogueWarps; ++w)
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

  const int num_kb = (k + (kBlockK << elem8) - 1) / (kBlockK << elem8);
  // This CTA's k-blocks: consecutive ranges in rank order (a range may be empty when there are
  // fewer k-blocks than CTAs; its partial tile is then zero).
  const long long share = static_cast<long long>(group) * ranks + rank, shares = static_cast<long long>(groups) * ranks;
  const int kb_begin = static_cast<int>(share * num_kb / shares);
  const int kb_end = static_cast<int>((share + 1) * num_kb / shares);
  const int m0 = (tile / tiles_n) * kBlockM;
  const int n0 = (tile % tiles_n) * kBlockN;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer ------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      const bool placed =
          HC_CHECK(status, abort_flag, HC_CHECK_TILE_COORDINATES,
                   tile >= 0 && group >= 0 && group < groups && m0 < m + kBlockM && n0 / kBlockN < tiles_n && rank < ranks) &&
          HC_CHECK(status, abort_flag, HC_CHECK_K_BLOCKS, kb_begin >= 0 && kb_begin <= kb_end && kb_end <= num_kb);
      for (int kb = kb_begin; placed && kb < kb_end; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag))
          break;
        if (!HC_CHECK(status, abort_flag, HC_CHECK_RING_STAGE,
                      stage < kStages && smem_base + (stage + 1) * kStageBytes <= epi_base) ||
            !HC_CHECK(status, abort_flag, HC_CHECK_TMA_COORDINATES,
                      m0 >= 0 && n0 >= 0 && ((n0 * 2) & 15) == 0 &&
                          ((((kb * kBlockK) << elem8) * (elem8 ? 1 : 2)) & 15) == 0))
          break;
        const uint32_t a_dst = smem_base + stage * kStageBytes;
        const uint32_t b_dst = a_dst + kATileBytes;
        mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
        tma_load_2d(a_dst, &tmap_a, full_bar(stage), (kb * kBlockK) << elem8, m0);
        if (b_layout == kBLayoutKN) {
#pragma unroll
          for (int j = 0; j < kBlockN / 64; ++j)
            tma_load_2d(b_dst + j * kBChunkBytes, &tmap_b, full_bar(stage), n0 + j * 64, kb * kBlockK);
        } else {
          tma_load_2d(b_dst, &tmap_b, full_bar(stage), (kb * kBlockK) << elem8, n0);
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer --------
    if (lane == 0) {
      auto mma_role = [&](auto f8) {
        constexpr bool kF8 = decltype(f8)::value;
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            ok = false;
            break;
          }
          tcgen05_fence_after_sync();
          const uint32_t a_addr = smem_base + stage * kStageBytes;
          const uint32_t b_addr = a_addr + kATileBytes;
          const uint64_t a_desc = make_smem_desc_sw128(a_addr, 16, 1024);
          const bool b_kn = b_layout == kBLayoutKN;
          const uint64_t b_desc = b_kn ? make_smem_desc_sw128(b_addr, kBChunkBytes, 1024)
                                       : make_smem_desc_sw128(b_addr, 16, 1024);
          const uint64_t b_step = b_kn ? 128 : 2;
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk)
            umma_ss<kF8>(tmem_base, a_desc + static_cast<uint64_t>(kk * 2), b_desc + static_cast<uint64_t>(kk) * b_step,
                         idesc, (kb != kb_begin || kk != 0) ? 1u : 0u);
          umma_commit(empty_bar(stage));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok && kb_end > kb_begin)
          umma_commit(tmem_full_bar);
      };
      if (elem8)
        mma_role(std::true_type{});
      else
        mma_role(std::false_type{});
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue, part 1 ---
    // Accumulator -> this CTA's partial tile in shared memory. Block (quarter, chunk) holds rows
    // 32 quarter .. + 31 and columns 32 chunk .. + 31 of the tile in the staging layout.
    const int quarter = warp & 3;             // the TMEM lanes a warp may read follow warp % 4
    const int column_part = (warp - 2) >> 2;  // which half of the tile's columns it drains
    bool ready = true;
    if (kb_end > kb_begin) {
      ready = mbar_wait(tmem_full_bar, 0u, abort_flag);
      ready = __all_sync(0xffffffffu, ready);
      tcgen05_fence_after_sync();
    }
    uint32_t r[32];
#pragma unroll 1
    for (int j = 0; j < 4; ++j) {
      const int chunk = column_part * 4 + j;
      if (kb_end > kb_begin && ready) {
        tmem_load_32x32b_x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + chunk * 32, r);
        tmem_load_wait_for(r);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          r[i] = 0u;
      }
      float *block = reinterpret_cast<float *>(smem_gen + static_cast<uint32_t>(quarter * 8 + chunk) * kBlockBytes);
      stage_row_shifted<0>(r, block, lane);
    }
    tcgen05_fence_before_sync();
    __syncwarp();
  }

  // Every partial tile of the cluster is complete (and visible cluster-wide) after this barrier.
  cluster_sync_all();

  if (warp >= 2) {
    // ------------------------------------------------------------ epilogue, part 2 ---
    const int e = warp - 2;
    float *stage_gen = reinterpret_cast<float *>(smem_gen + (epi_base - smem_base) + e * kBlockBytes);
    const uint32_t c_load_bar = bar_base + 128u + 8u * static_cast<uint32_t>(e);
    uint32_t c_load_phase = 0;
    ReduceArgs ra;
    ra.smem_base = smem_base;
    ra.ranks = ranks;
    ra.groups = groups;
    ra.group = group;
    ra.partials = partials + static_cast<size_t>(tile) * groups * (kPartialBytes / 4);
    ra.counters = counters + static_cast<size_t>(tile) * kCountersPerTile;
    ra.stage = stage_gen;
    ra.c_load_bar = c_load_bar;
    ra.abort_flag = abort_flag;
    ra.m = m;
    ra.n = n;
    ra.lane = lane;
    // Owned blocks b = rank + j * ranks, each in `parts` groups of rows (so that a CTA has at least
    // eight units of work); the eight epilogue warps take the units in turn.
    const int parts = ranks <= 4 ? 1 : static_cast<int>(ranks) / 4;
    const int units = (kBlocks / static_cast<int>(ranks)) * parts;
#pragma unroll 1
    for (int u = e; u < units; u += kEpilogueWarps) {
      const int block = static_cast<int>(rank) + (u / parts) * static_cast<int>(ranks);
      const int part = u % parts;
      const int first_row = part * (32 / parts);
      const int row_base = m0 + (block >> 3) * 32 + first_row;
      const int col_base = n0 + (block & 7) * 32;
      if (!HC_CHECK(status, abort_flag, HC_CHECK_PARTIAL_SLOT,
                    block >= 0 && block < kBlocks && first_row >= 0 && first_row + 32 / parts <= 32 &&
                        static_cast<uint32_t>(block) * kBlockBytes + static_cast<uint32_t>(first_row) * 128u +
                                (32u / static_cast<uint32_t>(parts)) * 128u <= kPartialBytes))
        break;
      if (row_base >= m || col_base >= n)
        continue;  // warp-uniform, and the same in every cluster of the tile: the rows lie outside C
      if (parts == 1)
        reduce_rows<8>(ra, block, first_row, row_base, col_base, c_load_phase, tmap_c, ep);
      else if (parts == 2)
        reduce_rows<4>(ra, block, first_row, row_base, col_base, c_load_phase, tmap_c, ep);
      else
        reduce_rows<2>(ra, block, first_row, row_base, col_base, c_load_phase, tmap_c, ep);
    }
    if (lane == 0)
      tma_store_wait_all();  // shared memory must outlive the stores that read it
    __syncwarp();
  }

  // No CTA may leave while another can still read its partial tile.
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
    tmem_dealloc(tmem_base, kTmemColumns);
}

} // namespace dense_cluster

int dense_cluster_capacity(int cluster_size) {
  using namespace dense_cluster;
  static thread_local int cached_device = -1;
  static thread_local int capacity[5];  // cluster sizes 1, 2, 4, 8, 16
  int slot = 0;
  while ((1 << slot) < cluster_size)
    ++slot;
  if (slot > 4 || (1 << slot) != cluster_size || cluster_size < 2)
    return 0;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess)
    return 0;
  if (cached_device != device) {
    if (cudaFuncSetAttribute(gemm_dense_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kSmemBytes)) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_dense_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) !=
            cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    for (int s = 1; s <= 4; ++s) {
      cudaLaunchConfig_t config = {};
      config.gridDim = dim3(static_cast<unsigned>(1 << s) * 16u, 1, 1);
      config.blockDim = dim3(kThreads, 1, 1);
      config.dynamicSmemBytes = kSmemBytes;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = static_cast<unsigned>(1 << s);
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      config.attrs = &attr;
      config.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, gemm_dense_cluster_kernel, &config) != cudaSuccess) {
        cudaGetLastError();  // a size the device does not offer
        clusters = 0;
      }
      capacity[s] = clusters;
    }
    capacity[0] = 0;
    if (std::getenv("HC_CUDA_CLUSTER_CAPACITY") != nullptr)  // tuning aid: print what the device offers
      std::fprintf(stderr, "hc-cuda: clusters at once: size 2: %d, 4: %d, 8: %d, 16: %d\n", capacity[1], capacity[2],
                   capacity[3], capacity[4]);
    cached_device = device;
  }
  return capacity[slot];
}

ClusterPlan dense_cluster_choose(long long m, long long n, long long k, int elem_bytes, int sm_count) {
  using namespace dense_cluster;
  ClusterPlan none{0, 0};
  // Clusters of size S that run at once on `sm_count` SMs with one CTA per SM: the CTAs of a cluster
  // share a GPC, and a GPC of 16 to 20 SMs does not divide evenly. A 148-SM B200 reports 74, 33, 15
  // and 7 for S = 2, 4, 8 and 16 (HC_CUDA_CLUSTER_CAPACITY prints what the device offers).
  auto capacity = [&](int size) {
    const int even = sm_count / size;
    return size == 2 ? even : (size == 4 ? even - even / 9 : (size == 8 ? even - even / 6 : even - even / 4));
  };
  int forced_size = -1, forced_groups = -1;
  if (const char *text = std::getenv("HC_CUDA_DENSE_CLUSTER"))  // tuning aid: 0 = never, 2/4/8/16 = that size
    forced_size = std::atoi(text);
  if (const char *text = std::getenv("HC_CUDA_DENSE_CLUSTER_GROUPS"))  // tuning aid: clusters per tile
    forced_groups = std::atoi(text);
  if (forced_size == 0)
    return none;
  const long long tiles = ((m + kBlockM - 1) / kBlockM) * ((n + kBlockN - 1) / kBlockN);
  const long long num_kb = (k * elem_bytes + kBlockK * 2 - 1) / (kBlockK * 2);
  // Estimated time of a choice, in microseconds: the k-loop of one CTA at the rate an SM pulls
  // operands it has not touched before (about 50 GB/s, measured), the sum through distributed shared
  // memory, and, with several clusters per tile, the partial tiles through global memory (the last
  // cluster's CTAs each read `groups` slices of 128 KiB / S at about 100 GB/s).
  double best_time = 0.0;
  ClusterPlan best = none;
  for (int size = 16; size >= 2; size >>= 1) {
    if (forced_size >= 2 && size != forced_size)
      continue;
    long long most = capacity(size) / tiles;
    if (forced_size >= 2 && most < 1)
      most = 1;
    if (most > 16)
      most = 16;
    for (long long groups = 1; groups <= most; ++groups) {
      if (forced_groups >= 1 && groups != forced_groups)
        continue;
      const long long kb_per_cta = (num_kb + size * groups - 1) / (size * groups);
      if (kb_per_cta < 4 && !(forced_size >= 2 && num_kb >= size * groups))
        continue;
      double t = static_cast<double>(kb_per_cta) * kStageBytes / 50000.0 + 3.0;
      if (groups > 1)
        t += 3.0 + static_cast<double>(groups) * (kPartialBytes / size) / 100000.0;
      if (best.cluster_size == 0 || t < best_time) {
        best_time = t;
        best.cluster_size = size;
        best.groups = static_cast<int>(groups);
      }
    }
  }
  return best;
}

size_t dense_cluster_partials_bytes(long long tiles, int groups) {
  return groups > 1 ? static_cast<size_t>(tiles) * groups * dense_cluster::kPartialBytes : 0;
}

size_t dense_cluster_counters_bytes(long long tiles) {
  return static_cast<size_t>(tiles) * dense_cluster::kCountersPerTile * sizeof(unsigned);
}

cudaError_t launch_gemm_dense_cluster(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, const CUtensorMap &tmap_c,
                                      int m, int n, int k, int dtype, int cluster_size, int groups, float *partials,
                                      unsigned *counters, int b_layout, const Epilogue &ep, int *status,
                                      cudaStream_t stream) {
  using namespace dense_cluster;
  if (dense_cluster_capacity(cluster_size) <= 0)
    return cudaErrorInvalidValue;  // (the caller asks dense_cluster_capacity before it encodes tmap_c)
  const int tiles_m = (m + kBlockM - 1) / kBlockM;
  const int tiles_n = (n + kBlockN - 1) / kBlockN;
  const long long num_tiles = static_cast<long long>(tiles_m) * tiles_n;
  if (num_tiles <= 0 || groups < 1 || num_tiles * groups * cluster_size > 0x7fffffffLL)
    return cudaErrorInvalidValue;
  if (groups > 1 && (partials == nullptr || counters == nullptr))
    return cudaErrorInvalidValue;
  if (ep.c_dtype != kCTypeF32 || ep.push_count != 0)
    return cudaErrorInvalidValue;  // the caller keeps these on the counter-based split
  const int elem8 = dtype_is_8bit(dtype) ? 1 : 0;
  if (elem8 && b_layout != kBLayoutNK)
    return cudaErrorInvalidValue;
  const uint32_t idesc = make_idesc_f16(dtype_format(dtype), /*a_mn_major=*/false,
                                        /*b_mn_major=*/b_layout == kBLayoutKN, kBlockM, kBlockN);
  Epilogue launch_ep = ep;
  launch_ep.accumulate_by_tma = (ep.accumulate != 0 && ep.op_count == 0) ? 1 : 0;
  launch_ep.accumulate_by_tma_load = (ep.accumulate != 0 && ep.op_count != 0) ? 1 : 0;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(num_tiles * groups * cluster_size), 1, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = static_cast<unsigned>(cluster_size);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  config.attrs = &attr;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, gemm_dense_cluster_kernel, tmap_a, tmap_b, tmap_c, m, n, k, idesc, tiles_n,
                            groups, partials, counters, b_layout, elem8, launch_ep, status);
}

int dense_cluster_store_rows(int cluster_size) { return cluster_size <= 4 ? 32 : 128 / cluster_size; }

} // namespace sm100
} // namespace hc
