// Skinny GEMM for sm_100a:  C[M,N] (fp32) = A[M,K] * B[K,N] with M <= 64, where the time
// is the time to stream B from HBM once. Same contract as the dense kernel (the hc example
// kernel examples/amdgpu_gfx11_wmma_matmul.py:301-326: fp32 accumulate, out-of-range
// elements count as 0, only in-range C is written), different mapping:
//
//   * The product is computed transposed, C^T = B^T * A^T, so that the long N axis sits on
//     the 128 TMEM lanes and the short M axis (padded to 16/32/64) on the UMMA N side.
//     B is N-major in memory, which tcgen05.mma accepts directly as an MN-major operand:
//     no register staging and no transposing loads, TMA -> shared memory -> tensor core.
//   * Work unit = (block of 128 columns of C, one of `splits` ranges of k). Units are
//     spread over persistent CTAs, each with its own multi-stage TMA ring so that enough
//     bytes are in flight to cover HBM latency: two CTAs per SM with 6/5/4 stages, or, when the
//     grid has no more CTAs than there are SMs, one with 12/11/9.
//   * Split-k partial sums go to scratch memory; a per-32-column arrival counter tells the
//     last warp to finish a column block to add the partials in split order 0..S-1 (so the
//     result does not depend on which unit finished last) and to write C with coalesced
//     128-byte row segments. The counters are reset to zero by that warp.
//
// Warp roles: warp 0 TMA producer, warp 1 TMEM owner + tcgen05.mma issuer, warps 2-5
// epilogue (TMEM -> registers -> partials / C).
#include "gemm_epilogue.cuh"
#include "device_checks.cuh"
#include "gemm_launch.h"
#include "sm100_ptx.cuh"

#include <cstdlib>
#include <cstring>
#include <type_traits>

namespace hc {
namespace sm100 {

namespace skinny {

constexpr int kBlockN = 128;  // TMEM lanes
constexpr int kBlockK = 64;
constexpr int kUmmaK = 16;
constexpr int kNumThreads = 192;
constexpr int kCtasPerSm = 2;
constexpr uint32_t kBChunkBytes = 64 * kBlockK * 2;                   // 64 columns x 64 k-rows
constexpr uint32_t kBTileBytes = kBChunkBytes * (kBlockN / 64);       // 16 KiB
constexpr int kMaxStages = 16;
constexpr uint32_t kBarrierBytes = 512;  // full/empty[kMaxStages], TMEM barriers, slot, abort flag
constexpr uint32_t kMaxSmemPerCta = 232448;  // 227 KiB

template <int kMp>
struct Config {
  static constexpr uint32_t kATileBytes = kMp * kBlockK * 2;
  static constexpr uint32_t kStageBytes = kBTileBytes + kATileBytes;
  static constexpr uint32_t kTmemColumns = 2 * kMp < 32 ? 32 : 2 * kMp;
  // Ring depth: as deep as shared memory allows, for two resident CTAs per SM or, when the grid
  // does not exceed the SM count anyway, for one (twice the bytes in flight per CTA).
  static constexpr int stages_for(uint32_t smem_budget) {
    const int fit = static_cast<int>((smem_budget - kBarrierBytes - 1024) / kStageBytes);
    return fit > kMaxStages ? kMaxStages : fit;
  }
  static constexpr int kStagesShared = stages_for(kMaxSmemPerCta / 2 - 1024);  // 6 / 5 / 4
  static constexpr int kStagesAlone = stages_for(kMaxSmemPerCta);              // 12 / 11 / 9
  static constexpr uint32_t smem_bytes(int stages) { return stages * kStageBytes + kBarrierBytes + 1024; }
};

template <int kMp>
__global__ void __launch_bounds__(kNumThreads, kCtasPerSm)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_a,
                   const __grid_constant__ CUtensorMap tmap_b, void *c_any, int m, int n,
                   int k, long long ldc, uint32_t idesc, int n_tiles, int splits, int num_stages,
                   int b_layout, int elem8, Epilogue ep,
                   float *__restrict__ partials, unsigned *__restrict__ counters, int *status) {
  using Cfg = Config<kMp>;
  float *__restrict__ c = static_cast<float *>(c_any);  // the float32 view (accumulation reads it)
  const uint32_t kStages = static_cast<uint32_t>(num_stages);  // ring depth of this launch
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - raw_addr);

  const uint32_t bar_base = smem_base + kStages * Cfg::kStageBytes;
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (kMaxStages + s); };
  auto tmem_full_bar = [&](uint32_t a) { return bar_base + 8u * (2 * kMaxStages + a); };
  auto tmem_empty_bar = [&](uint32_t a) { return bar_base + 8u * (2 * kMaxStages + 2 + a); };
  const uint32_t misc_off = (bar_base - smem_base) + 8u * (2 * kMaxStages + 4);
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
      mbar_init(tmem_empty_bar(a), 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_descriptor(&tmap_a);
    tma_prefetch_descriptor(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), Cfg::kTmemColumns);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int kb_total = (k + (kBlockK << elem8) - 1) / (kBlockK << elem8);  // 8-bit: twice the k per stage
  const int num_units = n_tiles * splits;
  const int n_pad = n_tiles * kBlockN;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer ------
    if (lane == 0) {
      const uint64_t stream_policy = l2_policy_evict_first();  // B is read exactly once
      const uint64_t keep_policy = l2_policy_evict_last();     // A is re-read by every unit
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; ok && unit < num_units; unit += gridDim.x) {
        const int n_tile = unit % n_tiles;
        const int split = unit / n_tiles;
        const int kb_begin = static_cast<int>(static_cast<long long>(split) * kb_total / splits);
        const int kb_end = static_cast<int>(static_cast<long long>(split + 1) * kb_total / splits);
        const int n0 = n_tile * kBlockN;
        if (!HC_CHECK(status, abort_flag, HC_CHECK_TILE_COORDINATES, n_tile >= 0 && n_tile < n_tiles) ||
            !HC_CHECK(status, abort_flag, HC_CHECK_K_BLOCKS,
                      split >= 0 && split < splits && kb_begin >= 0 && kb_begin <= kb_end && kb_end <= kb_total))
          break;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          if (!HC_CHECK(status, abort_flag, HC_CHECK_RING_STAGE,
                        stage < kStages && smem_base + (stage + 1) * Cfg::kStageBytes <= bar_base) ||
              !HC_CHECK(status, abort_flag, HC_CHECK_TMA_COORDINATES,
                        ((n0 * 2) & 15) == 0 && ((((kb * kBlockK) << elem8) * (elem8 ? 1 : 2)) & 15) == 0)) {
            ok = false;
            break;
          }
          const uint32_t b_dst = smem_base + stage * Cfg::kStageBytes;
          const uint32_t a_dst = b_dst + kBTileBytes;
          mbar_arrive_expect_tx(full_bar(stage), Cfg::kStageBytes);
          if (b_layout == kBLayoutKN) {
#pragma unroll
            for (int j = 0; j < kBlockN / 64; ++j)
              tma_load_2d_hint(b_dst + j * kBChunkBytes, &tmap_b, full_bar(stage), n0 + j * 64,
                               kb * kBlockK, stream_policy);
          } else {
            // B stored [N, K]: 128 rows (n) x 64 k in one box, K-major.
            tma_load_2d_hint(b_dst, &tmap_b, full_bar(stage), (kb * kBlockK) << elem8, n0, stream_policy);
          }
          tma_load_2d_hint(a_dst, &tmap_a, full_bar(stage), (kb * kBlockK) << elem8, 0, keep_policy);
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
          const int split = unit / n_tiles;
          const int kb_begin = static_cast<int>(static_cast<long long>(split) * kb_total / splits);
          const int kb_end = static_cast<int>(static_cast<long long>(split + 1) * kb_total / splits);
          const uint32_t acc = iter & 1u;
          const uint32_t acc_phase = (iter >> 1) & 1u;
          if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag))
            break;
          tcgen05_fence_after_sync();
          const uint32_t d_tmem = tmem_base + acc * kMp;
          for (int kb = kb_begin; kb < kb_end; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
              ok = false;
              break;
            }
            tcgen05_fence_after_sync();
            const uint32_t bt_addr = smem_base + stage * Cfg::kStageBytes;
            const uint32_t a_addr = bt_addr + kBTileBytes;
            // UMMA "A" operand = B^T tile (128 n x 64 k): MN-major when B is stored [K, N] (n
            // contiguous), K-major when it is stored [N, K].
            const bool b_kn = b_layout == kBLayoutKN;
            const uint64_t bt_desc = b_kn ? make_smem_desc_sw128(bt_addr, kBChunkBytes, 1024)
                                          : make_smem_desc_sw128(bt_addr, 16, 1024);
            const uint64_t bt_step = b_kn ? 128 : 2;
            // UMMA "B" operand = A tile (kMp rows x 64 k), k contiguous: K-major.
            const uint64_t a_desc = make_smem_desc_sw128(a_addr, 16, 1024);
#pragma unroll
            for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
              umma_ss<kF8>(d_tmem, bt_desc + static_cast<uint64_t>(kk) * bt_step, a_desc + static_cast<uint64_t>(kk * 2),
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
    const int quarter = warp & 3;
    uint32_t iter = 0;
    for (int unit = blockIdx.x; unit < num_units; unit += gridDim.x, ++iter) {
      const int n_tile = unit % n_tiles;
      const int split = unit / n_tiles;
      const uint32_t acc = iter & 1u;
      const uint32_t acc_phase = (iter >> 1) & 1u;
      if (ep.accumulate && splits == 1) {
        // C is read before it is written: fetch this warp's 128-byte piece of every row into L2
        // while B is still streaming (one lane per row).
        const int first_col = n_tile * kBlockN + quarter * 32;
        for (int mm = lane; mm < m; mm += 32)
          if (first_col < n)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(c + static_cast<long long>(mm) * ldc + first_col));
      }
      const bool ready = mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag);
      if (!__all_sync(0xffffffffu, ready))
        break;
      tcgen05_fence_after_sync();
      // Lane `lane` of this warp holds column (n_tile*128 + quarter*32 + lane) of C; its
      // TMEM columns are the rows of C.
      uint32_t r[kMp];
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kMp;
      if (!HC_CHECK(status, abort_flag, HC_CHECK_TMEM_COLUMNS, acc * kMp + kMp <= Cfg::kTmemColumns) ||
          !HC_CHECK(status, abort_flag, HC_CHECK_OUTPUT_RANGE, n_tile >= 0 && n_tile < n_tiles) ||
          !HC_CHECK(status, abort_flag, HC_CHECK_PARTIAL_SLOT, split >= 0 && split < splits))
        break;
#pragma unroll
      for (int g = 0; g < kMp / 16; ++g) {
        uint32_t part[16];
        tmem_load_32x32b_x16(taddr + g * 16, part);
#pragma unroll
        for (int i = 0; i < 16; ++i)
          r[g * 16 + i] = part[i];
      }
      tmem_load_wait();
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(tmem_empty_bar(acc));

      const int col = n_tile * kBlockN + quarter * 32 + lane;
      const bool fused = ep.accumulate != 0 || ep.op_count != 0;
      if (splits == 1) {
        if (!fused) {
#pragma unroll
          for (int mm = 0; mm < kMp; ++mm)
            if (mm < m && col < n)
              store_c_element(c_any, static_cast<long long>(mm) * ldc + col, __uint_as_float(r[mm]), ep.c_dtype);
          continue;
        }
        // Reads first (the previous contents of eight rows, the bias once), then the stores.
        const float bias = (ep.bias != nullptr && col < n) ? __ldg(ep.bias + col) : 0.0f;
#pragma unroll
        for (int mm0 = 0; mm0 < kMp; mm0 += 8) {
          float previous[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            previous[j] = (ep.accumulate && mm0 + j < m && col < n)
                              ? __ldcs(c + static_cast<long long>(mm0 + j) * ldc + col) : 0.0f;
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            v[j] = __uint_as_float(r[mm0 + j]) + previous[j];
          apply_ops_to_column(v, bias, ep);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (mm0 + j < m && col < n)
              store_c_element(c_any, static_cast<long long>(mm0 + j) * ldc + col, v[j], ep.c_dtype);
        }
        continue;
      }
      float *my_partial = partials + static_cast<size_t>(split) * m * n_pad + col;
#pragma unroll
      for (int mm = 0; mm < kMp; ++mm)
        if (mm < m)
          __stcg(my_partial + static_cast<size_t>(mm) * n_pad, __uint_as_float(r[mm]));
      __threadfence();
      __syncwarp();
      unsigned arrived = 0;
      unsigned *counter = counters + n_tile * 4 + quarter;
      if (lane == 0)
        arrived = atomicAdd(counter, 1u);
      arrived = __shfl_sync(0xffffffffu, arrived, 0);
      if (arrived == static_cast<unsigned>(splits - 1)) {
        // Every split of this 32-column block has published its partial sums.
        __threadfence();
        const float *col_partials = partials + col;
        const float bias = (fused && ep.bias != nullptr && col < n) ? __ldg(ep.bias + col) : 0.0f;
        // Eight rows at a time, their loads issued together: the additions of one row stay in
        // split order, but the L2 round trips of different rows and splits overlap.
        for (int mm0 = 0; mm0 < m; mm0 += 8) {
          float sums[8];  // an accumulating kernel's sums start from C
#pragma unroll
          for (int j = 0; j < 8; ++j)
            sums[j] = (ep.accumulate && mm0 + j < m && col < n)
                          ? __ldcs(c + static_cast<long long>(mm0 + j) * ldc + col) : 0.0f;
#pragma unroll 4
          for (int s = 0; s < splits; ++s) {
            float part[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              part[j] = mm0 + j < m ? __ldcg(col_partials + (static_cast<size_t>(s) * m + mm0 + j) * n_pad) : 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              sums[j] += part[j];
          }
          if (fused)
            apply_ops_to_column(sums, bias, ep);
          if (col < n) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (mm0 + j < m)
                store_c_element(c_any, static_cast<long long>(mm0 + j) * ldc + col, sums[j], ep.c_dtype);
          }
        }
        if (lane == 0)
          *counter = 0u;
      }
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  if (*abort_flag != 0) {
    if (threadIdx.x == 0)
      atomicCAS(status, 0, kStatusDeviceWaitTimeout);  // (a failed check recorded earlier stays)
    const long long start = clock64();
    while (clock64() - start < 2000000LL) {
    }
    __syncthreads();
  }
  if (warp == 1)
    tmem_dealloc(tmem_base, Cfg::kTmemColumns);
}

template <int kMp>
cudaError_t launch(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, void *c, int m, int n,
                   int k, long long ldc, int dtype, int splits, float *partials,
                   unsigned *counters, int max_ctas, int sm_count, int b_layout, const Epilogue &ep,
                   int *status, cudaStream_t stream) {
  using Cfg = Config<kMp>;
  static thread_local int configured_device = -1;
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess)
    return err;
  if (configured_device != device) {
    err = cudaFuncSetAttribute(gemm_skinny_kernel<kMp>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(Cfg::smem_bytes(Cfg::kStagesAlone)));
    if (err != cudaSuccess)
      return err;
    configured_device = device;
  }
  const int n_tiles = (n + kBlockN - 1) / kBlockN;
  const long long units = static_cast<long long>(n_tiles) * splits;
  const int grid = static_cast<int>(units < max_ctas ? units : max_ctas);
  const int num_stages = skinny_ring_stages(m, grid, sm_count);
  const int elem8 = dtype_is_8bit(dtype) ? 1 : 0;
  if (elem8 && b_layout != kBLayoutNK)
    return cudaErrorInvalidValue;  // 8-bit operands are K-major: the caller transposes a [K, N] B first
  const uint32_t idesc = make_idesc_f16(dtype_format(dtype), /*a_mn_major=*/b_layout == kBLayoutKN,
                                        /*b_mn_major=*/false, kBlockN, kMp);
  // (The first flag describes the UMMA "A" operand, which is B^T here.)
  gemm_skinny_kernel<kMp><<<grid, kNumThreads, Cfg::smem_bytes(num_stages), stream>>>(
      tmap_a, tmap_b, c, m, n, k, ldc, idesc, n_tiles, splits, num_stages, b_layout, elem8, ep, partials, counters, status);
  return cudaGetLastError();
}

inline int padded_m(int m) { return m <= 16 ? 16 : (m <= 32 ? 32 : 64); }

} // namespace skinny

SkinnyShape skinny_shape(int m) {
  SkinnyShape s;
  s.block_n = skinny::kBlockN;
  s.block_k = skinny::kBlockK;
  s.max_m = 64;
  const int mp = skinny::padded_m(m);
  if (mp == 16) {
    s.stages = skinny::Config<16>::kStagesAlone;
    s.smem_bytes = skinny::Config<16>::smem_bytes(s.stages);
  } else if (mp == 32) {
    s.stages = skinny::Config<32>::kStagesAlone;
    s.smem_bytes = skinny::Config<32>::smem_bytes(s.stages);
  } else {
    s.stages = skinny::Config<64>::kStagesAlone;
    s.smem_bytes = skinny::Config<64>::smem_bytes(s.stages);
  }
  return s;
}

int skinny_choose_splits(int n, int k, int sm_count) {
  // Splitting k costs a round trip of partial sums through L2 and a counter handshake per
  // unit, and measurements show that B streams at full HBM rate as soon as roughly 0.8 CTAs
  // per SM are loading. So: no split when there are that many column blocks (8x16384x8192:
  // 128 blocks, 43 us unsplit against 52-66 us with 2-16 splits); otherwise just enough
  // splits to get there, each keeping at least 4 k-blocks so that its ring fills.
  const int n_tiles = (n + skinny::kBlockN - 1) / skinny::kBlockN;
  const int kb_total = (k + skinny::kBlockK - 1) / skinny::kBlockK;
  const int wanted_units = sm_count * 4 / 5 > 0 ? sm_count * 4 / 5 : 1;
  if (n_tiles >= wanted_units)
    return 1;
  int splits = (wanted_units + n_tiles - 1) / n_tiles;
  const int most = kb_total / 4 > 0 ? kb_total / 4 : 1;
  if (splits > most)
    splits = most;
  if (splits > 32)
    splits = 32;
  return splits < 1 ? 1 : splits;
}

int skinny_ring_stages(int m, int grid, int sm_count) {
  // A grid with no more CTAs than SMs leaves every CTA alone on its SM, so each may take all of
  // the shared memory (twice the bytes in flight); a larger grid shares an SM between two.
  bool alone = grid <= sm_count;
  if (const char *forced = std::getenv("HC_CUDA_SKINNY_RING")) {  // tuning aid: "shallow" or "deep"
    if (std::strcmp(forced, "shallow") == 0)
      alone = false;
    else if (std::strcmp(forced, "deep") == 0 && grid <= sm_count)
      alone = true;
  }
  const int mp = skinny::padded_m(m);
  if (mp == 16)
    return alone ? skinny::Config<16>::kStagesAlone : skinny::Config<16>::kStagesShared;
  if (mp == 32)
    return alone ? skinny::Config<32>::kStagesAlone : skinny::Config<32>::kStagesShared;
  return alone ? skinny::Config<64>::kStagesAlone : skinny::Config<64>::kStagesShared;
}

size_t skinny_partials_bytes(int m, int n, int splits) {
  if (splits <= 1)
    return 0;
  const size_t n_tiles = (static_cast<size_t>(n) + skinny::kBlockN - 1) / skinny::kBlockN;
  return static_cast<size_t>(splits) * static_cast<size_t>(m) * n_tiles * skinny::kBlockN *
         sizeof(float);
}

size_t skinny_counters_bytes(int n) {
  const size_t n_tiles = (static_cast<size_t>(n) + skinny::kBlockN - 1) / skinny::kBlockN;
  return n_tiles * 4 * sizeof(unsigned);
}

cudaError_t launch_gemm_skinny(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, void *c,
                               int m, int n, int k, long long ldc, int dtype, int splits,
                               float *partials, unsigned *counters, int max_ctas, int sm_count,
                               int b_layout, const Epilogue &ep, int *status, cudaStream_t stream) {
  if (m < 1 || m > 64 || splits < 1 || sm_count < 1)
    return cudaErrorInvalidValue;
  const int mp = skinny::padded_m(m);
  if (mp == 16)
    return skinny::launch<16>(tmap_a, tmap_b, c, m, n, k, ldc, dtype, splits, partials, counters,
                              max_ctas, sm_count, b_layout, ep, status, stream);
  if (mp == 32)
    return skinny::launch<32>(tmap_a, tmap_b, c, m, n, k, ldc, dtype, splits, partials, counters,
                              max_ctas, sm_count, b_layout, ep, status, stream);
  return skinny::launch<64>(tmap_a, tmap_b, c, m, n, k, ldc, dtype, splits, partials, counters,
                            max_ctas, sm_count, b_layout, ep, status, stream);
}

} // namespace sm100
} // namespace hc
