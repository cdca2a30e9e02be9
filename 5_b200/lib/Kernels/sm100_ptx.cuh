// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the GEMM kernels use:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM allocation, UMMA issue, commit,
// TMEM loads) and the shared-memory / instruction descriptors that tcgen05.mma consumes.
//
// Every wait in this file is bounded: `mbar_wait` gives up after kWaitTimeoutCycles
// and reports failure so that the calling kernel can record a status code and leave
// instead of spinning forever.
#pragma once

#include <cuda.h>  // CUtensorMap (type only; the driver library is never linked)
#include <cstdint>

namespace hc {
namespace sm100 {

// Roughly two seconds at B200 clocks; far longer than any legitimate wait in these kernels.
constexpr long long kWaitTimeoutCycles = 4000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier ----------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(arrivals) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Waits for the phase with the given parity to complete. Returns false when the wait ran
// out of time or when another role of the CTA has already raised `*abort_flag` (a word
// in shared memory); the caller then stops its role loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          long long timeout_cycles = kWaitTimeoutCycles) {
  if (mbar_try_wait(bar, parity))
    return true;
  const long long start = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xffu) == 0) {
      if (*abort_flag != 0)
        return false;
      if (clock64() - start > timeout_cycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

// ---------------------------------------------------------------- TMA ---------------

__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

__device__ __forceinline__ uint64_t l2_policy_evict_normal() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

// 2-D tiled load global -> shared, completion counted in bytes on `bar`.
// x is the innermost (contiguous) coordinate in elements; x * element size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap *map,
                                            uint32_t bar, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Tile store, shared memory -> global, through the same tensor-map machinery: elements of the box
// that fall outside the tensor are not written. Belongs to the issuing thread's bulk group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src_smem, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(map)), "r"(src_smem), "r"(x), "r"(y)
               : "memory");
}

// Same box, added to what global memory holds (fp32 add performed at the memory side): C += tile
// without the kernel ever reading C.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap *map, uint32_t src_smem, int32_t x, int32_t y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(map)), "r"(src_smem), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Until the stores this thread committed have finished *reading* shared memory (the source may
// then be overwritten) ...
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// ... or have completed altogether.
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Orders this thread's async-proxy operations (completed TMA stores) and generic-proxy
// operations on all memory against each other.
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Makes this thread's ordinary shared-memory writes visible to the async proxy (TMA).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst_smem, const CUtensorMap *map,
                                                 uint32_t bar, int32_t x, int32_t y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      :
      : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y),
        "l"(policy)
      : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM ----

// Whole-warp operations (.sync.aligned): every lane of one warp must call them together.
__device__ __forceinline__ void tmem_alloc(uint32_t result_slot_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   result_slot_smem),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_alloc_permit() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t tmem_addr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_addr),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; 16-bit inputs, fp32 accumulate. One thread issues it.
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same for 8-bit floats: kind::f8f6f4, 32 of k per instruction. Both kinds read 32 bytes of k per
// operand row, so descriptors and their per-step advance are the same in bytes. (The kind is a
// template argument of the issue loops, chosen by one branch per ring stage: a pair of oppositely
// predicated instructions per step, one of each kind, measured 10-30 % slower kernels.)
__device__ __forceinline__ void umma_f8_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <bool kF8>
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
  if constexpr (kF8)
    umma_f8_ss(tmem_d, desc_a, desc_b, idesc, accumulate);
  else
    umma_f16_ss(tmem_d, desc_a, desc_b, idesc, accumulate);
}

// Makes `bar` receive one arrival once every tcgen05.mma issued so far by this thread has
// finished (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// TMEM -> registers: the calling warp reads its own 32 lanes, `N` consecutive 32-bit
// columns per lane (lane l of the warp gets TMEM lane base+l).
__device__ __forceinline__ void tmem_load_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_load_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_load_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The same wait, tied to the registers of an earlier tmem_load_32x32b_x32 so that no use of
// them can be scheduled ahead of it (needed when other work is placed between load and wait).
__device__ __forceinline__ void tmem_load_wait_for(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                 "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]),
                 "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]),
                 "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]),
                 "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

// ---------------------------------------------------------------- CTA pairs ----------
// Helpers for kernels launched as clusters of two CTAs that drive one tcgen05.mma
// (.cta_group::2) together: the even CTA of the pair issues the instruction, operands and
// accumulator are split over the shared memory and TMEM of both.

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}

// Address, in the cluster-wide shared window, of the same shared-memory location in CTA
// `cta_rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta_rank) {
  uint32_t mapped;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(mapped) : "r"(smem_addr), "r"(cta_rank));
  return mapped;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t cluster_cta_count() {
  uint32_t count;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(count));
  return count;
}

__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t id;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(id));
  return id;
}

// 16 bytes from the shared memory of any CTA of the cluster (`cluster_addr` from map_to_cta).
__device__ __forceinline__ float4 ld_shared_cluster_f4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}

// Arrive on an mbarrier that may live in the other CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
}

// Pair form of tma_load_2d: the completion bytes may be counted on an mbarrier of either CTA of
// the pair (`cluster_bar` is an address in the cluster-wide shared window).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap *map,
                                                 uint32_t cluster_bar, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t dst_smem, const CUtensorMap *map,
                                                      uint32_t cluster_bar, int32_t x, int32_t y,
                                                      uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      :
      : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y),
        "l"(policy)
      : "memory");
}

// TMEM allocation for a pair: one warp of EACH CTA executes these together; the same columns are
// allocated in both CTAs and the address is written to `result_slot_smem` of each.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t result_slot_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   result_slot_smem),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_alloc_permit_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t tmem_addr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_addr), "r"(columns)
               : "memory");
}

// D (rows split over the TMEM of both CTAs) (+)= A (rows split over both CTAs' shared memory) *
// B (columns split over both CTAs' shared memory). Issued by one thread of the even CTA.
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_f8_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <bool kF8>
__device__ __forceinline__ void umma_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  if constexpr (kF8)
    umma_f8_ss_pair(tmem_d, desc_a, desc_b, idesc, accumulate);
  else
    umma_f16_ss_pair(tmem_d, desc_a, desc_b, idesc, accumulate);
}

// One arrival on `cluster_bar` (either CTA's) once all pair MMAs issued so far have finished.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   cluster_bar)
               : "memory");
}

// ---------------------------------------------------------------- descriptors -------

// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile whose base is
// 1024-byte aligned. `leading_bytes` / `stride_bytes` are the LBO / SBO fields:
//   K-major  (K contiguous):  SBO = distance between groups of 8 rows; LBO unused.
//   MN-major (M or N contiguous): LBO = distance between 64-element chunks along M/N,
//                                 SBO = distance between groups of 8 along K.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr,
                                                         uint32_t leading_bytes,
                                                         uint32_t stride_bytes) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);         // bits [0,14)
  desc |= static_cast<uint64_t>((leading_bytes >> 4) & 0x3fffu) << 16; // bits [16,30)
  desc |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3fffu) << 32;  // bits [32,46)
  desc |= static_cast<uint64_t>(1) << 46;                             // descriptor version
  desc |= static_cast<uint64_t>(2) << 61;                             // 128-byte swizzle
  return desc;
}

// Instruction descriptor for tcgen05.mma.kind::f16 and kind::f8f6f4 with fp32 accumulation (the
// two kinds share the field layout).
//   in_format: kind::f16: 0 = fp16, 1 = bf16; kind::f8f6f4: 0 = e4m3, 1 = e5m2.
//   *_mn_major: operand is contiguous along M (or N).
__host__ __device__ constexpr uint32_t make_idesc_f16(uint32_t in_format, bool a_mn_major,
                                                      bool b_mn_major, uint32_t umma_m,
                                                      uint32_t umma_n) {
  return (1u << 4)                              // D format: fp32
         | (in_format << 7)                     // A format
         | (in_format << 10)                    // B format
         | ((a_mn_major ? 1u : 0u) << 15)       // A major-ness
         | ((b_mn_major ? 1u : 0u) << 16)       // B major-ness
         | ((umma_n >> 3) << 17)                // N / 8
         | ((umma_m >> 4) << 24);               // M / 16
}

} // namespace sm100
} // namespace hc
