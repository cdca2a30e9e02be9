// Index checks inside the kernels, compiled in by -DHC_CUDA_CHECKED (the "checked" build of the
// library, lib/libhc_cuda_checked.so).
//
// A checked kernel verifies the indices it is about to use -- tile coordinates, ring stages, shared
// memory offsets, tensor-memory columns, TMA coordinates, partial-tile slots -- and, when one is out
// of range, records the number of the check in the launch's status word (first failure wins) and
// leaves through the same bounded give-up path as a wait that ran out: no trap, no device assert,
// the bad access is not made and the context stays usable. The host reports
// HC_CUDA_ERR_DEVICE_CHECK with that number at the next synchronise. In the ordinary build the
// macro costs nothing (its condition is not evaluated).
#pragma once

#include "gemm_launch.h"

namespace hc {
namespace sm100 {

// What a failed check stores in the status word: kStatusCheckFailed in the low byte, the number of
// the check above it.
__device__ __forceinline__ bool report_failed_check(int *status, volatile uint32_t *abort_flag, int check) {
  atomicCAS(status, 0, kStatusCheckFailed | (check << 8));
  if (abort_flag != nullptr)
    *abort_flag = 1;  // every role of the CTA stops at its next wait
  return false;
}

} // namespace sm100
} // namespace hc

#ifdef HC_CUDA_CHECKED
#define HC_CHECK(status, abort_flag, check, condition) \
  ((condition) ? true : ::hc::sm100::report_failed_check((status), (abort_flag), (check)))
#else
#define HC_CHECK(status, abort_flag, check, condition) (true)
#endif

// Numbers of the checks (reported with HC_CUDA_ERR_DEVICE_CHECK).
#define HC_CHECK_TILE_COORDINATES 1   /* a tile's block coordinates lie inside the tile grid */
#define HC_CHECK_K_BLOCKS 2           /* a unit's range of k-blocks lies inside [0, number of k-blocks] */
#define HC_CHECK_RING_STAGE 3         /* a ring stage index and its shared-memory range lie inside the ring */
#define HC_CHECK_TMA_COORDINATES 4    /* TMA coordinates are non-negative and 16-byte aligned along x */
#define HC_CHECK_TMEM_COLUMNS 5       /* a tensor-memory read stays inside the allocated columns */
#define HC_CHECK_OUTPUT_RANGE 6       /* the rows and columns a warp is about to write start inside the tile grid */
#define HC_CHECK_PARTIAL_SLOT 7       /* a partial tile's slot and a cluster block's offset lie inside their buffers */
#define HC_CHECK_SELFTEST 99          /* hcCudaSelfTestDeviceCheck: an index made up to be out of range */
