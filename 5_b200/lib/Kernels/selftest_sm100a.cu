// Self-test of the bounded-wait mechanism every GEMM kernel relies on.
//
// The kernels never spin without limit: `mbar_wait` gives up after a cycle budget, the CTA
// records a status code and returns, and the host reports HC_CUDA_ERR_DEVICE_TIMEOUT at the
// next synchronise while the context stays usable. This file makes that path observable without
// faulting or hanging anything: one thread waits, with a budget of about a millisecond, on an
// mbarrier that nothing ever signals, and then follows the same give-up path as the GEMM
// kernels (abort flag -> status word -> return).
#include "device_checks.cuh"
#include "gemm_launch.h"
#include "sm100_ptx.cuh"

namespace hc {
namespace sm100 {

namespace {

__global__ void __launch_bounds__(32) wait_that_runs_out_kernel(long long budget_cycles, int *status) {
  __shared__ __align__(8) unsigned long long barrier;
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(smem_u32(&barrier), 1);
    mbar_fence_init();
    const bool completed = mbar_wait(smem_u32(&barrier), 0, &abort_word, budget_cycles);
    if (!completed && abort_word != 0)
      atomicExch(status, kStatusDeviceWaitTimeout);
  }
}

// The checked build's self-test: an index past the end of a small array is checked, found out of
// range, recorded, and the access is skipped.
__global__ void __launch_bounds__(32) check_that_fails_kernel(int *status, int index, int *sink) {
  __shared__ int values[8];
  if (threadIdx.x < 8)
    values[threadIdx.x] = static_cast<int>(threadIdx.x);
  __syncthreads();
  if (threadIdx.x == 0 && HC_CHECK(status, nullptr, HC_CHECK_SELFTEST, index >= 0 && index < 8))
    *sink = values[index];  // (not reached with the index the host passes)
}

} // namespace

bool library_is_checked() {
#ifdef HC_CUDA_CHECKED
  return true;
#else
  return false;
#endif
}

cudaError_t launch_check_selftest(int *status, cudaStream_t stream) {
  if (!library_is_checked())
    return cudaErrorNotSupported;
  check_that_fails_kernel<<<1, 32, 0, stream>>>(status, 8, status);
  return cudaGetLastError();
}

cudaError_t launch_wait_selftest(long long budget_cycles, int *status, cudaStream_t stream) {
  if (budget_cycles < 1000)
    budget_cycles = 1000;
  if (budget_cycles > 200000000LL)
    budget_cycles = 200000000LL;  // never more than ~0.1 s
  wait_that_runs_out_kernel<<<1, 32, 0, stream>>>(budget_cycles, status);
  return cudaGetLastError();
}

} // namespace sm100
} // namespace hc
