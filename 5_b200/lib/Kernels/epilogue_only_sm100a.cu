// The degenerate member of the GEMM family: k == 0 with element-wise work fused into the store.
// There is no product, so C = ops(accumulate ? C : 0). In the hc kernel this is the launch whose
// k-loop runs zero times: the accumulators keep their starting values, the element-wise
// statements after the loop still run, and the store still happens.
#include "gemm_epilogue.cuh"
#include "gemm_launch.h"

namespace hc {
namespace sm100 {

namespace {

__global__ void __launch_bounds__(256)
epilogue_only_kernel(void *c, int m, int n, long long ldc, Epilogue ep) {
  const long long total = static_cast<long long>(m) * n;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(idx / n);
    const int col = static_cast<int>(idx - static_cast<long long>(row) * n);
    const long long index = row * ldc + col;
    // (Accumulation is only offered for a float32 C.)
    const float v = finish_value(0.0f, static_cast<const float *>(c) + index, col, ep);
    store_c_element(c, index, v, ep.c_dtype);
  }
}

} // namespace

cudaError_t launch_epilogue_only(void *c, int m, int n, long long ldc, const Epilogue &ep,
                                 cudaStream_t stream) {
  if (m <= 0 || n <= 0)
    return cudaSuccess;
  const long long total = static_cast<long long>(m) * n;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 8)
    blocks = 148LL * 8;
  epilogue_only_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(c, m, n, ldc, ep);
  return cudaGetLastError();
}

} // namespace sm100
} // namespace hc
