// Pitch repack for 16-bit matrices. TMA needs every row of a tensor to start on a 16-byte
// boundary; a row-major fp16/bf16 matrix whose column count is not a multiple of 8 (for
// instance K = 1031 or N = 3073) does not satisfy that. This kernel copies such a matrix
// once into scratch memory with the pitch rounded up to 8 elements, after which the TMA
// kernels read the copy (the tensor map still carries the true extent, so everything past
// it is zero-filled as the hc kernel's masked loads require,
// examples/amdgpu_gfx11_wmma_matmul.py:316-323).
//
// One thread produces 8 consecutive destination elements (one 128-bit store). The source
// row may start at any 2-byte boundary, so it is read with 16-bit loads; neighbouring
// threads read neighbouring addresses, so the loads of a warp still coalesce.
#include "gemm_launch.h"

namespace hc {
namespace sm100 {

namespace {

__global__ void __launch_bounds__(256)
repack_pitch_kernel(const uint16_t *__restrict__ src, long long src_ld, uint16_t *__restrict__ dst,
                    long long dst_ld, int rows, int cols) {
  const int pieces_per_row = (cols + 7) >> 3;
  const long long total = static_cast<long long>(rows) * pieces_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(idx / pieces_per_row);
    const int col0 = static_cast<int>(idx - static_cast<long long>(row) * pieces_per_row) << 3;
    const uint16_t *s = src + row * src_ld + col0;
    uint16_t v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      v[i] = (col0 + i < cols) ? __ldg(s + i) : static_cast<uint16_t>(0);
    uint4 packed;
    packed.x = v[0] | (static_cast<uint32_t>(v[1]) << 16);
    packed.y = v[2] | (static_cast<uint32_t>(v[3]) << 16);
    packed.z = v[4] | (static_cast<uint32_t>(v[5]) << 16);
    packed.w = v[6] | (static_cast<uint32_t>(v[7]) << 16);
    *reinterpret_cast<uint4 *>(dst + row * dst_ld + col0) = packed;
  }
}

} // namespace

cudaError_t launch_repack_pitch(const void *src, long long src_ld, void *dst, long long dst_ld,
                                int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0)
    return cudaSuccess;
  if ((dst_ld & 7) != 0 || (reinterpret_cast<uintptr_t>(dst) & 15) != 0)
    return cudaErrorInvalidValue;
  const long long total = static_cast<long long>(rows) * ((cols + 7) >> 3);
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 16)
    blocks = 148LL * 16;
  repack_pitch_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const uint16_t *>(src), src_ld, static_cast<uint16_t *>(dst), dst_ld, rows, cols);
  return cudaGetLastError();
}

} // namespace sm100
} // namespace hc
