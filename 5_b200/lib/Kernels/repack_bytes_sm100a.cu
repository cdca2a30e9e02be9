// Repack for 8-bit (float8) operands: copy, or transpose, a matrix of bytes into scratch memory
// with a TMA-friendly pitch.
//
// tcgen05.mma.kind::f8f6f4 is fed K-major operands here (k contiguous): A as [M, K] and B as
// [N, K]. An hc kernel whose float8 `b` is `Buffer[K, N]` stores B the other way round, so that B
// is transposed once into scratch before the GEMM reads it; a float8 operand that is already
// K-major but whose pitch or base TMA cannot address (not a multiple of 16 bytes) is copied the
// same way the 16-bit repack does. The tensor map still carries the true extents, so everything
// past them is zero-filled as the hc kernel's masked loads require
// (examples/amdgpu_gfx11_wmma_matmul.py:316-323).
//
// HBM-bound helper kernels: bytes read + bytes written = 2 x rows x cols.
#include "gemm_launch.h"

namespace hc {
namespace sm100 {

namespace {

constexpr int kTile = 64;

// dst[c][r] = src[r][c]: 64 x 64 byte tiles through shared memory, so that both the reads (along
// a source row) and the writes (along a destination row) touch consecutive bytes.
__global__ void __launch_bounds__(256)
transpose_bytes_kernel(const uint8_t *__restrict__ src, long long src_ld, uint8_t *__restrict__ dst,
                       long long dst_ld, int rows, int cols) {
  __shared__ uint8_t tile[kTile][kTile + 4];
  const int tx = static_cast<int>(threadIdx.x & 63), ty = static_cast<int>(threadIdx.x >> 6);
  const int tiles_c = (cols + kTile - 1) / kTile;
  const long long tiles = static_cast<long long>((rows + kTile - 1) / kTile) * tiles_c;
  for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
    const int r0 = static_cast<int>(t / tiles_c) * kTile, c0 = static_cast<int>(t % tiles_c) * kTile;
    for (int r = ty; r < kTile; r += 4)
      if (r0 + r < rows && c0 + tx < cols)
        tile[r][tx] = __ldg(src + static_cast<long long>(r0 + r) * src_ld + c0 + tx);
    __syncthreads();
    for (int c = ty; c < kTile; c += 4)
      if (c0 + c < cols && r0 + tx < rows)
        dst[static_cast<long long>(c0 + c) * dst_ld + r0 + tx] = tile[tx][c];
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256)
copy_bytes_kernel(const uint8_t *__restrict__ src, long long src_ld, uint8_t *__restrict__ dst, long long dst_ld,
                  int rows, int cols) {
  const long long total = static_cast<long long>(rows) * cols;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / cols, c = idx - r * cols;
    dst[r * dst_ld + c] = __ldg(src + r * src_ld + c);
  }
}

} // namespace

cudaError_t launch_repack_bytes(const void *src, long long src_ld, void *dst, long long dst_ld, int rows,
                                int cols, bool transpose, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0)
    return cudaSuccess;
  if ((dst_ld & 15) != 0 || (reinterpret_cast<uintptr_t>(dst) & 15) != 0)
    return cudaErrorInvalidValue;
  const uint8_t *s = static_cast<const uint8_t *>(src);
  uint8_t *d = static_cast<uint8_t *>(dst);
  if (transpose) {
    const long long tiles = static_cast<long long>((rows + kTile - 1) / kTile) * ((cols + kTile - 1) / kTile);
    const unsigned grid = static_cast<unsigned>(tiles < 148LL * 16 ? tiles : 148LL * 16);
    transpose_bytes_kernel<<<grid, 256, 0, stream>>>(s, src_ld, d, dst_ld, rows, cols);
  } else {
    const long long total = static_cast<long long>(rows) * cols;
    long long blocks = (total + 255) / 256;
    if (blocks > 148LL * 16)
      blocks = 148LL * 16;
    copy_bytes_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(s, src_ld, d, dst_ld, rows, cols);
  }
  return cudaGetLastError();
}

} // namespace sm100
} // namespace hc
