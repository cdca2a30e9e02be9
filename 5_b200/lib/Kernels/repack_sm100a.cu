// Pitch repack for 16-bit matrices. TMA needs every row of a tensor to start on a 16-byte
// boundary; a row-major fp16/bf16 matrix whose column count is not a multiple of 8 (for
// instance K = 1031 or N = 3073) does not satisfy that. This kernel copies such a matrix
// once into scratch memory with the pitch rounded up to 8 elements, after which the TMA
// kernels read the copy (the tensor map still carries the true extent, so everything past
// it is zero-filled as the hc kernel's masked loads require,
// examples/amdgpu_gfx11_wmma_matmul.py:316-323).
//
// One thread produces 8 consecutive destination elements (one 128-bit store). The source
// row may start at any 2-byte boundary: where its 8 elements start on a 4-byte boundary they
// are read with four 32-bit loads, otherwise with a 16-bit load, three 32-bit loads and a
// 16-bit load (the last piece of a row, which may be shorter, with 16-bit loads); neighbouring
// threads read neighbouring addresses, so the loads of a warp still coalesce.
#include "gemm_launch.h"

namespace hc {
namespace sm100 {

namespace {

struct RepackJob {
  const uint16_t *src;
  long long src_ld;
  uint16_t *dst;
  long long dst_ld;
  int rows;
  int cols;
};

// Blocks [0, blocks0) copy job0, the rest copy job1 (which may be empty): both operands of a
// GEMM are repacked by one launch.
__global__ void __launch_bounds__(256)
repack_pitch_kernel(RepackJob job0, RepackJob job1, int blocks0) {
  const bool second = static_cast<int>(blockIdx.x) >= blocks0;
  const RepackJob job = second ? job1 : job0;
  const long long block = second ? blockIdx.x - blocks0 : blockIdx.x;
  const long long blocks = second ? gridDim.x - blocks0 : blocks0;
  const int pieces_per_row = (job.cols + 7) >> 3;
  const long long total = static_cast<long long>(job.rows) * pieces_per_row;
  for (long long idx = block * blockDim.x + threadIdx.x; idx < total; idx += blocks * blockDim.x) {
    // (A 32-bit division when the number of pieces allows: the 64-bit one costs a hundred cycles.)
    const int row = total <= 0x7fffffffLL ? static_cast<int>(static_cast<unsigned>(idx) / static_cast<unsigned>(pieces_per_row))
                                          : static_cast<int>(idx / pieces_per_row);
    const int col0 = static_cast<int>(idx - static_cast<long long>(row) * pieces_per_row) << 3;
    const uint16_t *s = job.src + row * job.src_ld + col0;
    uint4 packed;
    if (col0 + 8 <= job.cols) {
      if ((reinterpret_cast<uintptr_t>(s) & 3) == 0) {
        const uint32_t *w = reinterpret_cast<const uint32_t *>(s);
        packed = make_uint4(__ldg(w), __ldg(w + 1), __ldg(w + 2), __ldg(w + 3));
      } else {
        // s + 1 is 4-byte aligned: elements 1..6 come as three words, 0 and 7 on their own.
        const uint32_t *w = reinterpret_cast<const uint32_t *>(s + 1);
        const uint32_t first = __ldg(s), w0 = __ldg(w), w1 = __ldg(w + 1), w2 = __ldg(w + 2), last = __ldg(s + 7);
        packed.x = first | (w0 << 16);
        packed.y = (w0 >> 16) | (w1 << 16);
        packed.z = (w1 >> 16) | (w2 << 16);
        packed.w = (w2 >> 16) | (last << 16);
      }
    } else {
      uint16_t v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        v[i] = (col0 + i < job.cols) ? __ldg(s + i) : static_cast<uint16_t>(0);
      packed.x = v[0] | (static_cast<uint32_t>(v[1]) << 16);
      packed.y = v[2] | (static_cast<uint32_t>(v[3]) << 16);
      packed.z = v[4] | (static_cast<uint32_t>(v[5]) << 16);
      packed.w = v[6] | (static_cast<uint32_t>(v[7]) << 16);
    }
    *reinterpret_cast<uint4 *>(job.dst + row * job.dst_ld + col0) = packed;
  }
}

int blocks_for(const RepackJob &job) {
  if (job.rows <= 0 || job.cols <= 0)
    return 0;
  const long long total = static_cast<long long>(job.rows) * ((job.cols + 7) >> 3);
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 8)
    blocks = 148LL * 8;
  return static_cast<int>(blocks);
}

bool valid_destination(const RepackJob &job) {
  return (job.dst_ld & 7) == 0 && (reinterpret_cast<uintptr_t>(job.dst) & 15) == 0;
}

} // namespace

cudaError_t launch_repack_pitch_two(const void *src0, long long src0_ld, void *dst0, long long dst0_ld,
                                    int rows0, int cols0, const void *src1, long long src1_ld, void *dst1,
                                    long long dst1_ld, int rows1, int cols1, cudaStream_t stream) {
  const RepackJob job0{static_cast<const uint16_t *>(src0), src0_ld, static_cast<uint16_t *>(dst0), dst0_ld,
                       rows0, cols0};
  const RepackJob job1{static_cast<const uint16_t *>(src1), src1_ld, static_cast<uint16_t *>(dst1), dst1_ld,
                       rows1, cols1};
  const int blocks0 = blocks_for(job0), blocks1 = blocks_for(job1);
  if (blocks0 + blocks1 == 0)
    return cudaSuccess;
  if ((blocks0 > 0 && !valid_destination(job0)) || (blocks1 > 0 && !valid_destination(job1)))
    return cudaErrorInvalidValue;
  repack_pitch_kernel<<<static_cast<unsigned>(blocks0 + blocks1), 256, 0, stream>>>(job0, job1, blocks0);
  return cudaGetLastError();
}

} // namespace sm100
} // namespace hc
