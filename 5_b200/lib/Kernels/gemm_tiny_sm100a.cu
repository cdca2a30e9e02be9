// Small products:  C = ops((C +) A * B) with a short k, on the float32 pipes, one small CTA per
// 16x16 tile of C.
//
// Below about a million multiply-adds the tensor-core kernels are all overhead: tensor-memory
// allocation, barrier set-up, the first TMA round trip, the drain through shared memory and the
// TMA store cost about 8 us whatever the product (benchmark configuration 1, 64^3: 7.9 us of
// kernel time). This kernel has none of that: a CTA of 64 threads computes a 16 x 16 tile (so that
// even a 64 x 64 product runs on 16 SMs at once), stages its rows of A and columns of B for up to
// 128 values of k in shared memory with ordinary loads (any pitch, any alignment: no repack), each
// thread keeps 2 x 2 outputs in registers, and the tile is stored with plain stores.
//
// It also computes exactly what the reference simulator computes for the hc kernel
// (examples/amdgpu_gfx11_wmma_matmul.py:180-190, 315-324): every accumulator starts at +0 (or at
// C's previous value in the accumulating member) and takes its products one k at a time in
// ascending order, each product and each sum rounded to float32 on its own -- __fmul_rn and
// __fadd_rn, no fused multiply-add (the product of two 16-bit values is exact in float32 unless it
// underflows, which is the one case where fusing would show). The element-wise operations then run
// in float32 in their order and a 16-bit C is rounded to nearest even. The result is therefore
// bit-identical to the simulator's, where the tensor-core kernels agree with it to rounding.
#include "gemm_epilogue.cuh"
#include "gemm_launch.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace hc {
namespace sm100 {

namespace {

constexpr int kTile = 16;     // rows and columns of C per CTA: a 64x64 product spreads over 16 SMs
constexpr int kThreads = 64;  // 8 x 8, a thread owns 2 x 2 outputs
constexpr int kChunk = 128;   // k staged per step: the whole k-loop of the products AUTO sends here
constexpr int kPitch = kTile + 2;  // floats; keeps the 8-byte reads aligned

__device__ __forceinline__ float widen(const void *base, long long index, int dtype) {
  if (dtype == kDTypeF16)
    return __half2float(static_cast<const __half *>(base)[index]);
  return __bfloat162float(static_cast<const __nv_bfloat16 *>(base)[index]);
}

__global__ void __launch_bounds__(kThreads)
gemm_tiny_kernel(const void *__restrict__ a, long long lda, const void *__restrict__ b, long long ldb, void *c_any,
                 long long ldc, int m, int n, int k, int dtype, int b_layout, Epilogue ep) {
  __shared__ __align__(8) float a_s[kChunk * kPitch];  // a_s[kk][row]
  __shared__ __align__(8) float b_s[kChunk * kPitch];  // b_s[kk][column]
  const int row0 = blockIdx.y * kTile, col0 = blockIdx.x * kTile;
  const int ty = threadIdx.x >> 3, tx = threadIdx.x & 7;

  float acc[2][2];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int row = row0 + ty * 2 + i, col = col0 + tx * 2 + j;
      // (Accumulation is only offered for a float32 C.)
      acc[i][j] = (ep.accumulate && row < m && col < n)
                      ? static_cast<const float *>(c_any)[static_cast<long long>(row) * ldc + col] : 0.0f;
    }

  for (int k0 = 0; k0 < k; k0 += kChunk) {
    const int depth = min(kChunk, k - k0);
    __syncthreads();  // the previous chunk has been read
    // The usual case first: rows of A and B that can be read 16 bytes at a time (aligned bases and
    // pitches, whole groups of eight k, a full tile of columns). All of a thread's loads -- four per
    // operand at most -- are issued before anything is stored, so the CTA pays one memory latency;
    // with two warps per CTA nothing else would hide more.
    const bool whole = depth % 8 == 0;
    const bool a_wide = whole && (reinterpret_cast<uintptr_t>(a) & 15) == 0 && (lda & 7) == 0;
    const bool b_wide = (reinterpret_cast<uintptr_t>(b) & 15) == 0 && (ldb & 7) == 0 &&
                        (b_layout == kBLayoutKN ? col0 + kTile <= n : whole);
    if (a_wide && b_wide) {
      constexpr int kSlots = kTile * kChunk / 8 / kThreads;  // 4 vectors of eight values per thread and operand
      uint4 av[kSlots], bv[kSlots];
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int i = 0; i < kSlots; ++i) {
        const int v = i * kThreads + static_cast<int>(threadIdx.x);
        const int row = v / (kChunk / 8), q = v % (kChunk / 8);  // A, and B stored [n, k]: eight k of one row
        av[i] = (q * 8 < depth && row0 + row < m)
                    ? __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(a) +
                                                            static_cast<long long>(row0 + row) * lda + k0 + q * 8))
                    : zero;
        if (b_layout == kBLayoutKN) {
          const int kk = v / 2, half = v % 2;  // eight columns of one k
          bv[i] = kk < depth ? __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(b) +
                                                                     static_cast<long long>(k0 + kk) * ldb + col0 + half * 8))
                             : zero;
        } else {
          bv[i] = (q * 8 < depth && col0 + row < n)
                      ? __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(b) +
                                                              static_cast<long long>(col0 + row) * ldb + k0 + q * 8))
                      : zero;
        }
      }
      auto widen_bits = [&](uint32_t word, int upper) {
        const uint16_t bits = static_cast<uint16_t>(upper ? word >> 16 : word & 0xffffu);
        return dtype == kDTypeF16 ? __half2float(__ushort_as_half(bits)) : __bfloat162float(__ushort_as_bfloat16(bits));
      };
#pragma unroll
      for (int i = 0; i < kSlots; ++i) {
        const int v = i * kThreads + static_cast<int>(threadIdx.x);
        const int row = v / (kChunk / 8), q = v % (kChunk / 8);
        const uint32_t aw[4] = {av[i].x, av[i].y, av[i].z, av[i].w};
        const uint32_t bw[4] = {bv[i].x, bv[i].y, bv[i].z, bv[i].w};
        if (q * 8 < depth) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            a_s[(q * 8 + j) * kPitch + row] = widen_bits(aw[j / 2], j % 2);
        }
        if (b_layout == kBLayoutKN) {
          const int kk = v / 2, half = v % 2;
          if (kk < depth) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              b_s[kk * kPitch + half * 8 + j] = widen_bits(bw[j / 2], j % 2);
          }
        } else if (q * 8 < depth) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            b_s[(q * 8 + j) * kPitch + row] = widen_bits(bw[j / 2], j % 2);
        }
      }
    } else {
    // Sixteen elements per thread and batch: all loads of a batch are issued before the first
    // store to shared memory, so their latencies overlap. Element e of a staged piece is
    // (e / kChunk, e % kChunk) or (e / kTile, e % kTile): divisions by constants, since with two
    // warps per CTA a run-time division is a hundred cycles of dependent instructions nothing hides.
    auto stage = [&](float *dst, auto value_of, auto place_of) {
#pragma unroll 1
      for (int e0 = 0; e0 < kTile * kChunk; e0 += 16 * kThreads) {
        float value[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          value[i] = value_of(e0 + i * kThreads + static_cast<int>(threadIdx.x));
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int place = place_of(e0 + i * kThreads + static_cast<int>(threadIdx.x));
          if (place >= 0)
            dst[place] = value[i];
        }
      }
    };
    // A is stored [m, k]: consecutive threads take consecutive k of one row.
    stage(a_s,
          [&](int e) {
            const int row = e / kChunk, kk = e % kChunk;
            return (kk < depth && row0 + row < m) ? widen(a, static_cast<long long>(row0 + row) * lda + k0 + kk, dtype)
                                                  : 0.0f;
          },
          [&](int e) { return e % kChunk < depth ? (e % kChunk) * kPitch + e / kChunk : -1; });
    if (b_layout == kBLayoutKN) {
      // B stored [k, n]: consecutive threads take consecutive columns of one k.
      stage(b_s,
            [&](int e) {
              const int kk = e / kTile, col = e % kTile;
              return (kk < depth && col0 + col < n) ? widen(b, static_cast<long long>(k0 + kk) * ldb + col0 + col, dtype)
                                                    : 0.0f;
            },
            [&](int e) { return e / kTile < depth ? (e / kTile) * kPitch + e % kTile : -1; });
    } else {
      // B stored [n, k]: consecutive threads take consecutive k of one column.
      stage(b_s,
            [&](int e) {
              const int col = e / kChunk, kk = e % kChunk;
              return (kk < depth && col0 + col < n) ? widen(b, static_cast<long long>(col0 + col) * ldb + k0 + kk, dtype)
                                                    : 0.0f;
            },
            [&](int e) { return e % kChunk < depth ? (e % kChunk) * kPitch + e / kChunk : -1; });
    }
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < depth; ++kk) {
      const float2 av = *reinterpret_cast<const float2 *>(a_s + kk * kPitch + ty * 2);
      const float2 bv = *reinterpret_cast<const float2 *>(b_s + kk * kPitch + tx * 2);
      acc[0][0] = __fadd_rn(acc[0][0], __fmul_rn(av.x, bv.x));
      acc[0][1] = __fadd_rn(acc[0][1], __fmul_rn(av.x, bv.y));
      acc[1][0] = __fadd_rn(acc[1][0], __fmul_rn(av.y, bv.x));
      acc[1][1] = __fadd_rn(acc[1][1], __fmul_rn(av.y, bv.y));
    }
  }

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + ty * 2 + i;
    if (row >= m)
      continue;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int col = col0 + tx * 2 + j;
      if (col >= n)
        continue;
      float v = acc[i][j];
      for (int op = 0; op < ep.op_count; ++op) {
        const int kind = ep.op_kind[op];
        const float x = kind == kEpilogueBiasColumn ? __ldg(ep.bias + col) : ep.op_value[op];
        // np.maximum / np.minimum as the simulator's NumPy computes them: a NaN stays, and of two
        // equal values (zeros of either sign) the constant is taken.
        v = kind == kEpilogueScale ? __fmul_rn(v, x)
          : kind == kEpilogueMax   ? ((v > x || v != v) ? v : x)
          : kind == kEpilogueMin   ? ((v < x || v != v) ? v : x)
                                   : __fadd_rn(v, x);
      }
      store_c_element(c_any, static_cast<long long>(row) * ldc + col, v, ep.c_dtype);
    }
  }
}

} // namespace

bool tiny_takes(long long m, long long n, long long k, int dtype, int sm_count) {
  // Where it beats the 8 us floor of the tensor-core kernels without question: C no larger than
  // 64 x 64 (sixteen tiles) and a k-loop that is staged in one go. The kernel itself takes any shape.
  (void)sm_count;
  return !dtype_is_8bit(dtype) && m >= 1 && n >= 1 && k >= 1 && m <= 64 && n <= 64 && k <= kChunk;
}

int tiny_tile() { return kTile; }

cudaError_t launch_gemm_tiny(const void *a, long long lda, const void *b, long long ldb, void *c, long long ldc, int m,
                             int n, int k, int dtype, int b_layout, const Epilogue &ep, cudaStream_t stream) {
  if (m <= 0 || n <= 0)
    return cudaSuccess;
  if (dtype_is_8bit(dtype) || ep.push_count != 0 || (ep.c_dtype != kCTypeF32 && ep.accumulate != 0))
    return cudaErrorInvalidValue;
  const dim3 grid(static_cast<unsigned>((n + kTile - 1) / kTile), static_cast<unsigned>((m + kTile - 1) / kTile), 1);
  if (grid.y > 65535u)
    return cudaErrorInvalidValue;
  gemm_tiny_kernel<<<grid, kThreads, 0, stream>>>(a, lda, b, ldb, c, ldc, m, n, k, dtype, b_layout, ep);
  return cudaGetLastError();
}

} // namespace sm100
} // namespace hc
