// Masked element-wise map for sm_100a:  out[i] = ops(x[i] [, y[i]])  for i in [0, n), float32.
//
// The hc kernel class behind it is the one-dimensional masked load / compute / store kernel of the
// reference's simulator tests (tests/test_simulator.py:210-224):
//
//     gid = group.work_offset[0]
//     vec = group.vload(x[gid:], shape=(G,))     # elements past the end of x are inactive
//     group.store(y[gid:], vec + 2)              # only active elements inside y are written
//
// with work_shape=(W,), group_shape=(G,): every element below W is loaded once, transformed and
// stored once, nothing past the end is touched (hc/simulator.py:1338-1357, 1441-1458). The group
// size is not observable, so the launch is re-tiled: a persistent grid of a multiple of the SM
// count walks the array in 128-bit vectors. The kernel is HBM-bound (4 bytes read per input and 4
// written per element): coalesced 16-byte accesses, eight of them in flight per thread and input,
// streaming cache hints (each byte is used once), and an operation loop whose dispatch is paid once
// per 32 values.
//
// The arithmetic is what NumPy does on float32 arrays with float32 (or weak Python) constants: one
// correctly rounded float32 operation per statement. __fmul_rn / __fadd_rn keep the compiler from
// contracting a multiply and an add into a fused multiply-add, which would round once instead of
// twice; maximum / minimum propagate NaN as NumPy's do. The result is therefore bit-identical to
// the reference simulator's.
#include "gemm_launch.h"

#include <cstdlib>

namespace hc {
namespace sm100 {

namespace {

// maximum / minimum as NumPy computes them on float32 arrays (x86: the SIMD max/min select, plus
// NaN propagation): the first operand if it is greater (smaller) or a NaN, otherwise the second. A
// NaN in either operand therefore gives NaN, and two zeros of opposite sign give the second one.
__device__ __forceinline__ float numpy_max(float first, float second) {
  return ((first > second) | (first != first)) ? first : second;  // (no short-circuit: branch-free)
}
__device__ __forceinline__ float numpy_min(float first, float second) {
  return ((first < second) | (first != first)) ? first : second;
}

constexpr int kThreads = 256;

// The operations on the N values a thread holds. The kind of each operation is the same for the
// whole grid, so it is branched on once per operation and batch of values, not per element; every
// operation is one correctly rounded float32 instruction per value.
template <int N>
__device__ __forceinline__ void apply_map_ops(float (&v)[N], const float (&w)[N], const MapOps &ops) {
#pragma unroll 1
  for (int i = 0; i < ops.count; ++i) {
    const int kind = ops.kind[i];
    const float c = ops.value[i];
    switch (kind) {
    case kMapScale: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = __fmul_rn(v[j], c);
      break;
    }
    case kMapAdd: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = __fadd_rn(v[j], c);
      break;
    }
    case kMapMax: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = numpy_max(v[j], c);
      break;
    }
    case kMapMin: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = numpy_min(v[j], c);
      break;
    }
    case kMapReverseSub: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = __fsub_rn(c, v[j]);
      break;
    }
    case kMapReverseMax: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = numpy_max(c, v[j]);
      break;
    }
    case kMapReverseMin: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = numpy_min(c, v[j]);
      break;
    }
    case kMapAddOther: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = __fadd_rn(v[j], w[j]);
      break;
    }
    case kMapSubOther: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = __fsub_rn(v[j], w[j]);
      break;
    }
    case kMapReverseSubOther: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = __fsub_rn(w[j], v[j]);
      break;
    }
    case kMapMulOther: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = __fmul_rn(v[j], w[j]);
      break;
    }
    case kMapMaxOther: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = numpy_max(v[j], w[j]);
      break;
    }
    case kMapMinOther: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = numpy_min(v[j], w[j]);
      break;
    }
    case kMapReverseMaxOther: {
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = numpy_max(w[j], v[j]);
      break;
    }
    default: {  // kMapReverseMinOther
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = numpy_min(w[j], v[j]);
      break;
    }
    }
  }
}

// kVec: all pointers are 16-byte aligned, so the body runs on float4; the tail (n % 4) and the
// unaligned case use 4-byte accesses (still coalesced).
// kVectorsPerThread: independent 16-byte loads in flight per thread and input, and the number of
// values (4 x that) one pass of the operation loop works on.
template <bool kVec, bool kTwoInputs, int kVectorsPerThread>
__global__ void __launch_bounds__(kThreads)
map_f32_kernel(const float *__restrict__ x, const float *__restrict__ y, float *__restrict__ out,
               long long n, MapOps ops) {
  constexpr int kValues = 4 * kVectorsPerThread;
  const long long tid = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
  const long long threads = static_cast<long long>(gridDim.x) * kThreads;
  if (kVec) {
    const long long vectors = n >> 2;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    const float4 *y4 = reinterpret_cast<const float4 *>(y);
    float4 *o4 = reinterpret_cast<float4 *>(out);
    // A CTA's pass covers kVectorsPerThread x 4 KB in a row (vector j of a thread lies 4 KB behind
    // vector j - 1), and the passes of the grid follow one another through the array.
    constexpr long long kStride = kThreads;
    for (long long base = static_cast<long long>(blockIdx.x) * (kThreads * kVectorsPerThread) + threadIdx.x;
         base < vectors; base += threads * kVectorsPerThread) {
      float v[kValues], w[kValues];
#pragma unroll
      for (int j = 0; j < kVectorsPerThread; ++j) {
        const long long i = base + j * kStride;
        float4 xv = make_float4(0.f, 0.f, 0.f, 0.f), yv = xv;
        if (i < vectors) {
          xv = __ldcs(x4 + i);
          if (kTwoInputs)
            yv = __ldcs(y4 + i);
        }
        v[4 * j] = xv.x, v[4 * j + 1] = xv.y, v[4 * j + 2] = xv.z, v[4 * j + 3] = xv.w;
        w[4 * j] = yv.x, w[4 * j + 1] = yv.y, w[4 * j + 2] = yv.z, w[4 * j + 3] = yv.w;
      }
      apply_map_ops(v, w, ops);
#pragma unroll
      for (int j = 0; j < kVectorsPerThread; ++j) {
        const long long i = base + j * kStride;
        if (i < vectors)
          __stcs(o4 + i, make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
      }
    }
    const long long tail = vectors << 2;
    if (tid < n - tail) {
      float v[1] = {x[tail + tid]}, w[1] = {kTwoInputs ? y[tail + tid] : 0.0f};
      apply_map_ops(v, w, ops);
      out[tail + tid] = v[0];
    }
  } else {
    for (long long base = static_cast<long long>(blockIdx.x) * (kThreads * kValues) + threadIdx.x; base < n;
         base += threads * kValues) {
      float v[kValues], w[kValues];
#pragma unroll
      for (int j = 0; j < kValues; ++j) {
        const long long i = base + j * kThreads;
        v[j] = i < n ? __ldcs(x + i) : 0.0f;
        w[j] = (kTwoInputs && i < n) ? __ldcs(y + i) : 0.0f;
      }
      apply_map_ops(v, w, ops);
#pragma unroll
      for (int j = 0; j < kValues; ++j) {
        const long long i = base + j * kThreads;
        if (i < n)
          __stcs(out + i, v[j]);
      }
    }
  }
}

} // namespace

int map_grid(long long n, int sm_count) {
  // Persistent grid: eight CTAs of 256 threads per SM (all 2048 thread slots), fewer when the
  // array is too short to give every thread a vector.
  const long long wanted = (n / 4 + kThreads - 1) / kThreads;
  long long per_sm = 8;
  if (const char *forced = std::getenv("HC_CUDA_MAP_CTAS_PER_SM")) {  // tuning aid
    const long long v = std::atoll(forced);
    if (v >= 1 && v <= 64)
      per_sm = v;
  }
  const long long most = static_cast<long long>(sm_count > 0 ? sm_count : 148) * per_sm;
  const long long grid = wanted < 1 ? 1 : (wanted < most ? wanted : most);
  return static_cast<int>(grid);
}

cudaError_t launch_map_f32(const float *x, const float *y, float *out, long long n, const MapOps &ops,
                           int sm_count, cudaStream_t stream) {
  if (n <= 0)
    return cudaSuccess;
  if (ops.count < 0 || ops.count > kMaxMapOps)
    return cudaErrorInvalidValue;
  const bool two = y != nullptr;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) |
                         (two ? reinterpret_cast<uintptr_t>(y) : 0);
  const bool vec = (bits & 15) == 0;
  const int grid = map_grid(n, sm_count);
  // Eight vectors (32 values) per pass of the operation loop: the dispatch of an operation costs a
  // fixed hundred or so issue slots, so a chain of seven operations ran at 1.7 / 3.3 / 5.7 TB/s with
  // 2 / 4 / 8 vectors per pass (a single operation: 6.0 / 6.4 / 6.5 TB/s).
  int vectors = 8;
  if (const char *forced = std::getenv("HC_CUDA_MAP_VECTORS"))  // tuning aid: 2, 4 or 8
    vectors = std::atoi(forced);
#define HC_LAUNCH_MAP(V)                                                                          \
  do {                                                                                            \
    if (vec && two)                                                                               \
      map_f32_kernel<true, true, V><<<grid, kThreads, 0, stream>>>(x, y, out, n, ops);            \
    else if (vec)                                                                                 \
      map_f32_kernel<true, false, V><<<grid, kThreads, 0, stream>>>(x, y, out, n, ops);           \
    else if (two)                                                                                 \
      map_f32_kernel<false, true, V><<<grid, kThreads, 0, stream>>>(x, y, out, n, ops);           \
    else                                                                                          \
      map_f32_kernel<false, false, V><<<grid, kThreads, 0, stream>>>(x, y, out, n, ops);          \
  } while (0)
  if (vectors == 4)
    HC_LAUNCH_MAP(4);
  else if (vectors == 2)
    HC_LAUNCH_MAP(2);
  else
    HC_LAUNCH_MAP(8);
#undef HC_LAUNCH_MAP
  return cudaGetLastError();
}

} // namespace sm100
} // namespace hc
