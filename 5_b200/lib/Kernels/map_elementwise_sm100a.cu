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
// written per element), so that is all there is to it: coalesced 16-byte accesses, enough of them
// in flight per thread, streaming cache hints (each byte is used once).
//
// The arithmetic is what NumPy does on float32 arrays with float32 (or weak Python) constants: one
// correctly rounded float32 operation per statement. __fmul_rn / __fadd_rn keep the compiler from
// contracting a multiply and an add into a fused multiply-add, which would round once instead of
// twice; maximum / minimum propagate NaN as NumPy's do. The result is therefore bit-identical to
// the reference simulator's.
#include "gemm_launch.h"

namespace hc {
namespace sm100 {

namespace {

__device__ __forceinline__ float map_max_nan(float a, float b) {
  float d;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}
__device__ __forceinline__ float map_min_nan(float a, float b) {
  float d;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}

__device__ __forceinline__ float apply_map_ops(float v, float w, const MapOps &ops) {
#pragma unroll
  for (int i = 0; i < kMaxMapOps; ++i) {
    if (i < ops.count) {
      const int kind = ops.kind[i];
      const float x = kind >= kMapAddOther ? w : ops.value[i];
      switch (kind) {
      case kMapScale:
      case kMapMulOther:
        v = __fmul_rn(v, x);
        break;
      case kMapAdd:
      case kMapAddOther:
        v = __fadd_rn(v, x);
        break;
      case kMapSubOther:
        v = __fsub_rn(v, x);
        break;
      case kMapReverseSub:
      case kMapReverseSubOther:
        v = __fsub_rn(x, v);
        break;
      case kMapMax:
      case kMapMaxOther:
        v = map_max_nan(v, x);
        break;
      default:  // kMapMin, kMapMinOther
        v = map_min_nan(v, x);
        break;
      }
    }
  }
  return v;
}

constexpr int kThreads = 256;
constexpr int kVectorsPerThread = 4;  // independent 16-byte loads in flight per thread and input

// kVec: all pointers are 16-byte aligned, so the body runs on float4; the tail (n % 4) and the
// unaligned case use 4-byte accesses (still coalesced).
template <bool kVec, bool kTwoInputs>
__global__ void __launch_bounds__(kThreads)
map_f32_kernel(const float *__restrict__ x, const float *__restrict__ y, float *__restrict__ out,
               long long n, MapOps ops) {
  const long long tid = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
  const long long threads = static_cast<long long>(gridDim.x) * kThreads;
  if (kVec) {
    const long long vectors = n >> 2;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    const float4 *y4 = reinterpret_cast<const float4 *>(y);
    float4 *o4 = reinterpret_cast<float4 *>(out);
    for (long long base = tid; base < vectors; base += threads * kVectorsPerThread) {
      float4 xv[kVectorsPerThread], yv[kVectorsPerThread];
#pragma unroll
      for (int j = 0; j < kVectorsPerThread; ++j) {
        const long long i = base + j * threads;
        if (i < vectors) {
          xv[j] = __ldcs(x4 + i);
          if (kTwoInputs)
            yv[j] = __ldcs(y4 + i);
        }
      }
#pragma unroll
      for (int j = 0; j < kVectorsPerThread; ++j) {
        const long long i = base + j * threads;
        if (i < vectors) {
          float4 r;
          r.x = apply_map_ops(xv[j].x, kTwoInputs ? yv[j].x : 0.0f, ops);
          r.y = apply_map_ops(xv[j].y, kTwoInputs ? yv[j].y : 0.0f, ops);
          r.z = apply_map_ops(xv[j].z, kTwoInputs ? yv[j].z : 0.0f, ops);
          r.w = apply_map_ops(xv[j].w, kTwoInputs ? yv[j].w : 0.0f, ops);
          __stcs(o4 + i, r);
        }
      }
    }
    const long long tail = vectors << 2;
    if (tid < n - tail)
      out[tail + tid] = apply_map_ops(x[tail + tid], kTwoInputs ? y[tail + tid] : 0.0f, ops);
  } else {
    for (long long base = tid; base < n; base += threads * kVectorsPerThread) {
      float xv[kVectorsPerThread], yv[kVectorsPerThread];
#pragma unroll
      for (int j = 0; j < kVectorsPerThread; ++j) {
        const long long i = base + j * threads;
        if (i < n) {
          xv[j] = __ldcs(x + i);
          if (kTwoInputs)
            yv[j] = __ldcs(y + i);
        }
      }
#pragma unroll
      for (int j = 0; j < kVectorsPerThread; ++j) {
        const long long i = base + j * threads;
        if (i < n)
          __stcs(out + i, apply_map_ops(xv[j], kTwoInputs ? yv[j] : 0.0f, ops));
      }
    }
  }
}

} // namespace

int map_grid(long long n, int sm_count) {
  // Persistent grid: eight CTAs of 256 threads per SM (all 2048 thread slots), fewer when the
  // array is too short to give every thread a vector.
  const long long wanted = (n / 4 + kThreads - 1) / kThreads;
  const long long most = static_cast<long long>(sm_count > 0 ? sm_count : 148) * 8;
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
  const int grid = map_grid(vec ? n : n * 4, sm_count);
  if (vec && two)
    map_f32_kernel<true, true><<<grid, kThreads, 0, stream>>>(x, y, out, n, ops);
  else if (vec)
    map_f32_kernel<true, false><<<grid, kThreads, 0, stream>>>(x, y, out, n, ops);
  else if (two)
    map_f32_kernel<false, true><<<grid, kThreads, 0, stream>>>(x, y, out, n, ops);
  else
    map_f32_kernel<false, false><<<grid, kThreads, 0, stream>>>(x, y, out, n, ops);
  return cudaGetLastError();
}

} // namespace sm100
} // namespace hc
