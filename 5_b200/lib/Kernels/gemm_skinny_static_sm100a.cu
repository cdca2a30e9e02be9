// hcCudaGemmSkinnyStatic: the skinny GEMM for callers that must not allocate device memory.
//
// The regular path (hcCudaGemm) keeps the split-k partial sums and arrival counters of the
// skinny kernel in scratch memory that the context obtains with cudaMalloc and grows on
// demand. Some users of this library cannot afford that call at launch time:
//   * a process whose GPU memory is already handed out in full to another allocator (an
//     inference server that reserves the whole device for its own pool at start-up), where
//     a late cudaMalloc simply fails;
//   * a latency-sensitive loop that shares the GPU with other streams, because cudaMalloc
//     and cudaFree synchronise the whole device and would stall those streams.
// For them this file offers one entry point that allocates nothing: the scratch lives in a
// file-scope __device__ array that is part of the loaded module (so every GPU that loads the
// library holds kStaticScratchBytes of it until the process exits), and the caller passes
// only inputs and outputs.
//
// Consequences of the shared array, which callers must respect:
//   * Every call on a device uses the same scratch. Two calls whose kernels may overlap on
//     the GPU (different streams, no dependency) race on it; serialise them.
//   * The array keeps whatever the previous call left. The words that must start at zero
//     (status word, arrival counters) are cleared on the caller's stream before each launch;
//     the partial sums are fully rewritten before they are read.
//   * Problems whose scratch would not fit are rejected with HC_CUDA_ERR_UNSUPPORTED.
#include "hc-c/Cuda.h"

#include "gemm_launch.h"

#include <cstdio>
#include <mutex>
#include <string>

namespace {

// Layout of the static scratch: [status word, padded to 256 B][counters 16 KiB][partials 8 MiB].
constexpr size_t kStatusBytes = 256;
constexpr size_t kCounterBytes = 16 * 1024;             // n <= 131072 columns
constexpr size_t kPartialBytes = 8u * 1024u * 1024u;    // splits * m * round_up(n, 128) * 4 bytes
constexpr size_t kStaticScratchBytes = kStatusBytes + kCounterBytes + kPartialBytes;
static_assert(kStaticScratchBytes == HC_CUDA_STATIC_SCRATCH_BYTES, "header and array size differ");

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DeviceSetup {
  bool ready = false;
  unsigned char *scratch = nullptr;  // device address of g_static_scratch on this device
  int sm_count = 0;
  EncodeTiledFn encode = nullptr;
};

constexpr int kMaxDevices = 64;
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;
thread_local std::string g_static_error;

int fail(int status, const std::string &text) {
  g_static_error = text;
  return status;
}

// One-time set-up for the current device. `g_static_scratch` names a host-side handle of
// the device array, not a device address: the address kernels can use has to be asked for
// with cudaGetSymbolAddress while the device is current, once per device.
int setup_current_device(int device, DeviceSetup **out) {
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  DeviceSetup &s = g_setup[device];
  if (!s.ready) {
    cudaDeviceProp prop;
    cudaError_t err = cudaGetDeviceProperties(&prop, device);
    if (err != cudaSuccess)
      return fail(HC_CUDA_ERR_CUDA, std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(err));
    if (prop.major != 10)
      return fail(HC_CUDA_ERR_NO_DEVICE, "the current device is not an sm_100 device");
    void *address = nullptr;
    err = cudaGetSymbolAddress(&address, g_static_scratch);
    if (err != cudaSuccess || address == nullptr)
      return fail(HC_CUDA_ERR_CUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(err));
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult query = cudaDriverEntryPointSymbolNotFound;
    err = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &query);
    if (err != cudaSuccess || query != cudaDriverEntryPointSuccess || fn == nullptr) {
      cudaGetLastError();
      return fail(HC_CUDA_ERR_CUDA, "the driver does not provide cuTensorMapEncodeTiled");
    }
    s.scratch = static_cast<unsigned char *>(address);
    s.sm_count = prop.multiProcessorCount;
    s.encode = reinterpret_cast<EncodeTiledFn>(fn);
    s.ready = true;
  }
  *out = &s;
  return HC_CUDA_OK;
}

int encode(const DeviceSetup &s, CUtensorMap *map, int dtype, const void *base, uint64_t inner,
           uint64_t outer, uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer) {
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUtensorMapDataType type =
      dtype == HC_CUDA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult res = s.encode(map, type, 2, const_cast<void *>(base), dims, strides, box, elem_strides,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS)
    return fail(HC_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(res)));
  return HC_CUDA_OK;
}

} // namespace

extern "C" {

int hcCudaGemmSkinnyStatic(const HcCudaGemmArgs *args, void *stream, int synchronize,
                           char *error_text, size_t error_text_bytes) {
  auto report = [&](int status) {
    if (status != HC_CUDA_OK && error_text != nullptr && error_text_bytes > 0)
      std::snprintf(error_text, error_text_bytes, "%s", g_static_error.c_str());
    return status;
  };
  if (args == nullptr)
    return report(fail(HC_CUDA_ERR_INVALID_ARGUMENT, "args must not be null"));
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess || device < 0 || device >= kMaxDevices) {
    cudaGetLastError();
    return report(fail(HC_CUDA_ERR_NO_DEVICE, "no current CUDA device"));
  }
  DeviceSetup *setup = nullptr;
  if (int rc = setup_current_device(device, &setup))
    return report(rc);

  if (args->dtype != HC_CUDA_F16 && args->dtype != HC_CUDA_BF16)
    return report(fail(HC_CUDA_ERR_UNSUPPORTED, "the static-scratch entry point multiplies float16 or bfloat16 "
                                                "matrices (8-bit operands may need a transposing repack)"));
  if (args->accumulate != 0 || args->epilogue_count != 0 || args->c_dtype != HC_CUDA_C_F32)
    return report(fail(HC_CUDA_ERR_UNSUPPORTED, "the static-scratch entry point computes a float32 C = A*B only "
                                                "(no accumulate, no fused operations, no 16-bit C)"));
  // Same validation and split choice as the regular path.
  HcCudaGemmArgs forced = *args;
  forced.variant = HC_CUDA_GEMM_SKINNY;
  HcCudaGemmPlanInfo plan;
  if (int rc = hcCudaGemmPlan(&forced, setup->sm_count, &plan))
    return report(fail(rc, hcCudaContextLastError(nullptr)));
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  const int m = static_cast<int>(args->m), n = static_cast<int>(args->n), k = static_cast<int>(args->k);
  if (plan.variant == HC_CUDA_GEMM_NOOP)
    return HC_CUDA_OK;
  bool launched_kernel = false;
  if (plan.variant == HC_CUDA_GEMM_ZERO_FILL) {
    err = cudaMemset2DAsync(args->c, static_cast<size_t>(args->ldc) * 4, 0, static_cast<size_t>(n) * 4,
                            static_cast<size_t>(m), cuda_stream);
    if (err != cudaSuccess)
      return report(fail(HC_CUDA_ERR_CUDA, std::string("cudaMemset2DAsync: ") + cudaGetErrorString(err)));
  } else {
    if (args->b_layout != HC_CUDA_B_KN)
      return report(fail(HC_CUDA_ERR_UNSUPPORTED, "the static-scratch entry point takes B stored [k, n] only"));

    if (plan.repack_a || plan.repack_b)
      return report(fail(HC_CUDA_ERR_UNSUPPORTED,
                         "the static-scratch entry point needs a and b 16-byte aligned with lda and ldb "
                         "multiples of 8 elements (a repack would need scratch it does not have)"));
    const size_t partial_bytes = hc::sm100::skinny_partials_bytes(m, n, plan.splits);
    const size_t counter_bytes = plan.splits > 1 ? hc::sm100::skinny_counters_bytes(n) : 0;
    if (partial_bytes > kPartialBytes || counter_bytes > kCounterBytes) {
      char text[256];
      std::snprintf(text, sizeof(text),
                    "problem needs %zu bytes of split-k partial sums and %zu bytes of counters; the static "
                    "scratch holds %zu and %zu",
                    partial_bytes, counter_bytes, kPartialBytes, kCounterBytes);
      return report(fail(HC_CUDA_ERR_UNSUPPORTED, text));
    }
    int *status_word = reinterpret_cast<int *>(setup->scratch);
    unsigned *counters = reinterpret_cast<unsigned *>(setup->scratch + kStatusBytes);
    float *partials = reinterpret_cast<float *>(setup->scratch + kStatusBytes + kCounterBytes);
    // The array keeps the previous call's contents: clear what must start at zero.
    err = cudaMemsetAsync(setup->scratch, 0, kStatusBytes + counter_bytes, cuda_stream);
    if (err != cudaSuccess)
      return report(fail(HC_CUDA_ERR_CUDA, std::string("cudaMemsetAsync: ") + cudaGetErrorString(err)));
    const hc::sm100::SkinnyShape shape = hc::sm100::skinny_shape(m);
    const uint32_t padded_m = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
    CUtensorMap tmap_a, tmap_b;
    if (int rc = encode(*setup, &tmap_a, args->dtype, args->a, k, m, static_cast<uint64_t>(args->lda) * 2,
                        shape.block_k, padded_m))
      return report(rc);
    if (int rc = encode(*setup, &tmap_b, args->dtype, args->b, n, k, static_cast<uint64_t>(args->ldb) * 2, 64,
                        shape.block_k))
      return report(rc);
    err = hc::sm100::launch_gemm_skinny(tmap_a, tmap_b, args->c, m, n, k, args->ldc, args->dtype, plan.splits,
                                        partials, counters, plan.grid, setup->sm_count, hc::sm100::kBLayoutKN,
                                        hc::sm100::Epilogue{}, status_word, cuda_stream);
    if (err != cudaSuccess)
      return report(fail(HC_CUDA_ERR_CUDA, std::string("launching the skinny kernel: ") + cudaGetErrorString(err)));
    launched_kernel = true;
  }
  if (synchronize) {
    // A zero fill launches no kernel, so there is no status to read: the word may still hold
    // what an earlier asynchronous call left there.
    int device_status = 0;
    err = launched_kernel ? cudaMemcpyAsync(&device_status, setup->scratch, sizeof(int), cudaMemcpyDeviceToHost,
                                            cuda_stream)
                          : cudaSuccess;
    if (err == cudaSuccess)
      err = cudaStreamSynchronize(cuda_stream);
    if (err != cudaSuccess)
      return report(fail(HC_CUDA_ERR_CUDA, std::string("waiting for the stream: ") + cudaGetErrorString(err)));
    if (device_status != 0) {
      // Reported once: the word starts at zero for whoever reads it next.
      err = cudaMemsetAsync(setup->scratch, 0, sizeof(int), cuda_stream);
      if (err == cudaSuccess)
        err = cudaStreamSynchronize(cuda_stream);
      if (err != cudaSuccess)
        cudaGetLastError();
      return report(fail(HC_CUDA_ERR_DEVICE_TIMEOUT,
                         "the kernel reported that a bounded device-side wait ran out; C is invalid"));
    }
  }
  return HC_CUDA_OK;
}

} // extern "C"
