// Implementation of include/hc-c/Cuda.h: the MLIR-free launch layer that sits where the
// reference keeps its C API (lib/CAPI/HC.cpp, lib/CAPI/HCFront.cpp). It validates the
// caller's buffers, chooses a kernel variant, encodes TMA tensor maps, manages the
// context's scratch memory and enqueues the sm_100a kernels of lib/Kernels.
//
// Nothing here computes a matrix product on the host: without a device the compute entry
// points fail.
#include "hc-c/Cuda.h"

#include "../Kernels/gemm_launch.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>  // types only; the library is opened at run time

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <initializer_list>
#include <mutex>
#include <vector>
#include <new>
#include <string>

namespace {

using hc::sm100::kDTypeBF16;

constexpr int kDefaultSmCount = 148;
constexpr int64_t kMaxDim = int64_t(1) << 30;
constexpr int64_t kMaxPitch = int64_t(1) << 38;
// Pitch granularity of operands the library lays out itself (repacked or staged copies): 64
// elements = 128 bytes, so that every 128-byte TMA box row is one aligned line. (TMA itself only
// needs 16 bytes; rows that straddle lines cost about a third more time on the ragged config.)
constexpr int64_t kRepackPitchBytes = 128;  // pitch of repacked / staged operands: whole cache lines

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct NcclApi {
  void *handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

NcclApi &nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char *override_path = std::getenv("HC_CUDA_NCCL_LIB");
    const char *names[] = {override_path, "libnccl.so.2", "libnccl.so"};
    for (const char *name : names) {
      if (name == nullptr || *name == '\0')
        continue;
      api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle != nullptr)
        break;
    }
    if (api.handle == nullptr)
      return;
    api.GetUniqueId =
        reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(api.handle, "ncclGetUniqueId"));
    api.CommInitRank =
        reinterpret_cast<decltype(api.CommInitRank)>(dlsym(api.handle, "ncclCommInitRank"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(api.handle, "ncclAllGather"));
    api.CommDestroy =
        reinterpret_cast<decltype(api.CommDestroy)>(dlsym(api.handle, "ncclCommDestroy"));
    api.GetErrorString =
        reinterpret_cast<decltype(api.GetErrorString)>(dlsym(api.handle, "ncclGetErrorString"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.AllGather && api.CommDestroy &&
             api.GetErrorString;
  });
  return api;
}

thread_local std::string g_thread_error;

} // namespace

struct HcCudaEvent {
  cudaEvent_t event = nullptr;
};

// One remembered cuTensorMapEncodeTiled result (see encode_map).
constexpr unsigned kMapCacheEntries = 16;
struct MapCacheEntry {
  bool valid = false;
  int dtype = 0;
  const void *base = nullptr;
  uint64_t inner = 0, outer = 0, pitch_bytes = 0;
  uint32_t box_inner = 0, box_outer = 0;
  CUtensorMap map;
};

struct HcCudaContext {
  int device = -1;
  cudaStream_t stream = nullptr;
  cudaDeviceProp prop{};
  int *status_dev = nullptr;
  int *status_host = nullptr;  // pinned
  void *scratch = nullptr;
  size_t scratch_bytes = 0;
  unsigned *counters = nullptr;
  size_t counters_bytes = 0;
  int4 *pairwise_leaves = nullptr;  // summation schedule of the pairwise kernel for `pairwise_h`
  int pairwise_h = -1, pairwise_leaf_count = 0;
  void *stage[3] = {nullptr, nullptr, nullptr};  // device staging for host-buffer calls
  size_t stage_bytes[3] = {0, 0, 0};
  // Host-buffer calls on large dense problems overlap copies with compute: A arrives in row
  // panels on `copy_in`, each panel's GEMM runs on `stream`, its rows of C leave on `copy_out`.
  static constexpr int kMaxPanels = 8;
  cudaStream_t copy_in = nullptr;
  cudaStream_t copy_out = nullptr;
  static constexpr int kMaxSteps = 2 * kMaxPanels;  // a panel of A and one of B per step
  cudaEvent_t panel_in[kMaxSteps] = {};
  cudaEvent_t panel_done[kMaxSteps] = {};
  bool planning_host_panels = false;  // plan_gemm then never splits k: see hcCudaGemmHost
  bool planning_push = false;         // plan_gemm then keeps to the kernels that can push tiles to peers
  cudaEvent_t fence_event = nullptr;
  EncodeTiledFn encode = nullptr;
  int group_n = 8;        // tile columns per group of the tile walk (256-column tiles)
  int group_n_wide = 16;  // the same for the 512x256-tile kernel (measured best of 4/8/12/16)
  bool c_tma_store = true;  // HC_CUDA_C_TMA_STORE=0 keeps ordinary stores (tuning aid)
  MapCacheEntry map_cache[kMapCacheEntries];  // recently encoded tensor maps, see encode_map
  unsigned map_cache_next = 0;
  ncclComm_t comm = nullptr;
  int nranks = 0;
  int rank = -1;
  mutable std::mutex mu;
  std::string last_error;
};

namespace {

int fail(const HcCudaContext *ctx, int status, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (ctx != nullptr)
    const_cast<HcCudaContext *>(ctx)->last_error = buf;
  else
    g_thread_error = buf;
  return status;
}

int fail_cuda(const HcCudaContext *ctx, cudaError_t err, const char *what) {
  const int status = err == cudaErrorMemoryAllocation ? HC_CUDA_ERR_OUT_OF_MEMORY : HC_CUDA_ERR_CUDA;
  return fail(ctx, status, "%s: %s (%s)", what, cudaGetErrorName(err), cudaGetErrorString(err));
}

#define HC_TRY_CUDA(ctx, expr)                                                                     \
  do {                                                                                             \
    cudaError_t hc_err__ = (expr);                                                                 \
    if (hc_err__ != cudaSuccess)                                                                   \
      return fail_cuda((ctx), hc_err__, #expr);                                                    \
  } while (0)

int64_t round_up(int64_t v, int64_t to) { return (v + to - 1) / to * to; }

bool ranges_overlap(const void *p, size_t pbytes, const void *q, size_t qbytes) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p), b = reinterpret_cast<uintptr_t>(q);
  return pbytes != 0 && qbytes != 0 && a < b + qbytes && b < a + pbytes;
}

// Validation + variant choice shared by hcCudaGemmPlan, hcCudaGemm and hcCudaGemmHost.
// `host_buffers`: the pointers are host memory that will be staged with aligned pitches, so
// no repack is ever needed.
int plan_gemm(const HcCudaContext *ctx, const HcCudaGemmArgs *args, int sm_count, bool host_buffers,
              HcCudaGemmPlanInfo *plan) {
  if (args == nullptr || plan == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "args and plan must not be null");
  std::memset(plan, 0, sizeof(*plan));
  plan->splits = 1;
  const int64_t m = args->m, n = args->n, k = args->k;
  if (m < 0 || n < 0 || k < 0)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "m, n, k must be non-negative (got %lld, %lld, %lld)",
                (long long)m, (long long)n, (long long)k);
  if (m > kMaxDim || n > kMaxDim || k > kMaxDim)
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "m, n, k must each be at most 2^30");
  if (args->dtype < HC_CUDA_F16 || args->dtype > HC_CUDA_F8E5M2)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "dtype must be an HcCudaDType (got %d)", args->dtype);
  const bool f8 = hc::sm100::dtype_is_8bit(args->dtype);
  const int64_t es = f8 ? 1 : 2;  // bytes per element of A and B
  if (args->variant != HC_CUDA_GEMM_AUTO && args->variant != HC_CUDA_GEMM_DENSE &&
      args->variant != HC_CUDA_GEMM_SKINNY && args->variant != HC_CUDA_GEMM_TINY)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "variant must be AUTO, DENSE, SKINNY or TINY (got %d)",
                args->variant);
  if (args->accumulate != 0 && args->accumulate != 1)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "accumulate must be 0 or 1 (got %d)", args->accumulate);
  if (args->epilogue_count < 0 || args->epilogue_count > HC_CUDA_MAX_EPILOGUE_OPS)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "epilogue_count must be 0..%d (got %d)",
                HC_CUDA_MAX_EPILOGUE_OPS, args->epilogue_count);
  int bias_ops = 0;
  for (int i = 0; i < args->epilogue_count; ++i) {
    const int kind = args->epilogue_kind[i];
    if (kind < HC_CUDA_EPILOGUE_SCALE || kind > HC_CUDA_EPILOGUE_BIAS_COLUMN)
      return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "epilogue_kind[%d] is not an HcCudaEpilogueOp (got %d)", i, kind);
    bias_ops += kind == HC_CUDA_EPILOGUE_BIAS_COLUMN ? 1 : 0;
  }
  if (bias_ops > 1)
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "at most one HC_CUDA_EPILOGUE_BIAS_COLUMN operation is supported");
  if (args->c_dtype != HC_CUDA_C_F32 && args->c_dtype != HC_CUDA_C_F16 && args->c_dtype != HC_CUDA_C_BF16)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "c_dtype must be an HcCudaCType (got %d)", args->c_dtype);
  if (args->c_dtype != HC_CUDA_C_F32 && args->accumulate != 0)
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "accumulate needs a float32 C");
  const size_t c_elem = args->c_dtype == HC_CUDA_C_F32 ? 4 : 2;
  if (sm_count <= 0)
    sm_count = kDefaultSmCount;

  if (m == 0 || n == 0) {
    plan->variant = HC_CUDA_GEMM_NOOP;
    return HC_CUDA_OK;
  }
  if (bias_ops != 0) {
    if (args->bias == nullptr || (reinterpret_cast<uintptr_t>(args->bias) & 3) != 0)
      return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "bias must be a 4-byte-aligned pointer to n floats");
  }
  if (args->c == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "c must not be null");
  if (args->ldc < n || args->ldc > kMaxPitch)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ldc (%lld) must be at least n (%lld)",
                (long long)args->ldc, (long long)n);
  if ((reinterpret_cast<uintptr_t>(args->c) & (c_elem - 1)) != 0)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "c must be %zu-byte aligned", c_elem);
  const size_t c_bytes = (static_cast<size_t>(m - 1) * args->ldc + n) * c_elem;
  if (bias_ops != 0 && ranges_overlap(args->c, c_bytes, args->bias, static_cast<size_t>(n) * 4))
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "c must not overlap bias");
  if (k == 0) {
    // No product to add: C becomes zero, stays as it is, or only receives the element-wise work.
    if (args->epilogue_count != 0) {
      plan->variant = HC_CUDA_GEMM_ELEMENTWISE;
      plan->kernel_launches = 1;
    } else {
      plan->variant = args->accumulate ? HC_CUDA_GEMM_NOOP : HC_CUDA_GEMM_ZERO_FILL;
    }
    return HC_CUDA_OK;
  }
  if (args->a == nullptr || args->b == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "a and b must not be null");
  if (args->lda < k || args->lda > kMaxPitch)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "lda (%lld) must be at least k (%lld)",
                (long long)args->lda, (long long)k);
  if (args->b_layout != HC_CUDA_B_KN && args->b_layout != HC_CUDA_B_NK)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "b_layout must be HC_CUDA_B_KN or HC_CUDA_B_NK (got %d)",
                args->b_layout);
  const bool b_nk = args->b_layout == HC_CUDA_B_NK;
  const int64_t b_rows = b_nk ? n : k, b_cols = b_nk ? k : n;  // as stored
  if (args->ldb < b_cols || args->ldb > kMaxPitch)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ldb (%lld) must be at least %s (%lld)",
                (long long)args->ldb, b_nk ? "k" : "n", (long long)b_cols);
  if ((reinterpret_cast<uintptr_t>(args->a) & (es - 1)) != 0 || (reinterpret_cast<uintptr_t>(args->b) & (es - 1)) != 0)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "a and b must be aligned to their element size");
  const size_t a_bytes = (static_cast<size_t>(m - 1) * args->lda + k) * es;
  const size_t b_bytes = (static_cast<size_t>(b_rows - 1) * args->ldb + b_cols) * es;
  if (ranges_overlap(args->c, c_bytes, args->a, a_bytes) ||
      ranges_overlap(args->c, c_bytes, args->b, b_bytes))
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "c must not overlap a or b");

  int variant = args->variant;
  const int skinny_max_m = hc::sm100::skinny_shape(1).max_m;
  if (variant == HC_CUDA_GEMM_SKINNY && m > skinny_max_m)
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "the skinny variant needs m <= %d (got %lld)",
                skinny_max_m, (long long)m);
  if (variant == HC_CUDA_GEMM_TINY && (f8 || (ctx != nullptr && ctx->planning_push)))
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "the tiny variant takes 16-bit operands and no push targets");
  if (variant == HC_CUDA_GEMM_AUTO && !(ctx != nullptr && (ctx->planning_push || ctx->planning_host_panels)) &&
      hc::sm100::tiny_takes(m, n, k, args->dtype, sm_count))
    variant = HC_CUDA_GEMM_TINY;
  if (variant == HC_CUDA_GEMM_TINY) {
    const int tile = hc::sm100::tiny_tile();
    plan->variant = variant;
    plan->tiles_m = static_cast<int32_t>((m + tile - 1) / tile);
    plan->tiles_n = static_cast<int32_t>((n + tile - 1) / tile);
    if (plan->tiles_m > 65535)
      return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "the tiny variant takes at most 65535 tile rows");
    plan->splits = 1;
    plan->grid = plan->tiles_m * plan->tiles_n;
    plan->kernel_launches = 1;
    plan->scratch_bytes = 0;
    return HC_CUDA_OK;
  }
  if (variant == HC_CUDA_GEMM_AUTO) {
    variant = m <= skinny_max_m ? HC_CUDA_GEMM_SKINNY : HC_CUDA_GEMM_DENSE;
    // 8 < m <= 64 with so few column blocks that the skinny kernel would split k: the dense tiles
    // shared among thread-block clusters (below) pull A once per 256 columns instead of once per 128
    // and add the partial sums through shared memory, where they can be used (measured on
    // 8192 x 8192: m = 64: 30.7 against 39.0 us, m = 32: 28.7 against 32.9; 64 x 2048 x 16384: 18.5
    // against 38.9; m = 8: no difference).
    if (variant == HC_CUDA_GEMM_SKINNY && m > 8 && !host_buffers && args->c_dtype == HC_CUDA_C_F32 &&
        (static_cast<size_t>(args->ldc) * c_elem) % 16 == 0 && (reinterpret_cast<uintptr_t>(args->c) & 15) == 0 &&
        (ctx == nullptr || (ctx->c_tma_store && !ctx->planning_push && !ctx->planning_host_panels)) &&
        std::getenv("HC_CUDA_DENSE_SPLITS") == nullptr && std::getenv("HC_CUDA_SKINNY_SPLITS") == nullptr &&
        hc::sm100::skinny_choose_splits(static_cast<int>(n), static_cast<int>((k * es + 1) / 2), sm_count) > 1) {
      const hc::sm100::DenseTileShape t = hc::sm100::dense_tile_shape();
      const int64_t tiles = ((m + t.block_m - 1) / t.block_m) * ((n + t.block_n - 1) / t.block_n);
      const int num_kb = static_cast<int>((k * es + 2 * t.block_k - 1) / (2 * t.block_k));
      long long first_split_tile = 0;
      if (hc::sm100::dense_choose_splits(tiles, sm_count, num_kb, &first_split_tile) > 1 && first_split_tile == 0 &&
          hc::sm100::dense_cluster_choose(m, n, k, static_cast<int>(es), sm_count).cluster_size >= 2)
        variant = HC_CUDA_GEMM_DENSE;
    }
  }
  plan->variant = variant;

  if (!host_buffers) {
    plan->repack_a = ((args->lda * es) % 16 != 0 || (reinterpret_cast<uintptr_t>(args->a) & 15) != 0) ? 1 : 0;
    plan->repack_b = ((args->ldb * es) % 16 != 0 || (reinterpret_cast<uintptr_t>(args->b) & 15) != 0) ? 1 : 0;
  }
  // 8-bit operands reach the tensor cores K-major only: a float8 B stored [K, N] is transposed
  // into scratch (one extra launch), whatever its pitch.
  if (f8 && !b_nk)
    plan->repack_b = 1;
  int64_t scratch = 0;
  if (plan->repack_a)
    scratch += round_up(m * round_up(k * es, kRepackPitchBytes), 1024);
  if (plan->repack_b)
    scratch += f8 && !b_nk ? round_up(n * round_up(k * es, kRepackPitchBytes), 1024)
                           : round_up(b_rows * round_up(b_cols * es, kRepackPitchBytes), 1024);
  // 16-bit operands share one repack launch; each 8-bit operand has its own.
  plan->kernel_launches = 1 + (f8 ? plan->repack_a + plan->repack_b : ((plan->repack_a || plan->repack_b) ? 1 : 0));

  if (variant == HC_CUDA_GEMM_DENSE) {
    const hc::sm100::DenseTileShape t = hc::sm100::dense_tile_shape();
    const bool pairs = hc::sm100::dense_uses_pairs(m, n, k, sm_count, ctx != nullptr && ctx->planning_push);
    // 512x256 tiles for products that fill the GPU with them, when the epilogue never has to read C
    // with ordinary loads (an accumulation must be one the TMA stores can perform) and the tiles go
    // nowhere but C. Decided again below if tiles turn out to be split over k.
    const bool c_tma_ok = (static_cast<size_t>(args->ldc) * c_elem) % 16 == 0 &&
                          (reinterpret_cast<uintptr_t>(args->c) & 15) == 0 && (ctx == nullptr || ctx->c_tma_store);
    bool wide = pairs && hc::sm100::dense_uses_wide(m, n, k, sm_count) &&
                (args->accumulate == 0 || (c_tma_ok && args->epilogue_count == 0)) &&
                !(ctx != nullptr && ctx->planning_push);
    int64_t tile_m = wide ? hc::sm100::kDenseWideTileM : (pairs ? 2 * t.block_m : t.block_m);
    if (wide) {
      const int64_t wide_tiles = ((m + tile_m - 1) / tile_m) * ((n + t.block_n - 1) / t.block_n);
      const int wide_kb = static_cast<int>((k + 64 * (2 / es) - 1) / (64 * (2 / es)));
      long long ignored = 0;
      const bool forced_split = std::getenv("HC_CUDA_DENSE_SPLITS") != nullptr;
      const char *forced_wide = std::getenv("HC_CUDA_DENSE_WIDE");  // "1": the tuning aid also rules out splits
      // With many rounds of tiles an underfilled last round is a per cent or two and not worth leaving
      // the wide tiles for; with few rounds the pair tiles split it over k instead.
      const bool many_rounds = wide_tiles >= 8LL * (sm_count / 2);
      const bool keep_wide = many_rounds || (forced_wide != nullptr && std::strcmp(forced_wide, "1") == 0);
      if (forced_split || (!keep_wide && !(ctx != nullptr && ctx->planning_host_panels) &&
                           hc::sm100::dense_choose_splits(wide_tiles, sm_count / 2, wide_kb, &ignored) > 1)) {
        wide = false;
        tile_m = 2 * t.block_m;
      }
    }
    plan->tiles_m = static_cast<int32_t>((m + tile_m - 1) / tile_m);
    plan->tiles_n = static_cast<int32_t>((n + t.block_n - 1) / t.block_n);
    plan->tile_n = static_cast<int32_t>(t.block_n);
    const int64_t tiles = static_cast<int64_t>(plan->tiles_m) * plan->tiles_n;
    if (tiles > 0x3fffffffLL)
      return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "too many tiles");
    // Tiles that do not fill a round of the persistent CTAs (all of them, or the last round's) are
    // split over k when k is long enough.
    const int block_k = (wide ? 64 : hc::sm100::dense_block_k(pairs)) * static_cast<int>(2 / es);  // same bytes per stage
    const int num_kb = static_cast<int>((k + block_k - 1) / block_k);
    const int slots = pairs ? sm_count / 2 : sm_count;
    long long first_split_tile = 0;
    // A small product with a short k whose 256-wide tiles would leave most SMs idle runs on 128 x 128
    // tiles (single CTAs, decided first: it is then not split over k).
    const bool narrow = !wide && !(ctx != nullptr && (ctx->planning_push || ctx->planning_host_panels)) &&
                        std::getenv("HC_CUDA_DENSE_SPLITS") == nullptr &&
                        hc::sm100::dense_uses_narrow(m, n, k, sm_count, pairs);
    plan->splits = narrow ? 1 : hc::sm100::dense_choose_splits(tiles, slots, num_kb, &first_split_tile);
    if (narrow)
      first_split_tile = 0;
    if (wide || (ctx != nullptr && ctx->planning_host_panels)) {
      // The 512x256 tiles are never split (they are only kept when no split is wanted), and the
      // panels of one host-buffer product must give the bits of the unsplit product.
      plan->splits = 1;
      first_split_tile = 0;
    } else if (const char *forced = std::getenv("HC_CUDA_DENSE_SPLITS")) {  // tuning aid: split every tile
      const int v = std::atoi(forced);
      if (v >= 1 && v <= num_kb && v <= 64) {
        plan->splits = v;
        first_split_tile = 0;
      }
    }
    // When every tile would be split (fewer tiles than CTAs), a float32 C that TMA can address gets the
    // cluster form instead: the CTAs that share a tile are one thread-block cluster and add their partial
    // tiles through distributed shared memory, not through global memory and counters.
    const char *cluster_env = std::getenv("HC_CUDA_DENSE_CLUSTER");  // tuning aid: a size forces the form
    const bool cluster_forced = cluster_env != nullptr && std::atoi(cluster_env) >= 2;
    if (((plan->splits > 1 && first_split_tile == 0 && std::getenv("HC_CUDA_DENSE_SPLITS") == nullptr) ||
         cluster_forced) &&
        c_tma_ok && args->c_dtype == HC_CUDA_C_F32 && !(ctx != nullptr && ctx->planning_push) &&
        !(ctx != nullptr && ctx->planning_host_panels)) {
      const hc::sm100::ClusterPlan cp = hc::sm100::dense_cluster_choose(m, n, k, static_cast<int>(es), sm_count);
      if (cp.cluster_size >= 2) {
        plan->cluster_size = cp.cluster_size;
        plan->tiles_m = static_cast<int32_t>((m + t.block_m - 1) / t.block_m);
        plan->tiles_n = static_cast<int32_t>((n + t.block_n - 1) / t.block_n);
        plan->splits = cp.cluster_size * cp.groups;
        plan->first_split_tile = 0;
        plan->grid = plan->tiles_m * plan->tiles_n * plan->splits;
        scratch += static_cast<int64_t>(hc::sm100::dense_cluster_partials_bytes(
            static_cast<long long>(plan->tiles_m) * plan->tiles_n, cp.groups));
        plan->scratch_bytes = scratch;
        return HC_CUDA_OK;
      }
    }
    if (narrow && plan->splits == 1 && plan->cluster_size == 0) {
      const int64_t narrow_n = hc::sm100::dense_narrow_block_n();
      plan->tile_n = static_cast<int32_t>(narrow_n);
      plan->tiles_m = static_cast<int32_t>((m + t.block_m - 1) / t.block_m);
      plan->tiles_n = static_cast<int32_t>((n + narrow_n - 1) / narrow_n);
      const int64_t narrow_tiles = static_cast<int64_t>(plan->tiles_m) * plan->tiles_n;
      plan->grid = static_cast<int32_t>(narrow_tiles < sm_count ? narrow_tiles : sm_count);
      plan->first_split_tile = 0;
      plan->scratch_bytes = scratch;
      return HC_CUDA_OK;
    }
    const int64_t split_tiles = plan->splits > 1 ? tiles - first_split_tile : 0;
    const int64_t units = tiles + split_tiles * (plan->splits - 1);
    plan->grid = static_cast<int32_t>((pairs ? 2 : 1) * (units < slots ? units : slots));
    scratch += static_cast<int64_t>(hc::sm100::dense_partials_bytes(split_tiles, plan->splits, pairs));
    plan->first_split_tile = static_cast<int32_t>(first_split_tile);
  } else {
    const hc::sm100::SkinnyShape s = hc::sm100::skinny_shape(static_cast<int>(m));
    plan->tiles_m = 1;
    plan->tiles_n = static_cast<int32_t>((n + s.block_n - 1) / s.block_n);
    // (k counted in 16-bit equivalents: a k-block is 128 bytes of k whatever the element width.)
    const int64_t k_units = (k * es + 1) / 2;
    plan->splits = hc::sm100::skinny_choose_splits(static_cast<int>(n), static_cast<int>(k_units), sm_count);
    if (const char *forced = std::getenv("HC_CUDA_SKINNY_SPLITS")) {  // tuning aid
      const int v = std::atoi(forced);
      const int64_t kb_total = (k_units + s.block_k - 1) / s.block_k;
      if (v >= 1 && v <= kb_total)
        plan->splits = v;
    }
    const int64_t units = static_cast<int64_t>(plan->tiles_n) * plan->splits;
    const int64_t slots = static_cast<int64_t>(sm_count) * 2;
    plan->grid = static_cast<int32_t>(units < slots ? units : slots);
    plan->ring_stages = hc::sm100::skinny_ring_stages(static_cast<int>(m), plan->grid, sm_count);
    scratch += static_cast<int64_t>(
        hc::sm100::skinny_partials_bytes(static_cast<int>(m), static_cast<int>(n), plan->splits));
  }
  plan->scratch_bytes = scratch;
  return HC_CUDA_OK;
}

int ensure_scratch(HcCudaContext *ctx, size_t bytes) {
  if (bytes <= ctx->scratch_bytes)
    return HC_CUDA_OK;
  if (ctx->scratch != nullptr) {
    HC_TRY_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    HC_TRY_CUDA(ctx, cudaFree(ctx->scratch));
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
  }
  const size_t grown = static_cast<size_t>(round_up(static_cast<int64_t>(bytes), 1 << 20));
  HC_TRY_CUDA(ctx, cudaMalloc(&ctx->scratch, grown));
  ctx->scratch_bytes = grown;
  return HC_CUDA_OK;
}

int ensure_counters(HcCudaContext *ctx, size_t bytes) {
  if (bytes <= ctx->counters_bytes)
    return HC_CUDA_OK;
  if (ctx->counters != nullptr) {
    HC_TRY_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    HC_TRY_CUDA(ctx, cudaFree(ctx->counters));
    ctx->counters = nullptr;
    ctx->counters_bytes = 0;
  }
  const size_t grown = static_cast<size_t>(round_up(static_cast<int64_t>(bytes), 4096));
  HC_TRY_CUDA(ctx, cudaMalloc(reinterpret_cast<void **>(&ctx->counters), grown));
  HC_TRY_CUDA(ctx, cudaMemsetAsync(ctx->counters, 0, grown, ctx->stream));
  ctx->counters_bytes = grown;
  return HC_CUDA_OK;
}

int ensure_stage(HcCudaContext *ctx, int which, size_t bytes) {
  if (bytes <= ctx->stage_bytes[which])
    return HC_CUDA_OK;
  if (ctx->stage[which] != nullptr) {
    HC_TRY_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    HC_TRY_CUDA(ctx, cudaFree(ctx->stage[which]));
    ctx->stage[which] = nullptr;
    ctx->stage_bytes[which] = 0;
  }
  const size_t grown = static_cast<size_t>(round_up(static_cast<int64_t>(bytes), 1 << 20));
  HC_TRY_CUDA(ctx, cudaMalloc(&ctx->stage[which], grown));
  ctx->stage_bytes[which] = grown;
  return HC_CUDA_OK;
}

constexpr int kMapFloat32 = -1;  // encode_map's dtype for C; otherwise an HcCudaDType

int encode_map(HcCudaContext *ctx, CUtensorMap *map, int dtype, const void *base, uint64_t inner,
               uint64_t outer, uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer) {
  // A tensor map is a pure function of these arguments, and callers launch the same product on
  // the same buffers over and over: keep the last few (the caller holds ctx->mu).
  for (MapCacheEntry &e : ctx->map_cache) {
    if (e.valid && e.base == base && e.inner == inner && e.outer == outer && e.pitch_bytes == pitch_bytes &&
        e.box_inner == box_inner && e.box_outer == box_outer && e.dtype == dtype) {
      *map = e.map;
      return HC_CUDA_OK;
    }
  }
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUtensorMapDataType type = dtype == kMapFloat32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : dtype == HC_CUDA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                   : hc::sm100::dtype_is_8bit(dtype) ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                                                     : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult res = ctx->encode(map, type, 2, const_cast<void *>(base), dims, strides, box,
                                   elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS)
    return fail(ctx, HC_CUDA_ERR_CUDA,
                "cuTensorMapEncodeTiled failed with CUresult %d (base %p, dims %llu x %llu, pitch %llu)",
                static_cast<int>(res), base, (unsigned long long)inner, (unsigned long long)outer,
                (unsigned long long)pitch_bytes);
  MapCacheEntry &slot = ctx->map_cache[ctx->map_cache_next];
  ctx->map_cache_next = (ctx->map_cache_next + 1) % kMapCacheEntries;
  slot = MapCacheEntry{true, dtype, base, inner, outer, pitch_bytes, box_inner, box_outer, *map};
  return HC_CUDA_OK;
}

// Enqueues the GEMM on device-resident buffers. The caller holds ctx->mu and has made the
// context's device current.
int enqueue_gemm(HcCudaContext *ctx, const HcCudaGemmArgs *args, const HcCudaGemmPlanInfo &plan,
                 const hc::sm100::Epilogue &push = hc::sm100::Epilogue{}) {
  if (plan.variant == HC_CUDA_GEMM_NOOP)
    return HC_CUDA_OK;
  const int m = static_cast<int>(args->m), n = static_cast<int>(args->n), k = static_cast<int>(args->k);
  hc::sm100::Epilogue ep = push;  // the push targets, if any; the fused work comes from args
  ep.accumulate = args->accumulate;
  ep.op_count = args->epilogue_count;
  for (int i = 0; i < args->epilogue_count; ++i) {
    ep.op_kind[i] = args->epilogue_kind[i];
    ep.op_value[i] = args->epilogue_value[i];
  }
  ep.bias = nullptr;  // non-null only when an operation reads it
  for (int i = 0; i < args->epilogue_count; ++i)
    if (args->epilogue_kind[i] == HC_CUDA_EPILOGUE_BIAS_COLUMN)
      ep.bias = args->bias;
  ep.c_dtype = args->c_dtype;
  const size_t c_elem = args->c_dtype == HC_CUDA_C_F32 ? 4 : 2;
  if (plan.variant == HC_CUDA_GEMM_ELEMENTWISE) {
    HC_TRY_CUDA(ctx, hc::sm100::launch_epilogue_only(args->c, m, n, args->ldc, ep, ctx->stream));
    return HC_CUDA_OK;
  }
  if (plan.variant == HC_CUDA_GEMM_ZERO_FILL) {
    HC_TRY_CUDA(ctx, cudaMemset2DAsync(args->c, static_cast<size_t>(args->ldc) * c_elem, 0,
                                       static_cast<size_t>(n) * c_elem, static_cast<size_t>(m), ctx->stream));
    return HC_CUDA_OK;
  }
  if (plan.variant == HC_CUDA_GEMM_TINY) {
    if (ep.push_count != 0)
      return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "the tiny variant has no push targets");
    HC_TRY_CUDA(ctx, hc::sm100::launch_gemm_tiny(args->a, args->lda, args->b, args->ldb, args->c, args->ldc, m, n, k,
                                                 args->dtype,
                                                 args->b_layout == HC_CUDA_B_NK ? hc::sm100::kBLayoutNK
                                                                                : hc::sm100::kBLayoutKN,
                                                 ep, ctx->stream));
    return HC_CUDA_OK;
  }
  if (int rc = ensure_scratch(ctx, static_cast<size_t>(plan.scratch_bytes)))
    return rc;

  const void *a = args->a;
  const void *b = args->b;
  int64_t lda = args->lda, ldb = args->ldb;
  const bool b_nk = args->b_layout == HC_CUDA_B_NK;
  const int b_rows = b_nk ? n : k, b_cols = b_nk ? k : n;  // B as stored
  char *cursor = static_cast<char *>(ctx->scratch);
  const bool f8 = hc::sm100::dtype_is_8bit(args->dtype);
  const int64_t es = f8 ? 1 : 2;  // bytes per element of A and B
  bool b_nk_now = b_nk;           // how B is laid out where the GEMM kernel reads it
  if (f8 && (plan.repack_a || plan.repack_b)) {
    if (plan.repack_a) {
      const int64_t pitch = round_up(static_cast<int64_t>(k), kRepackPitchBytes);
      HC_TRY_CUDA(ctx, hc::sm100::launch_repack_bytes(a, lda, cursor, pitch, m, k, /*transpose=*/false, ctx->stream));
      a = cursor;
      lda = pitch;
      cursor += round_up(static_cast<int64_t>(m) * pitch, 1024);
    }
    if (plan.repack_b) {
      // Stored [K, N]: transposed to [N, K]. Stored [N, K] with an odd pitch: copied.
      const int64_t pitch = round_up(static_cast<int64_t>(k), kRepackPitchBytes);
      HC_TRY_CUDA(ctx, hc::sm100::launch_repack_bytes(b, ldb, cursor, pitch, b_rows, b_cols, /*transpose=*/!b_nk,
                                                      ctx->stream));
      b = cursor;
      ldb = pitch;
      b_nk_now = true;
      cursor += round_up(static_cast<int64_t>(n) * pitch, 1024);
    }
  } else if (plan.repack_a || plan.repack_b) {
    // One launch copies whichever operands need it into scratch with 128-byte-aligned pitches.
    const void *src_a = nullptr, *src_b = nullptr;
    char *dst_a = nullptr, *dst_b = nullptr;
    int64_t pitch_a = 0, pitch_b = 0;
    if (plan.repack_a) {
      pitch_a = round_up(k, kRepackPitchBytes / 2);
      src_a = a;
      dst_a = cursor;
      cursor += round_up(static_cast<int64_t>(m) * pitch_a * 2, 1024);
    }
    if (plan.repack_b) {
      pitch_b = round_up(b_cols, kRepackPitchBytes / 2);
      src_b = b;
      dst_b = cursor;
      cursor += round_up(static_cast<int64_t>(b_rows) * pitch_b * 2, 1024);
    }
    HC_TRY_CUDA(ctx, hc::sm100::launch_repack_pitch_two(src_a, lda, dst_a, pitch_a, plan.repack_a ? m : 0, k,
                                                        src_b, ldb, dst_b, pitch_b, plan.repack_b ? b_rows : 0,
                                                        b_cols, ctx->stream));
    if (plan.repack_a) {
      a = dst_a;
      lda = pitch_a;
    }
    if (plan.repack_b) {
      b = dst_b;
      ldb = pitch_b;
    }
  }

  CUtensorMap tmap_a, tmap_b;
  const int b_layout = b_nk_now ? hc::sm100::kBLayoutNK : hc::sm100::kBLayoutKN;
  const uint32_t k_scale = static_cast<uint32_t>(2 / es);  // elements of k per 2 bytes: boxes are 128 bytes of k
  if (plan.variant == HC_CUDA_GEMM_DENSE) {
    const hc::sm100::DenseTileShape t = hc::sm100::dense_tile_shape();
    const bool narrow = plan.tile_n == hc::sm100::dense_narrow_block_n();  // 128 x 128 tiles on single CTAs
    const bool pairs = !narrow && hc::sm100::dense_uses_pairs(m, n, k, ctx->prop.multiProcessorCount, ep.push_count > 0);
    if (int rc = encode_map(ctx, &tmap_a, args->dtype, a, k, m, static_cast<uint64_t>(lda) * es,
                            t.block_k * k_scale, t.block_m))
      return rc;
    // B stored [K, N]: 64 (n) x 64 (k) boxes. Stored [N, K]: one box of 64 (k) x the CTA's rows
    // of n (256 on single CTAs, 128 per CTA of a pair).
    if (int rc = b_nk_now ? encode_map(ctx, &tmap_b, args->dtype, b, k, n, static_cast<uint64_t>(ldb) * es,
                                       t.block_k * k_scale,
                                       (narrow || (pairs && plan.cluster_size == 0)) ? t.block_n / 2 : t.block_n)
                          : encode_map(ctx, &tmap_b, args->dtype, b, n, k, static_cast<uint64_t>(ldb) * 2, 64,
                                       t.block_k))
      return rc;
    // C leaves through TMA stores when its rows start on 16-byte boundaries (the launcher falls
    // back to ordinary stores for fused work and push targets).
    CUtensorMap tmap_c;
    const CUtensorMap *c_map = nullptr;
    const bool c_rows_aligned = (static_cast<size_t>(args->ldc) * c_elem) % 16 == 0 &&
                                (reinterpret_cast<uintptr_t>(args->c) & 15) == 0;
    if (c_rows_aligned && ctx->c_tma_store) {
      // float32: 32 x 32 boxes; 16-bit: 64 columns x 32 rows (128-byte rows either way).
      const int map_type = args->c_dtype == HC_CUDA_C_F32 ? kMapFloat32
                           : args->c_dtype == HC_CUDA_C_BF16 ? HC_CUDA_BF16 : HC_CUDA_F16;
      if (int rc = encode_map(ctx, &tmap_c, map_type, args->c, n, m, static_cast<uint64_t>(args->ldc) * c_elem,
                              args->c_dtype == HC_CUDA_C_F32 ? 32 : 64, 32))
        return rc;
      c_map = &tmap_c;
    }
    if (plan.cluster_size > 1) {
      if (c_map == nullptr || args->c_dtype != HC_CUDA_C_F32 || ep.push_count != 0)
        return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "the cluster form needs a float32 C that TMA can address");
      // A planned size that this device does not offer is halved (with twice the clusters per tile, so
      // the k ranges stay the same).
      int size = plan.cluster_size, groups = plan.splits / plan.cluster_size;
      while (size > 2 && hc::sm100::dense_cluster_capacity(size) <= 0) {
        size >>= 1;
        groups <<= 1;
      }
      const long long cluster_tiles = static_cast<long long>(plan.tiles_m) * plan.tiles_n;
      float *partials = nullptr;
      if (groups > 1) {
        if (hc::sm100::dense_cluster_partials_bytes(cluster_tiles, groups) + (cursor - static_cast<char *>(ctx->scratch)) >
            ctx->scratch_bytes)
          return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "no cluster size of the plan is available on this device");
        if (int rc = ensure_counters(ctx, hc::sm100::dense_cluster_counters_bytes(cluster_tiles)))
          return rc;
        partials = reinterpret_cast<float *>(cursor);
      }
      CUtensorMap tmap_rows;  // C in boxes of as many rows as one warp finishes at a time
      if (int rc = encode_map(ctx, &tmap_rows, kMapFloat32, args->c, n, m, static_cast<uint64_t>(args->ldc) * 4, 32,
                              hc::sm100::dense_cluster_store_rows(size)))
        return rc;
      HC_TRY_CUDA(ctx, hc::sm100::launch_gemm_dense_cluster(tmap_a, tmap_b, tmap_rows, m, n, k, args->dtype, size,
                                                            groups, partials, ctx->counters, b_layout, ep,
                                                            ctx->status_dev, ctx->stream));
      return HC_CUDA_OK;
    }
    hc::sm100::SplitK split{plan.splits, plan.first_split_tile, nullptr, nullptr};
    CUtensorMap tmap_p;
    if (plan.splits > 1) {
      const long long split_tiles = static_cast<long long>(plan.tiles_m) * plan.tiles_n - plan.first_split_tile;
      if (int rc = ensure_counters(ctx, hc::sm100::dense_counters_bytes(split_tiles)))
        return rc;
      split.partials = reinterpret_cast<float *>(cursor);  // after the repacked operands, 1 KiB aligned
      split.counters = ctx->counters;
      const uint64_t tile_rows = static_cast<uint64_t>(pairs ? 2 * t.block_m : t.block_m);
      if (int rc = encode_map(ctx, &tmap_p, kMapFloat32, split.partials, static_cast<uint64_t>(t.block_n),
                              static_cast<uint64_t>(split_tiles) * plan.splits * tile_rows,
                              static_cast<uint64_t>(t.block_n) * 4, 32, 32))
        return rc;
    }
    // (plan_gemm chose 512x256 tiles iff it counted the rows of C in tiles of 512.)
    const bool wide = pairs && m >= 2 * hc::sm100::kDenseWideTileM && plan.splits == 1 &&
                      plan.tiles_m == (m + hc::sm100::kDenseWideTileM - 1) / hc::sm100::kDenseWideTileM;
    if (wide) {
      HC_TRY_CUDA(ctx, hc::sm100::launch_gemm_dense_wide(tmap_a, tmap_b, args->c, m, n, k, args->ldc, args->dtype,
                                                         ctx->group_n_wide, plan.grid, b_layout, ep, c_map,
                                                         ctx->status_dev, ctx->stream));
    } else if (pairs) {
      // Push targets as tensor maps (they are shaped and pitched like C): the epilogue then stores
      // every staged chunk to C and to each target through the TMA store engine instead of with
      // 16-byte stores from the warp. Off unless HC_CUDA_PUSH_TMA=1: measured on the sharded
      // benchmark it was 2.5 % faster at 2 GPUs (7.21 against 7.40 ms per product + gather) but 5 %
      // slower at 4 (4.19 against 3.97 ms): a warp has one staging block, and waiting until the store
      // engine has read it for three remote stores costs more than issuing the peer stores itself.
      hc::sm100::PushMaps push_maps;
      push_maps.count = 0;
      const char *push_tma = std::getenv("HC_CUDA_PUSH_TMA");
      if (ep.push_count > 0 && c_map != nullptr && args->c_dtype == HC_CUDA_C_F32 && push_tma != nullptr &&
          std::strcmp(push_tma, "1") == 0) {
        for (int t = 0; t < ep.push_count; ++t)
          if (int rc = encode_map(ctx, &push_maps.map[t], kMapFloat32, ep.push[t], n, m,
                                  static_cast<uint64_t>(args->ldc) * 4, 32, 32))
            return rc;
        push_maps.count = ep.push_count;
      }
      HC_TRY_CUDA(ctx, hc::sm100::launch_gemm_dense_pair(tmap_a, tmap_b, args->c, m, n, k, args->ldc,
                                                         args->dtype, ctx->group_n, plan.grid, b_layout, ep,
                                                         c_map, split, &tmap_p, ctx->status_dev, ctx->stream,
                                                         push_maps.count > 0 ? &push_maps : nullptr));
    } else {
      HC_TRY_CUDA(ctx, hc::sm100::launch_gemm_dense(tmap_a, tmap_b, args->c, m, n, k, args->ldc,
                                                    args->dtype, ctx->group_n, plan.grid, b_layout, ep,
                                                    c_map, split, &tmap_p, ctx->status_dev, ctx->stream,
                                                    narrow ? hc::sm100::dense_narrow_block_n() : t.block_n));
    }
    return HC_CUDA_OK;
  }

  const hc::sm100::SkinnyShape s = hc::sm100::skinny_shape(m);
  const uint32_t padded_m = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
  if (int rc = encode_map(ctx, &tmap_a, args->dtype, a, k, m, static_cast<uint64_t>(lda) * es,
                          s.block_k * k_scale, padded_m))
    return rc;
  if (int rc = b_nk_now ? encode_map(ctx, &tmap_b, args->dtype, b, k, n, static_cast<uint64_t>(ldb) * es,
                                     s.block_k * k_scale, s.block_n)
                        : encode_map(ctx, &tmap_b, args->dtype, b, n, k, static_cast<uint64_t>(ldb) * 2, 64,
                                     s.block_k))
    return rc;
  float *partials = nullptr;
  if (plan.splits > 1) {
    partials = reinterpret_cast<float *>(cursor);
    if (int rc = ensure_counters(ctx, hc::sm100::skinny_counters_bytes(n)))
      return rc;
  }
  HC_TRY_CUDA(ctx, hc::sm100::launch_gemm_skinny(tmap_a, tmap_b, args->c, m, n, k, args->ldc,
                                                 args->dtype, plan.splits, partials, ctx->counters,
                                                 plan.grid, ctx->prop.multiProcessorCount, b_layout, ep,
                                                 ctx->status_dev, ctx->stream));
  return HC_CUDA_OK;
}

int ensure_copy_streams(HcCudaContext *ctx) {
  if (ctx->copy_in != nullptr)
    return HC_CUDA_OK;
  HC_TRY_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking));
  HC_TRY_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking));
  for (int i = 0; i < HcCudaContext::kMaxSteps; ++i) {
    HC_TRY_CUDA(ctx, cudaEventCreateWithFlags(&ctx->panel_in[i], cudaEventDisableTiming));
    HC_TRY_CUDA(ctx, cudaEventCreateWithFlags(&ctx->panel_done[i], cudaEventDisableTiming));
  }
  HC_TRY_CUDA(ctx, cudaEventCreateWithFlags(&ctx->fence_event, cudaEventDisableTiming));
  return HC_CUDA_OK;
}

int synchronize_locked(HcCudaContext *ctx) {
  HC_TRY_CUDA(ctx, cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(int),
                                   cudaMemcpyDeviceToHost, ctx->stream));
  HC_TRY_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  const int device_status = *ctx->status_host;
  if (device_status != 0) {
    HC_TRY_CUDA(ctx, cudaMemsetAsync(ctx->status_dev, 0, sizeof(int), ctx->stream));
    // A kernel that gave up may have left split-k arrival counters half counted.
    if (ctx->counters != nullptr)
      HC_TRY_CUDA(ctx, cudaMemsetAsync(ctx->counters, 0, ctx->counters_bytes, ctx->stream));
    HC_TRY_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if ((device_status & 0xff) == hc::sm100::kStatusCheckFailed)
      return fail(ctx, HC_CUDA_ERR_DEVICE_CHECK,
                  "index check %d of a kernel failed (checked build): the access was not made; the output of that "
                  "launch is invalid",
                  device_status >> 8);
    return fail(ctx, HC_CUDA_ERR_DEVICE_TIMEOUT,
                "a kernel reported status %d: a bounded device-side wait ran out; the output of "
                "that launch is invalid",
                device_status);
  }
  return HC_CUDA_OK;
}

} // namespace

extern "C" {

int hcCudaApiVersion(void) { return HC_CUDA_API_VERSION; }

int hcCudaBuildFlags(void) { return hc::sm100::library_is_checked() ? 1 : 0; }

const char *hcCudaStatusString(int status) {
  switch (status) {
  case HC_CUDA_OK: return "HC_CUDA_OK";
  case HC_CUDA_ERR_INVALID_ARGUMENT: return "HC_CUDA_ERR_INVALID_ARGUMENT";
  case HC_CUDA_ERR_UNSUPPORTED: return "HC_CUDA_ERR_UNSUPPORTED";
  case HC_CUDA_ERR_CUDA: return "HC_CUDA_ERR_CUDA";
  case HC_CUDA_ERR_NO_DEVICE: return "HC_CUDA_ERR_NO_DEVICE";
  case HC_CUDA_ERR_DEVICE_TIMEOUT: return "HC_CUDA_ERR_DEVICE_TIMEOUT";
  case HC_CUDA_ERR_COMM: return "HC_CUDA_ERR_COMM";
  case HC_CUDA_ERR_OUT_OF_MEMORY: return "HC_CUDA_ERR_OUT_OF_MEMORY";
  case HC_CUDA_ERR_DEVICE_CHECK: return "HC_CUDA_ERR_DEVICE_CHECK";
  default: return "HC_CUDA_ERR_UNKNOWN";
  }
}

int hcCudaGetDeviceCount(int *count) {
  if (count == nullptr)
    return fail(nullptr, HC_CUDA_ERR_INVALID_ARGUMENT, "count must not be null");
  int n = 0;
  const cudaError_t err = cudaGetDeviceCount(&n);
  if (err != cudaSuccess) {
    cudaGetLastError();  // no driver / no device is an answer, not a failure
    n = 0;
  }
  *count = n;
  return HC_CUDA_OK;
}

int hcCudaContextCreate(int device, HcCudaContext **out) {
  if (out == nullptr)
    return fail(nullptr, HC_CUDA_ERR_INVALID_ARGUMENT, "out must not be null");
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    cudaGetLastError();
    count = 0;
  }
  if (device < 0 || device >= count)
    return fail(nullptr, HC_CUDA_ERR_NO_DEVICE, "device %d does not exist (%d CUDA device(s) visible)",
                device, count);
  HcCudaContext *ctx = new (std::nothrow) HcCudaContext();
  if (ctx == nullptr)
    return fail(nullptr, HC_CUDA_ERR_OUT_OF_MEMORY, "out of host memory");
  ctx->device = device;
  auto bail = [&](int status) {
    g_thread_error = ctx->last_error;
    hcCudaContextDestroy(ctx);
    return status;
  };
  cudaError_t err = cudaSetDevice(device);
  if (err == cudaSuccess)
    err = cudaGetDeviceProperties(&ctx->prop, device);
  if (err != cudaSuccess)
    return bail(fail_cuda(ctx, err, "selecting the device"));
  if (ctx->prop.major != 10)
    return bail(fail(ctx, HC_CUDA_ERR_NO_DEVICE,
                     "device %d (%s) has compute capability %d.%d; this backend needs sm_100 (10.x)",
                     device, ctx->prop.name, ctx->prop.major, ctx->prop.minor));
  err = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
  if (err == cudaSuccess)
    err = cudaMalloc(reinterpret_cast<void **>(&ctx->status_dev), sizeof(int));
  if (err == cudaSuccess)
    err = cudaMemset(ctx->status_dev, 0, sizeof(int));
  if (err == cudaSuccess)
    err = cudaHostAlloc(reinterpret_cast<void **>(&ctx->status_host), sizeof(int), cudaHostAllocDefault);
  if (err != cudaSuccess)
    return bail(fail_cuda(ctx, err, "creating the context's stream and status word"));
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult query = cudaDriverEntryPointSymbolNotFound;
  err = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &query);
  if (err != cudaSuccess || query != cudaDriverEntryPointSuccess || fn == nullptr) {
    cudaGetLastError();
    return bail(fail(ctx, HC_CUDA_ERR_CUDA, "the driver does not provide cuTensorMapEncodeTiled"));
  }
  ctx->encode = reinterpret_cast<EncodeTiledFn>(fn);
  if (const char *g = std::getenv("HC_CUDA_GROUP_N")) {
    const int v = std::atoi(g);
    if (v >= 1)
      ctx->group_n = ctx->group_n_wide = v;
  }
  if (const char *t = std::getenv("HC_CUDA_C_TMA_STORE"))
    ctx->c_tma_store = std::atoi(t) != 0;
  *out = ctx;
  return HC_CUDA_OK;
}

int hcCudaContextDestroy(HcCudaContext *ctx) {
  if (ctx == nullptr)
    return HC_CUDA_OK;
  if (ctx->device >= 0 && cudaSetDevice(ctx->device) == cudaSuccess) {
    if (ctx->stream != nullptr)
      cudaStreamSynchronize(ctx->stream);
    if (ctx->comm != nullptr && nccl_api().ok)
      nccl_api().CommDestroy(ctx->comm);
    for (void *p : ctx->stage)
      if (p != nullptr)
        cudaFree(p);
    for (int i = 0; i < HcCudaContext::kMaxSteps; ++i) {
      if (ctx->panel_in[i] != nullptr)
        cudaEventDestroy(ctx->panel_in[i]);
      if (ctx->panel_done[i] != nullptr)
        cudaEventDestroy(ctx->panel_done[i]);
    }
    if (ctx->fence_event != nullptr)
      cudaEventDestroy(ctx->fence_event);
    if (ctx->copy_in != nullptr)
      cudaStreamDestroy(ctx->copy_in);
    if (ctx->copy_out != nullptr)
      cudaStreamDestroy(ctx->copy_out);
    if (ctx->scratch != nullptr)
      cudaFree(ctx->scratch);
    if (ctx->counters != nullptr)
      cudaFree(ctx->counters);
    if (ctx->pairwise_leaves != nullptr)
      cudaFree(ctx->pairwise_leaves);
    if (ctx->status_dev != nullptr)
      cudaFree(ctx->status_dev);
    if (ctx->status_host != nullptr)
      cudaFreeHost(ctx->status_host);
    if (ctx->stream != nullptr)
      cudaStreamDestroy(ctx->stream);
    cudaGetLastError();
  }
  delete ctx;
  return HC_CUDA_OK;
}

const char *hcCudaContextLastError(const HcCudaContext *ctx) {
  if (ctx == nullptr)
    return g_thread_error.c_str();
  return ctx->last_error.c_str();
}

int hcCudaContextGetDeviceInfo(HcCudaContext *ctx, HcCudaDeviceInfo *out) {
  if (ctx == nullptr || out == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx and out must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  std::memset(out, 0, sizeof(*out));
  std::snprintf(out->name, sizeof(out->name), "%.127s", ctx->prop.name);
  out->device = ctx->device;
  out->cc_major = ctx->prop.major;
  out->cc_minor = ctx->prop.minor;
  out->sm_count = ctx->prop.multiProcessorCount;
  out->total_memory_bytes = static_cast<int64_t>(ctx->prop.totalGlobalMem);
  out->l2_bytes = ctx->prop.l2CacheSize;
  int khz = 0;
  if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device) != cudaSuccess)
    cudaGetLastError();
  out->sm_clock_khz = khz;
  return HC_CUDA_OK;
}

int hcCudaContextSynchronize(HcCudaContext *ctx) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  return synchronize_locked(ctx);
}

int hcCudaMalloc(HcCudaContext *ctx, size_t bytes, void **device_ptr) {
  if (ctx == nullptr || device_ptr == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx and device_ptr must not be null");
  *device_ptr = nullptr;
  std::lock_guard<std::mutex> lock(ctx->mu);
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  if (bytes == 0)
    return HC_CUDA_OK;
  HC_TRY_CUDA(ctx, cudaMalloc(device_ptr, bytes));
  return HC_CUDA_OK;
}

int hcCudaFree(HcCudaContext *ctx, void *device_ptr) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  if (device_ptr == nullptr)
    return HC_CUDA_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HC_TRY_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  HC_TRY_CUDA(ctx, cudaFree(device_ptr));
  return HC_CUDA_OK;
}

int hcCudaHostAlloc(size_t bytes, void **host_ptr) {
  if (host_ptr == nullptr)
    return fail(nullptr, HC_CUDA_ERR_INVALID_ARGUMENT, "host_ptr must not be null");
  *host_ptr = nullptr;
  if (bytes == 0)
    return HC_CUDA_OK;
  HC_TRY_CUDA(nullptr, cudaHostAlloc(host_ptr, bytes, cudaHostAllocPortable));
  return HC_CUDA_OK;
}

int hcCudaHostFree(void *host_ptr) {
  if (host_ptr == nullptr)
    return HC_CUDA_OK;
  HC_TRY_CUDA(nullptr, cudaFreeHost(host_ptr));
  return HC_CUDA_OK;
}

int hcCudaMemcpyHtoD(HcCudaContext *ctx, void *device_dst, const void *host_src, size_t bytes) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  if (bytes == 0)
    return HC_CUDA_OK;
  if (device_dst == nullptr || host_src == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "copy pointers must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HC_TRY_CUDA(ctx, cudaMemcpyAsync(device_dst, host_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  HC_TRY_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return HC_CUDA_OK;
}

int hcCudaMemcpyDtoH(HcCudaContext *ctx, void *host_dst, const void *device_src, size_t bytes) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  if (bytes == 0)
    return HC_CUDA_OK;
  if (host_dst == nullptr || device_src == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "copy pointers must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HC_TRY_CUDA(ctx, cudaMemcpyAsync(host_dst, device_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  HC_TRY_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return HC_CUDA_OK;
}

int hcCudaMemcpy2DHtoD(HcCudaContext *ctx, void *device_dst, size_t dst_pitch, const void *host_src,
                       size_t src_pitch, size_t width_bytes, size_t rows) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  if (width_bytes == 0 || rows == 0)
    return HC_CUDA_OK;
  if (device_dst == nullptr || host_src == nullptr || dst_pitch < width_bytes || src_pitch < width_bytes)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "bad 2-D copy arguments");
  std::lock_guard<std::mutex> lock(ctx->mu);
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(device_dst, dst_pitch, host_src, src_pitch, width_bytes, rows,
                                     cudaMemcpyHostToDevice, ctx->stream));
  HC_TRY_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return HC_CUDA_OK;
}

int hcCudaMemcpy2DDtoH(HcCudaContext *ctx, void *host_dst, size_t dst_pitch, const void *device_src,
                       size_t src_pitch, size_t width_bytes, size_t rows) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  if (width_bytes == 0 || rows == 0)
    return HC_CUDA_OK;
  if (host_dst == nullptr || device_src == nullptr || dst_pitch < width_bytes || src_pitch < width_bytes)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "bad 2-D copy arguments");
  std::lock_guard<std::mutex> lock(ctx->mu);
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(host_dst, dst_pitch, device_src, src_pitch, width_bytes, rows,
                                     cudaMemcpyDeviceToHost, ctx->stream));
  HC_TRY_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return HC_CUDA_OK;
}

int hcCudaMemset(HcCudaContext *ctx, void *device_ptr, int byte_value, size_t bytes) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  if (bytes == 0)
    return HC_CUDA_OK;
  if (device_ptr == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "device_ptr must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HC_TRY_CUDA(ctx, cudaMemsetAsync(device_ptr, byte_value, bytes, ctx->stream));
  return HC_CUDA_OK;
}

int hcCudaGemmPlan(const HcCudaGemmArgs *args, int sm_count, HcCudaGemmPlanInfo *out) {
  return plan_gemm(nullptr, args, sm_count, /*host_buffers=*/false, out);
}

int hcCudaGemm(HcCudaContext *ctx, const HcCudaGemmArgs *args) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  HcCudaGemmPlanInfo plan;
  if (int rc = plan_gemm(ctx, args, ctx->prop.multiProcessorCount, false, &plan))
    return rc;
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  return enqueue_gemm(ctx, args, plan);
}

int hcCudaGemmPush(HcCudaContext *ctx, const HcCudaGemmArgs *args, float *const *targets, int n_targets) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (n_targets < 0 || n_targets > HC_CUDA_MAX_PUSH_TARGETS || (n_targets > 0 && targets == nullptr))
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "n_targets must be in [0, %d] with a non-null array",
                HC_CUDA_MAX_PUSH_TARGETS);
  if (args == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "args must not be null");
  HcCudaGemmArgs dense = *args;
  if (dense.variant == HC_CUDA_GEMM_AUTO)
    dense.variant = HC_CUDA_GEMM_DENSE;
  if (dense.variant != HC_CUDA_GEMM_DENSE)
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "pushing C to other buffers is implemented by the dense kernels only");
  if (dense.c_dtype != HC_CUDA_C_F32 && n_targets > 0)
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "pushing C to other buffers needs a float32 C");
  HcCudaGemmPlanInfo plan;
  ctx->planning_push = n_targets > 0;
  const int plan_rc = plan_gemm(ctx, &dense, ctx->prop.multiProcessorCount, false, &plan);
  ctx->planning_push = false;
  if (plan_rc)
    return plan_rc;
  hc::sm100::Epilogue push{};
  if (plan.variant == HC_CUDA_GEMM_DENSE && n_targets > 0) {
    if ((dense.ldc & 3) != 0 || (reinterpret_cast<uintptr_t>(dense.c) & 15) != 0)  // (float32 C here)
      return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "pushing needs c 16-byte aligned and ldc a multiple of 4");
    const size_t c_bytes = (static_cast<size_t>(dense.m - 1) * dense.ldc + dense.n) * 4;
    for (int i = 0; i < n_targets; ++i) {
      if (targets[i] == nullptr || (reinterpret_cast<uintptr_t>(targets[i]) & 15) != 0)
        return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "push target %d must be a 16-byte-aligned device pointer", i);
      if (ranges_overlap(targets[i], c_bytes, dense.c, c_bytes))
        return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "push target %d overlaps c", i);
      push.push[i] = targets[i];
    }
    push.push_count = n_targets;
  } else if (n_targets > 0 && dense.k == 0 && dense.m > 0 && dense.n > 0) {
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "k == 0 with push targets is not supported");
  }
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  return enqueue_gemm(ctx, &dense, plan, push);
}

int hcCudaIpcExport(HcCudaContext *ctx, const void *device_ptr, void *handle, size_t handle_bytes) {
  static_assert(sizeof(cudaIpcMemHandle_t) <= HC_CUDA_IPC_HANDLE_BYTES, "handle buffer too small");
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (device_ptr == nullptr || handle == nullptr || handle_bytes < sizeof(cudaIpcMemHandle_t))
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "device_ptr and a handle buffer of at least %zu bytes are required",
                sizeof(cudaIpcMemHandle_t));
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaIpcMemHandle_t h;
  HC_TRY_CUDA(ctx, cudaIpcGetMemHandle(&h, const_cast<void *>(device_ptr)));
  std::memset(handle, 0, handle_bytes);
  std::memcpy(handle, &h, sizeof(h));
  return HC_CUDA_OK;
}

int hcCudaIpcOpen(HcCudaContext *ctx, const void *handle, size_t handle_bytes, void **device_ptr) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (device_ptr == nullptr || handle == nullptr || handle_bytes < sizeof(cudaIpcMemHandle_t))
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "a handle of at least %zu bytes and device_ptr are required",
                sizeof(cudaIpcMemHandle_t));
  *device_ptr = nullptr;
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  HC_TRY_CUDA(ctx, cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return HC_CUDA_OK;
}

int hcCudaIpcClose(HcCudaContext *ctx, void *device_ptr) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  if (device_ptr == nullptr)
    return HC_CUDA_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HC_TRY_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  HC_TRY_CUDA(ctx, cudaIpcCloseMemHandle(device_ptr));
  return HC_CUDA_OK;
}

int hcCudaGemmHost(HcCudaContext *ctx, const HcCudaGemmArgs *args) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  HcCudaGemmPlanInfo plan;
  if (int rc = plan_gemm(ctx, args, ctx->prop.multiProcessorCount, true, &plan))
    return rc;
  if (plan.variant == HC_CUDA_GEMM_NOOP)
    return HC_CUDA_OK;
  const size_t m = static_cast<size_t>(args->m), n = static_cast<size_t>(args->n),
               k = static_cast<size_t>(args->k);
  const size_t ce = args->c_dtype == HC_CUDA_C_F32 ? 4 : 2;  // bytes per element of C
  char *const host_c = static_cast<char *>(args->c);
  const size_t host_c_pitch = static_cast<size_t>(args->ldc) * ce;
  if (plan.variant == HC_CUDA_GEMM_ZERO_FILL) {
    for (size_t i = 0; i < m; ++i)
      std::memset(host_c + i * host_c_pitch, 0, n * ce);
    return HC_CUDA_OK;
  }
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  bool has_bias = false;
  for (int i = 0; i < args->epilogue_count; ++i)
    has_bias = has_bias || args->epilogue_kind[i] == HC_CUDA_EPILOGUE_BIAS_COLUMN;
  // Device copies get pitches that satisfy TMA (16 bytes), so no repack pass is needed.
  const size_t es = hc::sm100::dtype_is_8bit(args->dtype) ? 1 : 2;  // bytes per element of A and B
  const size_t lda = static_cast<size_t>(round_up(args->k, kRepackPitchBytes / static_cast<int64_t>(es)));
  const bool b_nk = args->b_layout == HC_CUDA_B_NK;
  const size_t b_rows = b_nk ? n : k, b_cols = b_nk ? k : n;  // B as stored
  const size_t ldb = static_cast<size_t>(round_up(static_cast<int64_t>(b_cols), kRepackPitchBytes / static_cast<int64_t>(es)));
  const size_t ldc = static_cast<size_t>(round_up(args->n, 16 / static_cast<int64_t>(ce)));  // 16-byte rows: TMA stores
  if (int rc = ensure_stage(ctx, 0, m * lda * es))
    return rc;
  if (int rc = ensure_stage(ctx, 1, b_rows * ldb * es))
    return rc;
  // C's staging buffer also holds the bias vector, after the last row.
  if (int rc = ensure_stage(ctx, 2, round_up(static_cast<int64_t>(m * ldc * ce), 16) + (has_bias ? n * 4 : 0)))
    return rc;
  HcCudaGemmArgs dev = *args;
  char *const dev_c = static_cast<char *>(ctx->stage[2]);
  float *bias_dev = reinterpret_cast<float *>(dev_c + round_up(static_cast<int64_t>(m * ldc * ce), 16));
  if (has_bias) {
    dev.bias = bias_dev;
    HC_TRY_CUDA(ctx, cudaMemcpyAsync(bias_dev, args->bias, n * 4, cudaMemcpyHostToDevice, ctx->stream));
  }
  dev.a = ctx->stage[0];
  dev.lda = static_cast<int64_t>(lda);
  dev.b = ctx->stage[1];
  dev.ldb = static_cast<int64_t>(ldb);
  dev.c = dev_c;
  dev.ldc = static_cast<int64_t>(ldc);

  const size_t total_bytes = (m * k + k * n) * es + m * n * ce;
  if (plan.variant == HC_CUDA_GEMM_ELEMENTWISE) {
    if (args->accumulate)
      HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(dev_c, ldc * ce, host_c, host_c_pitch, n * ce, m, cudaMemcpyHostToDevice,
                                         ctx->stream));
    if (int rc = plan_gemm(ctx, &dev, ctx->prop.multiProcessorCount, false, &plan))
      return rc;
    if (int rc = enqueue_gemm(ctx, &dev, plan))
      return rc;
    HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(host_c, host_c_pitch, dev_c, ldc * ce, n * ce, m, cudaMemcpyDeviceToHost,
                                       ctx->stream));
    return synchronize_locked(ctx);
  }
  // (8-bit operands take the sequential path: a float8 B stored [K, N] is transposed on the device as
  // a whole before the product, which the panel pipeline below does not provide for.)
  const bool pipelined = plan.variant == HC_CUDA_GEMM_DENSE && m >= 1024 && total_bytes >= (size_t(32) << 20) &&
                         es == 2 && std::getenv("HC_CUDA_NO_COPY_OVERLAP") == nullptr;
  if (!pipelined) {
    HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(ctx->stage[0], lda * es, args->a, static_cast<size_t>(args->lda) * es,
                                       k * es, m, cudaMemcpyHostToDevice, ctx->stream));
    HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(ctx->stage[1], ldb * es, args->b, static_cast<size_t>(args->ldb) * es,
                                       b_cols * es, b_rows, cudaMemcpyHostToDevice, ctx->stream));
    if (args->accumulate)
      HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(dev_c, ldc * ce, host_c, host_c_pitch, n * ce, m, cudaMemcpyHostToDevice,
                                         ctx->stream));
    if (int rc = plan_gemm(ctx, &dev, ctx->prop.multiProcessorCount, false, &plan))
      return rc;
    if (int rc = enqueue_gemm(ctx, &dev, plan))
      return rc;
    HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(host_c, host_c_pitch, dev_c, ldc * ce, n * ce, m, cudaMemcpyDeviceToHost,
                                       ctx->stream));
    return synchronize_locked(ctx);
  }

  if (int rc = ensure_copy_streams(ctx))
    return rc;
  // Everything already queued on the main stream comes first.
  HC_TRY_CUDA(ctx, cudaEventRecord(ctx->fence_event, ctx->stream));
  HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_in, ctx->fence_event, 0));
  HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, ctx->fence_event, 0));
  // Whatever way this call ends, no copy may still be running into the caller's arrays or the
  // staging buffers when it returns: an error return in the middle of the panel loop waits for
  // all three streams first (the success path waits in finish()).
  struct DrainOnExit {
    HcCudaContext *ctx;
    bool armed = true;
    ~DrainOnExit() {
      if (!armed)
        return;
      for (cudaStream_t s : {ctx->copy_in, ctx->copy_out, ctx->stream})
        if (cudaStreamSynchronize(s) != cudaSuccess)
          cudaGetLastError();
    }
  } drain_guard{ctx};
  struct PanelsPlanning {  // the sub-products below are planned without k-splits
    HcCudaContext *ctx;
    explicit PanelsPlanning(HcCudaContext *c) : ctx(c) { ctx->planning_host_panels = true; }
    ~PanelsPlanning() { ctx->planning_host_panels = false; }
  } planning_guard(ctx);

  // One sub-product C[row0:row0+rows, col0:col0+cols] on the staged operands, then its way home.
  int done_events = 0;
  auto multiply_and_fetch = [&](size_t row0, size_t rows, size_t col0, size_t cols, cudaEvent_t inputs_ready) -> int {
    HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, inputs_ready, 0));
    HcCudaGemmArgs part = dev;
    part.m = static_cast<int64_t>(rows);
    part.n = static_cast<int64_t>(cols);
    part.a = static_cast<const char *>(dev.a) + row0 * lda * 2;
    part.b = static_cast<const char *>(dev.b) + (b_nk ? col0 * ldb : col0) * 2;
    part.c = dev_c + (row0 * ldc + col0) * ce;
    if (has_bias)
      part.bias = dev.bias + col0;
    HcCudaGemmPlanInfo part_plan;
    if (int rc = plan_gemm(ctx, &part, ctx->prop.multiProcessorCount, false, &part_plan))
      return rc;
    if (int rc = enqueue_gemm(ctx, &part, part_plan))
      return rc;
    cudaEvent_t done = ctx->panel_done[done_events++];
    HC_TRY_CUDA(ctx, cudaEventRecord(done, ctx->stream));
    HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, done, 0));
    HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(host_c + row0 * host_c_pitch + col0 * ce, host_c_pitch, part.c, ldc * ce,
                                       cols * ce, rows, cudaMemcpyDeviceToHost, ctx->copy_out));
    return HC_CUDA_OK;
  };
  auto finish = [&]() -> int {
    HC_TRY_CUDA(ctx, cudaEventRecord(ctx->fence_event, ctx->copy_out));
    HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->fence_event, 0));
    const int rc = synchronize_locked(ctx);  // waits for the main stream, which waits for copy_out
    drain_guard.armed = rc != HC_CUDA_OK && rc != HC_CUDA_ERR_DEVICE_TIMEOUT;
    return rc;
  };
  // Panels are multiples of 256 rows (or columns); a remainder shorter than that joins the last one.
  auto panel_size = [](size_t total) {
    const size_t size = (total + HcCudaContext::kMaxPanels - 1) / HcCudaContext::kMaxPanels;
    return static_cast<size_t>(round_up(static_cast<int64_t>(size), 256));
  };
  auto panel_count = [](size_t total, size_t size) {
    const size_t count = total / size;
    return static_cast<int>(count == 0 || total - count * size >= 256 ? count + 1 : count);
  };
  auto panel_extent = [](size_t start, size_t total, size_t size) {
    return total - start < size + 256 ? total - start : size;
  };
  const size_t panel_rows = panel_size(m);
  const int row_panels = panel_count(m, panel_rows);

  // Pinned host memory can be copied in strided pieces at full rate; with it, and a C that does
  // not have to travel to the device first, A and B are sent in alternating panels (below).
  auto is_pinned = [](const void *p) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    return attr.type == cudaMemoryTypeHost;
  };
  const bool square = n >= 2048 && !args->accumulate && is_pinned(args->a) && is_pinned(args->b) &&
                      is_pinned(args->c) && std::getenv("HC_CUDA_ROW_PANELS_ONLY") == nullptr;
  if (!square) {
    // Row panels. PCIe carries both directions at once, so the rows of C of one panel travel back
    // while the next panels of A are still arriving and being multiplied; the call then takes
    // about (time to send B) + max(time to send A, time to fetch C) instead of the sum of all four.
    HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(ctx->stage[1], ldb * 2, args->b, static_cast<size_t>(args->ldb) * 2,
                                       b_cols * 2, b_rows, cudaMemcpyHostToDevice, ctx->copy_in));
    for (int p = 0; p < row_panels; ++p) {
      const size_t row0 = static_cast<size_t>(p) * panel_rows;
      const size_t rows = panel_extent(row0, m, panel_rows);
      HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(static_cast<char *>(ctx->stage[0]) + row0 * lda * 2, lda * 2,
                                         static_cast<const char *>(args->a) + row0 * static_cast<size_t>(args->lda) * 2,
                                         static_cast<size_t>(args->lda) * 2, k * 2, rows, cudaMemcpyHostToDevice,
                                         ctx->copy_in));
      if (args->accumulate)  // this panel's rows of C are the starting values of its sums
        HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(dev_c + row0 * ldc * ce, ldc * ce, host_c + row0 * host_c_pitch, host_c_pitch,
                                           n * ce, rows, cudaMemcpyHostToDevice, ctx->copy_in));
      HC_TRY_CUDA(ctx, cudaEventRecord(ctx->panel_in[p], ctx->copy_in));
      if (int rc = multiply_and_fetch(row0, rows, 0, n, ctx->panel_in[p]))
        return rc;
    }
    return finish();
  }

  // Alternating panels. Waiting for all of B before the first product leaves the return path idle
  // for the time B takes. Instead row panels of A and column panels of B are sent in turn, and
  // after each arrival everything that has become computable is multiplied and sent back: A_s
  // gives C[rows s, columns of B_0..B_{s-1}], B_s gives C[rows of A_0..A_s, columns s]. The
  // computable part of C grows with the square of what has arrived, so the return path starts after
  // one panel of each instead of after a whole operand, and both directions stay busy to the end.
  const size_t panel_cols = panel_size(n);
  const int col_panels = panel_count(n, panel_cols);
  int in_events = 0;
  size_t rows_sent = 0, cols_sent = 0;
  for (int step = 0; step < (row_panels > col_panels ? row_panels : col_panels); ++step) {
    if (step < row_panels) {
      const size_t row0 = rows_sent;
      const size_t rows = panel_extent(row0, m, panel_rows);
      HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(static_cast<char *>(ctx->stage[0]) + row0 * lda * 2, lda * 2,
                                         static_cast<const char *>(args->a) + row0 * static_cast<size_t>(args->lda) * 2,
                                         static_cast<size_t>(args->lda) * 2, k * 2, rows, cudaMemcpyHostToDevice,
                                         ctx->copy_in));
      cudaEvent_t arrived = ctx->panel_in[in_events++];
      HC_TRY_CUDA(ctx, cudaEventRecord(arrived, ctx->copy_in));
      rows_sent += rows;
      if (cols_sent > 0)
        if (int rc = multiply_and_fetch(row0, rows, 0, cols_sent, arrived))
          return rc;
    }
    if (step < col_panels) {
      const size_t col0 = cols_sent;
      const size_t cols = panel_extent(col0, n, panel_cols);
      if (b_nk) {  // stored [n, k]: the panel is a block of rows
        HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(static_cast<char *>(ctx->stage[1]) + col0 * ldb * 2, ldb * 2,
                                           static_cast<const char *>(args->b) + col0 * static_cast<size_t>(args->ldb) * 2,
                                           static_cast<size_t>(args->ldb) * 2, k * 2, cols, cudaMemcpyHostToDevice,
                                           ctx->copy_in));
      } else {     // stored [k, n]: a block of columns, k pieces of `cols` elements
        HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(static_cast<char *>(ctx->stage[1]) + col0 * 2, ldb * 2,
                                           static_cast<const char *>(args->b) + col0 * 2,
                                           static_cast<size_t>(args->ldb) * 2, cols * 2, k, cudaMemcpyHostToDevice,
                                           ctx->copy_in));
      }
      cudaEvent_t arrived = ctx->panel_in[in_events++];
      HC_TRY_CUDA(ctx, cudaEventRecord(arrived, ctx->copy_in));
      cols_sent += cols;
      if (rows_sent > 0)
        if (int rc = multiply_and_fetch(0, rows_sent, col0, cols, arrived))
          return rc;
    }
  }
  return finish();
}

int hcCudaGemmHostDeviceA(HcCudaContext *ctx, const HcCudaGemmArgs *args) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  HcCudaGemmPlanInfo plan;
  if (int rc = plan_gemm(ctx, args, ctx->prop.multiProcessorCount, true, &plan))
    return rc;
  if (plan.variant == HC_CUDA_GEMM_NOOP)
    return HC_CUDA_OK;
  if (args->accumulate != 0 || hc::sm100::dtype_is_8bit(args->dtype) || args->k == 0)
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "hcCudaGemmHostDeviceA computes C = ops(A*B) for float16 / bfloat16 "
                                              "operands with k > 0 (no accumulate, no 8-bit operands)");
  if ((reinterpret_cast<uintptr_t>(args->a) & 15) != 0 || (args->lda & 7) != 0)
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "the device-resident a must be 16-byte aligned with lda a multiple of 8");
  const size_t m = static_cast<size_t>(args->m), n = static_cast<size_t>(args->n), k = static_cast<size_t>(args->k);
  const size_t ce = args->c_dtype == HC_CUDA_C_F32 ? 4 : 2;
  char *const host_c = static_cast<char *>(args->c);
  const size_t host_c_pitch = static_cast<size_t>(args->ldc) * ce;
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  bool has_bias = false;
  for (int i = 0; i < args->epilogue_count; ++i)
    has_bias = has_bias || args->epilogue_kind[i] == HC_CUDA_EPILOGUE_BIAS_COLUMN;
  const bool b_nk = args->b_layout == HC_CUDA_B_NK;
  const size_t b_rows = b_nk ? n : k, b_cols = b_nk ? k : n;  // B as stored
  const size_t ldb = static_cast<size_t>(round_up(static_cast<int64_t>(b_cols), kRepackPitchBytes / 2));
  const size_t ldc = static_cast<size_t>(round_up(args->n, 16 / static_cast<int64_t>(ce)));
  if (int rc = ensure_stage(ctx, 1, b_rows * ldb * 2))
    return rc;
  if (int rc = ensure_stage(ctx, 2, round_up(static_cast<int64_t>(m * ldc * ce), 16) + (has_bias ? n * 4 : 0)))
    return rc;
  if (int rc = ensure_copy_streams(ctx))
    return rc;
  HcCudaGemmArgs dev = *args;
  char *const dev_c = static_cast<char *>(ctx->stage[2]);
  dev.b = ctx->stage[1];
  dev.ldb = static_cast<int64_t>(ldb);
  dev.c = dev_c;
  dev.ldc = static_cast<int64_t>(ldc);
  if (has_bias) {
    float *bias_dev = reinterpret_cast<float *>(dev_c + round_up(static_cast<int64_t>(m * ldc * ce), 16));
    dev.bias = bias_dev;
    HC_TRY_CUDA(ctx, cudaMemcpyAsync(bias_dev, args->bias, n * 4, cudaMemcpyHostToDevice, ctx->stream));
  }
  HC_TRY_CUDA(ctx, cudaEventRecord(ctx->fence_event, ctx->stream));
  HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_in, ctx->fence_event, 0));
  HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, ctx->fence_event, 0));
  struct Drain {  // no copy may still touch the caller's arrays when the call returns
    HcCudaContext *ctx;
    ~Drain() {
      for (cudaStream_t s : {ctx->copy_in, ctx->copy_out, ctx->stream})
        if (cudaStreamSynchronize(s) != cudaSuccess)
          cudaGetLastError();
    }
  } drain{ctx};
  struct PanelsPlanning {  // the sub-products are planned without k-splits: the bits of one launch
    HcCudaContext *ctx;
    explicit PanelsPlanning(HcCudaContext *c) : ctx(c) { ctx->planning_host_panels = true; }
    ~PanelsPlanning() { ctx->planning_host_panels = false; }
  } planning_guard(ctx);
  // Column panels of B (multiples of 256 columns, at most kMaxPanels): panel p + 1 arrives while
  // panel p is multiplied and the columns of C of panel p - 1 leave.
  size_t panel_cols = (n + HcCudaContext::kMaxPanels - 1) / HcCudaContext::kMaxPanels;
  panel_cols = static_cast<size_t>(round_up(static_cast<int64_t>(panel_cols), 256));
  if (plan.variant != HC_CUDA_GEMM_DENSE || n < 1024)
    panel_cols = n;
  int panel = 0;
  for (size_t col0 = 0; col0 < n; ++panel) {
    size_t cols = n - col0 < panel_cols + 256 ? n - col0 : panel_cols;
    if (b_nk)
      HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(static_cast<char *>(ctx->stage[1]) + col0 * ldb * 2, ldb * 2,
                                         static_cast<const char *>(args->b) + col0 * static_cast<size_t>(args->ldb) * 2,
                                         static_cast<size_t>(args->ldb) * 2, k * 2, cols, cudaMemcpyHostToDevice,
                                         ctx->copy_in));
    else
      HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(static_cast<char *>(ctx->stage[1]) + col0 * 2, ldb * 2,
                                         static_cast<const char *>(args->b) + col0 * 2,
                                         static_cast<size_t>(args->ldb) * 2, cols * 2, k, cudaMemcpyHostToDevice,
                                         ctx->copy_in));
    HC_TRY_CUDA(ctx, cudaEventRecord(ctx->panel_in[panel], ctx->copy_in));
    HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->panel_in[panel], 0));
    HcCudaGemmArgs part = dev;
    part.n = static_cast<int64_t>(cols);
    part.b = static_cast<const char *>(dev.b) + (b_nk ? col0 * ldb : col0) * 2;
    part.c = dev_c + col0 * ce;
    if (has_bias)
      part.bias = dev.bias + col0;
    HcCudaGemmPlanInfo part_plan;
    if (int rc = plan_gemm(ctx, &part, ctx->prop.multiProcessorCount, false, &part_plan))
      return rc;
    if (int rc = enqueue_gemm(ctx, &part, part_plan))
      return rc;
    HC_TRY_CUDA(ctx, cudaEventRecord(ctx->panel_done[panel], ctx->stream));
    HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, ctx->panel_done[panel], 0));
    HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(host_c + col0 * ce, host_c_pitch, part.c, ldc * ce, cols * ce, m,
                                       cudaMemcpyDeviceToHost, ctx->copy_out));
    col0 += cols;
  }
  HC_TRY_CUDA(ctx, cudaEventRecord(ctx->fence_event, ctx->copy_out));
  HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->fence_event, 0));
  return synchronize_locked(ctx);
}

namespace {

// Validation shared by hcCudaMap and hcCudaMapHost; fills `ops`.
int check_map_args(const HcCudaContext *ctx, const HcCudaMapArgs *args, hc::sm100::MapOps *ops) {
  if (args == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "args must not be null");
  if (args->n < 0)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "n must be non-negative (got %lld)", (long long)args->n);
  if (args->n > (int64_t(1) << 40))
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "n must be at most 2^40");
  if (args->op_count < 0 || args->op_count > HC_CUDA_MAX_MAP_OPS)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "op_count must be 0..%d (got %d)", HC_CUDA_MAX_MAP_OPS,
                args->op_count);
  bool uses_other = false;
  ops->count = args->op_count;
  for (int i = 0; i < args->op_count; ++i) {
    const int kind = args->op_kind[i];
    if (kind < HC_CUDA_MAP_SCALE || kind > HC_CUDA_MAP_REVERSE_MIN_OTHER)
      return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "op_kind[%d] is not an HcCudaMapOp (got %d)", i, kind);
    uses_other = uses_other || hc::sm100::map_op_uses_other(kind);
    ops->kind[i] = kind;
    ops->value[i] = args->op_value[i];
  }
  if (args->n == 0)
    return HC_CUDA_OK;
  if (args->x == nullptr || args->out == nullptr || (uses_other && args->y == nullptr))
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "x and out (and y, when an ..._OTHER operation is used) must "
                                                   "not be null");
  const size_t bytes = static_cast<size_t>(args->n) * 4;
  const void *inputs[2] = {args->x, uses_other ? args->y : nullptr};
  for (const void *in : inputs) {
    if (in == nullptr)
      continue;
    if ((reinterpret_cast<uintptr_t>(in) & 3) != 0 || (reinterpret_cast<uintptr_t>(args->out) & 3) != 0)
      return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "x, y and out must be 4-byte aligned");
    if (in != args->out && ranges_overlap(in, bytes, args->out, bytes))
      return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "out may be the same buffer as an input, but must not "
                                                     "partially overlap one");
  }
  return HC_CUDA_OK;
}

} // namespace

int hcCudaMap(HcCudaContext *ctx, const HcCudaMapArgs *args) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  hc::sm100::MapOps ops{};
  if (int rc = check_map_args(ctx, args, &ops))
    return rc;
  if (args->n == 0)
    return HC_CUDA_OK;
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HC_TRY_CUDA(ctx, hc::sm100::launch_map_f32(args->x, args->y, args->out, args->n, ops,
                                             ctx->prop.multiProcessorCount, ctx->stream));
  return HC_CUDA_OK;
}

int hcCudaMapHost(HcCudaContext *ctx, const HcCudaMapArgs *args) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  hc::sm100::MapOps ops{};
  if (int rc = check_map_args(ctx, args, &ops))
    return rc;
  if (args->n == 0)
    return HC_CUDA_OK;
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  bool two = false;
  for (int i = 0; i < ops.count; ++i)
    two = two || hc::sm100::map_op_uses_other(ops.kind[i]);
  const size_t n = static_cast<size_t>(args->n);
  // Chunks of 4 Mi elements (16 MiB per array): a ring of kMaxSteps device chunks per array, so
  // that chunk i + 1 arrives and chunk i - 1 leaves while chunk i is computed.
  constexpr size_t kChunk = size_t(4) << 20;
  constexpr int kRing = HcCudaContext::kMaxSteps;
  const size_t chunks = (n + kChunk - 1) / kChunk;
  const size_t ring = chunks < static_cast<size_t>(kRing) ? chunks : static_cast<size_t>(kRing);
  const size_t slot = (n < kChunk ? n : kChunk) * 4;
  if (int rc = ensure_stage(ctx, 0, ring * slot))
    return rc;
  if (two)
    if (int rc = ensure_stage(ctx, 1, ring * slot))
      return rc;
  if (int rc = ensure_stage(ctx, 2, ring * slot))
    return rc;
  if (int rc = ensure_copy_streams(ctx))
    return rc;
  HC_TRY_CUDA(ctx, cudaEventRecord(ctx->fence_event, ctx->stream));
  HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_in, ctx->fence_event, 0));
  HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, ctx->fence_event, 0));
  struct Drain {  // no copy may still touch the caller's arrays when the call returns
    HcCudaContext *ctx;
    ~Drain() {
      for (cudaStream_t s : {ctx->copy_in, ctx->copy_out, ctx->stream})
        if (cudaStreamSynchronize(s) != cudaSuccess)
          cudaGetLastError();
    }
  } drain{ctx};
  for (size_t chunk = 0; chunk < chunks; ++chunk) {
    const size_t begin = chunk * kChunk;
    const size_t count = n - begin < kChunk ? n - begin : kChunk;
    const int s = static_cast<int>(chunk % ring);
    float *dx = reinterpret_cast<float *>(static_cast<char *>(ctx->stage[0]) + s * slot);
    float *dy = two ? reinterpret_cast<float *>(static_cast<char *>(ctx->stage[1]) + s * slot) : nullptr;
    float *dout = reinterpret_cast<float *>(static_cast<char *>(ctx->stage[2]) + s * slot);
    // Ring slot s is free for new input once the kernel of its previous user has run, and its
    // output slot once that chunk's copy out has finished.
    if (chunk >= ring) {
      HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_in, ctx->panel_done[s], 0));
      HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->panel_in[s], 0));  // re-recorded below, after use
    }
    HC_TRY_CUDA(ctx, cudaMemcpyAsync(dx, args->x + begin, count * 4, cudaMemcpyHostToDevice, ctx->copy_in));
    if (two)
      HC_TRY_CUDA(ctx, cudaMemcpyAsync(dy, args->y + begin, count * 4, cudaMemcpyHostToDevice, ctx->copy_in));
    HC_TRY_CUDA(ctx, cudaEventRecord(ctx->fence_event, ctx->copy_in));
    HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->fence_event, 0));
    HC_TRY_CUDA(ctx, hc::sm100::launch_map_f32(dx, dy, dout, static_cast<long long>(count), ops,
                                               ctx->prop.multiProcessorCount, ctx->stream));
    HC_TRY_CUDA(ctx, cudaEventRecord(ctx->panel_done[s], ctx->stream));
    HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, ctx->panel_done[s], 0));
    HC_TRY_CUDA(ctx, cudaMemcpyAsync(args->out + begin, dout, count * 4, cudaMemcpyDeviceToHost, ctx->copy_out));
    HC_TRY_CUDA(ctx, cudaEventRecord(ctx->panel_in[s], ctx->copy_out));  // "output slot s has left"
  }
  HC_TRY_CUDA(ctx, cudaEventRecord(ctx->fence_event, ctx->copy_out));
  HC_TRY_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->fence_event, 0));
  return synchronize_locked(ctx);
}

namespace {

int check_pairwise_args(const HcCudaContext *ctx, const HcCudaPairwiseArgs *args) {
  if (args == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "args must not be null");
  if (args->w1 < 0 || args->w2 < 0 || args->h < 0)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "w1, w2 and h must be non-negative (got %lld, %lld, %lld)",
                (long long)args->w1, (long long)args->w2, (long long)args->h);
  if (args->w1 > 0x7fffffffLL || args->w2 > 0x7fffffffLL)
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "w1 and w2 must be below 2^31");
  if (args->h > hc::sm100::pairwise_max_h())
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "h must be at most %d (got %lld)", hc::sm100::pairwise_max_h(),
                (long long)args->h);
  if (args->op != HC_CUDA_PAIRWISE_EUCLIDEAN && args->op != HC_CUDA_PAIRWISE_SQUARED)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "op is not an HcCudaPairwiseOp (got %d)", args->op);
  if (args->w1 == 0 || args->w2 == 0 || args->h == 0)
    return HC_CUDA_OK;
  if (args->x1 == nullptr || args->x2 == nullptr || args->out == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "x1, x2 and out must not be null");
  if (((reinterpret_cast<uintptr_t>(args->x1) | reinterpret_cast<uintptr_t>(args->x2) |
        reinterpret_cast<uintptr_t>(args->out)) & 3) != 0)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "x1, x2 and out must be 4-byte aligned");
  if (args->ld1 < args->h || args->ld2 < args->h || args->ldo < args->w2 || args->ld1 > kMaxPitch ||
      args->ld2 > kMaxPitch || args->ldo > kMaxPitch)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ld1 and ld2 must be at least h (%lld) and ldo at least w2 (%lld)",
                (long long)args->h, (long long)args->w2);
  const size_t bytes1 = (static_cast<size_t>(args->w1 - 1) * args->ld1 + args->h) * 4;
  const size_t bytes2 = (static_cast<size_t>(args->w2 - 1) * args->ld2 + args->h) * 4;
  const size_t bytes_out = (static_cast<size_t>(args->w1 - 1) * args->ldo + args->w2) * 4;
  if (ranges_overlap(args->out, bytes_out, args->x1, bytes1) || ranges_overlap(args->out, bytes_out, args->x2, bytes2))
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "out must not overlap x1 or x2");
  return HC_CUDA_OK;
}

// The summation schedule for h on the device (kept until another h is asked for).
int ensure_pairwise_schedule(HcCudaContext *ctx, int h) {
  if (ctx->pairwise_h == h)
    return HC_CUDA_OK;
  const int count = hc::sm100::pairwise_schedule(h, nullptr, 0);
  std::vector<int4> leaves(static_cast<size_t>(count));
  hc::sm100::pairwise_schedule(h, leaves.data(), count);
  HC_TRY_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // no launch may still read the old schedule
  if (ctx->pairwise_leaves != nullptr) {
    HC_TRY_CUDA(ctx, cudaFree(ctx->pairwise_leaves));
    ctx->pairwise_leaves = nullptr;
    ctx->pairwise_h = -1;
  }
  HC_TRY_CUDA(ctx, cudaMalloc(reinterpret_cast<void **>(&ctx->pairwise_leaves), sizeof(int4) * static_cast<size_t>(count)));
  HC_TRY_CUDA(ctx, cudaMemcpy(ctx->pairwise_leaves, leaves.data(), sizeof(int4) * static_cast<size_t>(count),
                              cudaMemcpyHostToDevice));
  ctx->pairwise_h = h;
  ctx->pairwise_leaf_count = count;
  return HC_CUDA_OK;
}

} // namespace

int hcCudaPairwise(HcCudaContext *ctx, const HcCudaPairwiseArgs *args) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (int rc = check_pairwise_args(ctx, args))
    return rc;
  if (args->w1 == 0 || args->w2 == 0 || args->h == 0)
    return HC_CUDA_OK;
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  if (int rc = ensure_pairwise_schedule(ctx, static_cast<int>(args->h)))
    return rc;
  HC_TRY_CUDA(ctx, hc::sm100::launch_pairwise_f32(args->x1, args->ld1, args->x2, args->ld2, args->out, args->ldo,
                                                  static_cast<int>(args->w1), static_cast<int>(args->w2),
                                                  static_cast<int>(args->h), args->op == HC_CUDA_PAIRWISE_EUCLIDEAN,
                                                  ctx->pairwise_leaves, ctx->pairwise_leaf_count, ctx->stream));
  return HC_CUDA_OK;
}

int hcCudaPairwiseHost(HcCudaContext *ctx, const HcCudaPairwiseArgs *args) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (int rc = check_pairwise_args(ctx, args))
    return rc;
  if (args->w1 == 0 || args->w2 == 0 || args->h == 0)
    return HC_CUDA_OK;
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  if (int rc = ensure_pairwise_schedule(ctx, static_cast<int>(args->h)))
    return rc;
  // Compact device copies with pitches that allow 16-byte accesses.
  const size_t w1 = static_cast<size_t>(args->w1), w2 = static_cast<size_t>(args->w2), h = static_cast<size_t>(args->h);
  const size_t ld_in = static_cast<size_t>(round_up(static_cast<int64_t>(h), 4));
  const size_t ld_out = static_cast<size_t>(round_up(static_cast<int64_t>(w2), 4));
  if (int rc = ensure_stage(ctx, 0, w1 * ld_in * 4))
    return rc;
  if (int rc = ensure_stage(ctx, 1, w2 * ld_in * 4))
    return rc;
  if (int rc = ensure_stage(ctx, 2, w1 * ld_out * 4))
    return rc;
  struct Drain {  // no copy may still touch the caller's arrays when the call returns
    HcCudaContext *ctx;
    ~Drain() {
      if (cudaStreamSynchronize(ctx->stream) != cudaSuccess)
        cudaGetLastError();
    }
  } drain{ctx};
  HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(ctx->stage[0], ld_in * 4, args->x1, static_cast<size_t>(args->ld1) * 4, h * 4, w1,
                                     cudaMemcpyHostToDevice, ctx->stream));
  HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(ctx->stage[1], ld_in * 4, args->x2, static_cast<size_t>(args->ld2) * 4, h * 4, w2,
                                     cudaMemcpyHostToDevice, ctx->stream));
  HC_TRY_CUDA(ctx, hc::sm100::launch_pairwise_f32(static_cast<const float *>(ctx->stage[0]), static_cast<long long>(ld_in),
                                                  static_cast<const float *>(ctx->stage[1]), static_cast<long long>(ld_in),
                                                  static_cast<float *>(ctx->stage[2]), static_cast<long long>(ld_out),
                                                  static_cast<int>(w1), static_cast<int>(w2), static_cast<int>(h),
                                                  args->op == HC_CUDA_PAIRWISE_EUCLIDEAN, ctx->pairwise_leaves,
                                                  ctx->pairwise_leaf_count, ctx->stream));
  HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(args->out, static_cast<size_t>(args->ldo) * 4, ctx->stage[2], ld_out * 4, w2 * 4, w1,
                                     cudaMemcpyDeviceToHost, ctx->stream));
  return synchronize_locked(ctx);
}

namespace {

int check_row_sum_args(const HcCudaContext *ctx, const HcCudaRowSumArgs *args) {
  if (args == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "args must not be null");
  if (args->w < 0 || args->h < 0)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "w and h must be non-negative (got %lld, %lld)",
                (long long)args->w, (long long)args->h);
  if (args->w > 0x7fffffffLL)
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "w must be below 2^31");
  if (args->h > hc::sm100::pairwise_max_h())
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "h must be at most %d (got %lld)", hc::sm100::pairwise_max_h(),
                (long long)args->h);
  if ((args->flags & ~(HC_CUDA_ROW_SUM_SQUARE | HC_CUDA_ROW_SUM_SQRT)) != 0)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "flags has bits that are no HcCudaRowSumFlags (got %d)", args->flags);
  if (args->w == 0 || args->h == 0)
    return HC_CUDA_OK;
  if (args->x == nullptr || args->out == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "x and out must not be null");
  if (((reinterpret_cast<uintptr_t>(args->x) | reinterpret_cast<uintptr_t>(args->out)) & 3) != 0)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "x and out must be 4-byte aligned");
  if (args->ldx < args->h || args->ldx > kMaxPitch)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ldx must be at least h (%lld)", (long long)args->h);
  const size_t bytes_x = (static_cast<size_t>(args->w - 1) * args->ldx + args->h) * 4;
  if (ranges_overlap(args->out, static_cast<size_t>(args->w) * 4, args->x, bytes_x))
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "out must not overlap x");
  return HC_CUDA_OK;
}

} // namespace

int hcCudaRowSum(HcCudaContext *ctx, const HcCudaRowSumArgs *args) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (int rc = check_row_sum_args(ctx, args))
    return rc;
  if (args->w == 0 || args->h == 0)
    return HC_CUDA_OK;
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  if (int rc = ensure_pairwise_schedule(ctx, static_cast<int>(args->h)))
    return rc;
  HC_TRY_CUDA(ctx, hc::sm100::launch_row_sum_f32(args->x, args->ldx, args->out, static_cast<int>(args->w),
                                                 static_cast<int>(args->h), args->flags & HC_CUDA_ROW_SUM_SQUARE,
                                                 args->flags & HC_CUDA_ROW_SUM_SQRT, ctx->pairwise_leaves,
                                                 ctx->pairwise_leaf_count, ctx->stream));
  return HC_CUDA_OK;
}

int hcCudaRowSumHost(HcCudaContext *ctx, const HcCudaRowSumArgs *args) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (int rc = check_row_sum_args(ctx, args))
    return rc;
  if (args->w == 0 || args->h == 0)
    return HC_CUDA_OK;
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  if (int rc = ensure_pairwise_schedule(ctx, static_cast<int>(args->h)))
    return rc;
  // A compact device copy with a pitch that allows 16-byte loads.
  const size_t w = static_cast<size_t>(args->w), h = static_cast<size_t>(args->h);
  const size_t ld = static_cast<size_t>(round_up(static_cast<int64_t>(h), 4));
  if (int rc = ensure_stage(ctx, 0, w * ld * 4))
    return rc;
  if (int rc = ensure_stage(ctx, 2, w * 4))
    return rc;
  struct Drain {  // no copy may still touch the caller's arrays when the call returns
    HcCudaContext *ctx;
    ~Drain() {
      if (cudaStreamSynchronize(ctx->stream) != cudaSuccess)
        cudaGetLastError();
    }
  } drain{ctx};
  HC_TRY_CUDA(ctx, cudaMemcpy2DAsync(ctx->stage[0], ld * 4, args->x, static_cast<size_t>(args->ldx) * 4, h * 4, w,
                                     cudaMemcpyHostToDevice, ctx->stream));
  HC_TRY_CUDA(ctx, hc::sm100::launch_row_sum_f32(static_cast<const float *>(ctx->stage[0]), static_cast<long long>(ld),
                                                 static_cast<float *>(ctx->stage[2]), static_cast<int>(w),
                                                 static_cast<int>(h), args->flags & HC_CUDA_ROW_SUM_SQUARE,
                                                 args->flags & HC_CUDA_ROW_SUM_SQRT, ctx->pairwise_leaves,
                                                 ctx->pairwise_leaf_count, ctx->stream));
  HC_TRY_CUDA(ctx, cudaMemcpyAsync(args->out, ctx->stage[2], w * 4, cudaMemcpyDeviceToHost, ctx->stream));
  return synchronize_locked(ctx);
}

int hcCudaSelfTestDeviceTimeout(HcCudaContext *ctx, int64_t budget_cycles) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HC_TRY_CUDA(ctx, hc::sm100::launch_wait_selftest(budget_cycles, ctx->status_dev, ctx->stream));
  return HC_CUDA_OK;
}

int hcCudaSelfTestDeviceCheck(HcCudaContext *ctx) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (!hc::sm100::library_is_checked())
    return fail(ctx, HC_CUDA_ERR_UNSUPPORTED, "this library is not the checked build");
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HC_TRY_CUDA(ctx, hc::sm100::launch_check_selftest(ctx->status_dev, ctx->stream));
  return HC_CUDA_OK;
}

int hcCudaEventCreate(HcCudaContext *ctx, HcCudaEvent **out) {
  if (ctx == nullptr || out == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx and out must not be null");
  *out = nullptr;
  std::lock_guard<std::mutex> lock(ctx->mu);
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HcCudaEvent *ev = new (std::nothrow) HcCudaEvent();
  if (ev == nullptr)
    return fail(ctx, HC_CUDA_ERR_OUT_OF_MEMORY, "out of host memory");
  const cudaError_t err = cudaEventCreate(&ev->event);
  if (err != cudaSuccess) {
    delete ev;
    return fail_cuda(ctx, err, "cudaEventCreate");
  }
  *out = ev;
  return HC_CUDA_OK;
}

int hcCudaEventDestroy(HcCudaContext *ctx, HcCudaEvent *event) {
  if (event == nullptr)
    return HC_CUDA_OK;
  if (ctx != nullptr)
    cudaSetDevice(ctx->device);
  if (event->event != nullptr)
    cudaEventDestroy(event->event);
  delete event;
  return HC_CUDA_OK;
}

int hcCudaEventRecord(HcCudaContext *ctx, HcCudaEvent *event) {
  if (ctx == nullptr || event == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx and event must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HC_TRY_CUDA(ctx, cudaEventRecord(event->event, ctx->stream));
  return HC_CUDA_OK;
}

int hcCudaEventElapsedMs(HcCudaContext *ctx, HcCudaEvent *start, HcCudaEvent *stop, float *milliseconds) {
  if (ctx == nullptr || start == nullptr || stop == nullptr || milliseconds == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx, events and milliseconds must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HC_TRY_CUDA(ctx, cudaEventSynchronize(stop->event));
  HC_TRY_CUDA(ctx, cudaEventElapsedTime(milliseconds, start->event, stop->event));
  return HC_CUDA_OK;
}

int hcCudaCommGetUniqueId(void *id, size_t id_bytes) {
  static_assert(sizeof(ncclUniqueId) <= HC_CUDA_COMM_ID_BYTES, "id buffer too small");
  if (id == nullptr || id_bytes < sizeof(ncclUniqueId))
    return fail(nullptr, HC_CUDA_ERR_INVALID_ARGUMENT, "id must hold at least %zu bytes",
                sizeof(ncclUniqueId));
  NcclApi &api = nccl_api();
  if (!api.ok)
    return fail(nullptr, HC_CUDA_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
  ncclUniqueId uid;
  const ncclResult_t res = api.GetUniqueId(&uid);
  if (res != ncclSuccess)
    return fail(nullptr, HC_CUDA_ERR_COMM, "ncclGetUniqueId: %s", api.GetErrorString(res));
  std::memset(id, 0, id_bytes);
  std::memcpy(id, &uid, sizeof(uid));
  return HC_CUDA_OK;
}

int hcCudaCommInitRank(HcCudaContext *ctx, const void *id, size_t id_bytes, int nranks, int rank) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (id == nullptr || id_bytes < sizeof(ncclUniqueId))
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "id must hold at least %zu bytes", sizeof(ncclUniqueId));
  if (nranks < 1 || rank < 0 || rank >= nranks)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "rank %d is not in [0, %d)", rank, nranks);
  if (ctx->comm != nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "the context already has a communicator");
  NcclApi &api = nccl_api();
  if (!api.ok)
    return fail(ctx, HC_CUDA_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  ncclUniqueId uid;
  std::memcpy(&uid, id, sizeof(uid));
  const ncclResult_t res = api.CommInitRank(&ctx->comm, nranks, uid, rank);
  if (res != ncclSuccess) {
    ctx->comm = nullptr;
    return fail(ctx, HC_CUDA_ERR_COMM, "ncclCommInitRank: %s", api.GetErrorString(res));
  }
  ctx->nranks = nranks;
  ctx->rank = rank;
  return HC_CUDA_OK;
}

int hcCudaCommAllGather(HcCudaContext *ctx, const void *send, void *recv, size_t bytes_per_rank) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (ctx->comm == nullptr)
    return fail(ctx, HC_CUDA_ERR_COMM, "no communicator: call hcCudaCommInitRank first");
  if (bytes_per_rank == 0)
    return HC_CUDA_OK;
  if (send == nullptr || recv == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "send and recv must not be null");
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  NcclApi &api = nccl_api();
  const ncclResult_t res = api.AllGather(send, recv, bytes_per_rank, ncclInt8, ctx->comm, ctx->stream);
  if (res != ncclSuccess)
    return fail(ctx, HC_CUDA_ERR_COMM, "ncclAllGather: %s", api.GetErrorString(res));
  return HC_CUDA_OK;
}

int hcCudaCommDestroy(HcCudaContext *ctx) {
  if (ctx == nullptr)
    return fail(ctx, HC_CUDA_ERR_INVALID_ARGUMENT, "ctx must not be null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (ctx->comm == nullptr)
    return HC_CUDA_OK;
  HC_TRY_CUDA(ctx, cudaSetDevice(ctx->device));
  HC_TRY_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  nccl_api().CommDestroy(ctx->comm);
  ctx->comm = nullptr;
  ctx->nranks = 0;
  ctx->rank = -1;
  return HC_CUDA_OK;
}

} // extern "C"
