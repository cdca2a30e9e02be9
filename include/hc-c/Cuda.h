/* hc-c/Cuda.h -- C ABI of the NVIDIA sm_100a (B200) launch backend for hc's tiled matmul.
 *
 * The reference project can execute its matmul kernel
 * (examples/amdgpu_gfx11_wmma_matmul.py:301-326, `tiled_gfx11_wmma_matmul`) only through
 * the host simulator (`hc.simulator.launch`, hc/simulator.py:165-186); the compiled handle
 * refuses to run (`CompiledKernel.__call__`, hc/_compile.py:57-62). This header is the
 * launch half that is missing there: a plain-C interface (pointers and sizes, no MLIR, no
 * C++ types) that `hc.compile(..., target="nvidia-sm100a")` binds through ctypes, placed
 * beside the reference's own C API (include/hc-c/HC.h:18-30, include/hc-c/Front.h:14-22)
 * and written in the same style (extern "C", an export macro, one prefix).
 *
 * Conventions
 *   - Every function returns an `HcCudaStatus` (0 = success). No C++ exception crosses the
 *     boundary. `hcCudaContextLastError` gives the text of the last failure on a context.
 *   - Buffers are caller-owned. The library never frees or reallocates caller memory; what
 *     it allocates itself (stream, scratch, status word) belongs to the context and is
 *     released by `hcCudaContextDestroy`.
 *   - One context per device. Calls on one context are serialised by an internal mutex;
 *     different contexts may be used from different threads concurrently.
 *   - Work is ordered on the context's own stream. Functions documented as asynchronous
 *     return once the work is enqueued; `hcCudaContextSynchronize` waits for it and reports
 *     device-side failures (a bounded wait inside a kernel that ran out).
 *   - There is no CPU fallback: without a usable sm_100 device every compute entry point
 *     fails with HC_CUDA_ERR_NO_DEVICE or HC_CUDA_ERR_UNSUPPORTED.
 */
#ifndef HC_C_CUDA_H
#define HC_C_CUDA_H

#include <stddef.h>
#include <stdint.h>

#if defined(_WIN32)
#define HC_CUDA_CAPI_EXPORTED __declspec(dllexport)
#else
#define HC_CUDA_CAPI_EXPORTED __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define HC_CUDA_API_VERSION 8

typedef enum HcCudaStatus {
  HC_CUDA_OK = 0,
  HC_CUDA_ERR_INVALID_ARGUMENT = 1, /* null/misaligned/overlapping pointer, bad size or enum */
  HC_CUDA_ERR_UNSUPPORTED = 2,      /* valid request this backend cannot serve */
  HC_CUDA_ERR_CUDA = 3,             /* a CUDA runtime/driver call failed */
  HC_CUDA_ERR_NO_DEVICE = 4,        /* no such device, or not an sm_100 device */
  HC_CUDA_ERR_DEVICE_TIMEOUT = 5,   /* a bounded wait inside a kernel ran out */
  HC_CUDA_ERR_COMM = 6,             /* NCCL missing, not initialised, or a collective failed */
  HC_CUDA_ERR_OUT_OF_MEMORY = 7,
  HC_CUDA_ERR_DEVICE_CHECK = 8      /* checked build: an index check inside a kernel failed (the access
                                       was not made); the message names the check */
} HcCudaStatus;

/* Element type of A and B. Accumulation is always float32 and C is float32 unless c_dtype says
 * otherwise, as in the reference kernel's `Buffer[M, N, np.float32]`
 * (examples/amdgpu_gfx11_wmma_matmul.py:310). */
typedef enum HcCudaDType {
  HC_CUDA_F16 = 0,
  HC_CUDA_BF16 = 1,
  /* 8-bit floats in the ml_dtypes / OCP encodings (float8_e4m3fn: no infinities, NaN = S.1111.111;
   * float8_e5m2: the upper byte of an fp16), multiplied by tcgen05.mma.kind::f8f6f4 with float32
   * accumulation. Every product of two such values is exact in float32, as for the 16-bit types.
   * The tensor cores take these operands with k contiguous, so a B stored [k, n] is transposed
   * once into context scratch (one extra launch); B stored [n, k] is read where it stands. */
  HC_CUDA_F8E4M3 = 2,
  HC_CUDA_F8E5M2 = 3
} HcCudaDType;

typedef enum HcCudaGemmVariant {
  HC_CUDA_GEMM_AUTO = 0,   /* tiny for m, n <= 64 with a short k, else skinny when m <= 64 (dense tiles
                              shared among clusters when that kernel would split k), dense otherwise */
  HC_CUDA_GEMM_DENSE = 1,  /* TMA ring + tcgen05.mma, persistent; 256x256 tiles on CTA pairs
                              (cta_group::2) or 128x256 on single CTAs, chosen per shape */
  HC_CUDA_GEMM_SKINNY = 2, /* m <= 64: B streamed once; split over k (ordered reduction) only
                              when there are too few column blocks to fill the GPU */
  HC_CUDA_GEMM_TINY = 6,   /* float32 pipes, one small CTA per 16x16 tile: products and sums rounded
                              one by one with k ascending, i.e. bit-identical to the reference
                              simulator; any pitch and alignment (no repack), 16-bit operands, no push
                              targets. AUTO picks it for m, n <= 64 and k <= 128 (benchmark
                              configuration 1), where the tensor-core kernels would be all set-up */
  /* Reported by hcCudaGemmPlan only: */
  HC_CUDA_GEMM_NOOP = 3,     /* m == 0 or n == 0: nothing to write */
  HC_CUDA_GEMM_ZERO_FILL = 4,    /* k == 0: C is set to zero, no kernel */
  HC_CUDA_GEMM_ELEMENTWISE = 5   /* k == 0 with fused element-wise work: one small kernel that
                                    applies it to C (accumulate) or to zeros */
} HcCudaGemmVariant;

/* Element type of C. The products are always accumulated in float32; a 16-bit C receives the
 * float32 value (after any fused operations) rounded to nearest even, which is what the
 * reference simulator's store does for a kernel whose `c` is `Buffer[M, N, np.float16]`
 * (with or without an explicit `acc.astype(np.float16)` before the store). */
typedef enum HcCudaCType { HC_CUDA_C_F32 = 0, HC_CUDA_C_F16 = 1, HC_CUDA_C_BF16 = 2 } HcCudaCType;

/* How B is laid out in memory. */
typedef enum HcCudaBLayout {
  HC_CUDA_B_KN = 0, /* B stored [k, n] row-major, pitch ldb >= n: the reference kernel's Buffer[K, N] */
  HC_CUDA_B_NK = 1  /* B stored transposed, [n, k] row-major, pitch ldb >= k: a kernel whose b is
                       Buffer[N, K] and whose k-loop loads b[col0:col0+16, k0:k0+16] */
} HcCudaBLayout;

/* Element-wise operations fused into the store of C, applied in the order given. They mirror
 * the element-wise statements an hc kernel may apply to its accumulators between the k-loop and
 * the store (the v1 tensor operations of doc/langref.md:405-414: `*`, `+`, `-`, `maximum`,
 * `minimum` with a scalar, and the addition of a per-column vector). */
typedef enum HcCudaEpilogueOp {
  HC_CUDA_EPILOGUE_SCALE = 1,      /* v = v * value */
  HC_CUDA_EPILOGUE_ADD = 2,        /* v = v + value */
  HC_CUDA_EPILOGUE_MAX = 3,        /* v = max(v, value) */
  HC_CUDA_EPILOGUE_MIN = 4,        /* v = min(v, value) */
  HC_CUDA_EPILOGUE_BIAS_COLUMN = 5 /* v = v + bias[column]; value is ignored */
} HcCudaEpilogueOp;
#define HC_CUDA_MAX_EPILOGUE_OPS 4

/* C[m,n] = A[m,k] * B[k,n]; all three row-major with element pitches lda/ldb/ldc.
 * Mirrors the launch arguments of the reference kernel, `(a, b, c)` with
 * a: Buffer[M, K], b: Buffer[K, N], c: Buffer[M, N] (examples/...:306-311), the symbols
 * M, N, K being what `_bind_buffer` derives from the array shapes (hc/simulator.py:752-768).
 * Every in-range element of C is overwritten; nothing outside C is written; A and B are
 * read only. A, B, C aligned to their element sizes; other alignments and pitches are accepted
 * (a or b not 16-byte aligned, or a pitch lda/ldb that is not a multiple of 16 bytes, costs one
 * repack launch through context scratch memory). */
typedef struct HcCudaGemmArgs {
  int64_t m, n, k;
  int32_t dtype;   /* HcCudaDType */
  int32_t variant; /* HcCudaGemmVariant: AUTO, DENSE, SKINNY or TINY */
  const void *a;
  int64_t lda;
  const void *b;
  int64_t ldb;
  void *c;         /* float32 unless c_dtype says otherwise */
  int64_t ldc;
  int32_t b_layout;   /* HcCudaBLayout */
  int32_t accumulate; /* 0: C = A*B. 1: C = C + A*B, the kernel that loads its accumulators from
                         `c` before the k-loop instead of zeroing them; every in-range element of
                         C is then read once and written once */
  int32_t epilogue_count;                          /* 0..HC_CUDA_MAX_EPILOGUE_OPS */
  int32_t epilogue_kind[HC_CUDA_MAX_EPILOGUE_OPS]; /* HcCudaEpilogueOp, applied in order to
                                                      (C +) A*B before it is stored */
  float epilogue_value[HC_CUDA_MAX_EPILOGUE_OPS];
  int32_t c_dtype;   /* HcCudaCType; 16-bit C is not available together with accumulate or with
                        push targets (HC_CUDA_ERR_UNSUPPORTED) */
  const float *bias; /* n floats, 4-byte aligned; read by HC_CUDA_EPILOGUE_BIAS_COLUMN (at most
                        one such operation), NULL otherwise. Host memory for hcCudaGemmHost,
                        device memory elsewhere */
} HcCudaGemmArgs;

/* What a GEMM call will do; computed on the host without touching a device. */
typedef struct HcCudaGemmPlanInfo {
  int32_t variant;         /* DENSE, SKINNY, NOOP or ZERO_FILL */
  int32_t tiles_m;         /* C tiles along m (dense) or 1 (skinny) */
  int32_t tiles_n;         /* C tiles along n */
  int32_t splits;          /* k-splits: of every column block (skinny), or of the dense tiles from
                              first_split_tile on; 1 when nothing is split */
  int32_t grid;            /* CTAs of the GEMM kernel */
  int32_t repack_a;        /* 1: A is first copied to a 128-byte-aligned pitch */
  int32_t repack_b;        /* 1: B likewise */
  int32_t kernel_launches; /* kernels this call enqueues (the GEMM, plus one repack if needed) */
  int64_t scratch_bytes;   /* context scratch the call needs */
  int32_t first_split_tile; /* dense with splits > 1: tiles before this one are computed whole (the
                               full rounds of the persistent CTAs); 0 when every tile is split */
  int32_t ring_stages;      /* skinny: stages of the CTA's shared-memory ring for this grid on
                               `sm_count` SMs -- the deep ring (all of an SM's shared memory) when
                               no two CTAs share an SM, else the shallow one; 0 for other variants */
  int32_t cluster_size;     /* dense, few tiles and a long k: CTAs per thread-block cluster that share
                               one 128x256 tile (each a range of k, `splits` == cluster_size, partial
                               tiles added through distributed shared memory); 0 otherwise */
  int32_t tile_n;           /* dense: columns of a tile of C -- 256, or 128 for small products whose
                               256-wide tiles would leave most SMs idle (single CTAs, never split
                               over k); 0 for other variants */
} HcCudaGemmPlanInfo;

typedef struct HcCudaDeviceInfo {
  char name[128];
  int32_t device;
  int32_t cc_major, cc_minor;
  int32_t sm_count;
  int64_t total_memory_bytes;
  int32_t l2_bytes;
  int32_t sm_clock_khz; /* nominal max SM clock */
} HcCudaDeviceInfo;

typedef struct HcCudaContext HcCudaContext;
typedef struct HcCudaEvent HcCudaEvent;

/* ---- library ------------------------------------------------------------------------ */

/* Bit 0: the library is the checked build (libhc_cuda_checked.so, compiled with -DHC_CUDA_CHECKED):
 * its GEMM kernels verify tile coordinates, k-block ranges, ring stages, TMA coordinates,
 * tensor-memory columns, output ranges and partial-tile slots before using them, and a failure is
 * reported as HC_CUDA_ERR_DEVICE_CHECK at the next synchronise instead of becoming a wild access. */
HC_CUDA_CAPI_EXPORTED int hcCudaBuildFlags(void);

/* Returns HC_CUDA_API_VERSION of the built library. */
HC_CUDA_CAPI_EXPORTED int hcCudaApiVersion(void);

/* Static, never-null name of a status code. */
HC_CUDA_CAPI_EXPORTED const char *hcCudaStatusString(int status);

/* Number of CUDA devices visible; 0 with HC_CUDA_OK when there is no driver or device. */
HC_CUDA_CAPI_EXPORTED int hcCudaGetDeviceCount(int *count);

/* ---- context ------------------------------------------------------------------------ */

/* Creates the context of `device` (stream, status word, scratch bookkeeping). Fails with
 * HC_CUDA_ERR_NO_DEVICE when the device does not exist or is not compute capability 10.x.
 * Replaces the process-wide, idempotent registration entry point of the reference C API
 * (`mlirRegisterHCAllPasses`, lib/CAPI/HC.cpp:22-29) as the library's set-up call. */
HC_CUDA_CAPI_EXPORTED int hcCudaContextCreate(int device, HcCudaContext **out);
HC_CUDA_CAPI_EXPORTED int hcCudaContextDestroy(HcCudaContext *ctx);

/* Text of the most recent failure on `ctx` ("" if none). Owned by the context; valid until
 * the next failing call on it. `ctx == NULL` reports failures of calls that take no context
 * (or a null one), per thread. */
HC_CUDA_CAPI_EXPORTED const char *hcCudaContextLastError(const HcCudaContext *ctx);

HC_CUDA_CAPI_EXPORTED int hcCudaContextGetDeviceInfo(HcCudaContext *ctx, HcCudaDeviceInfo *out);

/* Waits for all work enqueued on the context. Returns HC_CUDA_ERR_DEVICE_TIMEOUT if a
 * kernel reported that one of its waits ran out (the results of that launch are invalid;
 * the context stays usable). The reference launch is synchronous
 * (hc/simulator.py:165-186); `handle(a, b, c)` gets that behaviour by calling this. */
HC_CUDA_CAPI_EXPORTED int hcCudaContextSynchronize(HcCudaContext *ctx);

/* ---- memory ------------------------------------------------------------------------- */

HC_CUDA_CAPI_EXPORTED int hcCudaMalloc(HcCudaContext *ctx, size_t bytes, void **device_ptr);
HC_CUDA_CAPI_EXPORTED int hcCudaFree(HcCudaContext *ctx, void *device_ptr);

/* Page-locked host memory (full-speed, truly asynchronous copies). */
HC_CUDA_CAPI_EXPORTED int hcCudaHostAlloc(size_t bytes, void **host_ptr);
HC_CUDA_CAPI_EXPORTED int hcCudaHostFree(void *host_ptr);

/* Copies, ordered on the context stream; they return after the copy has completed. */
HC_CUDA_CAPI_EXPORTED int hcCudaMemcpyHtoD(HcCudaContext *ctx, void *device_dst,
                                           const void *host_src, size_t bytes);
HC_CUDA_CAPI_EXPORTED int hcCudaMemcpyDtoH(HcCudaContext *ctx, void *host_dst,
                                           const void *device_src, size_t bytes);
/* Strided forms: `rows` rows of `width_bytes`, pitches in bytes (column slabs of a
 * row-major host matrix to/from a compact device buffer). */
HC_CUDA_CAPI_EXPORTED int hcCudaMemcpy2DHtoD(HcCudaContext *ctx, void *device_dst,
                                             size_t dst_pitch, const void *host_src,
                                             size_t src_pitch, size_t width_bytes, size_t rows);
HC_CUDA_CAPI_EXPORTED int hcCudaMemcpy2DDtoH(HcCudaContext *ctx, void *host_dst, size_t dst_pitch,
                                             const void *device_src, size_t src_pitch,
                                             size_t width_bytes, size_t rows);
/* Asynchronous fill with a byte value. */
HC_CUDA_CAPI_EXPORTED int hcCudaMemset(HcCudaContext *ctx, void *device_ptr, int byte_value,
                                       size_t bytes);

/* ---- the hot path ------------------------------------------------------------------- */

/* Validates `args` exactly as hcCudaGemm does (pointers are checked for null, alignment
 * and overlap but never dereferenced) and reports what would be launched on a device with
 * `sm_count` SMs. Needs no device. */
HC_CUDA_CAPI_EXPORTED int hcCudaGemmPlan(const HcCudaGemmArgs *args, int sm_count,
                                         HcCudaGemmPlanInfo *out);

/* Asynchronous. a, b, c are device pointers on the context's device. This is what
 * `CompiledKernel.__call__` (hc/_compile.py:57-62) resolves to for device buffers. */
HC_CUDA_CAPI_EXPORTED int hcCudaGemm(HcCudaContext *ctx, const HcCudaGemmArgs *args);

/* Synchronous. a, b, c are host pointers (NumPy buffers): copies A and B to the device,
 * runs the GEMM, copies C back into the caller's array, returns when C is complete --
 * the in-place, synchronous behaviour of `hc.simulator.launch` (hc/simulator.py:165-186,
 * doc/simulator.md:201-207). Device staging memory is kept by the context between calls.
 * Large dense problems are pipelined in row panels so that the copy of C back overlaps the
 * copy of A in and the compute. Page-locked host buffers (hcCudaHostAlloc) make the copies
 * asynchronous and about twice as fast. */
HC_CUDA_CAPI_EXPORTED int hcCudaGemmHost(HcCudaContext *ctx, const HcCudaGemmArgs *args);

/* Synchronous. hcCudaGemmHost for a caller whose A already lives on the device: `a` is a device
 * pointer (16-byte aligned, lda a multiple of 8 elements), b and c are host pointers. B travels
 * in column panels, each panel's columns of C are multiplied as it arrives and leave while the
 * next panel arrives. This is the per-rank call of the N-sharded product from host arrays: every
 * rank uploads only its share of A's rows, the ranks exchange the shares over NVLink
 * (hcCudaCommAllGather), and each multiplies the gathered A with its own column slab of B.
 * float16 / bfloat16 operands, k > 0, no accumulate. No counterpart in the reference (its only
 * launch is the single-process hc.simulator.launch, hc/simulator.py:165-186). */
HC_CUDA_CAPI_EXPORTED int hcCudaGemmHostDeviceA(HcCudaContext *ctx, const HcCudaGemmArgs *args);

/* ---- the masked element-wise map ---------------------------------------------------------- */

/* Operations of hcCudaMap, applied in order to every element: with a float32 constant, or with the
 * element of the second input at the same index. They are the element-wise tensor operations of
 * doc/langref.md:405-414 that a one-dimensional load / compute / store kernel spells out. */
typedef enum HcCudaMapOp {
  HC_CUDA_MAP_SCALE = 1,             /* v = v * value */
  HC_CUDA_MAP_ADD = 2,               /* v = v + value */
  HC_CUDA_MAP_MAX = 3,               /* v = maximum(v, value) as NumPy computes it: a NaN operand gives NaN, and
                                        when neither operand is greater the second one is returned */
  HC_CUDA_MAP_MIN = 4,               /* v = minimum(v, value) */
  HC_CUDA_MAP_REVERSE_SUB = 5,       /* v = value - v */
  HC_CUDA_MAP_ADD_OTHER = 6,         /* v = v + y[i] */
  HC_CUDA_MAP_SUB_OTHER = 7,         /* v = v - y[i] */
  HC_CUDA_MAP_REVERSE_SUB_OTHER = 8, /* v = y[i] - v */
  HC_CUDA_MAP_MUL_OTHER = 9,         /* v = v * y[i] */
  HC_CUDA_MAP_MAX_OTHER = 10,        /* v = maximum(v, y[i]) */
  HC_CUDA_MAP_MIN_OTHER = 11,        /* v = minimum(v, y[i]) */
  /* maximum / minimum with the operands the other way round: NumPy returns the second operand when
   * neither is greater (two zeros of opposite sign), so the order is observable. */
  HC_CUDA_MAP_REVERSE_MAX = 12,      /* v = maximum(value, v) */
  HC_CUDA_MAP_REVERSE_MIN = 13,      /* v = minimum(value, v) */
  HC_CUDA_MAP_REVERSE_MAX_OTHER = 14, /* v = maximum(y[i], v) */
  HC_CUDA_MAP_REVERSE_MIN_OTHER = 15  /* v = minimum(y[i], v) */
} HcCudaMapOp;
#define HC_CUDA_MAX_MAP_OPS 8

/* out[i] = ops(x[i] [, y[i]]) for i in [0, n): the kernel class of the reference simulator's masked
 * vector test (tests/test_simulator.py:210-224) -- `vec = group.vload(x[gid:], shape=(G,))`,
 * element-wise statements, `group.store(out[gid:], vec)` with work_shape=(W,) -- whose loads and
 * stores are masked at the end of the buffers (hc/simulator.py:1338-1357, 1441-1458), so exactly
 * the first n elements are read and written. float32 buffers, 4-byte aligned; `out` may be the very
 * same buffer as x or y (in place) but must not partially overlap either. Every operation is one
 * correctly rounded float32 operation, so the result is bit-identical to NumPy's. */
typedef struct HcCudaMapArgs {
  int64_t n;
  const float *x;
  const float *y; /* second input, or NULL when no ..._OTHER operation is used */
  float *out;
  int32_t op_count; /* 0..HC_CUDA_MAX_MAP_OPS; 0 copies x to out */
  int32_t op_kind[HC_CUDA_MAX_MAP_OPS];
  float op_value[HC_CUDA_MAX_MAP_OPS];
} HcCudaMapArgs;

/* Asynchronous; x, y, out are device pointers on the context's device. What
 * `CompiledKernel.__call__` (hc/_compile.py:57-62) resolves to for a recognised element-wise
 * kernel on device buffers. */
HC_CUDA_CAPI_EXPORTED int hcCudaMap(HcCudaContext *ctx, const HcCudaMapArgs *args);

/* Synchronous; x, y, out are host pointers (NumPy buffers). The arrays travel in chunks so that
 * the copy in, the kernel and the copy out of successive chunks overlap; page-locked buffers make
 * the copies asynchronous. The in-place, synchronous behaviour of `hc.simulator.launch`
 * (hc/simulator.py:165-186). */
HC_CUDA_CAPI_EXPORTED int hcCudaMapHost(HcCudaContext *ctx, const HcCudaMapArgs *args);

/* ---- pairwise distances: the two-dimensional workgroup kernel of the simulator tests ---- */

typedef enum HcCudaPairwiseOp {
  HC_CUDA_PAIRWISE_EUCLIDEAN = 0, /* out[i, j] = sqrt(sum_h (x1[i, h] - x2[j, h])^2) */
  HC_CUDA_PAIRWISE_SQUARED = 1    /* the same without the square root */
} HcCudaPairwiseOp;

/* out[i, j] for i < w1, j < w2 from x1 (w1 x h) and x2 (w2 x h), all float32, row-major with
 * pitches ld1, ld2, ldo in elements: what the reference simulator computes for
 *
 *     gid = group.work_offset
 *     lhs = group.load(x1[gid[0]:], shape=(group.shape[0], x1.shape[1]))
 *     rhs = group.load(x2[gid[1]:], shape=(group.shape[1], x2.shape[1]))
 *     group.store(out[gid[0]:, gid[1]:], np.sqrt(((lhs[:, None, :] - rhs[None, :, :]) ** 2).sum(axis=2)))
 *
 * launched over work_shape=(w1, w2) (tests/test_simulator.py:142-167): loads and stores are masked
 * at the ends of the buffers, so exactly the w1 x w2 elements of out are written. Every operation
 * rounds once and the sum over h runs in the order of NumPy's float32 sum (hc/_sim_types.py:1100-1102),
 * so the result is bit-identical to the simulator's. h == 0 writes nothing (a reduction over no
 * active element is inactive, hc/_sim_types.py:1057-1063). h at most 2^20; out must not overlap
 * x1 or x2. */
typedef struct HcCudaPairwiseArgs {
  int64_t w1, w2, h;
  const float *x1;
  int64_t ld1;
  const float *x2;
  int64_t ld2;
  float *out;
  int64_t ldo;
  int32_t op; /* HcCudaPairwiseOp */
} HcCudaPairwiseArgs;

/* Asynchronous; x1, x2, out are device pointers on the context's device. What
 * `CompiledKernel.__call__` (hc/_compile.py:57-62) resolves to for a recognised pairwise kernel on
 * device buffers. */
HC_CUDA_CAPI_EXPORTED int hcCudaPairwise(HcCudaContext *ctx, const HcCudaPairwiseArgs *args);

/* Synchronous; x1, x2, out are host pointers (NumPy buffers): the in-place, synchronous behaviour
 * of `hc.simulator.launch` (hc/simulator.py:165-186). */
HC_CUDA_CAPI_EXPORTED int hcCudaPairwiseHost(HcCudaContext *ctx, const HcCudaPairwiseArgs *args);

/* ---- row sums: the one-dimensional workgroup kernel that reduces the rows it loads ------- */

typedef enum HcCudaRowSumFlags {
  HC_CUDA_ROW_SUM_SQUARE = 1, /* every value is multiplied by itself (one rounding) before it is added */
  HC_CUDA_ROW_SUM_SQRT = 2    /* the square root of the sum is stored */
} HcCudaRowSumFlags;

/* out[i] for i < w from x (w x h), float32, row-major with pitch ldx in elements: what the reference
 * simulator computes for
 *
 *     r0 = group.work_offset[0]
 *     rows = group.load(x[r0:], shape=(group.shape[0], x.shape[1]))
 *     group.store(out[r0:], rows.sum(axis=1))
 *
 * launched over work_shape=(w,) -- optionally `(rows * rows).sum(axis=1)` (HC_CUDA_ROW_SUM_SQUARE)
 * and `np.sqrt(...)` of the sum (HC_CUDA_ROW_SUM_SQRT). The load is masked at the end of the buffer
 * (hc/simulator.py:1338-1357) and a reduction keeps the active values only
 * (hc/_sim_types.py:1050-1102), so exactly the w elements of out are written, each the np.sum of its
 * row: float32 additions in the order of NumPy's sum of a contiguous vector, which the kernel
 * follows, so the result is bit-identical to the simulator's. h == 0 writes nothing (a reduction
 * over no active element is inactive). h at most 2^20; out must not overlap x. */
typedef struct HcCudaRowSumArgs {
  int64_t w, h;
  const float *x;
  int64_t ldx;
  float *out;
  int32_t flags; /* HcCudaRowSumFlags, or'ed */
} HcCudaRowSumArgs;

/* Asynchronous; x and out are device pointers on the context's device. What
 * `CompiledKernel.__call__` (hc/_compile.py:57-62) resolves to for a recognised row-sum kernel on
 * device buffers. */
HC_CUDA_CAPI_EXPORTED int hcCudaRowSum(HcCudaContext *ctx, const HcCudaRowSumArgs *args);

/* Synchronous; x and out are host pointers (NumPy buffers): the in-place, synchronous behaviour of
 * `hc.simulator.launch` (hc/simulator.py:165-186). */
HC_CUDA_CAPI_EXPORTED int hcCudaRowSumHost(HcCudaContext *ctx, const HcCudaRowSumArgs *args);

/* ---- the product fused with its gather (N-sharded GEMM, one process per GPU) ------------- */

#define HC_CUDA_MAX_PUSH_TARGETS 7
#define HC_CUDA_IPC_HANDLE_BYTES 64

/* Asynchronous. hcCudaGemm on device buffers (dense kernels; AUTO means DENSE here) whose
 * epilogue also stores every tile of C, at the same offsets and pitch, to `targets[0 ..
 * n_targets)`: device pointers usable from this device, normally the same window of a
 * row-major C in each peer GPU's memory, opened with hcCudaIpcOpen. The slab of C a rank
 * computes thus reaches all ranks over NVLink (plain peer stores) while later tiles are still
 * being multiplied, instead of in a separate all-gather afterwards; nothing is ever loaded from
 * a peer. c and the targets must be 16-byte aligned, ldc a multiple of 4. A rank's copy is
 * complete when every rank has synchronised its own launch (host barrier after
 * hcCudaContextSynchronize). No counterpart in the reference. */
HC_CUDA_CAPI_EXPORTED int hcCudaGemmPush(HcCudaContext *ctx, const HcCudaGemmArgs *args,
                                         float *const *targets, int n_targets);

/* Cross-process sharing of a device allocation on one node (CUDA IPC): export the handle of an
 * allocation made with hcCudaMalloc (pass its base pointer), carry the 64 bytes to another
 * process by any host channel, open it there (peer access is enabled on demand), close it
 * before the owner frees the memory. */
HC_CUDA_CAPI_EXPORTED int hcCudaIpcExport(HcCudaContext *ctx, const void *device_ptr, void *handle,
                                          size_t handle_bytes);
HC_CUDA_CAPI_EXPORTED int hcCudaIpcOpen(HcCudaContext *ctx, const void *handle, size_t handle_bytes,
                                        void **device_ptr);
HC_CUDA_CAPI_EXPORTED int hcCudaIpcClose(HcCudaContext *ctx, void *device_ptr);

/* ---- launching without allocating ---------------------------------------------------- */

/* Bytes of device memory every GPU that loads this library sets aside for the entry point
 * below (a file-scope __device__ array; held until the process exits). */
#define HC_CUDA_STATIC_SCRATCH_BYTES (256 + 16 * 1024 + 8 * 1024 * 1024)

/* The skinny GEMM (m <= 64) with all of its scratch in that static array: this call never
 * allocates or frees device memory, in contrast to hcCudaGemm, whose context grows its scratch
 * with cudaMalloc. It has no counterpart in the reference (which never touches a device); it is
 * for callers that cannot allocate at launch time -- a process whose GPU memory is already
 * reserved in full by another allocator, or a latency-critical loop that must avoid the
 * device-wide synchronisation cudaMalloc and cudaFree imply.
 *
 * Runs on the calling thread's current device and on `stream` (a cudaStream_t; NULL = the
 * default stream). a, b, c are device pointers; a and b must be 16-byte aligned with lda and ldb
 * multiples of 8 elements (no repack is possible without scratch). The split-k partial sums
 * must fit: splits * m * round_up(n, 128) * 4 <= 8 MiB and n <= 131072, otherwise
 * HC_CUDA_ERR_UNSUPPORTED. `synchronize` != 0 waits for the result and reports a device-side
 * timeout (once: the status word is cleared after it has been reported); with 0 the call returns
 * once the work is enqueued. A device-side timeout is observable ONLY through a call with
 * `synchronize` != 0: the status word lives in the shared array and every launch clears it, so
 * after an asynchronous call whose result matters, either make the last call of the batch a
 * synchronising one or check the result by other means. On failure a message is copied into
 * `error_text` (may be NULL).
 *
 * The first call on each device looks up the array's device address and the driver's tensor-map
 * encoder; make that first call outside any stream capture. All calls on a device share the one
 * array: calls whose kernels could overlap on the GPU (different streams) race and must be
 * serialised by the caller. The array keeps the previous call's contents; the call clears the
 * words that have to start at zero itself. */
HC_CUDA_CAPI_EXPORTED int hcCudaGemmSkinnyStatic(const HcCudaGemmArgs *args, void *stream,
                                                 int synchronize, char *error_text,
                                                 size_t error_text_bytes);

/* Asynchronous self-test of the bounded-wait path: enqueues a one-thread kernel that waits
 * `budget_cycles` SM cycles (clamped to [1e3, 2e8], i.e. at most about 0.1 s) on a barrier that
 * nothing signals and then gives up exactly as a GEMM kernel would. The next
 * hcCudaContextSynchronize therefore returns HC_CUDA_ERR_DEVICE_TIMEOUT, clears the status and
 * leaves the context usable. Nothing faults or hangs. No counterpart in the reference. */
HC_CUDA_CAPI_EXPORTED int hcCudaSelfTestDeviceTimeout(HcCudaContext *ctx, int64_t budget_cycles);

/* Checked build only (HC_CUDA_ERR_UNSUPPORTED otherwise): enqueues a one-thread kernel that checks
 * an index made up to be out of range, skips the access and records the failed check; the next
 * hcCudaContextSynchronize returns HC_CUDA_ERR_DEVICE_CHECK and the context stays usable. Makes
 * the checked build's reporting path observable without faulting anything. No counterpart in the
 * reference. */
HC_CUDA_CAPI_EXPORTED int hcCudaSelfTestDeviceCheck(HcCudaContext *ctx);

/* ---- timing ------------------------------------------------------------------------- */

HC_CUDA_CAPI_EXPORTED int hcCudaEventCreate(HcCudaContext *ctx, HcCudaEvent **out);
HC_CUDA_CAPI_EXPORTED int hcCudaEventDestroy(HcCudaContext *ctx, HcCudaEvent *event);
/* Records on the context stream (asynchronous). */
HC_CUDA_CAPI_EXPORTED int hcCudaEventRecord(HcCudaContext *ctx, HcCudaEvent *event);
/* Waits for `stop`, then returns the device time between the two records. */
HC_CUDA_CAPI_EXPORTED int hcCudaEventElapsedMs(HcCudaContext *ctx, HcCudaEvent *start,
                                               HcCudaEvent *stop, float *milliseconds);

/* ---- multi-GPU (one process per GPU; the N-sharded GEMM) ---------------------------- */

#define HC_CUDA_COMM_ID_BYTES 128

/* Rank 0 creates an id and hands it to the other ranks by any host channel. */
HC_CUDA_CAPI_EXPORTED int hcCudaCommGetUniqueId(void *id, size_t id_bytes);
/* Collective over all ranks: joins this context to a communicator of `nranks`. */
HC_CUDA_CAPI_EXPORTED int hcCudaCommInitRank(HcCudaContext *ctx, const void *id, size_t id_bytes,
                                             int nranks, int rank);
/* Asynchronous all-gather over NVLink: every rank contributes `bytes_per_rank` bytes from
 * `send`; `recv` (nranks * bytes_per_rank) receives them in rank order (slab-major C). */
HC_CUDA_CAPI_EXPORTED int hcCudaCommAllGather(HcCudaContext *ctx, const void *send, void *recv,
                                              size_t bytes_per_rank);
HC_CUDA_CAPI_EXPORTED int hcCudaCommDestroy(HcCudaContext *ctx);

#ifdef __cplusplus
}
#endif

#endif /* HC_C_CUDA_H */
