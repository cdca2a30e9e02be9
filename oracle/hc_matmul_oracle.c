/* CPU oracle for hc's tiled WMMA matmul. TEST INFRASTRUCTURE ONLY: it is the checker that
 * the parity tests, the smoke test and the benchmark's CPU-baseline leg compare the CUDA
 * path against. Nothing in the product links, loads or calls it.
 *
 * It restates, in plain C, the arithmetic that the reference executes when its simulator
 * runs examples/amdgpu_gfx11_wmma_matmul.py:
 *
 *   - one workgroup of 32 lanes per 16x16 tile of C, groups (ceil(M/16), ceil(N/16))
 *       (kernel decorator, examples/amdgpu_gfx11_wmma_matmul.py:301-305; _tile_origin :110-111)
 *   - accumulator fragment starts at +0.0f                       (init_wmma_acc :249-256)
 *   - k-loop in steps of 16; each step loads a 16x16 window of A and of B in which
 *     everything outside the matrix reads as 0
 *       (kernel body :315-323; masked copy hc/simulator.py:1338-1357; with_inactive(0)
 *        examples/...:178-179)
 *   - per lane: rows lane/16, lane/16+2, ... (8 rows), column lane%16; for each row
 *       acc += float(A[row,k]) * float(B[k,col]) for k = 0..15 ascending, every product and
 *       every sum rounded to fp32                                (wmma_gfx11 :180-190)
 *   - the accumulator carries unchanged from one k-step to the next (:324), so the k order
 *     is simply ascending from 0 to K-1
 *   - store: each lane writes its 8 values to C[row0+s : row0+16 : 2, col], clipped to the
 *     matrix                      (store_wmma_tile :284-298; hc/simulator.py:1441-1458)
 *
 * `hc_oracle_matmul_tiled` follows that structure literally (groups, k-steps, lanes,
 * masked loads, clipped stores). `hc_oracle_matmul` computes the same values with the loops
 * interchanged for speed (row of C at a time, k ascending, independent accumulators per
 * column); both are bit-identical, which tests/ verify, and both are bit-identical to the
 * reference simulator's own output on the committed golden fixtures.
 *
 * The product of two fp16 (11-bit significand) or two bf16 (8-bit) values is exact in
 * fp32, so a fused multiply-add would give the same bits; the file is still compiled with
 * -ffp-contract=off so that the statement above does not depend on that argument.
 *
 * Inputs are passed as raw bit patterns; `dtype` 0 = IEEE fp16, 1 = bfloat16 (16-bit elements),
 * 2 = float8 e4m3fn, 3 = float8 e5m2 (8-bit elements, the ml_dtypes / OCP encodings: e4m3fn has
 * no infinities and one NaN pattern per sign, S.1111.111; e5m2 is the upper byte of an fp16).
 * The simulator widens any NumPy element type with `np.float32(value)`, which is exact for all
 * four, and products of two 8-bit floats are exact in fp32 like the 16-bit ones.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

#define HC_ORACLE_F16 0
#define HC_ORACLE_BF16 1
#define HC_ORACLE_F8E4M3FN 2
#define HC_ORACLE_F8E5M2 3

static float bits_to_float(uint32_t bits) {
  float f;
  memcpy(&f, &bits, sizeof f);
  return f;
}

static float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0)
      return bits_to_float(sign);
    /* subnormal: renormalise */
    int shift = 0;
    while ((man & 0x400u) == 0) {
      man <<= 1;
      ++shift;
    }
    man &= 0x3ffu;
    return bits_to_float(sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13));
  }
  if (exp == 31)
    return bits_to_float(sign | 0x7f800000u | (man << 13));
  return bits_to_float(sign | ((exp + 127 - 15) << 23) | (man << 13));
}

static float bf16_to_float(uint16_t h) { return bits_to_float((uint32_t)h << 16); }

static float f8e4m3fn_to_float(uint8_t v) {
  const uint32_t sign = (uint32_t)(v & 0x80u) << 24;
  const uint32_t exp = (v >> 3) & 0xfu;
  uint32_t man = v & 0x7u;
  if (exp == 15 && man == 7)
    return bits_to_float(sign | 0x7fc00000u); /* the only NaN; there is no infinity */
  if (exp == 0) {
    if (man == 0)
      return bits_to_float(sign);
    int shift = 0; /* subnormal: man * 2^-9 */
    while ((man & 0x8u) == 0) {
      man <<= 1;
      ++shift;
    }
    man &= 0x7u;
    return bits_to_float(sign | ((uint32_t)(127 - 7 - shift + 1) << 23) | (man << 20));
  }
  return bits_to_float(sign | ((exp + 127 - 7) << 23) | (man << 20));
}

/* Element `index` of a matrix of `dtype` elements, widened to fp32 (exact). */
static float to_float(const void *base, int64_t index, int dtype) {
  if (dtype == HC_ORACLE_F8E4M3FN)
    return f8e4m3fn_to_float(((const uint8_t *)base)[index]);
  if (dtype == HC_ORACLE_F8E5M2)
    return half_to_float((uint16_t)(((const uint8_t *)base)[index]) << 8);
  const uint16_t v = ((const uint16_t *)base)[index];
  return dtype == HC_ORACLE_BF16 ? bf16_to_float(v) : half_to_float(v);
}

/* Marks a library that decodes the 8-bit element types (lets the loader spot a stale build). */
int hc_oracle_supports_f8(void) { return 1; }

int hc_oracle_max_threads(void) {
  const long online = sysconf(_SC_NPROCESSORS_ONLN);
  return online < 1 ? 1 : (online > 256 ? 256 : (int)online);
}

/* Widens a rows x cols matrix of 16- or 8-bit values to fp32 (exact). */
void hc_oracle_widen(const void *src, int64_t ld, float *dst, int64_t rows, int64_t cols,
                     int dtype) {
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c)
      dst[r * cols + c] = to_float(src, r * ld + c, dtype);
}

/* Literal restatement: workgroups, k-steps, lanes. Slow; for small shapes. Returns 0. */
int hc_oracle_matmul_tiled(const void *a, int64_t lda, const void *b, int64_t ldb, float *c,
                           int64_t ldc, int64_t m, int64_t n, int64_t k, int dtype) {
  enum { T = 16, LANES = 32, FRAG = 8 };
  const int64_t groups_m = (m + T - 1) / T, groups_n = (n + T - 1) / T;
  for (int64_t g1 = 0; g1 < groups_n; ++g1) {
    for (int64_t g0 = 0; g0 < groups_m; ++g0) { /* dimension 0 fastest, hc/simulator.py:1298-1301 */
      const int64_t row0 = g0 * T, col0 = g1 * T;
      float acc[FRAG][LANES];
      for (int r = 0; r < FRAG; ++r)
        for (int lane = 0; lane < LANES; ++lane)
          acc[r][lane] = 0.0f;
      for (int64_t k0 = 0; k0 < k; k0 += T) {
        float a_tile[T][T], b_tile[T][T];
        for (int i = 0; i < T; ++i)
          for (int j = 0; j < T; ++j) {
            const int64_t ar = row0 + i, ak = k0 + j;
            a_tile[i][j] = (ar < m && ak < k) ? to_float(a, ar * lda + ak, dtype) : 0.0f;
            const int64_t bk = k0 + i, bc = col0 + j;
            b_tile[i][j] = (bk < k && bc < n) ? to_float(b, bk * ldb + bc, dtype) : 0.0f;
          }
        for (int lane = 0; lane < LANES; ++lane) {
          const int col = lane % T;
          for (int index = 0; index < FRAG; ++index) {
            const int row = lane / 16 + 2 * index;
            float accum = acc[index][lane];
            for (int kk = 0; kk < T; ++kk) {
              const float prod = a_tile[row][kk] * b_tile[kk][col];
              accum = accum + prod;
            }
            acc[index][lane] = accum;
          }
        }
      }
      for (int lane = 0; lane < LANES; ++lane) {
        const int64_t col = col0 + lane % T;
        for (int index = 0; index < FRAG; ++index) {
          const int64_t row = row0 + lane / 16 + 2 * index;
          if (row < m && col < n)
            c[row * ldc + col] = acc[index][lane];
        }
      }
    }
  }
  return 0;
}

/* Work shared by the threads of hc_oracle_matmul_rows: rows are handed out one at a time
 * through an atomic cursor; which thread computes a row does not affect its value. */
typedef struct {
  const void *a;
  const void *b;
  float *bf;
  float *c;
  int64_t lda, ldb, ldc, n, k, row_end;
  int dtype;
  int64_t next_widen_row;
  int64_t next_row;
  /* Family members beyond the reference example (all zero for the example itself): */
  int accumulate;          /* accumulators start from C instead of +0.0f */
  int op_count;            /* element-wise statements between the k-loop and the store */
  const int *op_kind;      /* 1: v*x  2: v+x  3: max(v,x)  4: min(v,x)  5: v+bias[col] */
  const float *op_value;
  const float *bias;
} RowsJob;

static void *widen_worker(void *arg) {
  RowsJob *job = (RowsJob *)arg;
  for (;;) {
    const int64_t r = __atomic_fetch_add(&job->next_widen_row, 1, __ATOMIC_RELAXED);
    if (r >= job->k)
      return NULL;
    for (int64_t j = 0; j < job->n; ++j)
      job->bf[r * job->n + j] = to_float(job->b, r * job->ldb + j, job->dtype);
  }
}

static void *rows_worker(void *arg) {
  RowsJob *job = (RowsJob *)arg;
  const int64_t n = job->n;
  for (;;) {
    const int64_t r = __atomic_fetch_add(&job->next_row, 1, __ATOMIC_RELAXED);
    if (r >= job->row_end)
      return NULL;
    float *out = job->c + r * job->ldc;
    if (!job->accumulate)
      for (int64_t j = 0; j < n; ++j)
        out[j] = 0.0f;
    for (int64_t kk = 0; kk < job->k; ++kk) {
      const float av = to_float(job->a, r * job->lda + kk, job->dtype);
      const float *brow = job->bf + kk * n;
      for (int64_t j = 0; j < n; ++j) {
        const float prod = av * brow[j];
        out[j] = out[j] + prod;
      }
    }
    for (int i = 0; i < job->op_count; ++i) {
      const int kind = job->op_kind[i];
      const float x = job->op_value[i];
      for (int64_t j = 0; j < n; ++j) {
        const float v = out[j];
        out[j] = kind == 1 ? v * x
               : kind == 2 ? v + x
               : kind == 3 ? ((v > x || v != v) ? v : x) /* np.maximum: a NaN stays a NaN */
               : kind == 4 ? ((v < x || v != v) ? v : x) /* np.minimum likewise */
                           : v + job->bias[j];
      }
    }
  }
}

static void run_threads(void *(*fn)(void *), RowsJob *job, int threads) {
  pthread_t ids[256];
  int started = 0;
  for (int t = 1; t < threads && t < 256; ++t)
    if (pthread_create(&ids[started], NULL, fn, job) == 0)
      ++started;
  fn(job);
  for (int t = 0; t < started; ++t)
    pthread_join(ids[t], NULL);
}

/* Same values, loops interchanged: a row of C at a time, k ascending, one independent
 * accumulator per column. Rows [row_begin, row_end) of C are computed, so callers can time
 * or check a bounded sample of a large problem. `threads` <= 0 means one per online CPU.
 * Returns 0, or -1 if memory for the widened copy of B could not be obtained. */
static int matmul_rows_job(const void *a, int64_t lda, const void *b, int64_t ldb, float *c,
                           int64_t ldc, int64_t m, int64_t n, int64_t k, int dtype,
                           int64_t row_begin, int64_t row_end, int threads, const RowsJob *extra) {
  if (row_begin < 0)
    row_begin = 0;
  if (row_end > m)
    row_end = m;
  if (row_begin >= row_end || n <= 0)
    return 0;
  if (threads <= 0)
    threads = hc_oracle_max_threads();
  RowsJob job;
  memset(&job, 0, sizeof job);
  if (extra != NULL)
    job = *extra;
  job.a = a;
  job.b = b;
  job.c = c;
  job.lda = lda;
  job.ldb = ldb;
  job.ldc = ldc;
  job.n = n;
  job.k = k;
  job.row_end = row_end;
  job.dtype = dtype;
  job.next_row = row_begin;
  if (k > 0) {
    job.bf = (float *)malloc((size_t)k * (size_t)n * sizeof(float));
    if (job.bf == NULL)
      return -1;
    run_threads(widen_worker, &job, threads);
  }
  run_threads(rows_worker, &job, threads);
  free(job.bf);
  return 0;
}

int hc_oracle_matmul_rows(const void *a, int64_t lda, const void *b, int64_t ldb, float *c,
                          int64_t ldc, int64_t m, int64_t n, int64_t k, int dtype,
                          int64_t row_begin, int64_t row_end, int threads) {
  return matmul_rows_job(a, lda, b, ldb, c, ldc, m, n, k, dtype, row_begin, row_end, threads, NULL);
}

/* The kernel family around the example, as the reference simulator executes its members:
 * with `accumulate` the accumulators are loaded from C before the k-loop (out-of-range
 * elements read as 0 and are never stored), so each sum starts from C[i,j] and then takes
 * the products k ascending; after the k-loop `op_count` element-wise fp32 statements run in
 * order on every accumulator value (kinds as in RowsJob; kind 5 adds bias[column]). */
int hc_oracle_matmul_fused(const void *a, int64_t lda, const void *b, int64_t ldb, float *c,
                           int64_t ldc, int64_t m, int64_t n, int64_t k, int dtype, int accumulate,
                           int op_count, const int *op_kind, const float *op_value, const float *bias,
                           int threads) {
  RowsJob extra;
  memset(&extra, 0, sizeof extra);
  extra.accumulate = accumulate;
  extra.op_count = op_count;
  extra.op_kind = op_kind;
  extra.op_value = op_value;
  extra.bias = bias;
  return matmul_rows_job(a, lda, b, ldb, c, ldc, m, n, k, dtype, 0, m, threads, &extra);
}

int hc_oracle_matmul(const void *a, int64_t lda, const void *b, int64_t ldb, float *c,
                     int64_t ldc, int64_t m, int64_t n, int64_t k, int dtype, int threads) {
  return hc_oracle_matmul_rows(a, lda, b, ldb, c, ldc, m, n, k, dtype, 0, m, threads);
}
