/*
 * native_oracle.c — CPU restatement of the Sarek *Native* backend's arithmetic
 * for the dense-GEMM and element-wise map kernels.
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It is the checker the CUDA path is
 * compared against and the timed CPU baseline; it is never linked into, loaded
 * by or called from the product library.
 *
 * Parity status: the reference is OCaml and no OCaml toolchain exists on the
 * build machine, so the reference binary cannot be run.  The restatement is
 * pinned against every closed-form fixture the reference's own tests hold for
 * these kernels (tolerances 1e-3 / 1e-5, see tests/test_oracle_golden.py);
 * for the stricter bounds used by the GPU parity tests (1 ulp, 1e-5*sqrt(K),
 * 2e-3) parity is unpinned by the reference's tests and rests on the rules
 * below, each read from the reference source.
 *
 * Rules of the Native backend that every function here follows:
 *  R1  a float32 vector load widens the value exactly to double
 *      (sarek/core/Vector.ml:80-91, Bigarray float32 get);
 *  R2  every float32 + - * / in a kernel body is an OCaml double operation,
 *      float literals are doubles, mutable accumulators are double refs,
 *      shared tiles are double arrays; no intermediate float32 rounding and
 *      no fused multiply-add (sarek/ppx/Sarek_native_gen.ml:96-118,279-290,
 *      533-539,746-772; sarek/sarek/Sarek_cpu_runtime.ml:74-109);
 *  R3  a float32 vector store narrows double -> float once, round to nearest
 *      even (sarek/core/Vector.ml:139-143, Bigarray unsafe_set);
 *  R4  float32 scalar kernel arguments arrive as un-rounded doubles
 *      (sarek/ppx/Sarek_native_gen.ml:1129-1134);
 *  R5  GEMM sums k ascending into one accumulator per output element, in the
 *      naive kernel and in the tiled one alike
 *      (benchmarks/bench_matrix_mul.ml:55-73,
 *       benchmarks/bench_matrix_mul_tiled.ml:55-94).
 *
 * Build with -ffp-contract=off so the compiler never fuses a*b+c.
 */
#include <math.h>
#include <pthread.h>
#include <stdatomic.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define SO_EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* Seeded synthetic inputs: one counter-based generator shared (as an        */
/* algorithm) by the oracle, the numpy test helpers and the CUDA fill kernel */
/* ------------------------------------------------------------------------ */

static inline uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

static inline uint64_t so_u64(uint64_t seed, uint64_t stream, uint64_t i) {
  return splitmix64(seed ^ (stream * 0x9E3779B97F4A7C15ull) ^ i);
}

/* uniform on the 24-bit grid of [-1,1): exactly representable in float32 */
static inline float so_unit(uint64_t seed, uint64_t stream, uint64_t i) {
  uint64_t u = so_u64(seed, stream, i) >> 40; /* 24 bits */
  return (float)((double)u * (1.0 / 8388608.0) - 1.0);
}

/* kind 0: U[-1,1); kind 1: U[-0.1,0.1) = fl32(unit * 0.1f);
 * kind 2: N(0, sigma) by Box-Muller in double on two 24-bit uniforms of
 * (0,1], rounded once to float32. */
SO_EXPORT void so_fill(float *dst, int64_t n, uint64_t seed, uint64_t stream,
                       int kind, double sigma, int64_t first) {
  for (int64_t j = 0; j < n; ++j) {
    uint64_t i = (uint64_t)(first + j);
    if (kind == 0) {
      dst[j] = so_unit(seed, stream, i);
    } else if (kind == 1) {
      dst[j] = so_unit(seed, stream, i) * 0.1f;
    } else {
      uint64_t r = so_u64(seed, stream, i);
      double u1 = ((double)((r >> 40) + 1)) * (1.0 / 16777216.0);
      double u2 = ((double)((r >> 16) & 0xFFFFFF)) * (1.0 / 16777216.0);
      double z = sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2);
      dst[j] = (float)(z * sigma);
    }
  }
}

/* ------------------------------------------------------------------------ */
/* Element-wise kernels                                                      */
/* ------------------------------------------------------------------------ */

/* vector_add: if tid < n then c.(tid) <- a.(tid) +. b.(tid)
 * (benchmarks/bench_vector_add.ml:47-55; sarek/tests/e2e/test_vector_add.ml:21-29) */
static inline void k_vector_add(const float *a, const float *b, float *c,
                                int64_t i) {
  c[i] = (float)((double)a[i] + (double)b[i]);
}

/* stream_triad: if tid < n then a.(tid) <- b.(tid) +. (c.(tid) *. scalar)
 * (benchmarks/bench_stream_triad.ml:22-31); scalar is a double (R4). */
static inline void k_triad(float *a, const float *b, const float *c,
                           double scalar, int64_t i) {
  a[i] = (float)((double)b[i] + ((double)c[i] * scalar));
}

/* second kernel of the a = b + 3c ; d = a*a + b chain: d.(i) <- a.(i)*.a.(i)+.b.(i) */
static inline void k_sq_add(float *d, const float *a, const float *b,
                            int64_t i) {
  double av = (double)a[i];
  d[i] = (float)((av * av) + (double)b[i]);
}

SO_EXPORT void so_vector_add(const float *a, const float *b, float *c,
                             int64_t n) {
  for (int64_t i = 0; i < n; ++i) k_vector_add(a, b, c, i);
}

SO_EXPORT void so_stream_triad(float *a, const float *b, const float *c,
                               double scalar, int64_t n) {
  for (int64_t i = 0; i < n; ++i) k_triad(a, b, c, scalar, i);
}

/* The two-kernel chain as Native runs it: a fused kernel carries no native
 * function (sarek/sarek/Sarek_fusion.ml:546) so Native executes the unfused
 * kernels one after the other, storing (and rounding) the intermediate `a`.
 * `a_tmp` may be NULL, in which case the rounded intermediate is kept in a
 * register-sized temporary; the result in d is the same either way. */
SO_EXPORT void so_chain_triad_square(float *d, float *a_tmp, const float *b,
                                     const float *c, double scalar, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    float a = (float)((double)b[i] + ((double)c[i] * scalar));
    if (a_tmp) a_tmp[i] = a;
    double av = (double)a;
    d[i] = (float)((av * av) + (double)b[i]);
  }
}

/* ------------------------------------------------------------------------ */
/* GEMM                                                                      */
/* ------------------------------------------------------------------------ */

/* Epilogue descriptor: out = act(alpha*sum + beta*cin[row*n+col] + bias[col]),
 * all in double, one rounding at the store.  alpha=1, beta=0, no bias, act=0
 * is the plain matrix_mul store `c.(row*n+col) <- sum`. */
typedef struct {
  double alpha, beta;
  const float *cin;  /* may be NULL */
  const float *bias; /* may be NULL */
  int act;           /* 0 none, 1 relu (if x > 0.0 then x else 0.0) */
} so_epilogue;

static inline float epi_store(double sum, const so_epilogue *e, int64_t row,
                              int64_t col, int64_t n) {
  if (!e) return (float)sum;
  double x = e->alpha * sum;
  if (e->cin) x = x + e->beta * (double)e->cin[row * n + col];
  if (e->bias) x = x + (double)e->bias[col];
  if (e->act == 1) x = (x > 0.0) ? x : 0.0;
  return (float)x;
}

/* One output element exactly as the naive kernel's thread computes it
 * (benchmarks/bench_matrix_mul.ml:55-73). */
static inline double dot_naive(const float *a, const float *b, int64_t row,
                               int64_t col, int64_t n, int64_t k) {
  double sum = 0.0;
  for (int64_t i = 0; i < k; ++i)
    sum = sum + ((double)a[row * k + i] * (double)b[i * n + col]);
  return sum;
}

/* Rows [r0, r1) of C = epi(A*B).  The loop nest is k-outer / column-inner so
 * B is read along its rows; every output element still receives its products
 * in ascending k into a single double accumulator, so the values equal the
 * thread-per-element form bit for bit (R5).  `out` holds (r1-r0) x n. */
SO_EXPORT void so_matmul_rows(const float *a, const float *b, float *out,
                              int64_t m, int64_t n, int64_t k, int64_t r0,
                              int64_t r1, double alpha, double beta,
                              const float *cin, const float *bias, int act) {
  (void)m;
  so_epilogue e = {alpha, beta, cin, bias, act};
  double *acc = (double *)malloc(sizeof(double) * (size_t)(n > 0 ? n : 1));
  for (int64_t row = r0; row < r1; ++row) {
    for (int64_t j = 0; j < n; ++j) acc[j] = 0.0;
    for (int64_t i = 0; i < k; ++i) {
      double av = (double)a[row * k + i];
      const float *brow = b + i * n;
      for (int64_t j = 0; j < n; ++j) acc[j] = acc[j] + (av * (double)brow[j]);
    }
    for (int64_t j = 0; j < n; ++j)
      out[(row - r0) * n + j] = epi_store(acc[j], &e, row, j, n);
  }
  free(acc);
}

/* Selected single elements (row[i], col[i]) of epi(A*B). */
SO_EXPORT void so_matmul_points(const float *a, const float *b, float *out,
                                int64_t n, int64_t k, const int64_t *rows,
                                const int64_t *cols, int64_t count,
                                double alpha, double beta, const float *cin,
                                const float *bias, int act) {
  so_epilogue e = {alpha, beta, cin, bias, act};
  for (int64_t t = 0; t < count; ++t)
    out[t] = epi_store(dot_naive(a, b, rows[t], cols[t], n, k), &e, rows[t],
                       cols[t], n);
}

/* Selected whole columns of epi(A*B): out is m x ncols (row-major). */
SO_EXPORT void so_matmul_cols(const float *a, const float *b, float *out,
                              int64_t m, int64_t n, int64_t k,
                              const int64_t *cols, int64_t ncols, double alpha,
                              double beta, const float *cin, const float *bias,
                              int act) {
  so_epilogue e = {alpha, beta, cin, bias, act};
  for (int64_t row = 0; row < m; ++row)
    for (int64_t t = 0; t < ncols; ++t)
      out[row * ncols + t] =
          epi_store(dot_naive(a, b, row, cols[t], n, k), &e, row, cols[t], n);
}

/* The tiled kernel, executed block by block the way the Native runtime's
 * barrier path does: 16x16 thread blocks, double shared tiles, zero padding
 * at the ragged edges, three supersteps per k-tile
 * (benchmarks/bench_matrix_mul_tiled.ml:55-94;
 *  sarek/sarek/Sarek_cpu_runtime.ml:686-782,918-1002).
 * Blocks [blk0, blk1) of the row-major grid (gx = ceil(n/16), gy = ceil(m/16)). */
#define TS 16
static void tiled_blocks(const float *a, const float *b, float *c, int64_t m,
                         int64_t n, int64_t k, int64_t blk0, int64_t blk1) {
  int64_t gx = (n + TS - 1) / TS;
  int64_t num_tiles = (k + TS - 1) / TS;
  double tile_a[TS * TS], tile_b[TS * TS], sum[TS * TS];
  for (int64_t blk = blk0; blk < blk1; ++blk) {
    int64_t by = blk / gx, bx = blk % gx;
    for (int i = 0; i < TS * TS; ++i) sum[i] = 0.0;
    for (int64_t t = 0; t < num_tiles; ++t) {
      for (int ty = 0; ty < TS; ++ty)
        for (int tx = 0; tx < TS; ++tx) {
          int64_t row = ty + TS * by, col = tx + TS * bx;
          int64_t a_col = t * TS + tx, b_row = t * TS + ty;
          tile_a[ty * TS + tx] =
              (row < m && a_col < k) ? (double)a[row * k + a_col] : 0.0;
          tile_b[ty * TS + tx] =
              (b_row < k && col < n) ? (double)b[b_row * n + col] : 0.0;
        }
      for (int ty = 0; ty < TS; ++ty)
        for (int tx = 0; tx < TS; ++tx) {
          double s = sum[ty * TS + tx];
          for (int i = 0; i < TS; ++i)
            s = s + (tile_a[ty * TS + i] * tile_b[i * TS + tx]);
          sum[ty * TS + tx] = s;
        }
    }
    for (int ty = 0; ty < TS; ++ty)
      for (int tx = 0; tx < TS; ++tx) {
        int64_t row = ty + TS * by, col = tx + TS * bx;
        if (row < m && col < n) c[row * n + col] = (float)sum[ty * TS + tx];
      }
  }
}

SO_EXPORT void so_matmul_tiled(const float *a, const float *b, float *c,
                               int64_t m, int64_t n, int64_t k) {
  int64_t gx = (n + TS - 1) / TS, gy = (m + TS - 1) / TS;
  tiled_blocks(a, b, c, m, n, k, 0, gx * gy);
}

/* The naive kernel over a range of global thread ids, literally:
 * row = tid / n; col = tid mod n; guarded store. */
static void naive_ids(const float *a, const float *b, float *c, int64_t m,
                      int64_t n, int64_t k, int64_t id0, int64_t id1,
                      const so_epilogue *e) {
  for (int64_t tid = id0; tid < id1; ++tid) {
    int64_t row = tid / n, col = tid % n;
    if (row < m && col < n)
      c[row * n + col] = epi_store(dot_naive(a, b, row, col, n, k), e, row, col, n);
  }
}

SO_EXPORT void so_matmul_naive(const float *a, const float *b, float *c,
                               int64_t m, int64_t n, int64_t k) {
  naive_ids(a, b, c, m, n, k, 0, m * n, NULL);
}

/* ------------------------------------------------------------------------ */
/* Timed CPU baseline: the Native runtime's work partition                   */
/* ------------------------------------------------------------------------ */
/* Barrier-free kernels: workers claim chunks of 256 global ids from a shared
 * atomic counter (sarek/sarek/Sarek_cpu_runtime.ml:1042-1174,1452-1458); the
 * reference uses recommended_domain_count()-1 workers (:1190).  Barrier
 * kernels: whole thread blocks are split across workers (:918-1002,1205-1273).
 * The caller passes the worker count it wants. */

typedef struct {
  int op; /* 0 vector_add, 1 triad, 2 sq_add, 3 naive matmul(+epilogue), 4 tiled */
  atomic_llong next;
  int64_t total, chunk, base; /* work items are base + [0, total) */
  const float *x0, *x1;
  float *y0;
  float *y1;
  double scalar;
  int64_t m, n, k;
  const so_epilogue *epi;
} par_job;

static void *par_worker(void *arg) {
  par_job *j = (par_job *)arg;
  for (;;) {
    int64_t s = atomic_fetch_add(&j->next, j->chunk);
    if (s >= j->total) break;
    int64_t e = s + j->chunk < j->total ? s + j->chunk : j->total;
    switch (j->op) {
      case 0: for (int64_t i = s; i < e; ++i) k_vector_add(j->x0, j->x1, j->y0, i); break;
      case 1: for (int64_t i = s; i < e; ++i) k_triad(j->y0, j->x0, j->x1, j->scalar, i); break;
      case 2: for (int64_t i = s; i < e; ++i) k_sq_add(j->y0, j->x0, j->x1, i); break;
      case 3: naive_ids(j->x0, j->x1, j->y0, j->m, j->n, j->k, j->base + s, j->base + e, j->epi); break;
      case 4: tiled_blocks(j->x0, j->x1, j->y0, j->m, j->n, j->k, j->base + s, j->base + e); break;
    }
  }
  return NULL;
}

static void par_run(par_job *j, int workers) {
  if (workers < 1) workers = 1;
  atomic_store(&j->next, 0);
  pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)workers);
  for (int w = 0; w < workers; ++w) pthread_create(&th[w], NULL, par_worker, j);
  for (int w = 0; w < workers; ++w) pthread_join(th[w], NULL);
  free(th);
}

SO_EXPORT void so_par_vector_add(const float *a, const float *b, float *c,
                                 int64_t n, int workers) {
  par_job j = {0};
  j.op = 0; j.total = n; j.chunk = 256; j.x0 = a; j.x1 = b; j.y0 = c;
  par_run(&j, workers);
}

SO_EXPORT void so_par_stream_triad(float *a, const float *b, const float *c,
                                   double scalar, int64_t n, int workers) {
  par_job j = {0};
  j.op = 1; j.total = n; j.chunk = 256; j.x0 = b; j.x1 = c; j.y0 = a; j.scalar = scalar;
  par_run(&j, workers);
}

/* The chain as two Native launches: a = b + scalar*c, then d = a*a + b. */
SO_EXPORT void so_par_chain_triad_square(float *d, float *a, const float *b,
                                         const float *c, double scalar,
                                         int64_t n, int workers) {
  so_par_stream_triad(a, b, c, scalar, n, workers);
  par_job j = {0};
  j.op = 2; j.total = n; j.chunk = 256; j.x0 = a; j.x1 = b; j.y0 = d;
  par_run(&j, workers);
}

/* Naive kernel on global ids [id0, id1) (a slab of rows when id0, id1 are
 * multiples of n), with optional epilogue. */
SO_EXPORT void so_par_matmul_naive(const float *a, const float *b, float *c,
                                   int64_t m, int64_t n, int64_t k, int64_t id0,
                                   int64_t id1, double alpha, double beta,
                                   const float *cin, const float *bias, int act,
                                   int use_epilogue, int workers) {
  so_epilogue e = {alpha, beta, cin, bias, act};
  par_job j = {0};
  j.op = 3; j.total = id1 - id0; j.base = id0; j.chunk = 256;
  j.x0 = a; j.x1 = b; j.y0 = c;
  j.m = m; j.n = n; j.k = k; j.epi = use_epilogue ? &e : NULL;
  par_run(&j, workers);
}

SO_EXPORT void so_par_matmul_tiled(const float *a, const float *b, float *c,
                                   int64_t m, int64_t n, int64_t k,
                                   int64_t blk0, int64_t blk1, int workers) {
  par_job j = {0};
  int64_t gx = (n + TS - 1) / TS, gy = (m + TS - 1) / TS;
  if (blk1 <= 0 || blk1 > gx * gy) blk1 = gx * gy;
  j.op = 4; j.total = blk1 - blk0; j.base = blk0; j.chunk = 1; j.x0 = a; j.x1 = b; j.y0 = c;
  j.m = m; j.n = n; j.k = k;
  par_run(&j, workers);
}

/* Shared-memory tree reduction, block by block, as the Native runtime runs the
 * reduce_sum / dot_product kernels (benchmarks/bench_reduction.ml:62-105,
 * benchmarks/bench_dot_product.ml:17-57): sdata is a double array (R2), thread
 * t loads f(gid) or 0.0, then for c = block/2 ... 1 threads t < c add
 * sdata[t + c] into sdata[t]; thread 0 stores sdata[0] rounded to float32.
 * b == NULL: plain sum of a; otherwise the dot-product map a[gid] * b[gid]. */
SO_EXPORT void so_block_tree_reduce(const float *a, const float *b, float *out,
                                    int64_t n, int64_t nblocks, int block) {
  double *sdata = (double *)malloc(sizeof(double) * (size_t)block);
  for (int64_t blk = 0; blk < nblocks; ++blk) {
    for (int t = 0; t < block; ++t) {
      int64_t gid = blk * block + t;
      if (gid < n)
        sdata[t] = b ? ((double)a[gid] * (double)b[gid]) : (double)a[gid];
      else
        sdata[t] = 0.0;
    }
    for (int c = block / 2; c >= 1; c /= 2)
      for (int t = 0; t < c; ++t) sdata[t] = sdata[t] + sdata[t + c];
    out[blk] = (float)sdata[0];
  }
  free(sdata);
}

/* float32 helpers the tests use to state tolerances in ulps */
SO_EXPORT int32_t so_ulp_distance(float x, float y) {
  int32_t ix, iy;
  memcpy(&ix, &x, 4);
  memcpy(&iy, &y, 4);
  if (ix < 0) ix = (int32_t)0x80000000 - ix;
  if (iy < 0) iy = (int32_t)0x80000000 - iy;
  int64_t d = (int64_t)ix - (int64_t)iy;
  if (d < 0) d = -d;
  return d > 0x7fffffff ? 0x7fffffff : (int32_t)d;
}
