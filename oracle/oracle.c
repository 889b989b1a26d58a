/*
 * oracle.c -- CPU restatement of the reference's FP32 BLAS hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA kernels are compared
 * against (tests/, the smoke check and the cpu_baseline leg of the benchmark).  Nothing
 * on the product path may call it; the library fails loudly without its CUDA kernels.
 *
 * Parity pinning: the reference ships no golden vectors or known-answer tests for this
 * path.  o_cpu_gemm is pinned bit-for-bit against the reference's own cpu_gemm compiled
 * from its sources (oracle/_ref, see oracle/Makefile) and by the committed fixtures in
 * tests/golden/.  SAXPY, SDOT and ABFT have no CPU code in the reference at all (it
 * verifies against cuBLAS on the GPU); they are restated from the kernels' arithmetic.
 *
 * Build: gcc -O2 -ffp-contract=off -fPIC -shared -pthread oracle.c -o liboracle.so -lm
 * (-ffp-contract=off keeps `a*b + c` as two roundings exactly where the reference's host
 * compiler produces two roundings; fused operations are written as fmaf explicitly).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------
 * Seeded input generator shared bit-for-bit with the device fill kernel.
 * Replaces generate_random_vector / generate_random_matrix (utils/utils.cu:28-44), which
 * draw from libc rand() and cannot be reproduced on a GPU.  The benchmark configurations ask for
 * i.i.d. uniform[-1,1] from a seed.
 * ---------------------------------------------------------------------------------- */
static inline uint64_t o_mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

float o_uniform_at(uint64_t seed, uint64_t i) {
  uint64_t h = o_mix64(o_mix64(seed) ^ (i * 0xD1342543DE82EF95ull));
  uint32_t u = (uint32_t)(h >> 40); /* 24 bits */
  return (float)u * (1.0f / 8388608.0f) - 1.0f; /* multiples of 2^-23 in [-1,1): exact */
}

void o_fill_uniform(float *dst, int64_t n, uint64_t seed) {
  for (int64_t i = 0; i < n; ++i) dst[i] = o_uniform_at(seed, (uint64_t)i);
}

/* ------------------------------------------------------------------------------------
 * cpu_gemm, utils/utils.cu:93-103: row-major square, i-j-k order, float accumulator,
 * separate multiply and add, then mat3 = alpha*temp + beta*mat3.
 * ---------------------------------------------------------------------------------- */
void o_cpu_gemm(float alpha, float beta, const float *mat1, const float *mat2, int n, float *mat3) {
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j) {
      float temp = 0;
      for (int k = 0; k < n; ++k) temp += mat1[i * n + k] * mat2[k * n + j];
      mat3[i * n + j] = alpha * temp + beta * mat3[i * n + j];
    }
}

/* ---- small thread pool helper: run fn(lo,hi,arg) over [0,n) on `threads` threads ---- */
typedef void (*o_range_fn)(int64_t lo, int64_t hi, void *arg);
typedef struct { o_range_fn fn; int64_t lo, hi; void *arg; } o_job;
static void *o_job_main(void *p) { o_job *j = (o_job *)p; j->fn(j->lo, j->hi, j->arg); return NULL; }
static void o_parallel_for(int64_t n, int threads, o_range_fn fn, void *arg) {
  if (threads < 1) threads = 1;
  if (threads > 256) threads = 256;
  if ((int64_t)threads > n) threads = (int)(n > 0 ? n : 1);
  if (threads == 1) { fn(0, n, arg); return; }
  pthread_t tid[256]; o_job jobs[256];
  int64_t chunk = (n + threads - 1) / threads;
  for (int t = 0; t < threads; ++t) {
    jobs[t].fn = fn; jobs[t].arg = arg;
    jobs[t].lo = t * chunk; jobs[t].hi = (t + 1) * chunk < n ? (t + 1) * chunk : n;
    if (jobs[t].lo > n) jobs[t].lo = n;
    pthread_create(&tid[t], NULL, o_job_main, &jobs[t]);
  }
  for (int t = 0; t < threads; ++t) pthread_join(tid[t], NULL);
}

typedef struct {
  int M, N, K; float alpha, beta;
  const float *A; int lda; const float *B; int ldb; float *C; int ldc;
  double *C64; double *absdot; int mode;
} o_gemm_args;

/* mode 0: cpu_gemm arithmetic (mul, add) generalised to MxNxK with leading dimensions.
 * mode 1: one fmaf per k in ascending k, epilogue fmaf(alpha, acc, beta*c) (alpha*acc when
 *         beta == 0, C not read) -- the exact arithmetic of the FFMA GPU path, which keeps
 *         one accumulator per output and walks k in order.
 * Rows [lo,hi). */
static void o_gemm_rows_f32(int64_t lo, int64_t hi, void *p) {
  o_gemm_args *a = (o_gemm_args *)p;
  float *acc = (float *)malloc(sizeof(float) * (size_t)(a->N > 0 ? a->N : 1));
  for (int64_t i = lo; i < hi; ++i) {
    for (int j = 0; j < a->N; ++j) acc[j] = 0.0f;
    /* k-outer keeps B row-contiguous; each acc[j] still sees k in ascending order. */
    for (int k = 0; k < a->K; ++k) {
      float aik = a->A[i * (int64_t)a->lda + k];
      const float *brow = a->B + (int64_t)k * a->ldb;
      if (a->mode == 0) for (int j = 0; j < a->N; ++j) acc[j] += aik * brow[j];
      else              for (int j = 0; j < a->N; ++j) acc[j] = fmaf(aik, brow[j], acc[j]);
    }
    float *crow = a->C + i * (int64_t)a->ldc;
    for (int j = 0; j < a->N; ++j) {
      if (a->mode == 0) crow[j] = a->alpha * acc[j] + a->beta * crow[j];
      else if (a->beta == 0.0f) crow[j] = a->alpha * acc[j];
      else crow[j] = fmaf(a->alpha, acc[j], a->beta * crow[j]);
    }
  }
  free(acc);
}

/* Row-major C = alpha*A*B + beta*C, float accumulate in k order (cpu_gemm arithmetic). */
void o_sgemm_f32(int M, int N, int K, float alpha, const float *A, int lda, const float *B, int ldb,
                 float beta, float *C, int ldc, int threads) {
  o_gemm_args a = {M, N, K, alpha, beta, A, lda, B, ldb, C, ldc, NULL, NULL, 0};
  o_parallel_for(M, threads, o_gemm_rows_f32, &a);
}

/* Same with fused multiply-add: bit-exact model of the GPU FFMA path. */
void o_sgemm_fma(int M, int N, int K, float alpha, const float *A, int lda, const float *B, int ldb,
                 float beta, float *C, int ldc, int threads) {
  o_gemm_args a = {M, N, K, alpha, beta, A, lda, B, ldb, C, ldc, NULL, NULL, 1};
  o_parallel_for(M, threads, o_gemm_rows_f32, &a);
}

static void o_gemm_rows_f64(int64_t lo, int64_t hi, void *p) {
  o_gemm_args *a = (o_gemm_args *)p;
  size_t n = (size_t)(a->N > 0 ? a->N : 1);
  double *acc = (double *)malloc(sizeof(double) * n), *ab = (double *)malloc(sizeof(double) * n);
  for (int64_t i = lo; i < hi; ++i) {
    for (int j = 0; j < a->N; ++j) { acc[j] = 0.0; ab[j] = 0.0; }
    for (int k = 0; k < a->K; ++k) {
      double aik = a->A[i * (int64_t)a->lda + k];
      const float *brow = a->B + (int64_t)k * a->ldb;
      for (int j = 0; j < a->N; ++j) { double pr = aik * (double)brow[j]; acc[j] += pr; ab[j] += fabs(pr); }
    }
    for (int j = 0; j < a->N; ++j) {
      double c0 = (a->beta == 0.0f) ? 0.0 : (double)a->beta * (double)a->C[i * (int64_t)a->ldc + j];
      a->C64[i * (int64_t)a->N + j] = (double)a->alpha * acc[j] + c0;
      /* denominator of the north-star metric: (|A|.|B|)_ij, plus |beta*C| so that the
       * epilogue's own rounding is measured on the same scale */
      a->absdot[i * (int64_t)a->N + j] = fabs((double)a->alpha) * ab[j] + fabs(c0);
    }
  }
  free(acc); free(ab);
}

/* Double-precision reference (dense MxN outputs, ld = N) and the denominator matrix
 * sum_k |a_ik||b_kj| of the tolerance  max|C - C_ref| / (|A|.|B|).  C (input) is only read. */
void o_sgemm_f64(int M, int N, int K, float alpha, const float *A, int lda, const float *B, int ldb,
                 float beta, const float *C, int ldc, double *C64, double *absdot, int threads) {
  o_gemm_args a = {M, N, K, alpha, beta, A, lda, B, ldb, (float *)C, ldc, C64, absdot, 2};
  o_parallel_for(M, threads, o_gemm_rows_f64, &a);
}

/* max_ij |got - ref| / absdot  (entries with absdot == 0 must match exactly, else +inf). */
double o_gemm_error(int M, int N, const float *got, int ld, const double *C64, const double *absdot) {
  double worst = 0.0;
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      double d = fabs((double)got[i * ld + j] - C64[i * N + j]);
      double den = absdot[i * N + j];
      double r = (den > 0.0) ? d / den : (d == 0.0 ? 0.0 : INFINITY);
      if (!(r <= worst)) worst = r; /* NaN propagates to the result */
    }
  return worst;
}

/* Column-major NT of kernel/ft_sgemm (oracle call kernel/ft_sgemm/sgemm.cu:111):
 * A is MxK lda=M, B is NxK ldb=N, C is MxN ldc=M; C = alpha*A*B^T + beta*C, fmaf in k order. */
void o_sgemm_colmajor_nt(int M, int N, int K, float alpha, const float *A, const float *B, float beta,
                         float *C) {
  for (int j = 0; j < N; ++j)
    for (int i = 0; i < M; ++i) {
      float acc = 0.0f;
      for (int k = 0; k < K; ++k) acc = fmaf(A[(int64_t)k * M + i], B[(int64_t)k * N + j], acc);
      float *c = &C[(int64_t)j * M + i];
      *c = (beta == 0.0f) ? alpha * acc : fmaf(alpha, acc, beta * *c);
    }
}

/* ------------------------------------------------------------------------------------
 * SAXPY: b[tid] = alpha*a[tid] + b[tid]  (kernel/saxpy/saxpy.cu:44-47), one FMA.
 * SDOT:  temp += a[tid]*b[tid]           (kernel/sdot/sdot.cu:15-19); the sum is taken in
 *        double here so that it is a reference value, not one particular summation order.
 * ---------------------------------------------------------------------------------- */
void o_saxpy(int64_t n, float alpha, const float *x, float *y) {
  for (int64_t i = 0; i < n; ++i) y[i] = fmaf(alpha, x[i], y[i]);
}

typedef struct { const float *x, *y; double *part, *apart; int64_t chunk; } o_dot_args;
static void o_dot_range(int64_t lo, int64_t hi, void *p) {
  o_dot_args *a = (o_dot_args *)p;
  for (int64_t c = lo; c < hi; ++c) {
    double s = 0.0, sa = 0.0;
    const float *x = a->x + c * a->chunk, *y = a->y + c * a->chunk;
    for (int64_t i = 0; i < a->chunk; ++i) { double pr = (double)x[i] * (double)y[i]; s += pr; sa += fabs(pr); }
    a->part[c] = s; a->apart[c] = sa;
  }
}

/* Returns sum x[i]*y[i] in double; *abs_out (optional) = sum |x[i]*y[i]|, the scale the
 * 1e-5 relative tolerance is taken against. */
double o_sdot(int64_t n, const float *x, const float *y, double *abs_out, int threads) {
  const int64_t chunk = 1 << 16;
  int64_t nfull = n / chunk;
  double s = 0.0, sa = 0.0;
  if (nfull > 0) {
    double *part = (double *)malloc(sizeof(double) * (size_t)nfull * 2);
    o_dot_args a = {x, y, part, part + nfull, chunk};
    o_parallel_for(nfull, threads, o_dot_range, &a);
    for (int64_t c = 0; c < nfull; ++c) { s += part[c]; sa += part[nfull + c]; }
    free(part);
  }
  for (int64_t i = nfull * chunk; i < n; ++i) { double pr = (double)x[i] * (double)y[i]; s += pr; sa += fabs(pr); }
  if (abs_out) *abs_out = sa;
  return s;
}

/* ------------------------------------------------------------------------------------
 * ABFT host model.  Checksum algebra of kernel/ft_sgemm/README.md:4-14 applied per
 * 128x128 output tile: for the tile T = A_t * B_t,
 *     column checksum  e^T T = (e^T A_t) B_t      row checksum  T e = A_t (B_t e),
 * encoded slab by slab in the mainloop (kernel/ft_sgemm/include/ft_sgemm_tall.cuh:178-267),
 * compared against the sums of the accumulators (ft_sgemm_huge.cuh:147-271); a tile whose
 * row r and column c both disagree by more than tau holds a fault at (r,c), which is
 * rebuilt from the row checksum (the reference subtracts the residual and leaves the
 * location unfinished, ft_sgemm_huge.cuh:296-371).
 *
 * o_ft_fault_effect: for one planned fault, walk the accumulator of that element exactly
 * as the FFMA path does (fmaf, ascending k), flip `bit` after slab k_step (slab = 32 of
 * K), finish, and return the clean and faulty final accumulators.
 * ---------------------------------------------------------------------------------- */
typedef struct { int32_t tile_m, tile_n, row, col, k_step, bit; } o_fault;

void o_ft_fault_effect(int M, int N, int K, const float *A, int lda, const float *B, int ldb,
                       const o_fault *f, float *clean_out, float *faulty_out, int *in_range) {
  int64_t i = (int64_t)f->tile_m * 128 + f->row, j = (int64_t)f->tile_n * 128 + f->col;
  *in_range = (i < M && j < N && f->row >= 0 && f->col >= 0 && f->row < 128 && f->col < 128 && K > 0);
  *clean_out = 0.0f; *faulty_out = 0.0f;
  if (!*in_range) return;
  int nslab = (K + 31) / 32;
  int ks = f->k_step < 0 ? 0 : (f->k_step >= nslab ? nslab - 1 : f->k_step);
  int kflip = (ks + 1) * 32 < K ? (ks + 1) * 32 : K; /* flip after this many k */
  float acc = 0.0f, bad = 0.0f;
  for (int k = 0; k < K; ++k) {
    float a = A[i * lda + k], b = B[(int64_t)k * ldb + j];
    acc = fmaf(a, b, acc);
    bad = fmaf(a, b, bad);
    if (k + 1 == kflip) {
      uint32_t u; memcpy(&u, &bad, 4); u ^= (1u << (f->bit & 31)); memcpy(&bad, &u, 4);
    }
  }
  *clean_out = acc; *faulty_out = bad;
}

/* Row / column checksums of one 128x128 tile the way the encoder forms them, in double
 * (reference values for the tests of the checksum algebra). rowchk[128], colchk[128]. */
void o_abft_tile_checksums(int M, int N, int K, const float *A, int lda, const float *B, int ldb,
                           int tile_m, int tile_n, double *rowchk, double *colchk) {
  int m0 = tile_m * 128, n0 = tile_n * 128;
  int mh = M - m0 < 128 ? M - m0 : 128, nh = N - n0 < 128 ? N - n0 : 128;
  for (int r = 0; r < 128; ++r) rowchk[r] = 0.0;
  for (int c = 0; c < 128; ++c) colchk[c] = 0.0;
  for (int k = 0; k < K; ++k) {
    double br = 0.0, ac = 0.0;
    for (int c = 0; c < nh; ++c) br += B[(int64_t)k * ldb + n0 + c];
    for (int r = 0; r < mh; ++r) ac += A[(int64_t)(m0 + r) * lda + k];
    for (int r = 0; r < mh; ++r) rowchk[r] += (double)A[(int64_t)(m0 + r) * lda + k] * br;
    for (int c = 0; c < nh; ++c) colchk[c] += ac * (double)B[(int64_t)k * ldb + n0 + c];
  }
}

/* verify_matrix, utils/utils.cu:75-91: absolute tolerance 1e-2, first failure wins. */
int o_verify_matrix(const float *mat1, const float *mat2, int n) {
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j) {
      double diff = fabs((double)mat1[i * n + j] - (double)mat2[i * n + j]);
      if (diff > 1e-2) return 0;
    }
  return 1;
}

/* verify_vector, utils/utils.cu:60-73: relative 5e-3 against the SIGNED reference value
 * (so any negative reference passes -- kept as in the reference). */
int o_verify_vector(const float *vec1, const float *vec2, int n) {
  for (int i = 0; i < n; ++i) {
    double diff = fabs((double)vec1[i] - (double)vec2[i]);
    if (diff / (double)vec1[i] > 5e-3) return 0;
  }
  return 1;
}
