// ABFT (fault-tolerant) SGEMM entry points: b2_ft_sgemm on both math paths, the reference's column-major NT layout
// (kernel/ft_sgemm/include/ft_sgemm_huge.cuh:21, include_code_gen/ft_sgemm_wide.cuh:11) and the reference-shaped
// shims.  The kernels themselves are the FT instantiations of sgemm_ffma_kernel (sgemm_ffma.cu) and of the 3xTF32
// kernels (sgemm_3xtf32.cu); this file holds the threshold policy (defaults, scale-aware thresholds) and the routing.
#include <math.h>

#include "common.cuh"

namespace b2 {
int sgemm_ffma_dispatch(Context *ctx, int trans_a, int M, int N, int K, float alpha, const float *A, int lda,
                        const float *B, int ldb, float beta, float *C, int ldc, cudaStream_t s);
int sgemm_ffma_dispatch_ft(Context *ctx, int trans_a, int M, int N, int K, float alpha, const float *A, int lda,
                           const float *B, int ldb, float beta, float *C, int ldc, const FtArgs *ft, cudaStream_t s);
int sgemm_3xtf32_dispatch(Context *ctx, int M, int N, int K, float alpha, const float *A, int lda, const float *B, int ldb,
                          float beta, float *C, int ldc, const FtArgs *ft, cudaStream_t s);
void set_ft_level_knob(int level);
size_t ffma_workspace_bytes(int M, int N, int K);
size_t ft_tables_bytes(int M, int N, int K);
size_t tf32_workspace_bytes(int M, int N, int K);
void set_ffma_transpose_a_knob(int on);

// Sum of squares of a rows x cols matrix (pitch ld) added to *out: one block per row stripe.
__global__ void __launch_bounds__(256) sumsq_kernel(const float *__restrict__ X, int rows, int cols, int ld, double *out) {
  float acc = 0.f;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const float *row = X + (size_t)r * ld;
    for (int c = threadIdx.x; c < cols; c += 256) acc = __fmaf_rn(row[c], row[c], acc);
  }
  double d = (double)acc;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
  __shared__ double part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = d;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < 8; ++w) t += part[w];
    atomicAdd(out, t);
  }
}
__global__ void ft_scale_kernel(double *ss, double n1, double n2, float *scale) {
  const double r1 = sqrt(ss[0] / n1), r2 = sqrt(ss[1] / n2);
  *scale = (float)(3.0 * r1 * r2);   // uniform [-1, 1) has mean square 1/3
}

int ft_data_scale(Context *ctx, const float *X1, int rows1, int cols1, int ld1, const float *X2, int rows2, int cols2,
                  int ld2, cudaStream_t s, const float **scale_dev) {
  double *ss = (double *)((char *)ctx->fixed + kFixedFtScale);
  float *scale = (float *)(ss + 2);
  B2_CUDA(cudaMemsetAsync(ss, 0, 2 * sizeof(double), s));
  const int g1 = rows1 < 1184 ? rows1 : 1184, g2 = rows2 < 1184 ? rows2 : 1184;
  sumsq_kernel<<<g1, 256, 0, s>>>(X1, rows1, cols1, ld1, ss);
  sumsq_kernel<<<g2, 256, 0, s>>>(X2, rows2, cols2, ld2, ss + 1);
  ft_scale_kernel<<<1, 1, 0, s>>>(ss, (double)rows1 * cols1, (double)rows2 * cols2, scale);
  B2_CUDA(cudaGetLastError());
  *scale_dev = scale;
  return B2_OK;
}

// The ABFT SGEMM on a resolved context (arguments already validated).
int ft_sgemm_on(Context *ctx, int path, int M, int N, int K, float alpha, const float *A, int lda, const float *B, int ldb,
                float beta, float *C, int ldc, const b2_fault *plan_dev, int n_faults, float tau, b2_ft_report *report_dev,
                cudaStream_t s) {
  FtArgs ft;
  ft.nbands_pad = 0;
  ft.plan = plan_dev;
  ft.n_faults = n_faults;
  ft.report = report_dev ? (int *)report_dev : (int *)((char *)ctx->fixed + kFixedFtReport);
  ft.A = A;
  ft.B = B;
  ft.lda = lda;
  ft.ldb = ldb;
  ft.tau_scale = nullptr;
  if (tau < 0.f && K > 0) {
    // scale-aware default: one pass over A and B for their root mean squares
    int st = ft_data_scale(ctx, A, M, K, lda, B, K, N, ldb, s, &ft.tau_scale);
    if (st != B2_OK) return st;
  }
  if (path == B2_PATH_3XTF32) {
    ft.tau = tau > 0.f ? tau : 0.f;   // 0: the path's own default, which depends on where the checksums are formed
    return sgemm_3xtf32_dispatch(ctx, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, &ft, s);
  }
  // default threshold: 2e-6 per unit of K for operands of unit scale, about 16 sigma of the
  // rounding noise between the two ways a block's sum is formed
  ft.tau = tau > 0.f ? tau : fmaxf(2e-6f * (float)K, 4e-5f);
  return sgemm_ffma_dispatch_ft(ctx, 0, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, &ft, s);
}

// Plain or fault-tolerant SGEMM on either math path: what the host-buffer pipeline and the multi-GPU schedule call
// per panel.
int sgemm_dispatch(Context *ctx, int path, bool abft, int M, int N, int K, float alpha, const float *A, int lda, const float *B,
                   int ldb, float beta, float *C, int ldc, b2_ft_report *report_dev, cudaStream_t s) {
  if (M == 0 || N == 0) return B2_OK;
  if (abft) return ft_sgemm_on(ctx, path, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, nullptr, 0, 0.f, report_dev, s);
  if (path == B2_PATH_3XTF32) return sgemm_3xtf32_dispatch(ctx, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, nullptr, s);
  return sgemm_ffma_dispatch(ctx, 0, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, s);
}
}  // namespace b2

using namespace b2;

extern "C" {

// Reference-shaped shim for the plain column-major NT family (kernel/ft_sgemm/include_code_gen/sgemm_huge.cuh:11).
int ref_sgemm_colmajor_nt(int M, int N, int K, float *A, float *B, float *C, float alpha, float beta) {
  Context *ctx = default_context();
  B2_REQUIRE(ctx != nullptr, B2_ERR_CUDA, "ref_sgemm_colmajor_nt: no context (%s)", b2_last_error());
  return sgemm_ffma_dispatch(ctx, 1, N, M, K, alpha, B, N, A, M, beta, C, M, nullptr);
}

int b2_ft_sgemm(b2_handle h, int path, int M, int N, int K, float alpha, const float *A, int lda, const float *B, int ldb,
                float beta, float *C, int ldc, const b2_fault *plan_dev, int n_faults, float tau, b2_ft_report *report_dev,
                void *stream) {
  B2_REQUIRE(path == B2_PATH_FFMA || path == B2_PATH_3XTF32, B2_ERR_INVALID_ARG, "b2_ft_sgemm: unknown path %d", path);
  B2_REQUIRE(M >= 0 && N >= 0 && K >= 0, B2_ERR_INVALID_ARG, "b2_ft_sgemm: negative dimension (M=%d N=%d K=%d)", M, N, K);
  B2_REQUIRE(n_faults >= 0 && (n_faults == 0 || plan_dev != nullptr), B2_ERR_INVALID_ARG, "b2_ft_sgemm: bad fault plan");
  if (M == 0 || N == 0) return B2_OK;
  B2_REQUIRE(C != nullptr, B2_ERR_INVALID_ARG, "b2_ft_sgemm: C is NULL");
  B2_REQUIRE(ldc >= N, B2_ERR_INVALID_ARG, "b2_ft_sgemm: ldc = %d < N = %d", ldc, N);
  if (K > 0) {
    B2_REQUIRE(A != nullptr && B != nullptr, B2_ERR_INVALID_ARG, "b2_ft_sgemm: A or B is NULL");
    B2_REQUIRE(lda >= K, B2_ERR_INVALID_ARG, "b2_ft_sgemm: lda = %d < K = %d", lda, K);
    B2_REQUIRE(ldb >= N, B2_ERR_INVALID_ARG, "b2_ft_sgemm: ldb = %d < N = %d", ldb, N);
  }
  B2_CONTEXT(ctx, h, "b2_ft_sgemm");
  return ft_sgemm_on(ctx, path, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, plan_dev, n_faults, tau, report_dev,
                     (cudaStream_t)stream);
}

// Column-major NT form of the ABFT SGEMM (the layout of the reference's ft_sgemm_* kernels):
// A is M x K (lda = M), B is stored N x K (ldb = N), C is M x N (ldc = M), C = alpha*A*B^T + beta*C.
// Computed as the row-major product C^T = B * A^T with the transposed-A tile, so a fault planned
// at (row, col) of a 128 x 128 tile addresses C^T: row runs along N, col along M.
int b2_ft_sgemm_colmajor_nt(b2_handle h, int M, int N, int K, float alpha, const float *A, const float *B, float beta,
                            float *C, const b2_fault *plan_dev, int n_faults, float tau, b2_ft_report *report_dev,
                            void *stream) {
  B2_REQUIRE(M >= 0 && N >= 0 && K >= 0, B2_ERR_INVALID_ARG, "b2_ft_sgemm_colmajor_nt: negative dimension");
  B2_REQUIRE(n_faults >= 0 && (n_faults == 0 || plan_dev != nullptr), B2_ERR_INVALID_ARG, "b2_ft_sgemm_colmajor_nt: bad fault plan");
  if (M == 0 || N == 0) return B2_OK;
  B2_REQUIRE(C != nullptr && (K == 0 || (A != nullptr && B != nullptr)), B2_ERR_INVALID_ARG, "b2_ft_sgemm_colmajor_nt: null matrix");
  B2_CONTEXT(ctx, h, "b2_ft_sgemm_colmajor_nt");
  FtArgs ft;
  ft.nbands_pad = 0;
  ft.plan = plan_dev;
  ft.n_faults = n_faults;
  ft.tau = tau > 0.f ? tau : fmaxf(2e-6f * (float)K, 4e-5f);
  ft.tau_scale = nullptr;
  if (tau < 0.f && K > 0) {
    int st = ft_data_scale(ctx, A, K, M, M, B, K, N, N, (cudaStream_t)stream, &ft.tau_scale);
    if (st != B2_OK) return st;
  }
  ft.report = report_dev ? (int *)report_dev : (int *)((char *)ctx->fixed + kFixedFtReport);
  ft.A = B;   // left operand of C^T = B * A^T, held K x N in memory
  ft.B = A;   // right operand, held K x M in memory
  ft.lda = N;
  ft.ldb = M;
  return sgemm_ffma_dispatch_ft(ctx, 1, N, M, K, alpha, B, N, A, M, beta, C, M, &ft, (cudaStream_t)stream);
}

// Reference-shaped shim: ft_sgemm_<tile>(M, N, K, A, B, C, alpha, beta) of kernel/ft_sgemm
// (include/ft_sgemm_huge.cuh:21), default stream, no injection.
int ref_ft_sgemm_colmajor_nt(int M, int N, int K, float *A, float *B, float *C, float alpha, float beta) {
  return b2_ft_sgemm_colmajor_nt(nullptr, M, N, K, alpha, A, B, beta, C, nullptr, 0, 0.f, nullptr, nullptr);
}

// Workspace of the fault-tolerant SGEMM: the plain product's, plus on the FFMA path the two operand-checksum tables.
size_t b2_ft_sgemm_workspace_bytes(int path, int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (path == B2_PATH_3XTF32) return tf32_workspace_bytes(M, N, K);
  if (path != B2_PATH_FFMA) return 0;
  return ffma_workspace_bytes(M, N, K) + ft_tables_bytes(M, N, K);
}

int ft_sgemm(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C) {
  return b2_ft_sgemm(nullptr, B2_PATH_FFMA, M, N, K, alpha, A, K, B, N, beta, C, N, nullptr, 0, 0.f, nullptr, nullptr);
}

// ABFT encode granularity of the FFMA path: 1 block-level through shared memory (default), 2 thread-level in
// registers (128 x 128 tile only; other tiles keep the block-level encoder).
int b2_set_ft_level(int level) {
  B2_REQUIRE(level == 1 || level == 2, B2_ERR_INVALID_ARG, "b2_set_ft_level: %d is not 1 or 2", level);
  b2::set_ft_level_knob(level);
  return B2_OK;
}
// 1 (default): a row-major A is transposed into the workspace first when that pays; 0: never.
int b2_set_ffma_transpose_a(int on) {
  B2_REQUIRE(on == 0 || on == 1, B2_ERR_INVALID_ARG, "b2_set_ffma_transpose_a: %d is not 0 or 1", on);
  b2::set_ffma_transpose_a_knob(on);
  return B2_OK;
}

}  // extern "C"
