// Command-line driver in the shape of the reference's per-kernel main() programs, written against
// the C ABI only (include/b2blas.h + the CUDA runtime for allocation).
//
//   b2_driver sgemm <kernel_id 1..14> <start> <end> [threads_x]   kernel/sgemm/sgemm.cu:17-32,66-155,161-367
//   b2_driver ft_sgemm <start> <end> <gap>                        kernel/ft_sgemm/sgemm.cu:14-20,186-196
//   b2_driver saxpy                                                kernel/saxpy/saxpy.cu:57-135
//   b2_driver sdot                                                 kernel/sdot/sdot.cu:78-99,156-165
//
// Like the reference drivers it verifies one launch per size and then prints a GFLOPS row; unlike
// them it checks against the library's own naive kernel (rung 1) instead of cuBLAS, times with the
// CUDA-event timer of the harness, and turns every failure into a non-zero exit code.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "b2blas.h"

#define CK(call)                                                                          \
  do {                                                                                    \
    int st__ = (call);                                                                    \
    if (st__ < 0) {                                                                       \
      fprintf(stderr, "%s failed: %s (%s)\n", #call, b2_status_string(st__), b2_last_error()); \
      return 3;                                                                           \
    }                                                                                     \
  } while (0)
#define CU(call)                                                                 \
  do {                                                                           \
    cudaError_t e__ = (call);                                                    \
    if (e__ != cudaSuccess) {                                                    \
      fprintf(stderr, "%s failed: %s\n", #call, cudaGetErrorString(e__));        \
      return 4;                                                                  \
    }                                                                            \
  } while (0)

static int time_ms(b2_timer t, float *ms) { return b2_timer_elapsed_ms(t, ms); }

static int run_sgemm(int kernel_id, int start, int end, int threads_x) {
  const float alpha = 1.0f, beta = 0.5f;
  const size_t n2 = (size_t)end * end;
  float *dA, *dB, *dC, *dRef, *dC0;
  CU(cudaMalloc(&dA, n2 * 4)); CU(cudaMalloc(&dB, n2 * 4)); CU(cudaMalloc(&dC, n2 * 4));
  CU(cudaMalloc(&dRef, n2 * 4)); CU(cudaMalloc(&dC0, n2 * 4));
  CK(b2_fill_uniform(dA, (int64_t)n2, 1, nullptr));
  CK(b2_fill_uniform(dB, (int64_t)n2, 2, nullptr));
  CK(b2_fill_uniform(dC0, (int64_t)n2, 3, nullptr));
  b2_timer timer;
  CK(b2_timer_create(&timer));
  const int iters = 10;  // kernel/sgemm/sgemm.cu:165-174 times 10 launches
  for (int n = start; n <= end; n += 256) {
    // the same buffers are reinterpreted as an n x n matrix at every size, as in the reference (:66)
    CU(cudaMemcpy(dRef, dC0, (size_t)n * n * 4, cudaMemcpyDeviceToDevice));
    CU(cudaMemcpy(dC, dC0, (size_t)n * n * 4, cudaMemcpyDeviceToDevice));
    CK(b2_sgemm_series(1, 32, n, dA, dB, dRef, alpha, beta, nullptr));
    CK(b2_sgemm_series(kernel_id, threads_x, n, dA, dB, dC, alpha, beta, nullptr));
    float max_abs = 0.f;
    int bad = b2_verify_matrix(dRef, dC, n, n, n, 1e-2f, &max_abs, nullptr);  // verify_matrix, utils/utils.cu:75-91
    if (bad != 0) {
      printf("Failed to pass the correctness verification at n = %d (max |diff| = %g).\n", n, max_abs);
      return 5;
    }
    CK(b2_timer_start(timer, nullptr));
    for (int it = 0; it < iters; ++it) CK(b2_sgemm_series(kernel_id, threads_x, n, dA, dB, dC, alpha, beta, nullptr));
    CK(b2_timer_stop(timer, nullptr));
    float ms = 0.f;
    CK(time_ms(timer, &ms));
    printf("n = %5d  kernel %2d  %10.1f GFLOPS  (%.3f ms per launch, max |diff| vs naive %.2e)\n", n, kernel_id,
           2.0 * iters * (double)n * n * n / 1e9 / (ms / 1e3), ms / iters, max_abs);
  }
  CK(b2_check_status(nullptr, nullptr));
  b2_timer_destroy(timer);
  cudaFree(dA); cudaFree(dB); cudaFree(dC); cudaFree(dRef); cudaFree(dC0);
  return 0;
}

static int run_ft_sgemm(int start, int end, int gap) {
  const float alpha = 1.0f, beta = -1.5f;  // kernel/ft_sgemm/sgemm.cu:32-34
  const size_t n2 = (size_t)end * end;
  float *dA, *dB, *dC, *dRef, *dC0;
  b2_ft_report *drep;
  b2_fault *dplan;
  CU(cudaMalloc(&dA, n2 * 4)); CU(cudaMalloc(&dB, n2 * 4)); CU(cudaMalloc(&dC, n2 * 4));
  CU(cudaMalloc(&dRef, n2 * 4)); CU(cudaMalloc(&dC0, n2 * 4));
  CU(cudaMalloc(&drep, sizeof(b2_ft_report))); CU(cudaMalloc(&dplan, sizeof(b2_fault)));
  CK(b2_fill_uniform(dA, (int64_t)n2, 1, nullptr));
  CK(b2_fill_uniform(dB, (int64_t)n2, 2, nullptr));
  CK(b2_fill_uniform(dC0, (int64_t)n2, 3, nullptr));
  b2_timer timer;
  CK(b2_timer_create(&timer));
  const int iters = 20;  // kernel/ft_sgemm/sgemm.cu:23
  for (int n = start; n <= end; n += gap) {
    CU(cudaMemcpy(dRef, dC0, (size_t)n * n * 4, cudaMemcpyDeviceToDevice));
    CU(cudaMemcpy(dC, dC0, (size_t)n * n * 4, cudaMemcpyDeviceToDevice));
    CK(b2_sgemm(nullptr, B2_PATH_FFMA, n, n, n, alpha, dA, n, dB, n, beta, dRef, n, nullptr));
    // one planted bit flip (bit 27 of an accumulator in the last tile) must be found and repaired
    b2_fault f = {(n - 1) / 128, (n - 1) / 128, (n - 1) % 128, (n - 1) % 128, 1, 27};
    CU(cudaMemcpy(dplan, &f, sizeof f, cudaMemcpyHostToDevice));
    CU(cudaMemset(drep, 0, sizeof(b2_ft_report)));
    CK(b2_ft_sgemm(nullptr, B2_PATH_FFMA, n, n, n, alpha, dA, n, dB, n, beta, dC, n, dplan, 1, 0.f, drep, nullptr));
    b2_ft_report rep;
    CU(cudaMemcpy(&rep, drep, sizeof rep, cudaMemcpyDeviceToHost));
    float max_abs = 0.f;
    int bad = b2_verify_matrix(dRef, dC, n, n, n, 0.0f, &max_abs, nullptr);  // repaired result is bit-identical
    if (bad != 0 || rep.injected != 1 || rep.corrected != 1) {
      printf("ABFT check failed at n = %d: injected %d corrected %d max |diff| %g\n", n, rep.injected, rep.corrected, max_abs);
      return 5;
    }
    float ms_plain = 0.f, ms_ft = 0.f;
    CK(b2_timer_start(timer, nullptr));
    for (int it = 0; it < iters; ++it) CK(b2_sgemm(nullptr, B2_PATH_FFMA, n, n, n, alpha, dA, n, dB, n, beta, dC, n, nullptr));
    CK(b2_timer_stop(timer, nullptr));
    CK(time_ms(timer, &ms_plain));
    CK(b2_timer_start(timer, nullptr));
    for (int it = 0; it < iters; ++it) CK(b2_ft_sgemm(nullptr, B2_PATH_FFMA, n, n, n, alpha, dA, n, dB, n, beta, dC, n, nullptr, 0, 0.f, drep, nullptr));
    CK(b2_timer_stop(timer, nullptr));
    CK(time_ms(timer, &ms_ft));
    const double gf = 2.0 * iters * (double)n * n * n / 1e9;
    printf("n = %5d  sgemm %9.1f GFLOPS  ft_sgemm %9.1f GFLOPS  overhead %5.1f %%  (planted fault repaired)\n", n,
           gf / (ms_plain / 1e3), gf / (ms_ft / 1e3), 100.0 * (ms_ft / ms_plain - 1.0));
  }
  CK(b2_check_status(nullptr, nullptr));
  return 0;
}

static int run_vectors(bool dot) {
  const float alpha = 2.0f;
  const int iters = 100;                                 // kernel/saxpy/saxpy.cu:58
  const int64_t max_n = (int64_t)1 << 28;
  float *dx, *dy, *dres;
  CU(cudaMalloc(&dx, max_n * 4)); CU(cudaMalloc(&dy, max_n * 4)); CU(cudaMalloc(&dres, 4));
  CK(b2_fill_uniform(dx, max_n, 4, nullptr));
  b2_timer timer;
  CK(b2_timer_create(&timer));
  for (int64_t n = 1 << 20; n <= max_n; n <<= 4) {
    CK(b2_fill_const(dy, n, dot ? 1.0f : 0.0f, nullptr));
    float ms = 0.f;
    if (dot) {
      // x . 1 followed by (x+x) . 1 must double exactly
      float r1 = 0.f, r2 = 0.f;
      CK(b2_sdot(nullptr, n, dx, dy, dres, nullptr));
      CU(cudaMemcpy(&r1, dres, 4, cudaMemcpyDeviceToHost));
      CK(b2_fill_const(dy, n, 2.0f, nullptr));
      CK(b2_sdot(nullptr, n, dx, dy, dres, nullptr));
      CU(cudaMemcpy(&r2, dres, 4, cudaMemcpyDeviceToHost));
      if (r2 != 2.0f * r1) { printf("sdot linearity check failed at n = %lld: %g vs %g\n", (long long)n, r2, 2.0f * r1); return 5; }
      CK(b2_timer_start(timer, nullptr));
      for (int it = 0; it < iters; ++it) CK(b2_sdot(nullptr, n, dx, dy, dres, nullptr));
      CK(b2_timer_stop(timer, nullptr));
      CK(time_ms(timer, &ms));
      printf("sdot  n = %10lld  %8.1f GB/s  %8.1f GFLOPS\n", (long long)n, 8.0 * iters * n / 1e9 / (ms / 1e3), 2.0 * iters * n / 1e9 / (ms / 1e3));
    } else {
      // y = 0; y += 2x (exact); y += -2x  must give back exactly 0
      CK(b2_saxpy(nullptr, n, alpha, dx, dy, nullptr));
      CK(b2_saxpy(nullptr, n, -alpha, dx, dy, nullptr));
      CK(b2_sdot(nullptr, n, dy, dy, dres, nullptr));
      float r = 0.f;
      CU(cudaMemcpy(&r, dres, 4, cudaMemcpyDeviceToHost));
      if (r != 0.0f) { printf("saxpy round trip failed at n = %lld: %g\n", (long long)n, r); return 5; }
      CK(b2_timer_start(timer, nullptr));
      for (int it = 0; it < iters; ++it) CK(b2_saxpy(nullptr, n, alpha, dx, dy, nullptr));
      CK(b2_timer_stop(timer, nullptr));
      CK(time_ms(timer, &ms));
      printf("saxpy n = %10lld  %8.1f GB/s  %8.1f GFLOPS\n", (long long)n, 12.0 * iters * n / 1e9 / (ms / 1e3), 2.0 * iters * n / 1e9 / (ms / 1e3));
    }
  }
  return 0;
}

int main(int argc, char **argv) {
  if (argc < 2) {
    printf("usage: %s sgemm <kernel_id 1..14> <start> <end> [threads_x] | ft_sgemm <start> <end> <gap> | saxpy | sdot\n", argv[0]);
    return 1;
  }
  if (!strcmp(argv[1], "sgemm") && argc >= 5)
    return run_sgemm(atoi(argv[2]), atoi(argv[3]), atoi(argv[4]), argc > 5 ? atoi(argv[5]) : 32);
  if (!strcmp(argv[1], "ft_sgemm") && argc >= 5) return run_ft_sgemm(atoi(argv[2]), atoi(argv[3]), atoi(argv[4]));
  if (!strcmp(argv[1], "saxpy")) return run_vectors(false);
  if (!strcmp(argv[1], "sdot")) return run_vectors(true);
  printf("bad arguments\n");
  return 1;
}
