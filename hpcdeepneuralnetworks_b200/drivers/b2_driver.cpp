// Command-line driver in the shape of the reference's per-kernel main() programs, written against
// the C ABI only (include/b2blas.h + the CUDA runtime for allocation).
//
//   b2_driver sgemm <kernel_id 1..14> <start> <end> [threads_x]   kernel/sgemm/sgemm.cu:17-32,66-155,161-367
//   b2_driver ft_sgemm <start> <end> <gap>                        kernel/ft_sgemm/sgemm.cu:14-20,186-196
//   b2_driver saxpy                                                kernel/saxpy/saxpy.cu:57-135
//   b2_driver sdot                                                 kernel/sdot/sdot.cu:78-99,156-165
//   b2_driver small                        the small cases of the benchmark configurations timed from C++: SGEMM 256..1024
//                                          on both math paths and SAXPY/SDOT at 2^20 and 2^24, back-to-back launches on
//                                          rotating buffers (kernel/saxpy/saxpy.cu:79-80,126), so that the figures are the
//                                          kernels' and not a binding's
//   b2_driver tiles <n>                    every tile of the generated FFMA family, pinned, at n^3: the table the generator's
//                                          tile_measurements.json is filled from (code_gen/main.py:8-16 names the reference's tiles)
//   b2_driver sgemm_host <n> [path]        host arrays in, host array out (the drivers' malloc + cudaMemcpy + launch +
//                                          cudaMemcpy of kernel/sgemm/sgemm.cu:50-63 as one pipelined call)
//   b2_driver mg <rank> <world> <id file> <n> [panel_k]   one process per GPU: row-block sharded SGEMM and sharded SDOT;
//                                          rank 0 writes the communicator id to <id file>, the others wait for it
//
// Like the reference drivers it verifies one launch per size and then prints a GFLOPS row; unlike
// them it checks against the library's own naive kernel (rung 1) instead of cuBLAS, times with the
// CUDA-event timer of the harness, and turns every failure into a non-zero exit code.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <unistd.h>

#include <string>
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

static int run_sgemm_host(int n, int path) {
  const float alpha = 1.0f, beta = 0.5f;
  const size_t n2 = (size_t)n * n;
  float *hA, *hB, *hC, *hRef;
  CK(b2_host_alloc((void **)&hA, n2 * 4)); CK(b2_host_alloc((void **)&hB, n2 * 4));
  CK(b2_host_alloc((void **)&hC, n2 * 4)); CK(b2_host_alloc((void **)&hRef, n2 * 4));
  CK(b2_fill_uniform_host(hA, (int64_t)n2, 1)); CK(b2_fill_uniform_host(hB, (int64_t)n2, 2)); CK(b2_fill_uniform_host(hC, (int64_t)n2, 3));
  // the reference drivers' way: blocking copies around one launch
  float *dA, *dB, *dC;
  CU(cudaMalloc(&dA, n2 * 4)); CU(cudaMalloc(&dB, n2 * 4)); CU(cudaMalloc(&dC, n2 * 4));
  CU(cudaMemcpy(dA, hA, n2 * 4, cudaMemcpyHostToDevice)); CU(cudaMemcpy(dB, hB, n2 * 4, cudaMemcpyHostToDevice));
  CU(cudaMemcpy(dC, hC, n2 * 4, cudaMemcpyHostToDevice));
  b2_handle h;
  CK(b2_create(&h));
  CK(b2_sgemm(h, path, n, n, n, alpha, dA, n, dB, n, beta, dC, n, nullptr));
  CU(cudaMemcpy(hRef, dC, n2 * 4, cudaMemcpyDeviceToHost));
  b2_host_plan plan;
  CK(b2_host_plan_create(&plan, h, path, n, n, n, 0, 0, 0, 0));
  CK(b2_sgemm_host(plan, alpha, hA, n, hB, n, beta, hC, n, 0, nullptr));
  if (path == B2_PATH_FFMA && memcmp(hC, hRef, n2 * 4) != 0) {
    printf("sgemm_host: the pipelined result differs from the single device call at n = %d\n", n);
    return 5;
  }
  double worst = 0.0;
  for (size_t i = 0; i < n2; ++i) {
    const double d = (double)hC[i] - (double)hRef[i];
    if (d > worst) worst = d;
    if (-d > worst) worst = -d;
  }
  if (!(worst <= 1e-3 * n)) { printf("sgemm_host: result off by %g at n = %d\n", worst, n); return 5; }
  const int iters = 5;
  cudaEvent_t e0, e1;
  CU(cudaEventCreate(&e0)); CU(cudaEventCreate(&e1));
  CU(cudaEventRecord(e0, nullptr));
  for (int it = 0; it < iters; ++it) CK(b2_sgemm_host(plan, alpha, hA, n, hB, n, beta, hC, n, 0, nullptr));
  CU(cudaEventRecord(e1, nullptr));
  CU(cudaEventSynchronize(e1));
  float ms = 0.f;
  CU(cudaEventElapsedTime(&ms, e0, e1));
  printf("sgemm_host n = %5d  path %d  %9.1f GFLOPS end to end (%.3f ms per call, host copies included; max |diff| vs device call %.2e)\n",
         n, path, 2.0 * iters * (double)n * n * n / 1e9 / (ms / 1e3), ms / iters, worst);
  CK(b2_host_plan_destroy(plan));
  CK(b2_check_status(h, nullptr));
  CK(b2_destroy(h));
  return 0;
}

// Small cases through the C ABI alone: 200 back-to-back launches per figure, operands rotated through enough
// distinct buffers to exceed the 126 MB L2.
static int run_small() {
  b2_timer timer;
  CK(b2_timer_create(&timer));
  b2_handle h;
  CK(b2_create(&h));
  const int iters = 200;
  for (int n = 256; n <= 1024; n += 256) {
    const size_t n2 = (size_t)n * n;
    int sets = (int)((size_t)160 * 1024 * 1024 / (3 * n2 * 4)) + 1;
    if (sets > 64) sets = 64;
    float *buf;
    CU(cudaMalloc(&buf, (size_t)sets * 3 * n2 * 4));
    CK(b2_fill_uniform(buf, (int64_t)sets * 3 * n2, 7, nullptr));
    void *ws = nullptr;
    size_t wsb = b2_sgemm_workspace_bytes(B2_PATH_3XTF32, n, n, n);
    if (wsb < 8 * n2 * 4 + 4096) wsb = 8 * n2 * 4 + 4096;      // room for the parts of an 8-way split-K as well
    CU(cudaMalloc(&ws, wsb + 1024));
    CK(b2_set_workspace(h, (void *)(((uintptr_t)ws + 1023) & ~(uintptr_t)1023), wsb));
    for (int leg = 0; leg < 3; ++leg) {                 // FFMA, 3xTF32, FFMA with automatic split-K
      const int path = leg == 1 ? B2_PATH_3XTF32 : B2_PATH_FFMA;
      CK(b2_set_ffma_split_k(leg == 2 ? -1 : 0));
      for (int it = 0; it < 10; ++it) CK(b2_sgemm(h, path, n, n, n, 1.0f, buf, n, buf + n2, n, 0.5f, buf + 2 * n2, n, nullptr));
      CK(b2_timer_start(timer, nullptr));
      for (int it = 0; it < iters; ++it) {
        float *b = buf + (size_t)(it % sets) * 3 * n2;
        CK(b2_sgemm(h, path, n, n, n, 1.0f, b, n, b + n2, n, 0.5f, b + 2 * n2, n, nullptr));
      }
      CK(b2_timer_stop(timer, nullptr));
      float ms = 0.f;
      CK(time_ms(timer, &ms));
      printf("sgemm n = %4d  %-22s %8.2f us per call  %8.2f TFLOPS  (%d buffer sets in rotation)\n", n,
             leg == 0 ? "FFMA" : leg == 1 ? "3xTF32" : "FFMA, split-K automatic", 1e3 * ms / iters,
             2.0 * iters * (double)n * n * n / 1e12 / (ms / 1e3), sets);
    }
    CK(b2_set_ffma_split_k(0));
    CK(b2_set_workspace(h, nullptr, 0));
    CU(cudaFree(ws));
    CU(cudaFree(buf));
  }
  for (int lg = 20; lg <= 24; lg += 4) {
    const int64_t n = (int64_t)1 << lg;
    int sets = (int)(((int64_t)512 << 20) / (8 * n));
    if (sets > 64) sets = 64;
    if (sets < 1) sets = 1;
    float *x, *y, *res;
    CU(cudaMalloc(&x, (size_t)sets * n * 4)); CU(cudaMalloc(&y, (size_t)sets * n * 4)); CU(cudaMalloc(&res, 4));
    CK(b2_fill_uniform(x, sets * n, 4, nullptr));
    CK(b2_fill_uniform(y, sets * n, 5, nullptr));
    for (int which = 0; which < 2; ++which) {
      CK(b2_timer_start(timer, nullptr));
      for (int it = 0; it < iters; ++it) {
        const size_t o = (size_t)(it % sets) * n;
        if (which == 0) CK(b2_saxpy(h, n, 2.0f, x + o, y + o, nullptr));
        else CK(b2_sdot(h, n, x + o, y + o, res, nullptr));
      }
      CK(b2_timer_stop(timer, nullptr));
      float ms = 0.f;
      CK(time_ms(timer, &ms));
      printf("%s n = 2^%d  %8.2f us per call  %8.1f GB/s  (%d vector pairs in rotation)\n", which == 0 ? "saxpy" : "sdot ", lg,
             1e3 * ms / iters, (which == 0 ? 12.0 : 8.0) * iters * n / 1e9 / (ms / 1e3), sets);
    }
    CU(cudaFree(x)); CU(cudaFree(y)); CU(cudaFree(res));
  }
  CK(b2_check_status(h, nullptr));
  CK(b2_destroy(h));
  return 0;
}

// Throughput of every generated FFMA tile at one size (and of the automatic choice), back-to-back launches on rotating buffers.
static int run_tiles(int n) {
  b2_timer timer;
  CK(b2_timer_create(&timer));
  b2_handle h;
  CK(b2_create(&h));
  const size_t n2 = (size_t)n * n;
  int sets = (int)((size_t)160 * 1024 * 1024 / (3 * n2 * 4)) + 1;
  if (sets > 64) sets = 64;
  float *buf;
  CU(cudaMalloc(&buf, (size_t)sets * 3 * n2 * 4));
  CK(b2_fill_uniform(buf, (int64_t)sets * 3 * n2, 7, nullptr));
  const int iters = n <= 1024 ? 200 : (n <= 3072 ? 40 : 8);
  printf("{\"n\": %d, \"tflops\": {", n);
  for (int tile = -1; tile < b2_ffma_tile_count(); ++tile) {
    CK(b2_set_ffma_tile(tile));
    for (int it = 0; it < 3; ++it) CK(b2_sgemm(h, B2_PATH_FFMA, n, n, n, 1.0f, buf, n, buf + n2, n, 0.5f, buf + 2 * n2, n, nullptr));
    CK(b2_timer_start(timer, nullptr));
    for (int it = 0; it < iters; ++it) {
      float *b = buf + (size_t)(it % sets) * 3 * n2;
      CK(b2_sgemm(h, B2_PATH_FFMA, n, n, n, 1.0f, b, n, b + n2, n, 0.5f, b + 2 * n2, n, nullptr));
    }
    CK(b2_timer_stop(timer, nullptr));
    float ms = 0.f;
    CK(time_ms(timer, &ms));
    const char *name = "automatic";
    if (tile >= 0) CK(b2_ffma_tile_info(tile, nullptr, nullptr, nullptr, &name));
    printf("%s\"%s\": %.2f", tile >= 0 ? ", " : "", name, 2.0 * iters * (double)n * n * n / 1e12 / (ms / 1e3));
  }
  printf("}}\n");
  CK(b2_set_ffma_tile(-1));
  CK(b2_check_status(h, nullptr));
  CK(b2_destroy(h));
  CU(cudaFree(buf));
  return 0;
}

// One process per GPU.  Rank 0 draws the communicator id and publishes it through a file (written under another
// name and renamed, so that a reader never sees half of it).
static int run_mg(int rank, int world, const char *id_file, int n, int panel) {
  int ndev = 0;
  CU(cudaGetDeviceCount(&ndev));
  CU(cudaSetDevice(rank % (ndev > 0 ? ndev : 1)));
  unsigned char id[B2_MG_ID_BYTES];
  memset(id, 0, sizeof id);
  if (world > 1) {
    if (rank == 0) {
      CK(b2_mg_unique_id(id));
      std::string tmp = std::string(id_file) + ".tmp";
      FILE *f = fopen(tmp.c_str(), "wb");
      if (!f || fwrite(id, 1, sizeof id, f) != sizeof id) { fprintf(stderr, "cannot write %s\n", tmp.c_str()); return 6; }
      fclose(f);
      if (rename(tmp.c_str(), id_file) != 0) { fprintf(stderr, "cannot publish %s\n", id_file); return 6; }
    } else {
      FILE *f = nullptr;
      for (int tries = 0; tries < 600 && !(f = fopen(id_file, "rb")); ++tries) usleep(100000);
      if (!f || fread(id, 1, sizeof id, f) != sizeof id) { fprintf(stderr, "rank %d: no communicator id in %s after 60 s\n", rank, id_file); return 6; }
      fclose(f);
    }
  }
  b2_mg_handle mg;
  CK(b2_mg_create(&mg, nullptr, rank, world, world > 1 ? id : nullptr));
  int64_t start = 0, rows = 0;
  CK(b2_mg_row_block(n, rank, world, &start, &rows));
  const size_t n2 = (size_t)n * n, blk = (size_t)rows * n;
  float *dA, *dB, *dC, *dRef;
  CU(cudaMalloc(&dA, (blk ? blk : 1) * 4)); CU(cudaMalloc(&dB, n2 * 4)); CU(cudaMalloc(&dC, (blk ? blk : 1) * 4)); CU(cudaMalloc(&dRef, (blk ? blk : 1) * 4));
  CK(b2_fill_uniform(dA, (int64_t)blk, 1000 + rank, nullptr));
  CK(b2_fill_uniform(dC, (int64_t)blk, 3000 + rank, nullptr));
  CU(cudaMemcpy(dRef, dC, blk * 4, cudaMemcpyDeviceToDevice));
  if (rank == 0) CK(b2_fill_uniform(dB, (int64_t)n2, 2, nullptr));
  else CU(cudaMemset(dB, 0xff, n2 * 4));     // NaN pattern: a panel used before it landed would show
  const float alpha = 1.0f, beta = 0.5f;
  CK(b2_mg_sgemm(mg, B2_PATH_FFMA, 0, n, n, n, alpha, dA, n, dB, n, beta, dC, n, 0, panel, nullptr, nullptr));
  CU(cudaDeviceSynchronize());
  // B is now everywhere: the same K-panel schedule, locally, must give the same bits
  const int count = b2_mg_k_panel(n, panel, 0, nullptr, nullptr);
  for (int i = 0; i < count && rows > 0; ++i) {
    int k0 = 0, kw = 0;
    b2_mg_k_panel(n, panel, i, &k0, &kw);
    CK(b2_sgemm(nullptr, B2_PATH_FFMA, (int)rows, n, kw, alpha, dA + k0, n, dB + (size_t)k0 * n, n, i == 0 ? beta : 1.0f, dRef, n, nullptr));
  }
  float max_abs = 0.f;
  if (rows > 0 && b2_verify_matrix(dRef, dC, rows, n, n, 0.0f, &max_abs, nullptr) != 0) {
    printf("rank %d: sharded SGEMM differs from the local panel schedule (max |diff| %g)\n", rank, max_abs);
    return 5;
  }
  b2_timer timer;
  CK(b2_timer_create(&timer));
  CK(b2_timer_start(timer, nullptr));
  const int iters = 3;
  for (int it = 0; it < iters; ++it)
    CK(b2_mg_sgemm(mg, B2_PATH_FFMA, 0, n, n, n, alpha, dA, n, dB, n, 0.0f, dC, n, 0, panel, nullptr, nullptr));
  CK(b2_timer_stop(timer, nullptr));
  float ms = 0.f;
  CK(time_ms(timer, &ms));
  // sharded SDOT: every rank can rebuild every slice, so the expected sum is formed locally
  const int64_t nloc = (int64_t)1 << 22;
  float *dx, *dy, *dres;
  double *dsum, *dpart;
  CU(cudaMalloc(&dx, nloc * 4)); CU(cudaMalloc(&dy, nloc * 4)); CU(cudaMalloc(&dres, 4)); CU(cudaMalloc(&dsum, 8)); CU(cudaMalloc(&dpart, 8));
  double expect = 0.0;
  for (int r = 0; r < world; ++r) {
    CK(b2_fill_uniform(dx, nloc, 40 + r, nullptr));
    CK(b2_fill_uniform(dy, nloc, 50 + r, nullptr));
    CK(b2_sdot_partial(nullptr, nloc, dx, dy, dres, dpart, nullptr));
    double part = 0.0;
    CU(cudaMemcpy(&part, dpart, 8, cudaMemcpyDeviceToHost));
    expect += part;
  }
  CK(b2_fill_uniform(dx, nloc, 40 + rank, nullptr));
  CK(b2_fill_uniform(dy, nloc, 50 + rank, nullptr));
  CK(b2_mg_sdot(mg, nloc, dx, dy, dres, dsum, nullptr));
  double got = 0.0;
  CU(cudaMemcpy(&got, dsum, 8, cudaMemcpyDeviceToHost));
  const double tol = 1e-12 * (double)nloc * world;
  if (!(got - expect <= tol && expect - got <= tol)) { printf("rank %d: sharded SDOT %.17g, expected %.17g\n", rank, got, expect); return 5; }
  printf("rank %d of %d: mg sgemm n = %d rows %lld  %9.1f GFLOPS for the whole product (%.3f ms per call), bit-identical to the local panel schedule; mg sdot ok\n",
         rank, world, n, (long long)rows, 2.0 * iters * (double)n * n * n / 1e9 / (ms / 1e3), ms / iters);
  CK(b2_check_status(nullptr, nullptr));
  CK(b2_mg_destroy(mg));
  return 0;
}

int main(int argc, char **argv) {
  if (argc < 2) {
    printf("usage: %s sgemm <kernel_id 1..14> <start> <end> [threads_x] | ft_sgemm <start> <end> <gap> | saxpy | sdot | "
           "small | tiles <n> | sgemm_host <n> [path] | mg <rank> <world> <id file> <n> [panel_k]\n", argv[0]);
    return 1;
  }
  if (!strcmp(argv[1], "sgemm") && argc >= 5)
    return run_sgemm(atoi(argv[2]), atoi(argv[3]), atoi(argv[4]), argc > 5 ? atoi(argv[5]) : 32);
  if (!strcmp(argv[1], "ft_sgemm") && argc >= 5) return run_ft_sgemm(atoi(argv[2]), atoi(argv[3]), atoi(argv[4]));
  if (!strcmp(argv[1], "sgemm_host") && argc >= 3) return run_sgemm_host(atoi(argv[2]), argc > 3 ? atoi(argv[3]) : 0);
  if (!strcmp(argv[1], "mg") && argc >= 6) return run_mg(atoi(argv[2]), atoi(argv[3]), argv[4], atoi(argv[5]), argc > 6 ? atoi(argv[6]) : 0);
  if (!strcmp(argv[1], "small")) return run_small();
  if (!strcmp(argv[1], "tiles") && argc >= 3) return run_tiles(atoi(argv[2]));
  if (!strcmp(argv[1], "saxpy")) return run_vectors(false);
  if (!strcmp(argv[1], "sdot")) return run_vectors(true);
  printf("bad arguments\n");
  return 1;
}
