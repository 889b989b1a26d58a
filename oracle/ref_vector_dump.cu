// Test infrastructure, not product code: runs the REFERENCE's own SAXPY and SDOT kernels
// (kernel/saxpy/saxpy.cu:15-48, kernel/sdot/sdot.cu:9-35), included unmodified from the
// reference tree at build time with their main() renamed out of the way, on the seeded inputs
// the tests use, with the drivers' launch geometry (kernel/saxpy/saxpy.cu:74-78,109-112;
// kernel/sdot/sdot.cu:97-99,156), and writes the result to a file.
//
//   ref_vector_dump saxpy  <n multiple of 4> <alpha> <threads per block> <out.bin>   f128 kernel `saxpy`
//   ref_vector_dump saxpy2 <n>               <alpha> <threads per block> <out.bin>   scalar kernel `_saxpy`
//   ref_vector_dump sdot   <n>               <threads per block> <out.bin>           `_sdot` (adds into a zeroed scalar)
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

static uint64_t dump_mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
static void dump_fill(std::vector<float> &v, uint64_t seed) {
  const uint64_t ms = dump_mix64(seed);
  for (size_t i = 0; i < v.size(); ++i) {
    const uint64_t h = dump_mix64(ms ^ ((uint64_t)i * 0xD1342543DE82EF95ull));
    v[i] = (float)(uint32_t)(h >> 40) * (1.0f / 8388608.0f) - 1.0f;
  }
}

#define main reference_saxpy_main_unused
#include "kernel/saxpy/saxpy.cu"
#undef main
#undef multi
#undef PPP
#define main reference_sdot_main_unused
#include "kernel/sdot/sdot.cu"
#undef main

static int write_out(const char *path, const float *p, size_t count) {
  FILE *f = fopen(path, "wb");
  if (!f || fwrite(p, 4, count, f) != count) return 5;
  fclose(f);
  return 0;
}

int main(int argc, char **argv) {
  if (argc < 5) {
    fprintf(stderr, "usage: ref_vector_dump saxpy|saxpy2 <n> <alpha> <tpb> <out> | sdot <n> <tpb> <out>\n");
    return 2;
  }
  const bool is_dot = strcmp(argv[1], "sdot") == 0;
  const bool scalar = strcmp(argv[1], "saxpy2") == 0;
  const long n = atol(argv[2]);
  const float alpha = is_dot ? 0.f : (float)atof(argv[3]);
  const int tpb = atoi(argv[is_dot ? 3 : 4]);
  const char *out = argv[is_dot ? 4 : 5];
  if (n <= 0 || n > (1l << 28) || tpb < 32 || tpb > 1024 || (!is_dot && argc < 6) || (!is_dot && !scalar && n % 4 != 0)) {
    fprintf(stderr, "bad arguments\n");
    return 2;
  }
  std::vector<float> x((size_t)n), y((size_t)n);
  dump_fill(x, 4);
  dump_fill(y, 5);
  float *dx, *dy, *dc;
  if (cudaMalloc(&dx, n * 4) != cudaSuccess || cudaMalloc(&dy, n * 4) != cudaSuccess || cudaMalloc(&dc, 4) != cudaSuccess) return 3;
  cudaMemcpy(dx, x.data(), n * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(dy, y.data(), n * 4, cudaMemcpyHostToDevice);
  cudaMemset(dc, 0, 4);
  if (is_dot) {
    const long want = (n + tpb - 1) / tpb;
    const int blocks = (int)(want < 1024 ? want : 1024);
    _sdot<<<blocks, tpb>>>((int)n, dx, dy, dc);
  } else if (scalar) {
    _saxpy<<<(int)((n + tpb - 1) / tpb), tpb>>>((int)n, alpha, dx, dy);
  } else {
    saxpy<<<(int)((n / 4 + tpb - 1) / tpb), tpb>>>((int)(n / 4), alpha, (f128 *)dx, (f128 *)dy);
  }
  if (cudaDeviceSynchronize() != cudaSuccess) {
    fprintf(stderr, "kernel failed: %s\n", cudaGetErrorString(cudaGetLastError()));
    return 4;
  }
  if (is_dot) {
    float r = 0.f;
    cudaMemcpy(&r, dc, 4, cudaMemcpyDeviceToHost);
    return write_out(out, &r, 1);
  }
  cudaMemcpy(y.data(), dy, n * 4, cudaMemcpyDeviceToHost);
  return write_out(out, y.data(), (size_t)n);
}
