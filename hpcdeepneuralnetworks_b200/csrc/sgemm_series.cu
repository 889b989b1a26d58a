// The reference's SGEMM optimisation series, rungs 1..13, rebuilt as sm_100a kernels.
// Row-major square C = alpha*A*B + beta*C with the reference's argument order
// (N, A, B, C, alpha, beta).  Rung 14 and the north-star launcher live in sgemm_ffma.cu.
//
//   rung   reference                                   kernel here
//   1      kernel/sgemm/include/kernel_1.cuh:2         series_naive
//   2      kernel_2.cuh:1                              series_smem<T>
//   3,4,5  kernel_3.cuh:1, kernel_4.cuh:48, _5.cuh:1   series_reg1d<T, TRANSPOSE_A, VEC_SMEM>
//   6,7,8  kernel_6.cuh:1, kernel_7.cuh:2, _8.cuh:2    series_reg2d<BM, BK>
//   9,10   kernel_9.cuh:15, kernel_10.cuh:10           series_regtile<TM, false, 0>
//   11     kernel_11.cuh:15                            series_regtile<8, true, 0>
//   12,13  kernel_12.cuh:15, kernel_13.cuh:14          series_regtile<8, true, 1|2>
//
// Unlike the reference (kernel_12.cuh:46-50, kernel_13.cuh:48-53) the prefetching rungs do
// not read one K-slab past the end of A and B.  Like the reference, the rungs have no
// edge handling: N must be a multiple of the rung's block tile, which the launcher checks.
#include "common.cuh"

namespace b2 {

__device__ __forceinline__ float axpby(float alpha, float acc, float beta, float c) {
  return __fmaf_rn(alpha, acc, __fmul_rn(beta, c));
}

// Rung 1: one output per thread; x indexes the column so that a warp reads B and writes C
// coalesced (the point of kernel_1.cuh:8-9).
__global__ void series_naive(int N, const float *A, const float *B, float *C, float alpha, float beta) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;  // column
  const int j = blockIdx.y * blockDim.y + threadIdx.y;  // row
  if (i >= N || j >= N) return;
  float acc = 0.f;
  for (int k = 0; k < N; ++k) acc = __fmaf_rn(A[(size_t)j * N + k], B[(size_t)k * N + i], acc);
  C[(size_t)j * N + i] = axpby(alpha, acc, beta, C[(size_t)j * N + i]);
}

// Rung 2: T x T x T shared-memory block tiling, one output per thread.
template <int T>
__global__ void __launch_bounds__(T *T) series_smem(int N, const float *A, const float *B, float *C, float alpha,
                                                    float beta) {
  __shared__ float As[T][T], Bs[T][T];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int col = blockIdx.x * T + tx, row = blockIdx.y * T + ty;
  float acc = 0.f;
  for (int k0 = 0; k0 < N; k0 += T) {
    As[ty][tx] = A[(size_t)row * N + k0 + tx];
    Bs[ty][tx] = B[(size_t)(k0 + ty) * N + col];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < T; ++k) acc = __fmaf_rn(As[ty][k], Bs[k][tx], acc);
    __syncthreads();
  }
  C[(size_t)row * N + col] = axpby(alpha, acc, beta, C[(size_t)row * N + col]);
}

// Rungs 3-5: T x T x T tile, T x T/4 threads, each thread owns a 4-row x 1-column strip.
// TRANSPOSE_A stores the A tile k-major so the 4 rows of a strip are contiguous (rung 4);
// VEC_SMEM reads them with one 128-bit shared load (rung 5).
template <int T, bool TRANSPOSE_A, bool VEC_SMEM>
__global__ void __launch_bounds__(T *T / 4) series_reg1d(int N, const float *A, const float *B, float *C, float alpha,
                                                         float beta) {
  __shared__ __align__(16) float As[T * T];
  __shared__ __align__(16) float Bs[T * T];
  const int tx = threadIdx.x, ty = threadIdx.y;  // ty in [0, T/4)
  const int col = blockIdx.x * T + tx, row0 = blockIdx.y * T + ty * 4;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < N; k0 += T) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float a = A[(size_t)(row0 + r) * N + k0 + tx];
      if (TRANSPOSE_A) As[tx * T + ty * 4 + r] = a;  // As[k][m]
      else As[(ty * 4 + r) * T + tx] = a;            // As[m][k]
      Bs[(ty * 4 + r) * T + tx] = B[(size_t)(k0 + ty * 4 + r) * N + col];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < T; ++k) {
      const float b = Bs[k * T + tx];
      if (TRANSPOSE_A && VEC_SMEM) {
        const float4 a4 = *reinterpret_cast<const float4 *>(&As[k * T + ty * 4]);
        acc[0] = __fmaf_rn(a4.x, b, acc[0]);
        acc[1] = __fmaf_rn(a4.y, b, acc[1]);
        acc[2] = __fmaf_rn(a4.z, b, acc[2]);
        acc[3] = __fmaf_rn(a4.w, b, acc[3]);
      } else {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float a = TRANSPOSE_A ? As[k * T + ty * 4 + r] : As[(ty * 4 + r) * T + k];
          acc[r] = __fmaf_rn(a, b, acc[r]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    float *c = &C[(size_t)(row0 + r) * N + col];
    *c = axpby(alpha, acc[r], beta, *c);
  }
}

// Rungs 6-8: BM x BM x BK tile, (BM/4)^2 threads, 4x4 outputs per thread, 128-bit global
// loads and stores; A is stored k-major in shared memory.
template <int BM, int BK>
__global__ void __launch_bounds__((BM / 4) * (BM / 4)) series_reg2d(int N, const float *A, const float *B, float *C,
                                                                   float alpha, float beta) {
  constexpr int NT = (BM / 4) * (BM / 4);
  __shared__ __align__(16) float As[BK * BM];  // [k][m]
  __shared__ __align__(16) float Bs[BK * BM];  // [k][n]
  const int tid = threadIdx.y * (BM / 4) + threadIdx.x;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BM;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < N; k0 += BK) {
    // A tile: BM rows x BK/4 float4 ; B tile: BK rows x BM/4 float4
    for (int f = tid; f < BM * BK / 4; f += NT) {
      const int r = f / (BK / 4), kc = (f % (BK / 4)) * 4;
      const float4 v = *reinterpret_cast<const float4 *>(&A[(size_t)(m0 + r) * N + k0 + kc]);
      As[(kc + 0) * BM + r] = v.x;
      As[(kc + 1) * BM + r] = v.y;
      As[(kc + 2) * BM + r] = v.z;
      As[(kc + 3) * BM + r] = v.w;
      const int br = f / (BM / 4), bc = (f % (BM / 4)) * 4;
      *reinterpret_cast<float4 *>(&Bs[br * BM + bc]) = *reinterpret_cast<const float4 *>(&B[(size_t)(k0 + br) * N + n0 + bc]);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a = *reinterpret_cast<const float4 *>(&As[k * BM + ty * 4]);
      const float4 b = *reinterpret_cast<const float4 *>(&Bs[k * BM + tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float4 *cp = reinterpret_cast<float4 *>(&C[(size_t)(m0 + ty * 4 + i) * N + n0 + tx * 4]);
    float4 c = *cp;
    c.x = axpby(alpha, acc[i][0], beta, c.x);
    c.y = axpby(alpha, acc[i][1], beta, c.y);
    c.z = axpby(alpha, acc[i][2], beta, c.z);
    c.w = axpby(alpha, acc[i][3], beta, c.w);
    *cp = c;
  }
}

// Rungs 9-13: (16*TM)^2 x BK tile (BK = 64/TM), 256 threads, TM x TM outputs per thread.
// WARPTILE arranges the 8 warps 2 x 4 and the lanes 8 x 4 so that a warp covers 64 x 32
// (rung 11).  PIPE 0: load, sync, compute, sync.  PIPE 1: the next slab is fetched into
// registers while the current one is consumed (rung 12).  PIPE 2: plus a double-buffered
// shared tile and a single barrier per slab (rung 13).
template <int TM, bool WARPTILE, int PIPE>
__global__ void __launch_bounds__(256) series_regtile(int N, const float *A, const float *B, float *C, float alpha,
                                                      float beta) {
  constexpr int BM = 16 * TM, BK = 64 / TM, NBUF = (PIPE == 2) ? 2 : 1;
  __shared__ __align__(16) float As[NBUF][BK * BM];  // [k][m]
  __shared__ __align__(16) float Bs[NBUF][BK * BM];  // [k][n]
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BM;
  int rm, cn;  // first row / column of this thread's TM x TM block inside the tile
  if (WARPTILE) {
    const int w = tid >> 5, lane = tid & 31;
    rm = (w >> 2) * (BM / 2) + (lane >> 2) * TM;
    cn = (w & 3) * (BM / 4) + (lane & 3) * TM;
  } else {
    rm = (tid >> 4) * TM;
    cn = (tid & 15) * TM;
  }
  const int ar = tid / (BK / 4), akc = (tid % (BK / 4)) * 4;  // this thread's float4 of the A slab
  const int br = tid / (BM / 4), bc = (tid % (BM / 4)) * 4;   // and of the B slab
  const float *Ap = A + (size_t)(m0 + ar) * N + akc;
  const float *Bp = B + (size_t)br * N + n0 + bc;
  float acc[TM][TM] = {};
  float4 pa, pb;

  auto gload = [&](int k0) {
    pa = *reinterpret_cast<const float4 *>(Ap + k0);
    pb = *reinterpret_cast<const float4 *>(Bp + (size_t)k0 * N);
  };
  auto sstore = [&](int buf) {
    As[buf][(akc + 0) * BM + ar] = pa.x;
    As[buf][(akc + 1) * BM + ar] = pa.y;
    As[buf][(akc + 2) * BM + ar] = pa.z;
    As[buf][(akc + 3) * BM + ar] = pa.w;
    *reinterpret_cast<float4 *>(&Bs[buf][br * BM + bc]) = pb;
  };
  auto compute = [&](int buf) {
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float av[TM], bv[TM];
#pragma unroll
      for (int q = 0; q < TM / 4; ++q) {
        const float4 a = *reinterpret_cast<const float4 *>(&As[buf][k * BM + rm + 4 * q]);
        const float4 b = *reinterpret_cast<const float4 *>(&Bs[buf][k * BM + cn + 4 * q]);
        av[4 * q] = a.x; av[4 * q + 1] = a.y; av[4 * q + 2] = a.z; av[4 * q + 3] = a.w;
        bv[4 * q] = b.x; bv[4 * q + 1] = b.y; bv[4 * q + 2] = b.z; bv[4 * q + 3] = b.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TM; ++j) acc[i][j] = __fmaf_rn(av[i], bv[j], acc[i][j]);
    }
  };

  if (PIPE == 0) {
    for (int k0 = 0; k0 < N; k0 += BK) {
      gload(k0);
      sstore(0);
      __syncthreads();
      compute(0);
      __syncthreads();
    }
  } else if (PIPE == 1) {
    gload(0);
    for (int k0 = 0; k0 < N; k0 += BK) {
      sstore(0);
      __syncthreads();
      if (k0 + BK < N) gload(k0 + BK);  // in flight while this slab is consumed
      compute(0);
      __syncthreads();
    }
  } else {
    gload(0);
    sstore(0);
    __syncthreads();
    int buf = 0;
    for (int k0 = 0; k0 < N; k0 += BK) {
      const bool more = (k0 + BK < N);
      if (more) gload(k0 + BK);
      compute(buf);
      if (more) sstore(buf ^ 1);
      __syncthreads();
      buf ^= 1;
    }
  }

#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int q = 0; q < TM / 4; ++q) {
      float4 *cp = reinterpret_cast<float4 *>(&C[(size_t)(m0 + rm + i) * N + n0 + cn + 4 * q]);
      float4 c = *cp;
      c.x = axpby(alpha, acc[i][4 * q + 0], beta, c.x);
      c.y = axpby(alpha, acc[i][4 * q + 1], beta, c.y);
      c.z = axpby(alpha, acc[i][4 * q + 2], beta, c.z);
      c.w = axpby(alpha, acc[i][4 * q + 3], beta, c.w);
      *cp = c;
    }
}

}  // namespace b2

using namespace b2;

extern "C" int b2_sgemm_series(int kernel_id, int threads_x, int N, const float *A, const float *B, float *C, float alpha,
                               float beta, void *stream) {
  B2_REQUIRE(kernel_id >= 1 && kernel_id <= 14, B2_ERR_INVALID_ARG, "b2_sgemm_series: kernel id %d is not in 1..14", kernel_id);
  B2_REQUIRE(N >= 0, B2_ERR_INVALID_ARG, "b2_sgemm_series: N = %d is negative", N);
  if (N == 0) return B2_OK;
  B2_REQUIRE(A && B && C, B2_ERR_INVALID_ARG, "b2_sgemm_series: null matrix");
  if (kernel_id == 14) return b2_sgemm(nullptr, B2_PATH_FFMA, N, N, N, alpha, A, N, B, N, beta, C, N, stream);
  cudaStream_t s = (cudaStream_t)stream;
  int t = threads_x > 0 ? threads_x : 32;
  const bool al16 = ((((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) == 0);
  auto need = [&](int tile) -> bool { return N % tile == 0; };
#define B2_NEED(tile)                                                                                         \
  B2_REQUIRE(need(tile), B2_ERR_UNSUPPORTED, "b2_sgemm_series: rung %d needs N (%d) to be a multiple of %d", \
             kernel_id, N, (tile))
  if (kernel_id >= 6) B2_REQUIRE(al16, B2_ERR_UNSUPPORTED, "b2_sgemm_series: rung %d needs 16-byte aligned matrices", kernel_id);
  switch (kernel_id) {
    case 1: {
      B2_REQUIRE(t >= 1 && t <= 32, B2_ERR_UNSUPPORTED, "b2_sgemm_series: rung 1 block edge %d not in 1..32", t);
      dim3 blk(t, t), grd((N + t - 1) / t, (N + t - 1) / t);
      series_naive<<<grd, blk, 0, s>>>(N, A, B, C, alpha, beta);
      break;
    }
    case 2: {
      B2_REQUIRE(t == 16 || t == 32, B2_ERR_UNSUPPORTED, "b2_sgemm_series: rung 2 block edge %d must be 16 or 32", t);
      B2_NEED(t);
      dim3 blk(t, t), grd(N / t, N / t);
      if (t == 16) series_smem<16><<<grd, blk, 0, s>>>(N, A, B, C, alpha, beta);
      else series_smem<32><<<grd, blk, 0, s>>>(N, A, B, C, alpha, beta);
      break;
    }
    case 3: case 4: case 5: {
      B2_REQUIRE(t == 16 || t == 32, B2_ERR_UNSUPPORTED, "b2_sgemm_series: rung %d block edge %d must be 16 or 32", kernel_id, t);
      B2_NEED(t);
      dim3 blk(t, t / 4), grd(N / t, N / t);
#define B2_REG1D(T)                                                                               \
  if (kernel_id == 3) series_reg1d<T, false, false><<<grd, blk, 0, s>>>(N, A, B, C, alpha, beta); \
  else if (kernel_id == 4) series_reg1d<T, true, false><<<grd, blk, 0, s>>>(N, A, B, C, alpha, beta); \
  else series_reg1d<T, true, true><<<grd, blk, 0, s>>>(N, A, B, C, alpha, beta)
      if (t == 16) { B2_REG1D(16); } else { B2_REG1D(32); }
#undef B2_REG1D
      break;
    }
    case 6: { B2_NEED(32); series_reg2d<32, 32><<<dim3(N / 32, N / 32), dim3(8, 8), 0, s>>>(N, A, B, C, alpha, beta); break; }
    case 7: { B2_NEED(64); series_reg2d<64, 64><<<dim3(N / 64, N / 64), dim3(16, 16), 0, s>>>(N, A, B, C, alpha, beta); break; }
    case 8: { B2_NEED(64); series_reg2d<64, 16><<<dim3(N / 64, N / 64), dim3(16, 16), 0, s>>>(N, A, B, C, alpha, beta); break; }
    case 9: { B2_NEED(128); series_regtile<8, false, 0><<<dim3(N / 128, N / 128), 256, 0, s>>>(N, A, B, C, alpha, beta); break; }
    case 10: { B2_NEED(256); series_regtile<16, false, 0><<<dim3(N / 256, N / 256), 256, 0, s>>>(N, A, B, C, alpha, beta); break; }
    case 11: { B2_NEED(128); series_regtile<8, true, 0><<<dim3(N / 128, N / 128), 256, 0, s>>>(N, A, B, C, alpha, beta); break; }
    case 12: { B2_NEED(128); series_regtile<8, true, 1><<<dim3(N / 128, N / 128), 256, 0, s>>>(N, A, B, C, alpha, beta); break; }
    case 13: { B2_NEED(128); series_regtile<8, true, 2><<<dim3(N / 128, N / 128), 256, 0, s>>>(N, A, B, C, alpha, beta); break; }
    default: break;
  }
#undef B2_NEED
  B2_CUDA(cudaGetLastError());
  return B2_OK;
}
