// FP32 SIMT (FFMA) SGEMM for sm_100a: row-major C = alpha*A*B + beta*C, any M, N, K.
//
// Stands in for rung 14 of the reference series (kernel/sgemm/include/kernel_14.cuh:12:
// 128x128x32 block tile, 256 threads, 8x8 outputs per thread) and, through the
// column-major shim, for the plain tile family of kernel/ft_sgemm
// (include_code_gen/sgemm_huge.cuh:11).  What is different on Blackwell:
//   * A and B slabs are brought in by TMA (cp.async.bulk.tensor) into a 3-stage shared
//     ring guarded by full/empty mbarriers; no thread spends issue slots on global loads,
//     and out-of-range rows/columns/K are zero-filled by the copy engine, so any shape works.
//   * A stays K-contiguous in shared memory (TMA cannot transpose) under the 128-byte
//     swizzle; a thread reads a float4 ALONG K for each of its 8 rows, which costs the same
//     number of 128-bit shared loads as the reference's transposed store scheme
//     (kernel_9.cuh:37-40) and is bank-conflict free.
//   * 8 warps as 4 (M) x 2 (N), lanes as 4 (M) x 8 (N): the warp tiling idea of
//     kernel_11.cuh:22-27 with the lane shape chosen for the swizzled A reads.
//   * Optionally the inner product uses the packed fma.rn.f32x2 instruction (two FP32
//     FMAs per issue slot); per output the arithmetic is still one FMA per k in ascending k,
//     so results are bit-identical to the scalar form.
// Each output element is accumulated by exactly one thread in ascending k with one FMA per
// k, and the epilogue is fma(alpha, acc, beta*c) (alpha*acc when beta == 0; C is then not
// read).
#include <stdlib.h>

#include "common.cuh"

namespace b2 {

constexpr int FBM = 128, FBN = 128, FBK = 32, FSTAGES = 3;
constexpr int kStageA = FBM * FBK * 4;  // 16 KB, 128 rows of 128 bytes, 128B-swizzled
constexpr int kStageB = FBK * FBN * 4;  // 16 KB, 32 rows of 512 bytes, linear
constexpr int kFfmaSmem = 1024 + FSTAGES * (kStageA + kStageB) + 128;
constexpr int kGroupM = 16;  // tile rasterisation: 16 tile-rows share their B panels in L2

__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

struct FfmaArgs {
  float *C;
  int M, N, K, ldc;
  float alpha, beta;
  int vec_c;    // C rows are 16-byte aligned: 128-bit epilogue
  int *status;  // device status word: set to B2_ERR_TIMEOUT if a bounded wait runs out
};

// Accumulators of one thread: 8 rows x 8 columns.  Row i is tile row  wm*32 + lm + 4*i,
// column j is tile column  wn*64 + ln*4 + 32*(j/4) + j%4.
template <bool PACKED>
struct Acc;
template <>
struct Acc<false> {
  float v[8][8];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
  }
  __device__ __forceinline__ void step(const float (&a)[8], const float4 &b0, const float4 &b1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i][0] = __fmaf_rn(a[i], b0.x, v[i][0]);
      v[i][1] = __fmaf_rn(a[i], b0.y, v[i][1]);
      v[i][2] = __fmaf_rn(a[i], b0.z, v[i][2]);
      v[i][3] = __fmaf_rn(a[i], b0.w, v[i][3]);
      v[i][4] = __fmaf_rn(a[i], b1.x, v[i][4]);
      v[i][5] = __fmaf_rn(a[i], b1.y, v[i][5]);
      v[i][6] = __fmaf_rn(a[i], b1.z, v[i][6]);
      v[i][7] = __fmaf_rn(a[i], b1.w, v[i][7]);
    }
  }
  __device__ __forceinline__ float get(int i, int j) const { return v[i][j]; }
  __device__ __forceinline__ void set(int i, int j, float x) { v[i][j] = x; }
};
template <>
struct Acc<true> {
  uint64_t v[8][4];  // pairs of adjacent columns
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) v[i][j] = 0ull;
  }
  __device__ __forceinline__ void step(const float (&a)[8], const float4 &b0, const float4 &b1) {
    const uint64_t bp0 = pack2(b0.x, b0.y), bp1 = pack2(b0.z, b0.w), bp2 = pack2(b1.x, b1.y), bp3 = pack2(b1.z, b1.w);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint64_t aa = pack2(a[i], a[i]);
      v[i][0] = ffma2(aa, bp0, v[i][0]);
      v[i][1] = ffma2(aa, bp1, v[i][1]);
      v[i][2] = ffma2(aa, bp2, v[i][2]);
      v[i][3] = ffma2(aa, bp3, v[i][3]);
    }
  }
  __device__ __forceinline__ float get(int i, int j) const {
    float lo, hi;
    unpack2(v[i][j >> 1], lo, hi);
    return (j & 1) ? hi : lo;
  }
  __device__ __forceinline__ void set(int i, int j, float x) {
    float lo, hi;
    unpack2(v[i][j >> 1], lo, hi);
    if (j & 1) hi = x; else lo = x;
    v[i][j >> 1] = pack2(lo, hi);
  }
};

__device__ __forceinline__ void tile_of_block(int bid, int tiles_m, int tiles_n, int &tm, int &tn) {
  const int per_group = kGroupM * tiles_n;
  const int g = bid / per_group, r = bid - g * per_group;
  const int first = g * kGroupM;
  const int gsz = (tiles_m - first < kGroupM) ? (tiles_m - first) : kGroupM;
  tm = first + r % gsz;
  tn = r / gsz;
}

// Tile row of accumulator row i.  NN (A row-major, K contiguous): wm*32 + lm + 4*i, which makes
// the swizzled float4-along-K reads conflict free.  TN (A given K x M, M contiguous, as in the
// column-major family of kernel/ft_sgemm): wm*32 + lm*4 + (i&3) + 16*(i>>2), so that a thread
// reads two float4 along M per k.
template <bool TRANS_A>
__device__ __forceinline__ int acc_row(int wm, int lm, int i) {
  return TRANS_A ? (wm * 32 + lm * 4 + (i & 3) + 16 * (i >> 2)) : (wm * 32 + lm + 4 * i);
}

template <bool PACKED, int KCU, bool TRANS_A>
__global__ void __launch_bounds__(256, 2)
sgemm_ffma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const FfmaArgs p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char *sA = smem;
  unsigned char *sB = smem + FSTAGES * kStageA;
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + FSTAGES * (kStageA + kStageB));
  uint64_t *empty = full + FSTAGES;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 1, wn = warp & 1, lm = lane >> 3, ln = lane & 7;
  const int tiles_m = (p.M + FBM - 1) / FBM, tiles_n = (p.N + FBN - 1) / FBN;
  int tile_m, tile_n;
  tile_of_block(blockIdx.x, tiles_m, tiles_n, tile_m, tile_n);
  const int m0 = tile_m * FBM, n0 = tile_n * FBN;
  const int nkb = (p.K + FBK - 1) / FBK;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < FSTAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 8);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  __syncthreads();
  if (tid == 0) {
    for (int s = 0; s < FSTAGES && s < nkb; ++s) {
      mbar_expect_tx(&full[s], kStageA + kStageB);
      if (TRANS_A) tma_load_2d(sA + s * kStageA, &tmA, &full[s], m0, s * FBK);
      else tma_load_2d(sA + s * kStageA, &tmA, &full[s], s * FBK, m0);
      tma_load_2d(sB + s * kStageB, &tmB, &full[s], n0, s * FBK);
    }
  }

  Acc<PACKED> acc;
  acc.zero();
  // Byte offsets inside a stage.  A: row r at r*128, 16-byte chunk c of that row at
  // ((c ^ (r & 7)) << 4); rows of this thread are wm*32 + lm + 4*i, so r & 7 is lm for even
  // i and lm + 4 for odd i.  B: row k at k*512, column c at c*4.
  const uint32_t a_thread = TRANS_A ? (uint32_t)(wm * 32 + lm * 4) * 4u : (uint32_t)(wm * 32 + lm) * 128u;
  const uint32_t a_swz = (uint32_t)lm << 4;
  const uint32_t b_thread = (uint32_t)(wn * 64 + ln * 4) * 4u;
  bool ok = true;

  for (int kb = 0; kb < nkb; ++kb) {
    const int s = kb % FSTAGES;
    if (!mbar_wait(&full[s], (uint32_t)(kb / FSTAGES) & 1u)) {
      ok = false;
      break;
    }
    const unsigned char *As = sA + s * kStageA + a_thread;
    const unsigned char *Bs = sB + s * kStageB + b_thread;
    if (TRANS_A) {
#pragma unroll(KCU * 4)
      for (int k = 0; k < FBK; ++k) {
        const float4 a0 = *reinterpret_cast<const float4 *>(As + k * 512);
        const float4 a1 = *reinterpret_cast<const float4 *>(As + k * 512 + 64);
        const float4 b0 = *reinterpret_cast<const float4 *>(Bs + k * 512);
        const float4 b1 = *reinterpret_cast<const float4 *>(Bs + k * 512 + 128);
        const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        acc.step(a, b0, b1);
      }
    } else {
#pragma unroll(KCU)
      for (int kc = 0; kc < FBK / 4; ++kc) {
        const uint32_t y0 = ((uint32_t)kc << 4) ^ a_swz, y1 = y0 ^ 64u;
        float4 a4[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          a4[i] = *reinterpret_cast<const float4 *>(As + ((i & 1) ? y1 : y0) + i * 512);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const float4 b0 = *reinterpret_cast<const float4 *>(Bs + (kc * 4 + kk) * 512);
          const float4 b1 = *reinterpret_cast<const float4 *>(Bs + (kc * 4 + kk) * 512 + 128);
          float a[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) a[i] = (kk == 0) ? a4[i].x : (kk == 1) ? a4[i].y : (kk == 2) ? a4[i].z : a4[i].w;
          acc.step(a, b0, b1);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
    // Refill, one slab behind: the stage that slab kb-1 used gets slab kb-1+FSTAGES once all
    // 8 warps have released it.
    if (tid == 0 && kb >= 1) {
      const int kprev = kb - 1, knext = kprev + FSTAGES;
      if (knext < nkb) {
        const int sp = kprev % FSTAGES;
        if (!mbar_wait(&empty[sp], (uint32_t)(kprev / FSTAGES) & 1u)) {
          ok = false;
          break;
        }
        mbar_expect_tx(&full[sp], kStageA + kStageB);
        if (TRANS_A) tma_load_2d(sA + sp * kStageA, &tmA, &full[sp], m0, knext * FBK);
        else tma_load_2d(sA + sp * kStageA, &tmA, &full[sp], knext * FBK, m0);
        tma_load_2d(sB + sp * kStageB, &tmB, &full[sp], n0, knext * FBK);
      }
    }
  }
  if (!ok) {
    atomicExch(p.status, (int)B2_ERR_TIMEOUT);
    return;
  }

  // Epilogue straight from registers.
  const bool read_c = (p.beta != 0.f);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = m0 + acc_row<TRANS_A>(wm, lm, i);
    if (row >= p.M) continue;
    float *crow = p.C + (size_t)row * p.ldc;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int col = n0 + wn * 64 + ln * 4 + 32 * h;
      if (p.vec_c && col + 3 < p.N) {
        float4 c = make_float4(0.f, 0.f, 0.f, 0.f);
        if (read_c) c = *reinterpret_cast<const float4 *>(crow + col);
        float4 o;
        if (read_c) {
          o.x = __fmaf_rn(p.alpha, acc.get(i, 4 * h + 0), __fmul_rn(p.beta, c.x));
          o.y = __fmaf_rn(p.alpha, acc.get(i, 4 * h + 1), __fmul_rn(p.beta, c.y));
          o.z = __fmaf_rn(p.alpha, acc.get(i, 4 * h + 2), __fmul_rn(p.beta, c.z));
          o.w = __fmaf_rn(p.alpha, acc.get(i, 4 * h + 3), __fmul_rn(p.beta, c.w));
        } else {
          o.x = __fmul_rn(p.alpha, acc.get(i, 4 * h + 0));
          o.y = __fmul_rn(p.alpha, acc.get(i, 4 * h + 1));
          o.z = __fmul_rn(p.alpha, acc.get(i, 4 * h + 2));
          o.w = __fmul_rn(p.alpha, acc.get(i, 4 * h + 3));
        }
        *reinterpret_cast<float4 *>(crow + col) = o;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (col + e < p.N) {
            const float a = acc.get(i, 4 * h + e);
            crow[col + e] = read_c ? __fmaf_rn(p.alpha, a, __fmul_rn(p.beta, crow[col + e])) : __fmul_rn(p.alpha, a);
          }
        }
      }
    }
  }
}

// Fallback for operands TMA cannot describe (leading dimension not a multiple of 4 floats or
// a base pointer that is not 16-byte aligned): 64x64x16 tile, 256 threads, 4x4 outputs per
// thread, fully predicated scalar loads.  Same arithmetic order as the TMA kernel.
__global__ void __launch_bounds__(256) sgemm_generic_kernel(int M, int N, int K, float alpha, const float *A, int a_rs,
                                                            int a_ks, const float *B, int ldb, float beta, float *C, int ldc) {
  __shared__ float As[16][64 + 1];  // [k][m]
  __shared__ float Bs[16][64];      // [k][n]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int f = tid; f < 64 * 16; f += 256) {
      const int r = f >> 4, k = f & 15;
      As[k][r] = (m0 + r < M && k0 + k < K) ? A[(size_t)(m0 + r) * a_rs + (size_t)(k0 + k) * a_ks] : 0.f;
      const int bk = f >> 6, bc = f & 63;
      Bs[bk][bc] = (k0 + bk < K && n0 + bc < N) ? B[(size_t)(k0 + bk) * ldb + n0 + bc] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { av[i] = As[k][ty * 4 + i]; bv[i] = Bs[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      const int r = m0 + ty * 4 + i, c = n0 + tx * 4 + j;
      if (r < M && c < N) {
        float *cp = &C[(size_t)r * ldc + c];
        *cp = (beta != 0.f) ? __fmaf_rn(alpha, acc[i][j], __fmul_rn(beta, *cp)) : __fmul_rn(alpha, acc[i][j]);
      }
    }
}

// C = beta*C (K == 0 or alpha == 0 short cut; beta == 0 writes zeros without reading).
__global__ void scale_c_kernel(int M, int N, float beta, float *C, int ldc) {
  const int64_t total = (int64_t)M * N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / N, c = i - r * N;
    float *cp = &C[r * ldc + c];
    *cp = (beta != 0.f) ? __fmul_rn(beta, *cp) : 0.f;
  }
}

static int g_ffma_variant = -1;  // -1: pick from B2_FFMA_VARIANT (default packed)

static int ffma_variant() {
  if (g_ffma_variant < 0) {
    const char *e = getenv("B2_FFMA_VARIANT");
    g_ffma_variant = e ? atoi(e) : 2;
    if (g_ffma_variant < 0 || g_ffma_variant > 3) g_ffma_variant = 2;
  }
  return g_ffma_variant;
}

template <bool PACKED, int KCU, bool TRANS_A>
static int launch_ffma(const CUtensorMap &ta, const CUtensorMap &tb, const FfmaArgs &args, int grid, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    B2_CUDA(cudaFuncSetAttribute(sgemm_ffma_kernel<PACKED, KCU, TRANS_A>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFfmaSmem));
    B2_CUDA(cudaFuncSetAttribute(sgemm_ffma_kernel<PACKED, KCU, TRANS_A>, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    configured = true;
  }
  sgemm_ffma_kernel<PACKED, KCU, TRANS_A><<<grid, 256, kFfmaSmem, s>>>(ta, tb, args);
  B2_CUDA(cudaGetLastError());
  return B2_OK;
}

// trans_a = 0: A is M x K row-major (lda >= K).  trans_a = 1: A is given as K x M row-major
// (lda >= M), i.e. the column-major M x K operand of the kernel/ft_sgemm family.
int sgemm_ffma_dispatch(Context *ctx, int trans_a, int M, int N, int K, float alpha, const float *A, int lda,
                        const float *B, int ldb, float beta, float *C, int ldc, cudaStream_t s) {
  if (M == 0 || N == 0) return B2_OK;
  if (K == 0 || alpha == 0.f) {
    if (beta == 1.f) return B2_OK;
    scale_c_kernel<<<ctx->sm_count * 4, 256, 0, s>>>(M, N, beta, C, ldc);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
  }
  const bool tma_ok = ((((uintptr_t)A | (uintptr_t)B) & 15) == 0) && (lda % 4 == 0) && (ldb % 4 == 0);
  (void)trans_a;
  if (!tma_ok) {
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    sgemm_generic_kernel<<<grid, 256, 0, s>>>(M, N, K, alpha, A, trans_a ? 1 : lda, trans_a ? lda : 1, B, ldb, beta, C, ldc);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
  }
  CUtensorMap ta, tb;
  int st = trans_a ? make_tmap_2d(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, FBM, FBK, CU_TENSOR_MAP_SWIZZLE_NONE)
                   : make_tmap_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, FBK, FBM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != B2_OK) return st;
  st = make_tmap_2d(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, FBN, FBK, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (st != B2_OK) return st;
  FfmaArgs args;
  args.C = C; args.M = M; args.N = N; args.K = K; args.ldc = ldc; args.alpha = alpha; args.beta = beta;
  args.vec_c = ((((uintptr_t)C) & 15) == 0 && (ldc % 4) == 0) ? 1 : 0;
  args.status = (int *)((char *)ctx->fixed + kFixedStatus);
  const int grid = ((M + FBM - 1) / FBM) * ((N + FBN - 1) / FBN);
  if (trans_a) {
    return (ffma_variant() & 1) ? launch_ffma<true, 2, true>(ta, tb, args, grid, s)
                                : launch_ffma<false, 2, true>(ta, tb, args, grid, s);
  }
  switch (ffma_variant()) {
    case 0: return launch_ffma<false, 8, false>(ta, tb, args, grid, s);
    case 2: return launch_ffma<true, 2, false>(ta, tb, args, grid, s);
    case 3: return launch_ffma<false, 2, false>(ta, tb, args, grid, s);
    default: return launch_ffma<true, 8, false>(ta, tb, args, grid, s);
  }
}

}  // namespace b2

using namespace b2;

namespace b2 {
int sgemm_3xtf32_dispatch(Context *ctx, int M, int N, int K, float alpha, const float *A, int lda, const float *B, int ldb,
                          float beta, float *C, int ldc, cudaStream_t s);
}

extern "C" {

// Selects the inner-loop variant of the FFMA kernel (0 scalar FFMA, 1 packed f32x2, 2/3 the
// same with a shorter unrolled body).  For benchmarking; results are bit-identical.
int b2_set_ffma_variant(int v) {
  B2_REQUIRE(v >= 0 && v <= 3, B2_ERR_INVALID_ARG, "b2_set_ffma_variant: %d not in 0..3", v);
  b2::g_ffma_variant = v;
  return B2_OK;
}

// Reads and clears the device status word that bounded waits set; synchronises the stream.
int b2_check_status(b2_handle h, void *stream) {
  Context *ctx = h ? (Context *)h : default_context();
  B2_REQUIRE(ctx != nullptr, B2_ERR_CUDA, "b2_check_status: no context");
  int v = 0;
  int *dev = (int *)((char *)ctx->fixed + kFixedStatus);
  B2_CUDA(cudaMemcpyAsync(&v, dev, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  B2_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  if (v != 0) {
    B2_CUDA(cudaMemsetAsync(dev, 0, 4, (cudaStream_t)stream));
    set_error("a kernel reported status %d (%s)", v, b2_status_string(v));
  }
  return v;
}

int b2_sgemm(b2_handle h, int path, int M, int N, int K, float alpha, const float *A, int lda, const float *B, int ldb,
             float beta, float *C, int ldc, void *stream) {
  B2_REQUIRE(path == B2_PATH_FFMA || path == B2_PATH_3XTF32, B2_ERR_INVALID_ARG, "b2_sgemm: unknown path %d", path);
  B2_REQUIRE(M >= 0 && N >= 0 && K >= 0, B2_ERR_INVALID_ARG, "b2_sgemm: negative dimension (M=%d N=%d K=%d)", M, N, K);
  if (M == 0 || N == 0) return B2_OK;
  B2_REQUIRE(C != nullptr, B2_ERR_INVALID_ARG, "b2_sgemm: C is NULL");
  B2_REQUIRE(ldc >= N, B2_ERR_INVALID_ARG, "b2_sgemm: ldc = %d < N = %d", ldc, N);
  if (K > 0) {
    B2_REQUIRE(A != nullptr && B != nullptr, B2_ERR_INVALID_ARG, "b2_sgemm: A or B is NULL");
    B2_REQUIRE(lda >= K, B2_ERR_INVALID_ARG, "b2_sgemm: lda = %d < K = %d", lda, K);
    B2_REQUIRE(ldb >= N, B2_ERR_INVALID_ARG, "b2_sgemm: ldb = %d < N = %d", ldb, N);
  }
  B2_REQUIRE(((((uintptr_t)A | (uintptr_t)B | (uintptr_t)C)) & 3) == 0, B2_ERR_INVALID_ARG, "b2_sgemm: matrices must be 4-byte aligned");
  Context *ctx = h ? (Context *)h : default_context();
  B2_REQUIRE(ctx != nullptr, B2_ERR_CUDA, "b2_sgemm: no context (%s)", b2_last_error());
  if (path == B2_PATH_3XTF32)
    return sgemm_3xtf32_dispatch(ctx, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, (cudaStream_t)stream);
  return sgemm_ffma_dispatch(ctx, 0, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, (cudaStream_t)stream);
}

int sgemm(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C) {
  return b2_sgemm(nullptr, B2_PATH_FFMA, M, N, K, alpha, A, K, B, N, beta, C, N, nullptr);
}

int ref_sgemm_rowmajor(int N, float *A, float *B, float *C, float alpha, float beta) {
  return b2_sgemm(nullptr, B2_PATH_FFMA, N, N, N, alpha, A, N, B, N, beta, C, N, nullptr);
}

}  // extern "C"
