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
//   * 8 warps stacked along M, each spanning 16 rows x 128 columns, lanes as 4 (M) x 8 (N),
//     4 x 16 outputs per thread: the warp tiling idea of kernel_11.cuh:22-27 with a shape
//     chosen for the swizzled A reads and for the packed FMA below.
//   * The inner product uses the packed fma.rn.f32x2 instruction (two FP32 FMAs per issue
//     slot, pairs of adjacent columns); only the 4 A values per k have to be duplicated into
//     both halves of an operand.  Per output the arithmetic is still one FMA per k in
//     ascending k, so results are bit-identical to the scalar form (kept as a variant).
//     The K-slab body is fully unrolled: shorter unrolled bodies and register-free schemes
//     for the duplication (a per-warp shared region of (a,a) pairs) both measured slower.
// Each output element is accumulated by exactly one thread in ascending k with one FMA per
// k, and the epilogue is fma(alpha, acc, beta*c) (alpha*acc when beta == 0; C is then not
// read).
#include <stdlib.h>

#include "common.cuh"

namespace b2 {

constexpr int FBM = 128, FBN = 128, FBK = 32, FSTAGES = 3;
constexpr int kStageA = FBM * FBK * 4;  // 16 KB, 128 rows of 128 bytes, 128B-swizzled
constexpr int kStageB = FBK * FBN * 4;  // 16 KB, 32 rows of 512 bytes, linear
constexpr int kFfmaSmem = 1024 + FSTAGES * (kStageA + kStageB) + 1024;
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

__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

struct FfmaArgs {
  float *C;
  int M, N, K, ldc;
  float alpha, beta;
  int vec_c;    // C rows are 16-byte aligned: 128-bit epilogue
  int *status;  // device status word: set to B2_ERR_TIMEOUT if a bounded wait runs out
};

// Accumulators of one thread: 4 rows x 16 columns (a wide tile keeps the number of A values that
// must be duplicated into both halves of a packed operand at 4 per k).  Row i is tile row
// warp*16 + lm + 4*i (row-major A) or warp*16 + lm*4 + i (transposed A); column j is tile
// column ln*4 + 32*(j/4) + j%4, so one warp spans all 128 columns of 16 rows.
template <bool PACKED>
struct Acc;
template <>
struct Acc<false> {
  float v[4][16];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 16; ++j) v[i][j] = 0.f;
  }
  __device__ __forceinline__ void step(const float (&a)[4], const float4 (&b)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        v[i][4 * q + 0] = __fmaf_rn(a[i], b[q].x, v[i][4 * q + 0]);
        v[i][4 * q + 1] = __fmaf_rn(a[i], b[q].y, v[i][4 * q + 1]);
        v[i][4 * q + 2] = __fmaf_rn(a[i], b[q].z, v[i][4 * q + 2]);
        v[i][4 * q + 3] = __fmaf_rn(a[i], b[q].w, v[i][4 * q + 3]);
      }
  }
  __device__ __forceinline__ float get(int i, int j) const { return v[i][j]; }
  __device__ __forceinline__ void set(int i, int j, float x) { v[i][j] = x; }
};
template <>
struct Acc<true> {
  uint64_t v[4][8];  // pairs of adjacent columns
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0ull;
  }
  __device__ __forceinline__ void step(const float (&a)[4], const float4 (&b)[4]) {
    uint64_t bp[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      bp[2 * q] = pack2(b[q].x, b[q].y);
      bp[2 * q + 1] = pack2(b[q].z, b[q].w);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint64_t aa = pack2(a[i], a[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = ffma2(aa, bp[j], v[i][j]);
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

// Tile row of accumulator row i of a thread (see Acc) and tile column of accumulator column j.
template <bool TRANS_A>
__device__ __forceinline__ int acc_row(int warp, int lm, int i) {
  return TRANS_A ? (warp * 16 + lm * 4 + i) : (warp * 16 + lm + 4 * i);
}
__device__ __forceinline__ int acc_col(int ln, int j) { return ln * 4 + 32 * (j >> 2) + (j & 3); }

// ---- ABFT additions (FT = true) ----------------------------------------------------------
// Checksum algebra of kernel/ft_sgemm/README.md:4-14 per 128x128 output tile T = A_t * B_t:
//   row checksum   T e   = A_t (B_t e)      one value per tile row
//   col checksum   e^T T = (e^T A_t) B_t    one value per tile column
// Encoding happens slab by slab inside the mainloop, on the shared-memory stage the FMAs are
// about to consume (the reference encodes from the registers it prefetched,
// kernel/ft_sgemm/include/ft_sgemm_tall.cuh:178-267):
//   phase 1 (before the FMAs of the slab): warp w sums k-chunk w of the A slab over the 128
//           rows and rows 4w..4w+3 of the B slab over the 128 columns -> 32 + 32 slab sums in
//           shared memory, announced on a split-phase mbarrier;
//   phase 2 (after the FMAs, when every warp's sums have long arrived): threads 0..127 add
//           sum_k A[row][k] * Bsum[k] to their row checksum, threads 128..255 add
//           Asum[k] * B[k][4 columns] for 8 k to their partial column checksums.
// The epilogue compares the checksums with the row and column sums of the accumulators
// (the reference does this every 256 of K, ft_sgemm_huge.cuh:143-271); a single row and a
// single column out of tolerance locate the faulty accumulator, which is rebuilt as
// row checksum - (sum of the other accumulators of that row).
struct FtArgs {
  const b2_fault *plan;
  int n_faults;
  float tau;
  int *report;  // b2_ft_report as ints: tiles, injected, detected, corrected, uncorrectable
};

constexpr int kFtBarOff = FSTAGES * (kStageA + kStageB);  // full[3], empty[3], sums_ready[3]
constexpr int kFtSumOff = kFtBarOff + 128;                // float2 sAc[3][32] (each sum twice), float sBr[3][32]
constexpr int kFtInjOff = kFtSumOff + 3 * FSTAGES * 32 * 4;  // int inj[8]

template <bool PACKED, int KCU, bool TRANS_A, bool FT>
__global__ void __launch_bounds__(256, 2)
sgemm_ffma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const FfmaArgs p,
                  const FtArgs ft) {
  static_assert(!(FT && TRANS_A), "the ABFT encoder reads the row-major A stage");
  extern __shared__ unsigned char smem_raw[];
  // round the dynamic shared window up to 1024 bytes without leaving the shared address space
  unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char *sA = smem;
  unsigned char *sB = smem + FSTAGES * kStageA;
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + kFtBarOff);
  uint64_t *empty = full + FSTAGES;
  uint64_t *sums_ready = empty + FSTAGES;
  unsigned char *sAc = smem + kFtSumOff;               // [stage][32] column sums of the A slab, as (s,s) pairs
  unsigned char *sBr = sAc + FSTAGES * 256;            // [stage][32] row sums of the B slab
  int *inj = reinterpret_cast<int *>(smem + kFtInjOff);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int lm = lane >> 3, ln = lane & 7;
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
      if (FT) mbar_init(&sums_ready[s], 8);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (FT && warp == 1) {
    // first planned fault that names this tile (a plan holds at most one per tile)
    int found = 0x7fffffff;
    for (int f = lane; f < ft.n_faults; f += 32)
      if (ft.plan[f].tile_m == tile_m && ft.plan[f].tile_n == tile_n && f < found) found = f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) found = min(found, __shfl_xor_sync(0xffffffffu, found, o));
    if (lane == 0) {
      inj[0] = (found != 0x7fffffff);
      if (inj[0]) {
        inj[1] = ft.plan[found].row;
        inj[2] = ft.plan[found].col;
        inj[3] = ft.plan[found].k_step;
        inj[4] = ft.plan[found].bit;
      }
    }
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

  // planned fault: which slab, and (for the owning thread only) which accumulator
  int inj_kb = -1;  // slab after which this thread flips a bit (-1: never); the rest is re-read from inj[]
  if (FT && inj[0]) {
    const int r = inj[1], c = inj[2];
    const bool own = r >= 0 && r < FBM && c >= 0 && c < FBN && (r >> 4) == warp && (r & 3) == lm && ((c & 31) >> 2) == ln;
    if (own) {
      inj_kb = inj[3] < 0 ? 0 : (inj[3] >= nkb ? nkb - 1 : inj[3]);
    }
  }

  Acc<PACKED> acc;
  acc.zero();
  // Byte offsets inside a stage.  A: row r at r*128, 16-byte chunk c of that row at
  // ((c ^ (r & 7)) << 4); rows of this thread are warp*16 + lm + 4*i, so r & 7 is lm for even
  // i and lm + 4 for odd i.  B: row k at k*512, column c at c*4.
  const uint32_t a_thread = TRANS_A ? (uint32_t)(warp * 16 + lm * 4) * 4u : (uint32_t)(warp * 16 + lm) * 128u;
  const uint32_t a_swz = (uint32_t)lm << 4;
  const uint32_t b_thread = (uint32_t)(ln * 4) * 4u;
  // ABFT: per-thread byte offsets of the encoder, fixed for the whole kernel
  const uint32_t p1a_off = (uint32_t)lane * 128u + (uint32_t)((warp ^ (lane & 7)) << 4);   // A: rows lane+32q, k-chunk = warp
  const uint32_t p1b_off = (uint32_t)(warp * 4 + (lane >> 3)) * 512u + (uint32_t)(lane & 7) * 16u;  // B: row 4*warp + lane/8
  const uint32_t p2_off = (warp < 4) ? (uint32_t)tid * 128u : (uint32_t)(((tid - 128) >> 5) * 8) * 512u + (uint32_t)((tid - 128) & 31) * 16u;
  uint64_t chk2[2] = {0ull, 0ull};  // FT: packed running checksums (row: 2 pairs folded at the end; column: 4 columns)
  bool ok = true;

  for (int kb = 0; kb < nkb; ++kb) {
    const int s = kb % FSTAGES;
    const uint32_t parity = (uint32_t)(kb / FSTAGES) & 1u;
    if (!mbar_wait(&full[s], parity)) {
      ok = false;
      break;
    }
    const unsigned char *Ast = sA + s * kStageA;
    const unsigned char *Bst = sB + s * kStageB;
    if (FT) {
      // ---- phase 1: slab sums (packed adds; offsets precomputed) ----
      const unsigned char *pa_ptr = Ast + p1a_off;
      ulonglong2 v0 = *reinterpret_cast<const ulonglong2 *>(pa_ptr);
      ulonglong2 v1 = *reinterpret_cast<const ulonglong2 *>(pa_ptr + 32 * 128);
      ulonglong2 v2 = *reinterpret_cast<const ulonglong2 *>(pa_ptr + 64 * 128);
      ulonglong2 v3 = *reinterpret_cast<const ulonglong2 *>(pa_ptr + 96 * 128);
      const uint64_t pxy = fadd2(fadd2(v0.x, v1.x), fadd2(v2.x, v3.x));
      const uint64_t pzw = fadd2(fadd2(v0.y, v1.y), fadd2(v2.y, v3.y));
      float px, py, pz, pw;
      unpack2(pxy, px, py);
      unpack2(pzw, pz, pw);
      // 4 components x 32 lanes -> 4 totals: halve the live components while folding lanes
      const bool h16 = (lane & 16) != 0, h8 = (lane & 8) != 0;
      float k0 = h16 ? pz : px, k1 = h16 ? pw : py;
      k0 += __shfl_xor_sync(0xffffffffu, h16 ? px : pz, 16);
      k1 += __shfl_xor_sync(0xffffffffu, h16 ? py : pw, 16);
      float ka = h8 ? k1 : k0;
      ka += __shfl_xor_sync(0xffffffffu, h8 ? k0 : k1, 8);
      ka += __shfl_xor_sync(0xffffffffu, ka, 4);
      ka += __shfl_xor_sync(0xffffffffu, ka, 2);
      ka += __shfl_xor_sync(0xffffffffu, ka, 1);
      if ((lane & 7) == 0)
        *reinterpret_cast<float2 *>(sAc + s * 256 + (warp * 4 + (h16 ? 2 : 0) + (h8 ? 1 : 0)) * 8) = make_float2(ka, ka);
      const unsigned char *pb_ptr = Bst + p1b_off;
      v0 = *reinterpret_cast<const ulonglong2 *>(pb_ptr);
      v1 = *reinterpret_cast<const ulonglong2 *>(pb_ptr + 128);
      v2 = *reinterpret_cast<const ulonglong2 *>(pb_ptr + 256);
      v3 = *reinterpret_cast<const ulonglong2 *>(pb_ptr + 384);
      const uint64_t sb2 = fadd2(fadd2(fadd2(v0.x, v0.y), fadd2(v1.x, v1.y)), fadd2(fadd2(v2.x, v2.y), fadd2(v3.x, v3.y)));
      float sbx, sby;
      unpack2(sb2, sbx, sby);
      float sb = sbx + sby;
      sb += __shfl_xor_sync(0xffffffffu, sb, 1);
      sb += __shfl_xor_sync(0xffffffffu, sb, 2);
      sb += __shfl_xor_sync(0xffffffffu, sb, 4);
      if ((lane & 7) == 0) *reinterpret_cast<float *>(sBr + s * 128 + (warp * 4 + (lane >> 3)) * 4) = sb;
      __syncwarp();
      if (lane == 0) mbar_arrive(&sums_ready[s]);
    }
    const unsigned char *As = Ast + a_thread;
    const unsigned char *Bs = Bst + b_thread;
    if (TRANS_A) {
#pragma unroll(KCU * 4)
      for (int k = 0; k < FBK; ++k) {
        const float4 a4 = *reinterpret_cast<const float4 *>(As + k * 512);
        float4 b[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) b[q] = *reinterpret_cast<const float4 *>(Bs + k * 512 + q * 128);
        const float a[4] = {a4.x, a4.y, a4.z, a4.w};
        acc.step(a, b);
      }
    } else {
#pragma unroll(KCU)
      for (int kc = 0; kc < FBK / 4; ++kc) {
        const uint32_t y0 = ((uint32_t)kc << 4) ^ a_swz, y1 = y0 ^ 64u;
        float4 a4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          a4[i] = *reinterpret_cast<const float4 *>(As + ((i & 1) ? y1 : y0) + i * 512);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          float4 b[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) b[q] = *reinterpret_cast<const float4 *>(Bs + (kc * 4 + kk) * 512 + q * 128);
          float a[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) a[i] = (kk == 0) ? a4[i].x : (kk == 1) ? a4[i].y : (kk == 2) ? a4[i].z : a4[i].w;
          acc.step(a, b);
        }
      }
    }
    if (FT) {
      // ---- phase 2: fold the slab sums into the running checksums ----
      if (!mbar_wait(&sums_ready[s], parity)) {
        ok = false;
        break;
      }
      if (warp < 4) {
        // row checksum of tile row tid: sum_k A[tid][k] * Bsum[k], two packed chains
        const unsigned char *Arow = Ast + p2_off;
        const uint32_t sw = (uint32_t)(tid & 7) << 4;
        const unsigned char *br = sBr + s * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const ulonglong2 a = *reinterpret_cast<const ulonglong2 *>(Arow + (((uint32_t)c << 4) ^ sw));
          const ulonglong2 b = *reinterpret_cast<const ulonglong2 *>(br + c * 16);
          chk2[0] = ffma2(a.x, b.x, chk2[0]);
          chk2[1] = ffma2(a.y, b.y, chk2[1]);
        }
      } else {
        // partial checksums of 4 columns over 8 k: Asum[k] * B[k][4 columns]
        const unsigned char *Bcol = Bst + p2_off;
        const unsigned char *ac = sAc + s * 256 + ((tid - 128) >> 5) * 64;
#pragma unroll
        for (int kk = 0; kk < 8; kk += 2) {
          const ulonglong2 a2 = *reinterpret_cast<const ulonglong2 *>(ac + kk * 8);  // (s_k, s_k, s_k+1, s_k+1)
          const ulonglong2 b0 = *reinterpret_cast<const ulonglong2 *>(Bcol + kk * 512);
          const ulonglong2 b1 = *reinterpret_cast<const ulonglong2 *>(Bcol + (kk + 1) * 512);
          chk2[0] = ffma2(a2.x, b0.x, chk2[0]);
          chk2[1] = ffma2(a2.x, b0.y, chk2[1]);
          chk2[0] = ffma2(a2.y, b1.x, chk2[0]);
          chk2[1] = ffma2(a2.y, b1.y, chk2[1]);
        }
      }
      // ---- simulated soft error: flip one bit of one accumulator after this slab ----
      if (kb == inj_kb) {
        const int inj_i = (inj[1] & 15) >> 2, inj_j = (inj[2] >> 5) * 4 + (inj[2] & 3);
        const uint32_t inj_mask = 1u << (inj[4] & 31);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (i == inj_i && j == inj_j) acc.set(i, j, __uint_as_float(__float_as_uint(acc.get(i, j)) ^ inj_mask));
        atomicAdd(&ft.report[1], 1);
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

  if (FT) {
    // ---- verify, locate, correct (raw accumulators, before alpha/beta) ----
    __syncthreads();  // every stage has been consumed by every warp: the ring is scratch now
    float *scr = reinterpret_cast<float *>(sA);
    float *rowsum_s = scr;            // [128]     row sums (a warp spans all columns of its rows)
    float *colsum_s = scr + 128;      // [8][128]  partial column sums, one per warp
    float *rowchk_s = scr + 1152;     // [128]
    float *colchk_s = scr + 1280;     // [4][128]  partial column checksums, one per k-group
    float *fix_part = scr + 1792;     // [8]
    int *flags = reinterpret_cast<int *>(scr + 1800);  // nbad_r, nbad_c, bad_r, bad_c
    float rs[4], cs[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) rs[i] = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) cs[j] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float v = acc.get(i, j);
        rs[i] += v;
        cs[j] += v;
      }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      rs[i] += __shfl_xor_sync(0xffffffffu, rs[i], 1);
      rs[i] += __shfl_xor_sync(0xffffffffu, rs[i], 2);
      rs[i] += __shfl_xor_sync(0xffffffffu, rs[i], 4);
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      cs[j] += __shfl_xor_sync(0xffffffffu, cs[j], 8);
      cs[j] += __shfl_xor_sync(0xffffffffu, cs[j], 16);
    }
    if (ln == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) rowsum_s[acc_row<TRANS_A>(warp, lm, i)] = rs[i];
    }
    if (lm == 0) {
#pragma unroll
      for (int j = 0; j < 16; ++j) colsum_s[warp * 128 + acc_col(ln, j)] = cs[j];
    }
    {
      float c0, c1, c2, c3;
      unpack2(chk2[0], c0, c1);
      unpack2(chk2[1], c2, c3);
      if (warp < 4) {
        rowchk_s[tid] = (c0 + c1) + (c2 + c3);
      } else {
        const int j = tid - 128, cg = j & 31, kg = j >> 5;
        *reinterpret_cast<float4 *>(&colchk_s[kg * 128 + cg * 4]) = make_float4(c0, c1, c2, c3);
      }
    }
    if (tid < 4) flags[tid] = 0;
    __syncthreads();
    {
      float actual, expect;
      if (tid < 128) {
        actual = rowsum_s[tid];
        expect = rowchk_s[tid];
      } else {
        const int c = tid - 128;
        actual = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) actual += colsum_s[w * 128 + c];
        expect = (colchk_s[c] + colchk_s[128 + c]) + (colchk_s[256 + c] + colchk_s[384 + c]);
      }
      if (!(fabsf(actual - expect) <= ft.tau)) {  // NaN-safe: a NaN difference counts as out of tolerance
        atomicAdd(&flags[tid < 128 ? 0 : 1], 1);
        flags[tid < 128 ? 2 : 3] = tid & 127;
      }
    }
    __syncthreads();
    const int nbad_r = flags[0], nbad_c = flags[1];
    if (nbad_r | nbad_c) {  // uniform over the block
      if (nbad_r == 1 && nbad_c == 1) {
        const int br = flags[2], bc = flags[3];
        const bool own_row = (br >> 4) == warp && (br & 3) == lm;
        const int bi = (br & 15) >> 2;
        const bool own_col = own_row && ((bc & 31) >> 2) == ln;
        const int bj = (bc >> 5) * 4 + (bc & 3);
        if (own_row) {
          float part = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (i == bi && !(own_col && j == bj)) part += acc.get(i, j);
          fix_part[ln] = part;
        }
        __syncthreads();
        if (own_col) {
          float others = 0.f;
#pragma unroll
          for (int q = 0; q < 8; ++q) others += fix_part[q];
          const float rebuilt = rowchk_s[br] - others;
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (i == bi && j == bj) acc.set(i, j, rebuilt);
          atomicAdd(&ft.report[2], 1);
          atomicAdd(&ft.report[3], 1);
        }
      } else if (tid == 0) {
        if (nbad_r >= 1 && nbad_c >= 1) atomicAdd(&ft.report[2], 1);
        atomicAdd(&ft.report[4], 1);
      }
    }
    if (tid == 0) atomicAdd(&ft.report[0], 1);
  }

  // Epilogue straight from registers: per row, 8 lanes x 16 bytes = 128 contiguous bytes per store.
  const bool read_c = (p.beta != 0.f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = m0 + acc_row<TRANS_A>(warp, lm, i);
    if (row >= p.M) continue;
    float *crow = p.C + (size_t)row * p.ldc;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const int col = n0 + ln * 4 + 32 * h;
      if (p.vec_c && col + 3 < p.N) {
        float4 o;
        if (read_c) {
          const float4 c = *reinterpret_cast<const float4 *>(crow + col);
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
    g_ffma_variant = e ? atoi(e) : 1;
    if (g_ffma_variant < 0 || g_ffma_variant > 1) g_ffma_variant = 1;
  }
  return g_ffma_variant;
}

template <bool PACKED, int KCU, bool TRANS_A, bool FT = false>
static int launch_ffma(const CUtensorMap &ta, const CUtensorMap &tb, const FfmaArgs &args, int grid, cudaStream_t s,
                       const FtArgs &ft = FtArgs{nullptr, 0, 0.f, nullptr}) {
  static bool configured = false;
  if (!configured) {
    B2_CUDA(cudaFuncSetAttribute(sgemm_ffma_kernel<PACKED, KCU, TRANS_A, FT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFfmaSmem));
    B2_CUDA(cudaFuncSetAttribute(sgemm_ffma_kernel<PACKED, KCU, TRANS_A, FT>, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    configured = true;
  }
  sgemm_ffma_kernel<PACKED, KCU, TRANS_A, FT><<<grid, 256, kFfmaSmem, s>>>(ta, tb, args, ft);
  B2_CUDA(cudaGetLastError());
  return B2_OK;
}

int sgemm_ffma_dispatch_ft(Context *ctx, int trans_a, int M, int N, int K, float alpha, const float *A, int lda,
                           const float *B, int ldb, float beta, float *C, int ldc, const FtArgs *ft, cudaStream_t s);

// trans_a = 0: A is M x K row-major (lda >= K).  trans_a = 1: A is given as K x M row-major
// (lda >= M), i.e. the column-major M x K operand of the kernel/ft_sgemm family.
int sgemm_ffma_dispatch(Context *ctx, int trans_a, int M, int N, int K, float alpha, const float *A, int lda,
                        const float *B, int ldb, float beta, float *C, int ldc, cudaStream_t s) {
  return sgemm_ffma_dispatch_ft(ctx, trans_a, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, nullptr, s);
}

// ft == nullptr: plain SGEMM.  Otherwise the ABFT kernel (row-major A only; operands must be
// describable to TMA, i.e. 16-byte aligned with leading dimensions that are multiples of 4).
int sgemm_ffma_dispatch_ft(Context *ctx, int trans_a, int M, int N, int K, float alpha, const float *A, int lda,
                           const float *B, int ldb, float beta, float *C, int ldc, const FtArgs *ft, cudaStream_t s) {
  if (M == 0 || N == 0) return B2_OK;
  if (K == 0 || alpha == 0.f) {
    if (beta == 1.f) return B2_OK;
    scale_c_kernel<<<ctx->sm_count * 4, 256, 0, s>>>(M, N, beta, C, ldc);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
  }
  const bool tma_ok = ((((uintptr_t)A | (uintptr_t)B) & 15) == 0) && (lda % 4 == 0) && (ldb % 4 == 0);
  (void)trans_a;
  if (ft) {
    B2_REQUIRE(tma_ok && !trans_a, B2_ERR_UNSUPPORTED,
               "ft_sgemm: A and B must be 16-byte aligned with lda, ldb multiples of 4 (lda=%d ldb=%d)", lda, ldb);
  }
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
  const bool packed = ffma_variant() != 0;
  if (ft) return launch_ffma<true, 8, false, true>(ta, tb, args, grid, s, *ft);
  if (trans_a) return packed ? launch_ffma<true, 8, true>(ta, tb, args, grid, s) : launch_ffma<false, 8, true>(ta, tb, args, grid, s);
  return packed ? launch_ffma<true, 8, false>(ta, tb, args, grid, s) : launch_ffma<false, 8, false>(ta, tb, args, grid, s);
}

}  // namespace b2

using namespace b2;

namespace b2 {
int sgemm_3xtf32_dispatch(Context *ctx, int M, int N, int K, float alpha, const float *A, int lda, const float *B, int ldb,
                          float beta, float *C, int ldc, cudaStream_t s);
}

extern "C" {

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
  B2_REQUIRE(path == B2_PATH_FFMA, B2_ERR_UNSUPPORTED, "b2_ft_sgemm: ABFT is built on the FFMA path only");
  Context *ctx = h ? (Context *)h : default_context();
  B2_REQUIRE(ctx != nullptr, B2_ERR_CUDA, "b2_ft_sgemm: no context (%s)", b2_last_error());
  FtArgs ft;
  ft.plan = plan_dev;
  ft.n_faults = n_faults;
  // default threshold: 2e-6 per unit of K for operands of unit scale, about 16 sigma of the
  // rounding noise between the two ways the checksums are summed
  ft.tau = tau > 0.f ? tau : fmaxf(2e-6f * (float)K, 4e-5f);
  ft.report = report_dev ? (int *)report_dev : (int *)((char *)ctx->fixed + kFixedFtReport);
  return sgemm_ffma_dispatch_ft(ctx, 0, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, &ft, (cudaStream_t)stream);
}

int ft_sgemm(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C) {
  return b2_ft_sgemm(nullptr, B2_PATH_FFMA, M, N, K, alpha, A, K, B, N, beta, C, N, nullptr, 0, 0.f, nullptr, nullptr);
}

// Selects the inner-loop variant of the FFMA kernel (0 scalar FFMA, 1 packed f32x2).  For
// benchmarking; results are bit-identical.
int b2_set_ffma_variant(int v) {
  B2_REQUIRE(v >= 0 && v <= 1, B2_ERR_INVALID_ARG, "b2_set_ffma_variant: %d not in 0..1", v);
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
