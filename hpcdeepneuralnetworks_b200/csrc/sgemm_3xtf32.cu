// 3xTF32 split-precision SGEMM on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// The reference has no tensor-core path (every kernel of kernel/sgemm is FP32 FFMA); this
// path computes the same row-major C = alpha*A*B + beta*C with FP32-level accuracy:
//     x = hi + lo,  hi = tf32(x), lo = tf32(x - hi)          (round to nearest)
//     A*B ~= A_lo*B_hi + A_hi*B_lo + A_hi*B_hi               (lo*lo dropped, ~2^-22)
// Three tcgen05.mma.kind::tf32 per K-step accumulate into one FP32 accumulator tile in TMEM,
// small terms first.
//
// Kernels:
//   split_planes_kernel      one pass over A and B writing the hi/lo planes (low 13 mantissa
//   split_planes_t_kernel    bits already zero, so the tensor core's own treatment of them is
//                            irrelevant) into the workspace.  B is written transposed (N x K) so
//                            that both operands are K-major under the 128-byte swizzle.
//   sgemm_3xtf32_kernel      one 128 x 256 (or 128 x 128) output tile per CTA, K-slabs of 32; warp 0 =
//                            TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2..5 =
//                            epilogue (tcgen05.ld -> alpha/beta -> global).  2-stage ring of
//                            96 KB (A_hi, A_lo: 128x32; B_hi, B_lo: 256x32), all tiles under the
//                            128-byte swizzle.
//   sgemm_3xtf32_pair_kernel one 256 x 256 tile per cluster of two CTAs (tcgen05 cta_group::2): each CTA
//                            stages half of the A rows and half of the B columns (64 KB per slab, 3
//                            stages), the leader issues MMAs of M = 256 over both CTAs' tiles.  The
//                            form chosen for large problems; same warp roles, same epilogue.
//   sgemm_3xtf32_pair_persistent_kernel  as many clusters as the device holds, each walking several 256 x 256
//                            tiles with the accumulator double-buffered in tensor memory; plain (K <= 1024)
//                            and ABFT (CUDA-core checksums) forms.
//   sgemm_3xtf32_pair_chunked_kernel, sgemm_3xtf32_chunked_kernel  the default for plain calls with K > 1024:
//                            the K loop in chunks of 16 slabs whose sums the epilogue warps add up in FP32
//                            registers (bounds the tensor cores' truncation loss whatever K), C in and out by
//                            TMA; the pair form is persistent and cuts a partial last round of tiles along K
//                            (tf32_tail_fixup_kernel adds the runs).
//   sgemm_3xtf32_fused_kernel  very small products: the split inside the GEMM kernel (raw tiles by TMA, converted in
//                            shared memory by the warps that later run the epilogue); one launch, no workspace.
// The one-tile kernels and the persistent kernel have ABFT forms with the checksums on the CUDA cores (template
// FT); verification and repair sit in the shared epilogue.
// Every wait is bounded; a wait that runs out sets the status word, TMEM is still freed.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>

#include "common.cuh"

namespace b2 {

constexpr int TBM = 128;
// Two tile widths: 128 x 256 and 128 x 128 (for problem sizes whose 128 x 256 tile grid fills the
// last wave of 148 SMs badly).  K-slab depth TBK: 32 floats = one 128-byte swizzled row, or 16
// floats = one 64-byte swizzled row; the shallower slab doubles the number of stages that fit
// (more TMA bytes in flight for the same shared memory).
//
// FT adds ABFT.  A checksum covers one row of a group of 32 output columns: with s_g[k] = sum_{j<32} B[k][32g + j]
// (the plane S, 8 rows of plain FP32 sums per 256-column tile, written by the transposing split pre-pass),
// sum_j C[i][32g + j] = sum_k A[i][k] * s_g[k].  The checksums are formed on the CUDA cores: checksum warps read each
// stage next to the MMAs (their rows of A_hi and A_lo, all of S) and keep chk_g += (a_hi + a_lo) * s_g[k] for the 8
// groups in registers -- no extra MMA, a few percent of time.  An exact checksum does not follow the truncation of
// the tensor cores' accumulators, whose sum over a group falls short of it by a fraction of what the group held
// during the K loop; the checksum warps therefore also keep the sum over the slabs of each running checksum, and the
// epilogue expects the shortfall (tf32_epilogue).  That brings the clean residual from 5.9e-6*K down to 4e-7*K at
// K = 8192 and lets the default threshold sit at half the path's accuracy bound.  (An earlier form multiplied a
// split copy of S by the A tiles on the tensor cores, two more small MMAs per K-step: +20-30 % time and a residual
// of 2.2e-6*K, above what the bound allows; it was removed.)
constexpr int kFtCuda = 2;    // the value of the FT template parameter of the ABFT instantiations (0: plain)
// Measured on B200: every 32-deep K-slab (twelve MMAs) costs an accumulator about 4e-7 of its value (the hardware
// adds an MMA's products to the accumulator with truncation); the best fit is the same for uniform and normal
// operands of any scale and any K from 256 to 8192.
constexpr float kFtBiasPerSlab = 4e-7f;
template <int TBN, int TBK, int FT = 0>
struct Tf32Cfg {
  static constexpr int kTA = TBM * TBK * 4;          // bytes per A plane tile
  static constexpr int kTB = TBN * TBK * 4;          // bytes per B plane tile
  static constexpr int kTS = FT ? 8 * TBK * 4 : 0;  // bytes per checksum tile
  static constexpr int kStage = 2 * kTA + 2 * kTB + kTS;
  static constexpr int kStages = ((FT ? 208 : 192) * 1024) / kStage;
  static constexpr int kSmem = 1024 + kStages * kStage + 256 + (FT == kFtCuda ? 8192 : 0);   // + checksum table
  static constexpr int kTmemCols = TBN;             // FP32 accumulator: one TMEM column per output column
  static constexpr uint32_t kSwizzle = (TBK == 32) ? 2u : 4u;   // descriptor layout type: 128-byte / 64-byte swizzle
  static constexpr uint32_t kSbo = 8 * TBK * 4;                 // bytes between 8-row groups
};

__device__ __forceinline__ float tf32_rna(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r & 0xFFFFE000u);
}

// hi/lo planes of a rows x cols row-major matrix (pitch ld) into dense planes of pitch ldp
// (a multiple of 4): one thread per 4 consecutive columns, 128-bit loads when the source allows.
__global__ void __launch_bounds__(256) split_planes_kernel(const float *__restrict__ X, int rows, int cols, int ld,
                                                           float *__restrict__ hi, float *__restrict__ lo, int ldp, int vec) {
  const int c = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (c >= ldp) return;
  for (int r = blockIdx.y; r < rows; r += gridDim.y) {
    const float *src = X + (size_t)r * ld + c;
    float4 x;
    if (vec && c + 3 < cols) {
      x = __ldcs(reinterpret_cast<const float4 *>(src));
    } else {
      x.x = (c + 0 < cols) ? src[0] : 0.f;
      x.y = (c + 1 < cols) ? src[1] : 0.f;
      x.z = (c + 2 < cols) ? src[2] : 0.f;
      x.w = (c + 3 < cols) ? src[3] : 0.f;
    }
    float4 h, l;
    h.x = tf32_rna(x.x); l.x = tf32_rna(x.x - h.x);
    h.y = tf32_rna(x.y); l.y = tf32_rna(x.y - h.y);
    h.z = tf32_rna(x.z); l.z = tf32_rna(x.z - h.z);
    h.w = tf32_rna(x.w); l.w = tf32_rna(x.w - h.w);
    *reinterpret_cast<float4 *>(hi + (size_t)r * ldp + c) = h;
    *reinterpret_cast<float4 *>(lo + (size_t)r * ldp + c) = l;
  }
}

// Transposing variant: X is rows x cols (pitch ld); planes are cols x rows (pitch ldp >= rows,
// a multiple of 4).  Tiles of 128 rows x 64 columns of X through shared memory: reads run 256
// bytes along a row of X, writes 512 bytes along a row of the planes (the writes are two thirds of
// the traffic).
// With S != NULL it also writes the ABFT checksum plane (pitch ldp, 8 rows per 256-column tile): for every row r of
// X and group g of 32 columns inside tile t, S[8t + g][r] = sum_{j<32} X[r][256t + 32g + j].
constexpr int kSplitTK = 128, kSplitTN = 64;
__global__ void __launch_bounds__(256) split_planes_t_kernel(const float *__restrict__ X, int rows, int cols, int ld,
                                                             float *__restrict__ hi, float *__restrict__ lo, int ldp,
                                                             float *__restrict__ S) {
  __shared__ float t[kSplitTK][kSplitTN + 1];
  const int c0 = blockIdx.x * kSplitTN, r0 = blockIdx.y * kSplitTK, tid = threadIdx.x;
#pragma unroll 8
  for (int e = tid; e < kSplitTK * kSplitTN; e += 256) {
    const int rr = e / kSplitTN, cc = e % kSplitTN;
    const int r = r0 + rr, c = c0 + cc;
    t[rr][cc] = (r < rows && c < cols) ? __ldcs(X + (size_t)r * ld + c) : 0.f;
  }
  __syncthreads();
  // A warp takes 4 output rows x 8 quads of k at a time: lane (kq, nn) = (lane & 7, lane >> 3) reads
  // t[4kq + i][nn], 32 distinct banks under the pitch of 65, and each output row gets 128 contiguous bytes.
  {
    const int lane = tid & 31, warp = tid >> 5, kq = lane & 7, nn = lane >> 3;
    for (int w = warp; w < (kSplitTN / 4) * (kSplitTK / 32); w += 8) {
      const int cc = (w / (kSplitTK / 32)) * 4 + nn, rq = ((w % (kSplitTK / 32)) * 8 + kq) * 4;
      const int c = c0 + cc, r = r0 + rq;   // output row c, output columns r .. r+3
      if (c < cols && r < ldp) {
        float4 h, l;
        const float x0 = t[rq + 0][cc], x1 = t[rq + 1][cc], x2 = t[rq + 2][cc], x3 = t[rq + 3][cc];
        h.x = tf32_rna(x0); l.x = tf32_rna(x0 - h.x);
        h.y = tf32_rna(x1); l.y = tf32_rna(x1 - h.y);
        h.z = tf32_rna(x2); l.z = tf32_rna(x2 - h.z);
        h.w = tf32_rna(x3); l.w = tf32_rna(x3 - h.w);
        __stcs(reinterpret_cast<float4 *>(hi + (size_t)c * ldp + r), h);
        __stcs(reinterpret_cast<float4 *>(lo + (size_t)c * ldp + r), l);
      }
    }
  }
  if (S != nullptr) {
    const int rr = tid & (kSplitTK - 1), gg = tid >> 7;   // row r0 + rr of X, columns c0 + 32gg .. +31
    if (r0 + rr < ldp) {
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) sum += t[rr][32 * gg + j];
      const int g = (c0 % 256) / 32 + gg;
      S[((size_t)(c0 / 256) * 8 + g) * ldp + r0 + rr] = sum;
    }
  }
}

struct Tf32Args {
  float *C;
  int M, N, K, ldc;
  float alpha, beta;
  int vec_c;
  int *status;      // [0] sticky status word, [1] number of the launch that aborted (see record_timeout)
  unsigned int seq; // number of this launch on its handle
  FtArgs ft;        // used by the FT instantiations only
  float tau_elem;   // an output further than this from its recomputed value is replaced
  float ft_bias;    // FT = 2: expected loss of an accumulator per K-slab, as a fraction of its value (see tf32_epilogue)
};
// Where an accumulator tile goes and which k it covers: C itself with the call's alpha and beta for a whole tile, or,
// for a run of a tile cut along K, its workspace slot, unscaled, with the run's k range (the ABFT repair recomputes
// over that range only).
struct EpiOut {
  float *C;
  int ldc;
  float alpha, beta;
  int vec_c;
  int k_begin, k_end;
  __device__ __forceinline__ static EpiOut whole(const Tf32Args &p) { return EpiOut{p.C, p.ldc, p.alpha, p.beta, p.vec_c, 0, p.K}; }
};

// FP32 dot product of row `row` of A with column col0 + lane of B, from global memory (two
// interleaved chains over K).  Called by whole warps.
__device__ __forceinline__ float ft_recompute32(const Tf32Args &p, int k_begin, int k_end, int row, int col0, int lane) {
  const int col = col0 + lane;
  float acc0 = 0.f, acc1 = 0.f;
  if (row < p.M && col < p.N) {
    const float *a = p.ft.A + (size_t)row * p.ft.lda;
    const float *b = p.ft.B + col;
    int k = k_begin;
    const int kend = k_end;
    for (; k + 1 < kend; k += 2) {
      acc0 = __fmaf_rn(a[k], b[(size_t)k * p.ft.ldb], acc0);
      acc1 = __fmaf_rn(a[k + 1], b[(size_t)(k + 1) * p.ft.ldb], acc1);
    }
    if (k < kend) acc0 = __fmaf_rn(a[k], b[(size_t)k * p.ft.ldb], acc0);
  }
  return acc0 + acc1;
}

// Planned faults that land in this thread's row of this tile: at most one per 128 columns.
struct FtInj {
  int col0 = -1, col1 = -1;
  uint32_t mask0 = 0u, mask1 = 0u;
};
template <int TBN>
__device__ __forceinline__ FtInj ft_scan_plan(const Tf32Args &p, int my_row, int n0) {
  FtInj inj;
  for (int f = 0; f < p.ft.n_faults; ++f) {
    const b2_fault ff = p.ft.plan[f];
    const int gr = ff.tile_m * 128 + ff.row, gc = ff.tile_n * 128 + ff.col;
    if (gr == my_row && gr < p.M && gc >= n0 && gc < n0 + TBN && gc < p.N) {
      if (gc - n0 < 128) {
        if (inj.col0 < 0) { inj.col0 = gc - n0; inj.mask0 = 1u << (ff.bit & 31); }
      } else if (inj.col1 < 0) {
        inj.col1 = gc - n0; inj.mask1 = 1u << (ff.bit & 31);
      }
    }
  }
  return inj;
}

// CUDA-core checksums (FT = 2).  A warp owns 32 tile rows; lane (rb, kc) = (lane >> 3, lane & 7)
// takes rows rb + 4i (i = 0..7) and the four k of 16-byte chunk kc of each K-slab, so that a warp
// reads every A row once (8 lanes x 16 bytes = one 128-byte row, conflict-free) and S once per
// lane octet, and keeps 8 rows x 8 groups of partial sums in registers for the whole K loop.
// The tiles are K-major under the 128-byte swizzle: chunk j of row x sits at chunk j ^ (x & 7).
template <int RPL = 8>
struct FtCudaAcc {
  float v[RPL][8];   // [row i][group g]: running checksum
  float r[RPL][8];   // sum over the K-slabs so far of the running checksum (see tf32_epilogue: bias model)
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < RPL; ++i)
#pragma unroll
      for (int g = 0; g < 8; ++g) v[i][g] = r[i][g] = 0.f;
  }
};
// One K-slab: a warp covers 4 * RPL tile rows from row0 on; lane (rb, kc) takes rows row0 + rb + 4i, i < RPL.
template <int RPL>
__device__ __forceinline__ void ft_cuda_slab(const unsigned char *a_hi, const unsigned char *a_lo, const unsigned char *sg,
                                             int row0, int lane, FtCudaAcc<RPL> &acc) {
  const int rb = lane >> 3, kc = lane & 7;
  float4 s4[8];
#pragma unroll
  for (int g = 0; g < 8; ++g) s4[g] = *reinterpret_cast<const float4 *>(sg + g * 128 + ((kc ^ g) << 4));
#pragma unroll
  for (int i = 0; i < RPL; ++i) {
    const int r = row0 + rb + 4 * i;
    const int off = r * 128 + ((kc ^ (r & 7)) << 4);
    const float4 h = *reinterpret_cast<const float4 *>(a_hi + off);
    const float4 l = *reinterpret_cast<const float4 *>(a_lo + off);
    const float a0 = h.x + l.x, a1 = h.y + l.y, a2 = h.z + l.z, a3 = h.w + l.w;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float t = acc.v[i][g];
      t = __fmaf_rn(a0, s4[g].x, t);
      t = __fmaf_rn(a1, s4[g].y, t);
      t = __fmaf_rn(a2, s4[g].z, t);
      t = __fmaf_rn(a3, s4[g].w, t);
      acc.v[i][g] = t;
      acc.r[i][g] += t;
    }
  }
}
// End of the K loop: fold the eight k-chunk lanes of each row and leave, per tile row, the 8 checksums and the 8
// slab sums (less half the checksum: the checksum's mean over the slabs' MMAs) in the warp's rows of the shared
// table (float [128][16]); the epilogue thread of a row reads its own entries.
template <int RPL>
__device__ __forceinline__ void ft_cuda_finish(FtCudaAcc<RPL> &acc, float *table, int row0, int lane) {
  const int rb = lane >> 3, kc = lane & 7;
#pragma unroll
  for (int i = 0; i < RPL; ++i)
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float t = acc.v[i][g], u = acc.r[i][g];
      t += __shfl_xor_sync(0xffffffffu, t, 1);
      u += __shfl_xor_sync(0xffffffffu, u, 1);
      t += __shfl_xor_sync(0xffffffffu, t, 2);
      u += __shfl_xor_sync(0xffffffffu, u, 2);
      t += __shfl_xor_sync(0xffffffffu, t, 4);
      u += __shfl_xor_sync(0xffffffffu, u, 4);
      if (kc == g) {
        table[(row0 + rb + 4 * i) * 16 + g] = t;
        table[(row0 + rb + 4 * i) * 16 + 8 + g] = u - 0.5f * t;
      }
    }
  __syncwarp();
}

// Epilogue of one warp (TMEM lane quarter q): 32 rows x TBN columns of the accumulator tile ->
// alpha/beta -> global.  FT: each 32-column chunk is summed and compared with its two checksum
// columns first; a row-group out of tolerance is recomputed and repaired (see the file header).
// `ok` (warp-uniform) says the accumulator is complete; called by whole warps.
template <int TBN, int FT>
__device__ __forceinline__ void tf32_epilogue(const Tf32Args &p, uint32_t tmem_base, int q, int lane, int m0, int n0, bool ok,
                                              int nkb, const FtInj &inj, const float *chk_row, const EpiOut o_, bool count_tile = true) {
  const int inj_col0 = inj.col0, inj_col1 = inj.col1;
  const uint32_t inj_mask0 = inj.mask0, inj_mask1 = inj.mask1;
  const float tscale = (FT && p.ft.tau_scale) ? __ldg(p.ft.tau_scale) : 1.f;
  const float tau = p.ft.tau * tscale, tau_elem = p.tau_elem * tscale;
  float worst = 0.f;          // largest in-tolerance |group sum - checksum| this thread saw
  int n_inj = 0, n_det = 0, n_cor = 0, n_false = 0;
  const int row = m0 + q * 32 + lane;
  const bool read_c = (o_.beta != 0.f);
  float *crow = o_.C + (size_t)row * o_.ldc;
#pragma unroll 1
  for (int c = 0; c < TBN / 32; ++c) {
    uint32_t v[32];
    float expect = 0.f;
    if (ok && nkb > 0) {
      tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), v);
      if (FT) {
        // The tensor cores add each MMA's products to the accumulator with truncation, which pulls the
        // accumulator toward zero by a fraction of its value that is about the same for every MMA; over the
        // K loop a group of accumulators therefore loses ft_bias times the sum over the slabs of what the
        // group held at the time, and that sum is what the checksum warps kept beside the checksum.
        expect = chk_row[c] - p.ft_bias * chk_row[8 + c];
      }
      tmem_ld_wait();
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = 0u;
    }
    if (FT && ok && nkb > 0) {
      // simulated soft errors: flip one bit of an accumulator as it leaves TMEM
      if (inj_col0 >= 0 && (inj_col0 >> 5) == c) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j == (inj_col0 & 31)) v[j] ^= inj_mask0;
        ++n_inj;
      }
      if (TBN > 128 && inj_col1 >= 0 && (inj_col1 >> 5) == c) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j == (inj_col1 & 31)) v[j] ^= inj_mask1;
        ++n_inj;
      }
      {
        float g = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) g += __uint_as_float(v[j]);
        const float resid = fabsf(g - expect);
        const bool bad = !(resid <= tau);
        if (!bad) worst = fmaxf(worst, resid);
        unsigned m = __ballot_sync(0xffffffffu, bad);
        while (m) {
          const int L = __ffs(m) - 1;
          m &= m - 1;
          const int rowL = __shfl_sync(0xffffffffu, m0 + q * 32 + lane, L);
          const float ref = ft_recompute32(p, o_.k_begin, o_.k_end, rowL, n0 + c * 32, lane);
          int replaced = 0;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float r = __shfl_sync(0xffffffffu, ref, j);
            if (lane == L && !(fabsf(__uint_as_float(v[j]) - r) <= tau_elem)) {
              v[j] = __float_as_uint(r);
              ++replaced;
            }
          }
          if (lane == L) {
            if (replaced) { ++n_det; n_cor += replaced; } else { ++n_false; }
          }
        }
      }
    }
    if (!ok || row >= p.M) continue;
    const int col0 = n0 + c * 32;
    if (o_.vec_c && col0 + 31 < p.N) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 o;
        if (read_c) {
          const float4 cc = *reinterpret_cast<const float4 *>(crow + col0 + j);
          o.x = __fmaf_rn(o_.alpha, __uint_as_float(v[j + 0]), __fmul_rn(o_.beta, cc.x));
          o.y = __fmaf_rn(o_.alpha, __uint_as_float(v[j + 1]), __fmul_rn(o_.beta, cc.y));
          o.z = __fmaf_rn(o_.alpha, __uint_as_float(v[j + 2]), __fmul_rn(o_.beta, cc.z));
          o.w = __fmaf_rn(o_.alpha, __uint_as_float(v[j + 3]), __fmul_rn(o_.beta, cc.w));
        } else {
          o.x = __fmul_rn(o_.alpha, __uint_as_float(v[j + 0]));
          o.y = __fmul_rn(o_.alpha, __uint_as_float(v[j + 1]));
          o.z = __fmul_rn(o_.alpha, __uint_as_float(v[j + 2]));
          o.w = __fmul_rn(o_.alpha, __uint_as_float(v[j + 3]));
        }
        *reinterpret_cast<float4 *>(crow + col0 + j) = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (col0 + j < p.N) {
          const float a = __uint_as_float(v[j]);
          crow[col0 + j] = read_c ? __fmaf_rn(o_.alpha, a, __fmul_rn(o_.beta, crow[col0 + j])) : __fmul_rn(o_.alpha, a);
        }
      }
    }
  }
  if (FT) {
    // one set of atomics per warp
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      n_inj += __shfl_xor_sync(0xffffffffu, n_inj, o);
      n_det += __shfl_xor_sync(0xffffffffu, n_det, o);
      n_cor += __shfl_xor_sync(0xffffffffu, n_cor, o);
      n_false += __shfl_xor_sync(0xffffffffu, n_false, o);
      worst = fmaxf(worst, __shfl_xor_sync(0xffffffffu, worst, o));
    }
    if (lane == 0) {
      if (count_tile && q == 0 && m0 < p.M) atomicAdd(&p.ft.report[0], 1);   // a pair's second CTA may lie wholly below the matrix
      if (n_inj) atomicAdd(&p.ft.report[1], n_inj);
      if (n_det) atomicAdd(&p.ft.report[2], n_det);
      if (n_cor) atomicAdd(&p.ft.report[3], n_cor);
      if (n_false) atomicAdd(&p.ft.report[5], n_false);
      atomicMax(&p.ft.report[6], __float_as_int(worst));
    }
  }
}

template <int TBN, int TBK, int FT>
__global__ void __launch_bounds__(192, 1)
sgemm_3xtf32_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
                    const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
                    const __grid_constant__ CUtensorMap tmS, const Tf32Args p) {
  using Cfg = Tf32Cfg<TBN, TBK, FT>;
  constexpr int TSTAGES = Cfg::kStages, kTA = Cfg::kTA, kTB = Cfg::kTB, kTStage = Cfg::kStage;
  constexpr int kTmemCols = Cfg::kTmemCols;
  extern __shared__ unsigned char smem_raw[];
  // round the dynamic shared window up to 1024 bytes without leaving the shared address space
  unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + TSTAGES * kTStage);
  uint64_t *empty = full + TSTAGES;
  uint64_t *acc_ready = empty + TSTAGES;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_ready + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_n = (p.N + TBN - 1) / TBN;
  const int tile_m = blockIdx.x / tiles_n, tile_n = blockIdx.x % tiles_n;
  const int m0 = tile_m * TBM, n0 = tile_n * TBN;
  const int nkb = (p.K + TBK - 1) / TBK;

  {
    // an earlier CTA of this launch timed out: leave at once (one thread reads, so the whole CTA agrees)
    __shared__ int launch_aborted;
    if (threadIdx.x == 0) launch_aborted = b2::launch_aborted(p.status, p.seq) ? 1 : 0;
    __syncthreads();
    if (launch_aborted != 0) return;
  }
  if (tid == 0) {
    for (int s = 0; s < TSTAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], FT == kFtCuda ? 5 : 1);   // the MMA commit, and the four checksum warps
    }
    mbar_init(acc_ready, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmAh);
    tma_prefetch_desc(&tmAl);
    tma_prefetch_desc(&tmBh);
    tma_prefetch_desc(&tmBl);
    if (FT) tma_prefetch_desc(&tmS);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  uint32_t issued = 0;   // the producer thread: stages it has filled so far

  if (warp == 0) {
    // ---- TMA producer -----------------------------------------------------------------
    if (lane == 0) {
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % TSTAGES;
        if (!mbar_wait(&empty[s], ((uint32_t)(kb / TSTAGES) & 1u) ^ 1u)) {
          *abort_flag = 1;
          break;
        }
        unsigned char *st = smem + s * kTStage;
        mbar_expect_tx(&full[s], kTStage);
        issued = (uint32_t)kb + 1u;
        tma_load_2d(st, &tmAh, &full[s], kb * TBK, m0);
        tma_load_2d(st + kTA, &tmAl, &full[s], kb * TBK, m0);
        {
          tma_load_2d(st + 2 * kTA, &tmBh, &full[s], kb * TBK, n0);
          tma_load_2d(st + 2 * kTA + kTB, &tmBl, &full[s], kb * TBK, n0);
        }
        if (FT == kFtCuda) tma_load_2d(st + 2 * kTA + 2 * kTB, &tmS, &full[s], kb * TBK, tile_n * 8);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_tf32(TBM, TBN, 0, 0);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % TSTAGES;
        if (!mbar_wait(&full[s], (uint32_t)(kb / TSTAGES) & 1u)) {
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t st = smem_u32(smem + s * kTStage);
#pragma unroll
        for (int k4 = 0; k4 < TBK / 8; ++k4) {
          // K-major, 128B swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart; a K-step of
          // 8 floats is 32 bytes further along the row.
          const uint64_t a_hi = umma_smem_desc(st + k4 * 32, 16, Cfg::kSbo, Cfg::kSwizzle);
          const uint64_t a_lo = umma_smem_desc(st + kTA + k4 * 32, 16, Cfg::kSbo, Cfg::kSwizzle);
          const uint64_t b_hi = umma_smem_desc(st + 2 * kTA + k4 * 32, 16, Cfg::kSbo, Cfg::kSwizzle);
          const uint64_t b_lo = umma_smem_desc(st + 2 * kTA + kTB + k4 * 32, 16, Cfg::kSbo, Cfg::kSwizzle);
          umma_tf32(tmem_base, a_lo, b_hi, idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
          umma_tf32(tmem_base, a_hi, b_lo, idesc, 1u);
          umma_tf32(tmem_base, a_hi, b_hi, idesc, 1u);
        }
        umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
      }
      if (ok) umma_commit(acc_ready);
    }
  } else {
    // ---- epilogue: warps 2..5, TMEM lane quarter = warp % 4 -------------------------------
    const int q = warp & 3;
    bool ok = true;
    FtInj inj;
    if (FT) inj = ft_scan_plan<TBN>(p, m0 + q * 32 + lane, n0);
    float *table = reinterpret_cast<float *>(smem + TSTAGES * kTStage + 256);
    if (FT == kFtCuda) {
      // checksums on the CUDA cores: follow the stages next to the MMA issuer
      FtCudaAcc<8> acc;
      acc.zero();
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % TSTAGES;
        if (!mbar_wait(&full[s], (uint32_t)(kb / TSTAGES) & 1u)) {
          *abort_flag = 1;
          break;
        }
        const unsigned char *st = smem + s * kTStage;
        ft_cuda_slab(st, st + kTA, st + 2 * kTA + 2 * kTB, q * 32, lane, acc);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
      }
      ft_cuda_finish(acc, table, q * 32, lane);
    }
    if (nkb > 0) {
      // poll in slices so that an abort raised by the other roles is seen
      bool done = false;
      const uint64_t t0 = global_timer_ns();
      for (int it = 0; it < (1 << 14) && !done; ++it) {
        done = mbar_wait(acc_ready, 0, 1u << 10);
        if (!done && (*abort_flag || global_timer_ns() - t0 > 2000000000ull)) break;
      }
      ok = done;
    }
    ok = __all_sync(0xffffffffu, ok);   // the checksum pass below uses warp collectives
    if (!ok) *abort_flag = 1;
    tc_fence_after();
    tf32_epilogue<TBN, FT>(p, tmem_base, q, lane, m0, n0, ok, nkb, inj, table + (q * 32 + lane) * 16, EpiOut::whole(p));
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {   // the same answer in every thread: read after the barrier
    if (tid == 0) ring_settle(full, TSTAGES, issued);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tid == 0 && *abort_flag) record_timeout(p.status, p.seq);
}

// ---- CTA-pair form: one 256 x 256 output tile per cluster of two CTAs (tcgen05 cta_group::2) ----
// CTA r of the pair stages rows m0 + 128r.. of the A planes and columns n0 + 128r.. of the B planes
// (64 KB per K-slab instead of 96 KB, so three stages fit and each SM pulls a third fewer bytes out
// of L2 per flop); the leader (r = 0) issues MMAs of M = 256 that read both CTAs' tiles and write
// 128 accumulator rows into each CTA's TMEM.  Every TMA load is a plain per-CTA load that signals
// the leader's "full" barrier; the leader's commits free the stage in both CTAs.
// FT: both CTAs stage the tile's S rows; their checksum warps cover their own 128 accumulator rows.
constexpr int kPairBand = 8;   // tile rows per band of the pair kernel's tile order
// End of a pair kernel, after the cluster barrier that follows the roles: if a wait ran out anywhere in the pair
// (the leader's flag is set from both CTAs, and both read it here, so they take the same branch), the leader's
// producer thread lets the loads that signal its "full" barriers land before either CTA leaves.
__device__ __forceinline__ void pair_settle(volatile int *abort_flag, uint64_t *full, int stages, uint32_t issued, uint32_t rank,
                                            int tid) {
  if (ld_shared_cluster_u32(mapa_u32(smem_u32(const_cast<const int *>(abort_flag)), 0)) == 0) return;
  if (rank == 0 && tid == 0) ring_settle(full, stages, issued);
  cluster_sync_all();
}
template <int FT>
struct PairCfg {
  static constexpr int kTA = TBM * 32 * 4;           // bytes per A plane tile (128 rows)
  static constexpr int kTB = 128 * 32 * 4;           // bytes per B plane half tile (128 columns)
  static constexpr int kTS = FT ? 8 * 32 * 4 : 0;    // one S tile
  static constexpr int kStage = 2 * kTA + 2 * kTB + kTS;   // 64 KB (+1 KB)
  static constexpr int kStages = 3;
  static constexpr int kSmem = 1024 + kStages * kStage + 256 + (FT == kFtCuda ? 8192 : 0);   // + checksum table
  static constexpr int kTmemCols = 256;
};

template <int FT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
sgemm_3xtf32_pair_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
                         const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
                         const __grid_constant__ CUtensorMap tmS, const Tf32Args p) {
  using PC = PairCfg<FT>;
  constexpr int S = PC::kStages, kTA = PC::kTA, kTB = PC::kTB, kStage = PC::kStage;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + S * kStage);
  uint64_t *empty = full + S;
  uint64_t *acc_ready = empty + S;
  uint64_t *landed = acc_ready + 1;     // FT = 2, CTA 1: the leader's word that stage s is complete in both CTAs
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(landed + S);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  volatile int *gate = abort_flag + 1;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  // Tile order: bands of kPairBand tile rows, walked column by column, so that the pairs resident at one
  // time share few distinct A and B panels (more L2 hits than a row-major walk over all columns).
  const int tiles_n = (p.N + 255) / 256, tiles_m = (p.M + 255) / 256;
  const int pair = blockIdx.x >> 1;
  const int band = pair / (kPairBand * tiles_n), within = pair % (kPairBand * tiles_n);
  const int band_rows = min(kPairBand, tiles_m - band * kPairBand);
  const int tile_m = band * kPairBand + within % band_rows, tile_n = within / band_rows;
  const int m0 = tile_m * 256 + (int)rank * 128, n0 = tile_n * 256;
  const int nkb = (p.K + 31) / 32;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], FT == kFtCuda ? 5 : 1);
      mbar_init(&landed[s], 1);
    }
    mbar_init(acc_ready, 1);
    *abort_flag = 0;
    *gate = (rank == 0 && launch_aborted(p.status, p.seq)) ? 1 : 0;   // the leader decides for the pair
    mbar_fence_init();
    tma_prefetch_desc(&tmAh);
    tma_prefetch_desc(&tmAl);
    tma_prefetch_desc(&tmBh);
    tma_prefetch_desc(&tmBl);
    if (FT) tma_prefetch_desc(&tmS);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, PC::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();      // barriers of both CTAs are initialised before anything remote signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // an earlier CTA of this launch timed out: both CTAs of the pair skip the work (tensor memory is still freed below)
  const bool aborted = ld_shared_cluster_u32(mapa_u32(smem_u32(const_cast<const int *>(gate)), 0)) != 0;

  uint32_t issued = 0;   // the producer thread: stages it has filled so far
  if (aborted) {
  } else if (warp == 0) {
    // ---- TMA producer (one per CTA) ------------------------------------------------------
    if (lane == 0) {
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % S;
        if (!mbar_wait(&empty[s], ((uint32_t)(kb / S) & 1u) ^ 1u)) {
          pair_abort(abort_flag);
          break;
        }
        unsigned char *st = smem + s * kStage;
        const uint32_t leader_full = mapa_u32(smem_u32(&full[s]), 0);
        if (rank == 0) mbar_expect_tx(&full[s], 2 * kStage);   // the bytes of both CTAs
        issued = (uint32_t)kb + 1u;
        tma_load_2d_pair(st, &tmAh, leader_full, kb * 32, m0);
        tma_load_2d_pair(st + kTA, &tmAl, leader_full, kb * 32, m0);
        tma_load_2d_pair(st + 2 * kTA, &tmBh, leader_full, kb * 32, n0 + (int)rank * 128);
        tma_load_2d_pair(st + 2 * kTA + kTB, &tmBl, leader_full, kb * 32, n0 + (int)rank * 128);
        if (FT == kFtCuda) tma_load_2d_pair(st + 2 * kTA + 2 * kTB, &tmS, leader_full, kb * 32, tile_n * 8);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the leader CTA only -------------------------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_tf32(256, 256, 0, 0);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % S;
        if (!mbar_wait(&full[s], (uint32_t)(kb / S) & 1u)) {
          pair_abort(abort_flag);
          ok = false;
          break;
        }
        tc_fence_after();
        // Tell CTA 1's checksum warps.  Its tiles were written by its own TMA loads, whose completion
        // this thread has just observed on the "full" barrier, so they are in place before the arrival.
        if (FT == kFtCuda) mbar_arrive_remote(mapa_u32(smem_u32(&landed[s]), 1));
        const uint32_t st = smem_u32(smem + s * kStage);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const uint64_t a_hi = umma_smem_desc(st + k4 * 32, 16, 1024, 2);
          const uint64_t a_lo = umma_smem_desc(st + kTA + k4 * 32, 16, 1024, 2);
          const uint64_t b_hi = umma_smem_desc(st + 2 * kTA + k4 * 32, 16, 1024, 2);
          const uint64_t b_lo = umma_smem_desc(st + 2 * kTA + kTB + k4 * 32, 16, 1024, 2);
          umma_tf32_pair(tmem_base, a_lo, b_hi, idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
          umma_tf32_pair(tmem_base, a_hi, b_lo, idesc, 1u);
          umma_tf32_pair(tmem_base, a_hi, b_hi, idesc, 1u);
        }
        umma_commit_pair(&empty[s], (uint16_t)3);   // frees the stage in both CTAs
      }
      if (ok) umma_commit_pair(acc_ready, (uint16_t)3);
    }
  } else {
    // ---- epilogue: warps 2..5 of each CTA, its own 128 accumulator rows ---------------------
    const int q = warp & 3;
    bool ok = true;
    FtInj inj;
    if (FT) inj = ft_scan_plan<256>(p, m0 + q * 32 + lane, n0);
    float *table = reinterpret_cast<float *>(smem + S * kStage + 256);
    if (FT == kFtCuda) {
      // checksums on the CUDA cores: the leader's warps watch its "full" barrier, CTA 1's the word the
      // leader forwards once the stage is complete in both CTAs
      uint64_t *data_bar = (rank == 0) ? full : landed;
      FtCudaAcc<8> acc;
      acc.zero();
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % S;
        if (!mbar_wait(&data_bar[s], (uint32_t)(kb / S) & 1u)) {
          pair_abort(abort_flag);
          break;
        }
        const unsigned char *st = smem + s * kStage;
        ft_cuda_slab(st, st + kTA, st + 2 * kTA + 2 * kTB, q * 32, lane, acc);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
      }
      ft_cuda_finish(acc, table, q * 32, lane);
    }
    if (nkb > 0) {
      bool done = false;
      const uint64_t t0 = global_timer_ns();
      for (int it = 0; it < (1 << 14) && !done; ++it) {
        done = mbar_wait(acc_ready, 0, 1u << 10);
        if (!done && (*abort_flag || global_timer_ns() - t0 > 2000000000ull)) break;
      }
      ok = done;
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) pair_abort(abort_flag);
    tc_fence_after();
    tf32_epilogue<256, FT>(p, tmem_base, q, lane, m0, n0, ok, nkb, inj, table + (q * 32 + lane) * 16, EpiOut::whole(p));
  }

  // neither CTA leaves (or frees tensor memory) while the other may still be read by an MMA
  tc_fence_before();
  cluster_sync_all();
  pair_settle(abort_flag, full, S, issued, rank, tid);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, PC::kTmemCols);
  }
  if (tid == 0 && *abort_flag) record_timeout(p.status, p.seq);
}

// ---- persistent CTA-pair form (plain SGEMM only) -------------------------------------------------
// As many clusters as the device holds at once; cluster c computes tiles c, c + clusters, ... of the
// same band-ordered walk.  The accumulator is double-buffered in TMEM (2 x 256 columns): while the
// epilogue warps drain tile i, the MMA issuer is already accumulating tile i + 1 into the other
// buffer and the TMA producer runs ahead through the same 3-stage ring, so the per-tile prologue
// (barrier set-up, TMEM allocation, first loads in flight) is paid once and the epilogue (about
// 10 us a tile, a third of it waiting for C when beta != 0) hides behind the next tile's MMAs.
// Barriers beyond the ring: acc_full[b] in both CTAs (the leader's commit after a tile's last MMA),
// acc_empty[b] in the leader only (one arrival per epilogue warp of either CTA, CTA 1's by a relaxed
// remote arrive) which the MMA issuer waits on before it reuses buffer b.
__device__ __forceinline__ void pair_tile_origin(const Tf32Args &p, int t, uint32_t rank, int &m0, int &n0) {
  const int tiles_n = (p.N + 255) / 256, tiles_m = (p.M + 255) / 256;
  const int band = t / (kPairBand * tiles_n), within = t % (kPairBand * tiles_n);
  const int band_rows = min(kPairBand, tiles_m - band * kPairBand);
  m0 = (band * kPairBand + within % band_rows) * 256 + (int)rank * 128;
  n0 = (within / band_rows) * 256;
}

constexpr size_t kTailSlotBytes = 256 * 256 * sizeof(float);
constexpr size_t kTailSlotsMax = 80;   // one per cluster
struct ChunkWork {
  int tile, ch0, ch1;   // chunks [ch0, ch1) of this tile
  int slot;             // < 0: the whole tile, result to C; else the workspace slot of the run
};
struct ChunkWorkIter {
  int t, n_clusters, first_sk, nch, cluster, parts, tail_tiles;
  bool tail_done;
  __device__ __forceinline__ ChunkWorkIter(int cluster_, int n_clusters_, int first_sk_, int parts_, int tail_tiles_, int nch_)
      : t(cluster_), n_clusters(n_clusters_), first_sk(first_sk_), nch(nch_), cluster(cluster_), parts(parts_),
        tail_tiles(tail_tiles_), tail_done(false) {}
  __device__ __forceinline__ bool next(ChunkWork &w) {
    if (t < first_sk) {
      w.tile = t; w.ch0 = 0; w.ch1 = nch; w.slot = -1;
      t += n_clusters;
      return true;
    }
    if (!tail_done && parts > 0 && cluster < parts * tail_tiles) {
      tail_done = true;
      const int run = cluster / tail_tiles;
      w.tile = first_sk + cluster % tail_tiles;
      w.ch0 = (int)((long long)run * nch / parts);
      w.ch1 = (int)((long long)(run + 1) * nch / parts);
      w.slot = cluster;
      return w.ch1 > w.ch0;
    }
    return false;
  }
};

// FT = kFtCuda adds the ABFT form: eight more warps (6..13, 16 tile rows each) form the checksums of the tile being accumulated on the
// CUDA cores, beside the MMAs, exactly as in the one-tile kernel, and leave them in one of two shared tables
// (tab_full / tab_empty barriers, local to each CTA); the epilogue warps verify and repair the tile they drain
// against the table of the same parity.  Checksum warps and epilogue warps are different warps here, so the
// epilogue of tile i still overlaps the mainloop (MMAs and checksums) of tile i + 1.
template <int FT>
struct PersistCfg {
  static constexpr int kThreads = FT ? 448 : 192;     // FT: 8 checksum warps of 16 tile rows each
  static constexpr int kTable = FT ? 128 * 16 * 4 : 0;     // bytes per checksum table
  static constexpr int kSmem = 1024 + PairCfg<FT>::kStages * PairCfg<FT>::kStage + 256 + 2 * kTable;
};

template <int FT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PersistCfg<FT>::kThreads, 1)
sgemm_3xtf32_pair_persistent_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
                                    const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
                                    const __grid_constant__ CUtensorMap tmS, const Tf32Args p, int first_sk, int tail_parts,
                                    int tail_tiles, float *tail_ws) {
  static_assert(FT == 0 || FT == kFtCuda, "the persistent form has plain and CUDA-core-checksum variants");
  using PC = PairCfg<FT>;
  constexpr int S = PC::kStages, kTA = PC::kTA, kTB = PC::kTB, kStage = PC::kStage;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + S * kStage);
  uint64_t *empty = full + S;
  uint64_t *acc_full = empty + S;       // [2]
  uint64_t *acc_empty = acc_full + 2;   // [2], used in the leader
  uint64_t *landed = acc_empty + 2;     // [S]  FT, CTA 1: the leader's word that stage s is complete in both CTAs
  uint64_t *tab_full = landed + S;      // [2]  FT: the checksum warps have written table b
  uint64_t *tab_empty = tab_full + 2;   // [2]  FT: the epilogue warps have read table b
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tab_empty + 2);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  volatile int *gate = abort_flag + 1;
  float *tables = reinterpret_cast<float *>(smem + S * kStage + 256);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int nkb = (p.K + 31) / 32;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], FT ? 9 : 1);   // the MMA commit, and the eight checksum warps
      mbar_init(&landed[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);   // four epilogue warps in each of the two CTAs
      mbar_init(&tab_full[b], 8);
      mbar_init(&tab_empty[b], 4);
    }
    *abort_flag = 0;
    *gate = (rank == 0 && launch_aborted(p.status, p.seq)) ? 1 : 0;   // the leader decides for the pair
    mbar_fence_init();
    tma_prefetch_desc(&tmAh);
    tma_prefetch_desc(&tmAl);
    tma_prefetch_desc(&tmBh);
    tma_prefetch_desc(&tmBl);
    if (FT) tma_prefetch_desc(&tmS);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // an earlier CTA of this launch timed out: both CTAs of the pair skip the work (tensor memory is still freed below)
  const bool aborted = ld_shared_cluster_u32(mapa_u32(smem_u32(const_cast<const int *>(gate)), 0)) != 0;

  uint32_t issued = 0;   // the producer thread: stages it has filled so far
  if (aborted) {
  } else if (warp == 0) {
    // ---- TMA producer (one per CTA): one slab counter across all of this cluster's tiles ------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      ChunkWorkIter work(cluster, n_clusters, first_sk, tail_parts, tail_tiles, nkb);   // units of one K-slab
      ChunkWork w;
      while (ok && work.next(w)) {
        int m0, n0;
        pair_tile_origin(p, w.tile, rank, m0, n0);
        for (int kb = w.ch0; kb < w.ch1; ++kb, ++it) {
          const int s = it % S;
          if (!mbar_wait(&empty[s], ((it / S) & 1u) ^ 1u)) {
            pair_abort(abort_flag);
            ok = false;
            break;
          }
          unsigned char *st = smem + s * kStage;
          const uint32_t leader_full = mapa_u32(smem_u32(&full[s]), 0);
          if (rank == 0) mbar_expect_tx(&full[s], 2 * kStage);
          issued = it + 1u;
          tma_load_2d_pair(st, &tmAh, leader_full, kb * 32, m0);
          tma_load_2d_pair(st + kTA, &tmAl, leader_full, kb * 32, m0);
          tma_load_2d_pair(st + 2 * kTA, &tmBh, leader_full, kb * 32, n0 + (int)rank * 128);
          tma_load_2d_pair(st + 2 * kTA + kTB, &tmBl, leader_full, kb * 32, n0 + (int)rank * 128);
          if (FT) tma_load_2d_pair(st + 2 * kTA + 2 * kTB, &tmS, leader_full, kb * 32, (n0 >> 8) * 8);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the leader CTA only ------------------------------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_tf32(256, 256, 0, 0);
      uint32_t it = 0, n_done = 0;
      bool ok = true;
      ChunkWorkIter work(cluster, n_clusters, first_sk, tail_parts, tail_tiles, nkb);
      ChunkWork w;
      for (; ok && work.next(w); ++n_done) {
        const uint32_t buf = n_done & 1u;
        // the epilogue warps of both CTAs have drained this buffer (two tiles ago)
        if (!mbar_wait(&acc_empty[buf], ((n_done >> 1) & 1u) ^ 1u)) {
          pair_abort(abort_flag);
          break;
        }
        tc_fence_after();
        const uint32_t acc = tmem_base + buf * 256u;
        for (int kb = w.ch0; kb < w.ch1; ++kb, ++it) {
          const int s = it % S;
          if (!mbar_wait(&full[s], (it / S) & 1u)) {
            pair_abort(abort_flag);
            ok = false;
            break;
          }
          tc_fence_after();
          // CTA 1's checksum warps cannot watch this barrier: forward the word (its tiles were written by its
          // own TMA loads, whose completion this thread has just observed)
          if (FT) mbar_arrive_remote(mapa_u32(smem_u32(&landed[s]), 1));
          const uint32_t st = smem_u32(smem + s * kStage);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const uint64_t a_hi = umma_smem_desc(st + k4 * 32, 16, 1024, 2);
            const uint64_t a_lo = umma_smem_desc(st + kTA + k4 * 32, 16, 1024, 2);
            const uint64_t b_hi = umma_smem_desc(st + 2 * kTA + k4 * 32, 16, 1024, 2);
            const uint64_t b_lo = umma_smem_desc(st + 2 * kTA + kTB + k4 * 32, 16, 1024, 2);
            umma_tf32_pair(acc, a_lo, b_hi, idesc, (kb > w.ch0 || k4 > 0) ? 1u : 0u);
            umma_tf32_pair(acc, a_hi, b_lo, idesc, 1u);
            umma_tf32_pair(acc, a_hi, b_hi, idesc, 1u);
          }
          umma_commit_pair(&empty[s], (uint16_t)3);
        }
        if (ok) umma_commit_pair(&acc_full[buf], (uint16_t)3);
      }
    }
  } else if (warp < 6) {
    // ---- epilogue: warps 2..5 of each CTA ------------------------------------------------------
    const int q = warp & 3;
    uint32_t n_done = 0;
    const uint32_t leader_empty0 = mapa_u32(smem_u32(&acc_empty[0]), 0), leader_empty1 = mapa_u32(smem_u32(&acc_empty[1]), 0);
    ChunkWorkIter work(cluster, n_clusters, first_sk, tail_parts, tail_tiles, nkb);
    ChunkWork w;
    for (; work.next(w); ++n_done) {
      const uint32_t buf = n_done & 1u;
      int m0, n0;
      pair_tile_origin(p, w.tile, rank, m0, n0);
      FtInj inj;
      if (FT && w.ch0 == 0) inj = ft_scan_plan<256>(p, m0 + q * 32 + lane, n0);   // a planned fault strikes a tile's first run
      // one lane polls (the barrier words share the shared-memory pipe with the MMAs' operand reads); the others
      // then look once for themselves
      bool done = false;
      if (lane == 0) {
        const uint64_t t0 = global_timer_ns();
        for (int itw = 0; itw < (1 << 14) && !done; ++itw) {
          done = mbar_wait(&acc_full[buf], (n_done >> 1) & 1u, 1u << 10);
          if (!done && (*abort_flag || global_timer_ns() - t0 > 2000000000ull)) break;
        }
      }
      done = __shfl_sync(0xffffffffu, done ? 1 : 0, 0) != 0;
      if (done && lane != 0) done = mbar_wait(&acc_full[buf], (n_done >> 1) & 1u, 1u << 10);
      if (FT && done) done = mbar_wait(&tab_full[buf], (n_done >> 1) & 1u);
      const bool ok = __all_sync(0xffffffffu, done);
      if (!ok) {
        pair_abort(abort_flag);
        break;
      }
      tc_fence_after();
      // a whole tile goes to C; a run of a tile cut along K is verified and repaired against the checksums of its own k
      // range and stored unscaled in its workspace slot (row r of the tile at row r of the slot) for the fix-up kernel
      EpiOut eo = EpiOut::whole(p);
      if (w.slot >= 0) {
        int mt, nt;
        pair_tile_origin(p, w.tile, 0, mt, nt);
        eo.C = tail_ws + (size_t)w.slot * 256 * 256 - (ptrdiff_t)mt * 256 - nt;
        eo.ldc = 256;
        eo.alpha = 1.f;
        eo.beta = 0.f;
        eo.vec_c = 1;
        eo.k_begin = w.ch0 * 32;
        eo.k_end = min(w.ch1 * 32, p.K);
      }
      tf32_epilogue<256, FT>(p, tmem_base + buf * 256u, q, lane, m0, n0, true, w.ch1 - w.ch0, inj,
                             tables + buf * (PersistCfg<FT>::kTable / 4) + (q * 32 + lane) * 16, eo, w.ch0 == 0);
      // this warp's reads of the buffer are complete (every chunk waited for its tcgen05.ld): hand it back
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(&acc_empty[buf]);
        else mbar_arrive_remote(buf ? leader_empty1 : leader_empty0);
        if (FT) mbar_arrive(&tab_empty[buf]);
      }
    }
  } else if (FT) {
    // ---- checksum warps 6..13, 16 tile rows each: follow the stages beside the MMA issuer --------
    const int row0 = (warp - 6) * 16;
    uint64_t *data_bar = (rank == 0) ? full : landed;
    uint32_t it = 0, n_done = 0;
    bool ok = true;
    // the same sequence of work as ChunkWorkIter gives the other roles, with little state live across the slab loop:
    // this cluster's whole tiles, then at most one run of a tile of the last round
    const int n_whole = first_sk > cluster ? (first_sk - cluster + n_clusters - 1) / n_clusters : 0;
    const int n_works = n_whole + ((tail_parts > 0 && cluster < tail_parts * tail_tiles) ? 1 : 0);
    for (int i = 0; ok && i < n_works; ++i, ++n_done) {
      FtCudaAcc<4> acc;
      acc.zero();
      int kb = 0, kb_end = nkb;
      if (i >= n_whole) {
        const int run = cluster / tail_tiles;
        kb = (int)((long long)run * nkb / tail_parts);
        kb_end = (int)((long long)(run + 1) * nkb / tail_parts);
      }
      for (; kb < kb_end; ++kb, ++it) {
        const int s = it % S;
        if (!mbar_wait(&data_bar[s], (it / S) & 1u)) {
          ok = false;
          break;
        }
        const unsigned char *st = smem + s * kStage;
        ft_cuda_slab(st, st + kTA, st + 2 * kTA + 2 * kTB, row0, lane, acc);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
      }
      const uint32_t buf = n_done & 1u;
      // the epilogue warps have read this table (two tiles ago)
      if (ok && !mbar_wait(&tab_empty[buf], ((n_done >> 1) & 1u) ^ 1u)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        pair_abort(abort_flag);
        break;
      }
      ft_cuda_finish(acc, tables + buf * (PersistCfg<FT>::kTable / 4), row0, lane);
      if (lane == 0) mbar_arrive(&tab_full[buf]);
    }
  }

  tc_fence_before();
  cluster_sync_all();
  pair_settle(abort_flag, full, S, issued, rank, tid);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
  if (tid == 0 && *abort_flag) record_timeout(p.status, p.seq);
}

// ---- the epilogue side of chunked accumulation, shared by the two kernels below --------------------
// A warp owns 32 accumulator rows (its TMEM lane quarter) x 128 columns; thread = row, acc[j] = column j.

// Adds (first chunk: copies) the 128 columns at `src` of a finished chunk to the sums.
__device__ __forceinline__ void chunk_drain(uint32_t src, bool first, float (&acc)[128]) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint32_t v[16];
    tmem_ld_32x16(src + (uint32_t)(c * 16), v);
    tmem_ld_wait();
    if (first) {
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[c * 16 + j] = __uint_as_float(v[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[c * 16 + j] = __fadd_rn(acc[c * 16 + j], __uint_as_float(v[j]));
    }
  }
}

// The tile's last chunk is on its way: fetch the warp's first 32 x 32 block of C meanwhile (one lane).
__device__ __forceinline__ void chunk_fetch_c(const Tf32Args &p, const CUtensorMap *tmC, unsigned char *stg, uint64_t *cb,
                                              int row0, int colw) {
  if (p.beta != 0.f && p.vec_c && row0 < p.M && colw < (p.N & ~3)) {
    mbar_expect_tx(cb, 4096);
    tma_load_2d(stg, tmC, cb, colw, row0);
  }
}

// C = alpha*acc + beta*C for the warp's 32 x 128 part of the tile.  Registers hold one row per thread.  Each
// 32 x 32 block goes through the warp's 4 KB of shared memory in the 128-byte-swizzled layout of the tensor map of
// C: the block of C arrives there by TMA (the first one was asked for by chunk_fetch_c), every thread replaces its
// own row by the result, and a TMA store takes the block to C, clipped at the matrix edges.  No thread issues a
// global load or store, and the next block is fetched as soon as the store has read the staging area.  The tensor
// map ends at the last whole group of four columns (a TMA store writes whole 16-byte pieces, also at the edge);
// up to three columns beyond it, and everything when C is not 16-byte aligned, go element by element from the
// registers.  False: a wait ran out.
__device__ __forceinline__ bool chunk_store(const Tf32Args &p, const CUtensorMap *tmC, unsigned char *stg, uint64_t *cb,
                                            uint32_t &c_phase, const float (&acc)[128], int row0, int colw, int lane) {
  const bool read_c = (p.beta != 0.f);
  const int n4 = p.N & ~3;   // where the tensor map of C ends
  bool ok = true;
  if (p.vec_c) {
    if (row0 >= p.M) return true;
    if (n4 < p.N && colw <= n4 && n4 < colw + 128 && row0 + lane < p.M) {
      // the one to three columns after the last whole group of four
      float *ct = p.C + (size_t)(row0 + lane) * p.ldc + n4;
#pragma unroll
      for (int k = 0; k < 32; ++k) {
        if (colw + 4 * k == n4) {
#pragma unroll
          for (int e = 0; e < 3; ++e)
            if (n4 + e < p.N) ct[e] = read_c ? __fmaf_rn(p.alpha, acc[4 * k + e], __fmul_rn(p.beta, ct[e])) : __fmul_rn(p.alpha, acc[4 * k + e]);
        }
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col0 = colw + c * 32;
      if (col0 >= n4) break;   // uniform over the warp
      if (read_c) {
        if (!mbar_wait(cb, c_phase)) ok = false;
        c_phase ^= 1u;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float4 *slot = reinterpret_cast<float4 *>(stg + lane * 128 + ((k ^ (lane & 7)) << 4));
        float4 o;
        if (read_c) {
          const float4 cc = *slot;
          o.x = __fmaf_rn(p.alpha, acc[c * 32 + 4 * k + 0], __fmul_rn(p.beta, cc.x));
          o.y = __fmaf_rn(p.alpha, acc[c * 32 + 4 * k + 1], __fmul_rn(p.beta, cc.y));
          o.z = __fmaf_rn(p.alpha, acc[c * 32 + 4 * k + 2], __fmul_rn(p.beta, cc.z));
          o.w = __fmaf_rn(p.alpha, acc[c * 32 + 4 * k + 3], __fmul_rn(p.beta, cc.w));
        } else {
          o.x = __fmul_rn(p.alpha, acc[c * 32 + 4 * k + 0]);
          o.y = __fmul_rn(p.alpha, acc[c * 32 + 4 * k + 1]);
          o.z = __fmul_rn(p.alpha, acc[c * 32 + 4 * k + 2]);
          o.w = __fmul_rn(p.alpha, acc[c * 32 + 4 * k + 3]);
        }
        *slot = o;
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(tmC, stg, col0, row0);
        bulk_commit_group();
        bulk_wait_read_all();   // the staging area may be written again
        if (read_c && c < 3 && col0 + 32 < n4) {
          mbar_expect_tx(cb, 4096);
          tma_load_2d(stg, tmC, cb, col0 + 32, row0);
        }
      }
      __syncwarp();
    }
  } else {
    const int row = row0 + lane;
    if (row < p.M) {
      float *crow = p.C + (size_t)row * p.ldc;
#pragma unroll
      for (int j = 0; j < 128; ++j) {
        if (colw + j < p.N)
          crow[colw + j] = read_c ? __fmaf_rn(p.alpha, acc[j], __fmul_rn(p.beta, crow[colw + j])) : __fmul_rn(p.alpha, acc[j]);
      }
    }
    __syncwarp();
  }
  return ok;
}

// ---- persistent CTA-pair form with chunked accumulation (plain SGEMM) ------------------------------
// The tensor cores add every MMA's products to the accumulator with truncation: an accumulator loses a fixed
// fraction of what it holds per K-slab, so over a long K loop the loss grows with K and, for operands of one sign,
// adds up coherently.  Here the K loop is cut into chunks of `chunk` slabs.  Each chunk is accumulated from zero
// into one of the two TMEM buffers; eight epilogue warps per CTA (one 32-row lane quarter x one 128-column half
// each) add the finished chunk to FP32 sums that they keep in registers while the MMA issuer is already filling
// the other buffer with the next chunk - of the same tile or of the cluster's next tile.  The loss is then bounded
// by that of one chunk whatever K is, and the tile's last chunk goes to C straight from the registers, so a
// buffer is handed back as soon as it has been read and the global-memory part of the epilogue no longer holds
// tensor memory.  Barriers as in the persistent kernel above, counted in chunks instead of tiles.
//
// The last round.  n_tiles tiles on n_clusters clusters are whole rounds plus a remainder, and a remainder of R tiles
// would keep R clusters busy for a whole tile while the others idle (81 tiles on 74 clusters: two rounds for 1.09).
// When at least 2R clusters exist, the R tiles from first_sk on are therefore each cut along K into
// parts = n_clusters / R runs of whole chunks: cluster c < parts * R takes run c / R of tile first_sk + c % R, so
// that at any time the busy clusters read the same K-slabs of neighbouring tiles (shared A and B panels in L2, as
// in a whole round).  A run's FP32 sums go, unscaled, to slot c of the workspace (256 x 256 floats), from which
// tf32_tail_fixup_kernel adds a tile's runs in K order and applies alpha and beta.  Deterministic: the cut depends
// on the shape and the cluster count only.
// The warp's 32 x 128 sums, unscaled, to the workspace tile at (x0, y0) of the tensor map tmW, through its staging area.
__device__ __forceinline__ void chunk_store_raw(const CUtensorMap *tmW, unsigned char *stg, const float (&acc)[128], int x0,
                                                int y0, int lane) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
#pragma unroll
    for (int k = 0; k < 8; ++k)
      *reinterpret_cast<float4 *>(stg + lane * 128 + ((k ^ (lane & 7)) << 4)) =
          make_float4(acc[c * 32 + 4 * k], acc[c * 32 + 4 * k + 1], acc[c * 32 + 4 * k + 2], acc[c * 32 + 4 * k + 3]);
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tmW, stg, x0 + c * 32, y0);
      bulk_commit_group();
      bulk_wait_read_all();
    }
    __syncwarp();
  }
}

// One thread per four columns of a tail tile: adds the tile's runs in K order, C = alpha*sum + beta*C.
__global__ void __launch_bounds__(256) tf32_tail_fixup_kernel(const Tf32Args p, const float *__restrict__ ws, int first_sk,
                                                             int parts, int tail_tiles, int nch) {
  const int j = blockIdx.y;   // tail tile
  int m0, n0;
  pair_tile_origin(p, first_sk + j, 0, m0, n0);
  const int idx = blockIdx.x * 256 + threadIdx.x;   // 0 .. 256*64-1
  const int r = idx >> 6, c4 = (idx & 63) * 4;
  const int row = m0 + r, col = n0 + c4;
  if (row >= p.M || col >= p.N) return;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  bool first = true;
  for (int run = 0; run < parts; ++run) {
    if ((long long)(run + 1) * nch / parts <= (long long)run * nch / parts) continue;   // an empty run
    const int slot = run * tail_tiles + j;
    const float4 v = *reinterpret_cast<const float4 *>(ws + ((size_t)slot * 256 + r) * 256 + c4);
    if (first) sum = v;
    else { sum.x = __fadd_rn(sum.x, v.x); sum.y = __fadd_rn(sum.y, v.y); sum.z = __fadd_rn(sum.z, v.z); sum.w = __fadd_rn(sum.w, v.w); }
    first = false;
  }
  float *cp = p.C + (size_t)row * p.ldc + col;
  const float s4[4] = {sum.x, sum.y, sum.z, sum.w};
  if (p.vec_c && col + 3 < p.N) {
    float4 o;
    if (p.beta != 0.f) {
      const float4 cc = *reinterpret_cast<const float4 *>(cp);
      o.x = __fmaf_rn(p.alpha, sum.x, __fmul_rn(p.beta, cc.x));
      o.y = __fmaf_rn(p.alpha, sum.y, __fmul_rn(p.beta, cc.y));
      o.z = __fmaf_rn(p.alpha, sum.z, __fmul_rn(p.beta, cc.z));
      o.w = __fmaf_rn(p.alpha, sum.w, __fmul_rn(p.beta, cc.w));
    } else {
      o.x = __fmul_rn(p.alpha, sum.x); o.y = __fmul_rn(p.alpha, sum.y); o.z = __fmul_rn(p.alpha, sum.z); o.w = __fmul_rn(p.alpha, sum.w);
    }
    *reinterpret_cast<float4 *>(cp) = o;
  } else {
    for (int e = 0; e < 4; ++e)
      if (col + e < p.N) cp[e] = (p.beta != 0.f) ? __fmaf_rn(p.alpha, s4[e], __fmul_rn(p.beta, cp[e])) : __fmul_rn(p.alpha, s4[e]);
  }
}

constexpr int kChunkThreads = 320;   // TMA producer, MMA issuer, eight epilogue warps
constexpr int kChunkSmem = 1024 + PairCfg<0>::kStages * PairCfg<0>::kStage + 8 * 4096 + 256;   // ring, 4 KB of staging per epilogue warp, barriers
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kChunkThreads, 1)
sgemm_3xtf32_pair_chunked_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
                                 const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
                                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmW,
                                 const Tf32Args p, int first_sk, int tail_parts, int tail_tiles, int chunk) {
  using PC = PairCfg<0>;
  constexpr int S = PC::kStages, kTA = PC::kTA, kTB = PC::kTB, kStage = PC::kStage;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char *staging = smem + S * kStage;   // 4 KB per epilogue warp, each on a 1 KB boundary (128-byte swizzle)
  uint64_t *full = reinterpret_cast<uint64_t *>(staging + 8 * 4096);
  uint64_t *empty = full + S;
  uint64_t *acc_full = empty + S;       // [2]
  uint64_t *acc_empty = acc_full + 2;   // [2], used in the leader
  uint64_t *c_bar = acc_empty + 2;      // [8]  one per epilogue warp: its block of C has landed in its staging area
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(c_bar + 8);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  volatile int *gate = abort_flag + 1;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int nkb = (p.K + 31) / 32, nch = (nkb + chunk - 1) / chunk;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 16);   // eight epilogue warps in each of the two CTAs
    }
    for (int w = 0; w < 8; ++w) mbar_init(&c_bar[w], 1);
    *abort_flag = 0;
    *gate = (rank == 0 && launch_aborted(p.status, p.seq)) ? 1 : 0;   // the leader decides for the pair
    mbar_fence_init();
    tma_prefetch_desc(&tmAh);
    tma_prefetch_desc(&tmAl);
    tma_prefetch_desc(&tmBh);
    tma_prefetch_desc(&tmBl);
    tma_prefetch_desc(&tmC);
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool aborted = ld_shared_cluster_u32(mapa_u32(smem_u32(const_cast<const int *>(gate)), 0)) != 0;

  uint32_t issued = 0;   // the producer thread: stages it has filled so far
  if (aborted) {
  } else if (warp == 0) {
    // ---- TMA producer (one per CTA): one slab counter across all of this cluster's tiles ------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      ChunkWorkIter work(cluster, n_clusters, first_sk, tail_parts, tail_tiles, nch);
      ChunkWork w;
      while (ok && work.next(w)) {
        int m0, n0;
        pair_tile_origin(p, w.tile, rank, m0, n0);
        const int kb_end = min(w.ch1 * chunk, nkb);
        for (int kb = w.ch0 * chunk; kb < kb_end; ++kb, ++it) {
          const int s = it % S;
          if (!mbar_wait(&empty[s], ((it / S) & 1u) ^ 1u)) {
            pair_abort(abort_flag);
            ok = false;
            break;
          }
          unsigned char *st = smem + s * kStage;
          const uint32_t leader_full = mapa_u32(smem_u32(&full[s]), 0);
          if (rank == 0) mbar_expect_tx(&full[s], 2 * kStage);
          issued = it + 1u;
          tma_load_2d_pair(st, &tmAh, leader_full, kb * 32, m0);
          tma_load_2d_pair(st + kTA, &tmAl, leader_full, kb * 32, m0);
          tma_load_2d_pair(st + 2 * kTA, &tmBh, leader_full, kb * 32, n0 + (int)rank * 128);
          tma_load_2d_pair(st + 2 * kTA + kTB, &tmBl, leader_full, kb * 32, n0 + (int)rank * 128);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the leader CTA only; one accumulator buffer per chunk -----------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_tf32(256, 256, 0, 0);
      uint32_t it = 0, g = 0;
      bool ok = true;
      ChunkWorkIter work(cluster, n_clusters, first_sk, tail_parts, tail_tiles, nch);
      ChunkWork w;
      while (ok && work.next(w)) {
        for (int kb0 = w.ch0 * chunk; kb0 < min(w.ch1 * chunk, nkb) && ok; kb0 += chunk, ++g) {
          const uint32_t buf = g & 1u;
          // the epilogue warps of both CTAs have read this buffer (two chunks ago)
          if (!mbar_wait(&acc_empty[buf], ((g >> 1) & 1u) ^ 1u)) {
            pair_abort(abort_flag);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t acc = tmem_base + buf * 256u;
          const int kend = min(kb0 + chunk, nkb);
          for (int kb = kb0; kb < kend; ++kb, ++it) {
            const int s = it % S;
            if (!mbar_wait(&full[s], (it / S) & 1u)) {
              pair_abort(abort_flag);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t st = smem_u32(smem + s * kStage);
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              const uint64_t a_hi = umma_smem_desc(st + k4 * 32, 16, 1024, 2);
              const uint64_t a_lo = umma_smem_desc(st + kTA + k4 * 32, 16, 1024, 2);
              const uint64_t b_hi = umma_smem_desc(st + 2 * kTA + k4 * 32, 16, 1024, 2);
              const uint64_t b_lo = umma_smem_desc(st + 2 * kTA + kTB + k4 * 32, 16, 1024, 2);
              umma_tf32_pair(acc, a_lo, b_hi, idesc, (kb > kb0 || k4 > 0) ? 1u : 0u);
              umma_tf32_pair(acc, a_hi, b_lo, idesc, 1u);
              umma_tf32_pair(acc, a_hi, b_hi, idesc, 1u);
            }
            umma_commit_pair(&empty[s], (uint16_t)3);
          }
          if (ok) umma_commit_pair(&acc_full[buf], (uint16_t)3);
        }
      }
    }
  } else {
    // ---- epilogue: warps 2..9 of each CTA; lane quarter q, column half h -------------------------
    const int q = warp & 3, h = (warp - 2) >> 2;
    const uint32_t leader_empty0 = mapa_u32(smem_u32(&acc_empty[0]), 0), leader_empty1 = mapa_u32(smem_u32(&acc_empty[1]), 0);
    unsigned char *stg = staging + (warp - 2) * 4096;
    uint64_t *cb = &c_bar[warp - 2];
    uint32_t g = 0, c_phase = 0;
    bool ok = true;
    ChunkWorkIter work(cluster, n_clusters, first_sk, tail_parts, tail_tiles, nch);
    ChunkWork w;
    while (ok && work.next(w)) {
      int m0, n0;
      pair_tile_origin(p, w.tile, rank, m0, n0);
      const int row0 = m0 + q * 32, colw = n0 + h * 128;   // this warp's 32 rows x 128 columns
      const int kb_first = w.ch0 * chunk, kb_end = min(w.ch1 * chunk, nkb);
      float acc[128];
      for (int kb0 = kb_first; kb0 < kb_end; kb0 += chunk, ++g) {
        const uint32_t buf = g & 1u;
        if (w.slot < 0 && kb0 + chunk >= kb_end && lane == 0) chunk_fetch_c(p, &tmC, stg, cb, row0, colw);
        // one lane polls (the barrier words share the shared-memory pipe with the MMAs' operand reads); the
        // others then look once for themselves
        bool done = false;
        if (lane == 0) {
          const uint64_t t0 = global_timer_ns();
          for (int itw = 0; itw < (1 << 14) && !done; ++itw) {
            done = mbar_wait(&acc_full[buf], (g >> 1) & 1u, 1u << 10);
            if (!done && (*abort_flag || global_timer_ns() - t0 > 2000000000ull)) break;
          }
        }
        done = __shfl_sync(0xffffffffu, done ? 1 : 0, 0) != 0;
        if (done && lane != 0) done = mbar_wait(&acc_full[buf], (g >> 1) & 1u, 1u << 10);
        ok = __all_sync(0xffffffffu, done);
        if (!ok) {
          pair_abort(abort_flag);
          break;
        }
        tc_fence_after();
        chunk_drain(tmem_base + buf * 256u + (uint32_t)(h * 128) + ((uint32_t)(q * 32) << 16), kb0 == kb_first, acc);
        // this warp's reads of the buffer are complete: hand it back
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) mbar_arrive(&acc_empty[buf]);
          else mbar_arrive_remote(buf ? leader_empty1 : leader_empty0);
        }
      }
      if (!ok) break;
      if (w.slot >= 0) {
        chunk_store_raw(&tmW, stg, acc, h * 128, w.slot * 256 + (int)rank * 128 + q * 32, lane);
      } else if (!chunk_store(p, &tmC, stg, cb, c_phase, acc, row0, colw, lane)) {
        pair_abort(abort_flag);
        break;
      }
    }
    if (lane == 0) bulk_wait_all();   // this thread's stores to C are complete before the CTA goes
  }

  tc_fence_before();
  cluster_sync_all();
  pair_settle(abort_flag, full, S, issued, rank, tid);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
  if (tid == 0 && *abort_flag) record_timeout(p.status, p.seq);
}

// ---- single-CTA form with chunked accumulation (plain SGEMM, 128 x 128 tiles) -----------------------
// One tile per CTA, the same chunks in the same order as the pair kernel above (the two agree bit for bit): the MMA
// issuer alternates between two 128-column TMEM buffers, the four epilogue warps keep the sums of their 32 rows x
// 128 columns in registers and store the tile through their staging areas.
constexpr int kChunk1Smem = 1024 + Tf32Cfg<128, 32, 0>::kStages * Tf32Cfg<128, 32, 0>::kStage + 4 * 4096 + 256;
__global__ void __launch_bounds__(192, 1)
sgemm_3xtf32_chunked_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
                            const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
                            const __grid_constant__ CUtensorMap tmC, const Tf32Args p, int chunk) {
  using Cfg = Tf32Cfg<128, 32, 0>;
  constexpr int S = Cfg::kStages, kTA = Cfg::kTA, kTB = Cfg::kTB, kStage = Cfg::kStage;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char *staging = smem + S * kStage;
  uint64_t *full = reinterpret_cast<uint64_t *>(staging + 4 * 4096);
  uint64_t *empty = full + S;
  uint64_t *acc_full = empty + S;       // [2]
  uint64_t *acc_empty = acc_full + 2;   // [2]
  uint64_t *c_bar = acc_empty + 2;      // [4]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(c_bar + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_n = (p.N + 127) / 128;
  const int m0 = (blockIdx.x / tiles_n) * TBM, n0 = (blockIdx.x % tiles_n) * 128;
  const int nkb = (p.K + 31) / 32;

  {
    __shared__ int launch_aborted;
    if (threadIdx.x == 0) launch_aborted = b2::launch_aborted(p.status, p.seq) ? 1 : 0;
    __syncthreads();
    if (launch_aborted != 0) return;
  }
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    for (int w = 0; w < 4; ++w) mbar_init(&c_bar[w], 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmAh);
    tma_prefetch_desc(&tmAl);
    tma_prefetch_desc(&tmBh);
    tma_prefetch_desc(&tmBl);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  uint32_t issued = 0;   // the producer thread: stages it has filled so far

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % S;
        if (!mbar_wait(&empty[s], ((uint32_t)(kb / S) & 1u) ^ 1u)) {
          *abort_flag = 1;
          break;
        }
        unsigned char *st = smem + s * kStage;
        mbar_expect_tx(&full[s], kStage);
        issued = (uint32_t)kb + 1u;
        tma_load_2d(st, &tmAh, &full[s], kb * 32, m0);
        tma_load_2d(st + kTA, &tmAl, &full[s], kb * 32, m0);
        tma_load_2d(st + 2 * kTA, &tmBh, &full[s], kb * 32, n0);
        tma_load_2d(st + 2 * kTA + kTB, &tmBl, &full[s], kb * 32, n0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_tf32(TBM, 128, 0, 0);
      bool ok = true;
      uint32_t g = 0;
      for (int kb0 = 0; kb0 < nkb && ok; kb0 += chunk, ++g) {
        const uint32_t buf = g & 1u;
        if (!mbar_wait(&acc_empty[buf], ((g >> 1) & 1u) ^ 1u)) {
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t acc = tmem_base + buf * 128u;
        const int kend = min(kb0 + chunk, nkb);
        for (int kb = kb0; kb < kend; ++kb) {
          const int s = kb % S;
          if (!mbar_wait(&full[s], (uint32_t)(kb / S) & 1u)) {
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t st = smem_u32(smem + s * kStage);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const uint64_t a_hi = umma_smem_desc(st + k4 * 32, 16, Cfg::kSbo, Cfg::kSwizzle);
            const uint64_t a_lo = umma_smem_desc(st + kTA + k4 * 32, 16, Cfg::kSbo, Cfg::kSwizzle);
            const uint64_t b_hi = umma_smem_desc(st + 2 * kTA + k4 * 32, 16, Cfg::kSbo, Cfg::kSwizzle);
            const uint64_t b_lo = umma_smem_desc(st + 2 * kTA + kTB + k4 * 32, 16, Cfg::kSbo, Cfg::kSwizzle);
            umma_tf32(acc, a_lo, b_hi, idesc, (kb > kb0 || k4 > 0) ? 1u : 0u);
            umma_tf32(acc, a_hi, b_lo, idesc, 1u);
            umma_tf32(acc, a_hi, b_hi, idesc, 1u);
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;
    unsigned char *stg = staging + (warp - 2) * 4096;
    uint64_t *cb = &c_bar[warp - 2];
    const int row0 = m0 + q * 32, colw = n0;
    uint32_t g = 0, c_phase = 0;
    bool ok = true;
    float acc[128];
    for (int kb0 = 0; kb0 < nkb; kb0 += chunk, ++g) {
      const uint32_t buf = g & 1u;
      if (kb0 + chunk >= nkb && lane == 0) chunk_fetch_c(p, &tmC, stg, cb, row0, colw);
      bool done = false;
      if (lane == 0) {
        const uint64_t t0 = global_timer_ns();
        for (int itw = 0; itw < (1 << 14) && !done; ++itw) {
          done = mbar_wait(&acc_full[buf], (g >> 1) & 1u, 1u << 10);
          if (!done && (*abort_flag || global_timer_ns() - t0 > 2000000000ull)) break;
        }
      }
      done = __shfl_sync(0xffffffffu, done ? 1 : 0, 0) != 0;
      if (done && lane != 0) done = mbar_wait(&acc_full[buf], (g >> 1) & 1u, 1u << 10);
      ok = __all_sync(0xffffffffu, done);
      if (!ok) {
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      chunk_drain(tmem_base + buf * 128u + ((uint32_t)(q * 32) << 16), kb0 == 0, acc);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (ok && !chunk_store(p, &tmC, stg, cb, c_phase, acc, row0, colw, lane)) *abort_flag = 1;
    if (lane == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {   // the same answer in every thread: read after the barrier
    if (tid == 0) ring_settle(full, S, issued);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
  if (tid == 0 && *abort_flag) record_timeout(p.status, p.seq);
}

// ---- single-CTA form with the hi/lo split inside the kernel (plain SGEMM, very small problems) ----------
// Three launches (two split kernels, then the GEMM) cost a small product more than its arithmetic.  Here the TMA
// producer brings the RAW tiles of A (128 rows x 32 k, 128-byte swizzle) and B (32 k x 128 columns, as they lie in
// the row-major B) into a two-stage ring, and the four warps that will later be the epilogue convert them, between
// the loads and the MMAs, into the four K-major plane tiles the MMAs read: A_hi/A_lo element by element in place of
// the same swizzled layout, B_hi/B_lo transposed on the way (thread = column of B = row of the plane tile).  Same
// split arithmetic, same MMA order as the kernels behind the pre-pass: identical results.  Measured: a K-slab takes
// 1.4 us here against 0.6 us behind the pre-pass - the conversion puts 2.5 times the operand bytes through the
// SM's one shared-memory pipe (768 wavefronts of conversion + 512 of MMA operands + 256 of TMA writes per slab
// against the MMAs' 768 cycles of tensor time) - so the launch it saves pays only up to K = 512 on one wave of tiles
// (256^3: 23.6 us against 29.7 us); beyond that the dispatcher keeps the pre-pass, and a third raw stage or integer
// rounding in place of cvt.rna changed nothing.
constexpr int kFusedRaw = 2, kFusedPl = 2;
constexpr int kFusedTile = 128 * 32 * 4;                        // bytes of one 128 x 32 (or 32 x 128) FP32 tile
constexpr int kFusedSmem = 1024 + kFusedPl * 4 * kFusedTile + kFusedRaw * 2 * kFusedTile + 256;
__global__ void __launch_bounds__(192, 1)
sgemm_3xtf32_fused_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Tf32Args p) {
  constexpr int R = kFusedRaw, P = kFusedPl, kT = kFusedTile;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char *planes = smem;                     // stage ps: A_hi, A_lo, B_hi, B_lo
  unsigned char *raw = smem + P * 4 * kT;           // stage r: raw A, raw B
  uint64_t *raw_full = reinterpret_cast<uint64_t *>(raw + R * 2 * kT);
  uint64_t *raw_empty = raw_full + R;
  uint64_t *pl_full = raw_empty + R;
  uint64_t *pl_empty = pl_full + P;
  uint64_t *acc_ready = pl_empty + P;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_ready + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_n = (p.N + 127) / 128;
  const int m0 = (blockIdx.x / tiles_n) * TBM, n0 = (blockIdx.x % tiles_n) * 128;
  const int nkb = (p.K + 31) / 32;

  {
    __shared__ int launch_aborted;
    if (threadIdx.x == 0) launch_aborted = b2::launch_aborted(p.status, p.seq) ? 1 : 0;
    __syncthreads();
    if (launch_aborted != 0) return;
  }
  if (tid == 0) {
    for (int r = 0; r < R; ++r) {
      mbar_init(&raw_full[r], 1);
      mbar_init(&raw_empty[r], 4);   // the four converter warps
    }
    for (int s = 0; s < P; ++s) {
      mbar_init(&pl_full[s], 4);
      mbar_init(&pl_empty[s], 1);    // the MMA commit
    }
    mbar_init(acc_ready, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  uint32_t issued = 0;   // the producer thread: raw stages it has filled so far

  if (warp == 0) {
    // ---- TMA producer: raw tiles --------------------------------------------------------------
    if (lane == 0) {
      for (int kb = 0; kb < nkb; ++kb) {
        const int r = kb % R;
        if (!mbar_wait(&raw_empty[r], ((uint32_t)(kb / R) & 1u) ^ 1u)) {
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(&raw_full[r], 2 * kT);
        issued = (uint32_t)kb + 1u;
        tma_load_2d(raw + r * 2 * kT, &tmA, &raw_full[r], kb * 32, m0);
        tma_load_2d(raw + r * 2 * kT + kT, &tmB, &raw_full[r], n0, kb * 32);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -----------------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_tf32(TBM, 128, 0, 0);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int ps = kb % P;
        if (!mbar_wait(&pl_full[ps], (uint32_t)(kb / P) & 1u)) {
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t st = smem_u32(planes + ps * 4 * kT);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const uint64_t a_hi = umma_smem_desc(st + k4 * 32, 16, 1024, 2);
          const uint64_t a_lo = umma_smem_desc(st + kT + k4 * 32, 16, 1024, 2);
          const uint64_t b_hi = umma_smem_desc(st + 2 * kT + k4 * 32, 16, 1024, 2);
          const uint64_t b_lo = umma_smem_desc(st + 3 * kT + k4 * 32, 16, 1024, 2);
          umma_tf32(tmem_base, a_lo, b_hi, idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
          umma_tf32(tmem_base, a_hi, b_lo, idesc, 1u);
          umma_tf32(tmem_base, a_hi, b_hi, idesc, 1u);
        }
        umma_commit(&pl_empty[ps]);
      }
      if (ok) umma_commit(acc_ready);
    }
  } else {
    // ---- warps 2..5: converters during the K loop, epilogue after it -------------------------------
    const int t = (warp - 2) * 32 + lane;   // row of the A tile, column of the B tile
    const int q = warp & 3;
    bool ok = true;
    for (int kb = 0; kb < nkb; ++kb) {
      const int r = kb % R, ps = kb % P;
      if (!mbar_wait(&raw_full[r], (uint32_t)(kb / R) & 1u) || !mbar_wait(&pl_empty[ps], ((uint32_t)(kb / P) & 1u) ^ 1u)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        *abort_flag = 1;
        break;
      }
      const unsigned char *ra = raw + r * 2 * kT, *rb = ra + kT;
      unsigned char *pa = planes + ps * 4 * kT;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t off = (uint32_t)t * 128u + (uint32_t)((j ^ (t & 7)) << 4);
        // A: chunk j of row t, in place of the same swizzled position
        const float4 x = *reinterpret_cast<const float4 *>(ra + off);
        float4 h, l;
        h.x = tf32_rna(x.x); l.x = tf32_rna(x.x - h.x);
        h.y = tf32_rna(x.y); l.y = tf32_rna(x.y - h.y);
        h.z = tf32_rna(x.z); l.z = tf32_rna(x.z - h.z);
        h.w = tf32_rna(x.w); l.w = tf32_rna(x.w - h.w);
        *reinterpret_cast<float4 *>(pa + off) = h;
        *reinterpret_cast<float4 *>(pa + kT + off) = l;
        // B: k = 4j .. 4j+3 of column t become chunk j of row t of the transposed plane tiles
        float4 y;
        y.x = *reinterpret_cast<const float *>(rb + (4 * j + 0) * 512 + t * 4);
        y.y = *reinterpret_cast<const float *>(rb + (4 * j + 1) * 512 + t * 4);
        y.z = *reinterpret_cast<const float *>(rb + (4 * j + 2) * 512 + t * 4);
        y.w = *reinterpret_cast<const float *>(rb + (4 * j + 3) * 512 + t * 4);
        h.x = tf32_rna(y.x); l.x = tf32_rna(y.x - h.x);
        h.y = tf32_rna(y.y); l.y = tf32_rna(y.y - h.y);
        h.z = tf32_rna(y.z); l.z = tf32_rna(y.z - h.z);
        h.w = tf32_rna(y.w); l.w = tf32_rna(y.w - h.w);
        *reinterpret_cast<float4 *>(pa + 2 * kT + off) = h;
        *reinterpret_cast<float4 *>(pa + 3 * kT + off) = l;
      }
      fence_proxy_async();   // the MMAs read these tiles through the async proxy
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&pl_full[ps]);
        mbar_arrive(&raw_empty[r]);
      }
    }
    if (ok && nkb > 0) {
      bool done = false;
      const uint64_t t0 = global_timer_ns();
      for (int it = 0; it < (1 << 14) && !done; ++it) {
        done = mbar_wait(acc_ready, 0, 1u << 10);
        if (!done && (*abort_flag || global_timer_ns() - t0 > 2000000000ull)) break;
      }
      ok = done;
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) *abort_flag = 1;
    tc_fence_after();
    FtInj inj;
    tf32_epilogue<128, 0>(p, tmem_base, q, lane, m0, n0, ok, nkb, inj, nullptr, EpiOut::whole(p));
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {   // the same answer in every thread: read after the barrier
    if (tid == 0) ring_settle(raw_full, R, issued);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }
  if (tid == 0 && *abort_flag) record_timeout(p.status, p.seq);
}

static std::atomic<int> g_tf32_tile_n{0};  // 0: automatic; 128 or 256 pins the tile width
static std::atomic<int> g_tf32_slab_k{32}; // K-slab depth: 32 (128-byte swizzle) or 16 (64-byte swizzle, twice the stages)
static std::atomic<int> g_tf32_persistent{1};  // 1: the CTA-pair SGEMM runs as a persistent kernel with a double-buffered accumulator
static std::atomic<float> g_tf32_ft_bias{-1.f};  // < 0: default
static std::atomic<int> g_tf32_tail{1};    // 1: the last round of the chunked CTA-pair kernel is shared out in chunks over all clusters
constexpr int kDefaultChunk = 16;
static std::atomic<int> g_tf32_chunk{kDefaultChunk};  // plain SGEMM: K-slabs per accumulation chunk (0: one accumulation over all of K)
static std::atomic<int> g_tf32_fused{1};   // 1: small plain products split their operands inside the GEMM kernel; 0: always the pre-pass; 2: whenever the layout allows
static std::atomic<int> g_tf32_pair{1};    // CTA pairs (256 x 256 tiles, cta_group::2): 0 never, 1 when the wave model favours them, 2 always

// hi/lo planes of A (M x kp) and of B transposed (N x kp), plus the ABFT checksum planes
// (8 rows per 256 columns of B, x kp); every plane starts on a 1 KB boundary.
static size_t tf32_planes_bytes(int M, int N, int K) {
  const size_t kp = ((size_t)K + 3) & ~(size_t)3;
  const size_t srows = (((size_t)N + 255) / 256) * 8;
  return (2 * (size_t)M * kp + 2 * (size_t)N * kp + srows * kp) * sizeof(float) + 8 * 1024;
}
// ... plus, from K = 1024 on, the slots that the tail tiles' runs go
// through (one 256 x 256 tile per cluster, 80 clusters at most); a caller-supplied workspace without them is
// accepted and the last round then runs tile by tile.
size_t tf32_workspace_bytes(int M, int N, int K) {
  return tf32_planes_bytes(M, N, K) + (K >= 1024 ? kTailSlotsMax * kTailSlotBytes + 1024 : 0);
}

// How the chunked CTA-pair kernel treats `tiles` tiles on `clusters` clusters with `nkb` K-slabs in chunks of `chunk`:
// whole rounds for the tiles below *first; when the remaining R tiles would leave at least half of the clusters
// idle and the cut saves 16 K-slabs or more of time, each of them in *parts runs of whole chunks (run r = chunks
// [r*nch/parts, (r+1)*nch/parts), none empty; the longest has *longest chunks) on clusters r*R + j.  False: no cut.
bool tf32_tail_plan(int tiles, int clusters, int nkb, int chunk, int *first, int *parts, int *longest) {
  *first = tiles;
  *parts = 0;
  *longest = 0;
  if (tiles <= 0 || clusters <= 0 || chunk <= 0 || nkb <= 0) return false;
  const int nch = (nkb + chunk - 1) / chunk, rem = tiles % clusters;
  if (rem == 0) return false;
  const int p = clusters / rem < nch ? clusters / rem : nch;
  if (p < 2) return false;
  const int lg = (nch + p - 1) / p;
  if ((nch - lg) * chunk < 16) return false;
  *first = tiles - rem;
  *parts = p;
  *longest = lg;
  return true;
}

template <int TBN, int TBK, int FT>
static int launch_tf32(const Context *ctx, const CUtensorMap *maps, const Tf32Args &args, int grid, cudaStream_t s) {
  int st = ensure_func_attributes((const void *)sgemm_3xtf32_kernel<TBN, TBK, FT>, ctx->device, Tf32Cfg<TBN, TBK, FT>::kSmem);
  if (st != B2_OK) return st;
  sgemm_3xtf32_kernel<TBN, TBK, FT><<<grid, 192, Tf32Cfg<TBN, TBK, FT>::kSmem, s>>>(maps[0], maps[1], maps[2], maps[3],
                                                                                      maps[4], args);
  B2_CUDA(cudaGetLastError());
  return B2_OK;
}

int sgemm_ffma_dispatch_ft(Context *ctx, int trans_a, int M, int N, int K, float alpha, const float *A, int lda,
                           const float *B, int ldb, float beta, float *C, int ldc, const FtArgs *ft, cudaStream_t s);
size_t ffma_workspace_bytes(int M, int N, int K);

// The kernel forms the dispatcher chooses among (generated by gen_ft_sgemm.py from the tile parameters and the
// measured costs).
struct Tf32Tile {
  const char *name;
  int form;      // 0: one tile per CTA; 1: one 256 x 256 tile per CTA pair
  int tbn, tbk;
  double cost;   // time of one tile relative to a single-CTA 128 x 256 tile
};
#define B2_TF32_TILE(NAME, FORM, TBN, TBK, COST) {NAME, FORM, TBN, TBK, COST},
static const Tf32Tile g_tf32_tiles[] = {
#include "tf32_tiles.inc"
};
constexpr int kNumTf32Tiles = sizeof(g_tf32_tiles) / sizeof(g_tf32_tiles[0]);

// How many CTA pairs the device runs at once (one CTA per SM; a pair needs two SMs of one cluster
// domain).  Asked of the occupancy API once per device and handle; 0 (pairs are then not chosen automatically)
// if it will not say, e.g. on a partition that cannot schedule clusters.
static int max_resident_pairs(Context *ctx) {
  if (ctx->max_pairs >= 0) return ctx->max_pairs;
  int n = 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * ctx->sm_count, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = PairCfg<kFtCuda>::kSmem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (ensure_func_attributes((const void *)sgemm_3xtf32_pair_kernel<kFtCuda>, ctx->device, PairCfg<kFtCuda>::kSmem) != B2_OK ||
      cudaOccupancyMaxActiveClusters(&n, sgemm_3xtf32_pair_kernel<kFtCuda>, &cfg) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    n = 0;
  }
  ctx->max_pairs = n;
  return n;
}

// ft == NULL: plain 3xTF32 SGEMM; otherwise the ABFT form (checksum operand, verification and
// recompute-based repair in the epilogue).
int sgemm_3xtf32_dispatch(Context *ctx, int M, int N, int K, float alpha, const float *A, int lda, const float *B, int ldb,
                          float beta, float *C, int ldc, const FtArgs *ft, cudaStream_t s) {
  if (M == 0 || N == 0) return B2_OK;
  // nothing for the tensor cores to do: the FFMA path's scaling pass covers it
  if (K == 0 || alpha == 0.f) return sgemm_ffma_dispatch_ft(ctx, 0, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, ft, s);
  // Very small plain products (one wave of 128 x 128 tiles, K <= 512): the split inside the GEMM kernel, no workspace.
  {
    const int fused = g_tf32_fused.load();
    const long long tiles128 = (long long)((M + 127) / 128) * ((N + 127) / 128);
    const bool aligned = ((((uintptr_t)A) | ((uintptr_t)B)) & 15) == 0 && (lda % 4) == 0 && (ldb % 4) == 0;
    if (ft == nullptr && fused != 0 && aligned && g_tf32_tile_n == 0 && g_tf32_slab_k == 32 &&
        (fused == 2 || (g_tf32_pair == 1 && K <= 512 && tiles128 <= ctx->sm_count))) {   // an explicit choice of kernel form keeps the pre-pass
      CUtensorMap ta, tb;
      int st0 = make_tmap_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 32, 128, CU_TENSOR_MAP_SWIZZLE_128B);
      if (st0 != B2_OK) return st0;
      st0 = make_tmap_2d(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 128, 32, CU_TENSOR_MAP_SWIZZLE_NONE);
      if (st0 != B2_OK) return st0;
      Tf32Args fa;
      memset(&fa, 0, sizeof(fa));
      fa.C = C; fa.M = M; fa.N = N; fa.K = K; fa.ldc = ldc; fa.alpha = alpha; fa.beta = beta;
      fa.vec_c = ((((uintptr_t)C) & 15) == 0 && (ldc % 4) == 0) ? 1 : 0;
      fa.status = (int *)((char *)ctx->fixed + kFixedStatus);
      fa.seq = next_launch_seq(ctx);
      st0 = ensure_func_attributes((const void *)sgemm_3xtf32_fused_kernel, ctx->device, kFusedSmem);
      if (st0 != B2_OK) return st0;
      sgemm_3xtf32_fused_kernel<<<(int)tiles128, 192, kFusedSmem, s>>>(ta, tb, fa);
      B2_CUDA(cudaGetLastError());
      return B2_OK;
    }
  }
  // the planes are needed; the slots of the tail tiles only let the last round be shared out
  bool tail_slots = K >= 1024;
  if (tail_slots && ctx->ws && !ctx->ws_owned && ctx->ws_bytes < tf32_workspace_bytes(M, N, K)) tail_slots = false;
  int st = ensure_workspace(ctx, tail_slots ? tf32_workspace_bytes(M, N, K) : tf32_planes_bytes(M, N, K), s);
  if (st != B2_OK) return st;
  const int ftm = ft ? kFtCuda : 0;
  FtArgs ftl;
  if (ft) {
    // Default thresholds for operands of unit scale.  Checksums on the CUDA cores, corrected for the tensor
    // cores' truncation (ft_bias, see tf32_epilogue), leave a clean residual of at most 4.7e-7*K (K = 256 .. 8192,
    // uniform and normal data): 2.5e-6*K is five times that and half the path's tolerance of 2e-5*sum|a||b|
    // (5e-6*K for operands uniform in [-1, 1)).  Checksums accumulated by the tensor cores: residual 2.2e-6*K.
    ftl = *ft;
    if (!(ftl.tau > 0.f)) ftl.tau = fmaxf(2.5e-6f * (float)K, 6e-5f);
    ft = &ftl;
  }
  const int kp = (K + 3) & ~3;
  char *w = (char *)(((uintptr_t)ctx->ws + 1023) & ~(uintptr_t)1023);
  const size_t a_elems = (size_t)M * kp, b_elems = (size_t)N * kp;
  auto align1k = [](size_t bytes) { return (bytes + 1023) & ~(size_t)1023; };
  float *Ah = (float *)w;
  float *Al = (float *)(w + align1k(a_elems * 4));
  float *Bh = (float *)(w + 2 * align1k(a_elems * 4));
  float *Bl = (float *)(w + 2 * align1k(a_elems * 4) + align1k(b_elems * 4));
  const int srows = ((N + 255) / 256) * 8;
  float *S = (float *)(w + 2 * align1k(a_elems * 4) + 2 * align1k(b_elems * 4));

  {
    const int vec = ((((uintptr_t)A) & 15) == 0 && (lda % 4) == 0) ? 1 : 0;
    dim3 g((kp / 4 + 255) / 256, M < 16384 ? M : 16384);
    split_planes_kernel<<<g, 256, 0, s>>>(A, M, K, lda, Ah, Al, kp, vec);
    // the ABFT form covers whole 256-column tiles so that every checksum row is written
    dim3 gt(ft ? ((N + 255) / 256) * (256 / kSplitTN) : (N + kSplitTN - 1) / kSplitTN, (kp + kSplitTK - 1) / kSplitTK);
    split_planes_t_kernel<<<gt, 256, 0, s>>>(B, K, N, ldb, Bh, Bl, kp, ft ? S : nullptr);
  }
  B2_CUDA(cudaGetLastError());

  CUtensorMap maps[5];
  const int tbk = (g_tf32_slab_k == 32 || ft) ? 32 : 16;   // the ABFT form is built for the 32-deep slab only
  const CUtensorMapSwizzle swz = (tbk == 32) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  st = make_tmap_2d(&maps[0], Ah, (uint64_t)K, (uint64_t)M, (uint64_t)kp, tbk, TBM, swz);
  if (st != B2_OK) return st;
  st = make_tmap_2d(&maps[1], Al, (uint64_t)K, (uint64_t)M, (uint64_t)kp, tbk, TBM, swz);
  if (st != B2_OK) return st;
  // Kernel form and tile width by whole waves, from the generated table (tf32_tiles.inc: cost = time of one tile
  // relative to a single-CTA 128 x 256 tile); later rows win ties.  A pinned width selects the single-CTA kernel of that
  // width; the ABFT form exists for 256-column tiles only.
  const int pairs = ((M + 255) / 256) * ((N + 255) / 256);
  const int slots = max_resident_pairs(ctx);
  const bool pinned = (g_tf32_tile_n == 128 || g_tf32_tile_n == 256);
  int chosen = -1;
  double best_time = 1e300;
  for (int t = 0; t < kNumTf32Tiles; ++t) {
    const Tf32Tile &tl = g_tf32_tiles[t];
    if (tl.tbk != 32) continue;
    if (ft != nullptr && tl.tbn != 256) continue;
    double time;
    if (tl.form == 1) {
      if (tbk != 32 || pinned || g_tf32_pair == 0 || (g_tf32_pair == 1 && slots <= 0)) continue;
      time = g_tf32_pair == 2 ? -1.0 : tl.cost * ceil((double)pairs / (double)slots);
    } else {
      if (pinned && tl.tbn != g_tf32_tile_n) continue;
      const double tiles = (double)((M + TBM - 1) / TBM) * ((N + tl.tbn - 1) / tl.tbn);
      time = tl.cost * ceil(tiles / (double)ctx->sm_count);
    }
    if (time <= best_time) {
      best_time = time;
      chosen = t;
    }
  }
  B2_REQUIRE(chosen >= 0, B2_ERR_UNSUPPORTED, "3xTF32: no kernel form of the tile table fits this call");
  bool use_pair = g_tf32_tiles[chosen].form == 1;
  // Chunked accumulation (plain calls with more than two chunks of K-slabs, no pinned width): two forms exist, the
  // persistent CTA-pair kernel and single-CTA 128 x 128 tiles; whole waves decide between them as above.
  const int chunk = g_tf32_chunk.load();
  int tail_parts = 0;   // >= 2: each tile from tail_first on is cut along K into that many runs on different clusters
  int tail_first = pairs;
  const bool chunked = ft == nullptr && chunk > 0 && (K + 31) / 32 > 2 * chunk && tbk == 32 && !pinned;
  if (chunked) {
    const bool pair_ok = g_tf32_pair != 0 && slots > 0 && g_tf32_persistent != 0;
    double cost_pair = 0.9, cost_single = 0.55;
    for (int t = 0; t < kNumTf32Tiles; ++t) {
      if (g_tf32_tiles[t].form == 1) cost_pair = g_tf32_tiles[t].cost;
      else if (g_tf32_tiles[t].tbn == 128 && g_tf32_tiles[t].tbk == 32) cost_single = g_tf32_tiles[t].cost;
    }
    const double tiles128 = (double)((M + 127) / 128) * ((N + 127) / 128);
    double pair_rounds = pair_ok ? ceil((double)pairs / (double)slots) : 0.0;
    if (pair_ok) {
      int parts = 0, first = pairs, longest = 0;
      if (tail_slots && g_tf32_tail.load() != 0 && (size_t)slots <= kTailSlotsMax &&
          tf32_tail_plan(pairs, slots, (K + 31) / 32, chunk, &first, &parts, &longest)) {
        tail_parts = parts;
        tail_first = first;
        const int nch = ((K + 31) / 32 + chunk - 1) / chunk;
        pair_rounds = (double)(pairs / slots) + (double)longest / (double)nch;
      }
    }
    use_pair = pair_ok && (g_tf32_pair == 2 || cost_pair * pair_rounds <= cost_single * ceil(tiles128 / (double)ctx->sm_count));
  }
  if (use_pair) {
    st = make_tmap_2d(&maps[2], Bh, (uint64_t)K, (uint64_t)N, (uint64_t)kp, 32, 128, swz);
    if (st != B2_OK) return st;
    st = make_tmap_2d(&maps[3], Bl, (uint64_t)K, (uint64_t)N, (uint64_t)kp, 32, 128, swz);
    if (st != B2_OK) return st;
    if (ft) {
      st = make_tmap_2d(&maps[4], S, (uint64_t)K, (uint64_t)srows, (uint64_t)kp, 32, 8, swz);
      if (st != B2_OK) return st;
    } else {
      maps[4] = maps[2];
    }
    Tf32Args pa;
    memset(&pa, 0, sizeof(pa));
    pa.C = C; pa.M = M; pa.N = N; pa.K = K; pa.ldc = ldc; pa.alpha = alpha; pa.beta = beta;
    pa.vec_c = ((((uintptr_t)C) & 15) == 0 && (ldc % 4) == 0) ? 1 : 0;
    pa.status = (int *)((char *)ctx->fixed + kFixedStatus);
    pa.seq = next_launch_seq(ctx);
    if (ft) {
      pa.ft = *ft;
      pa.tau_elem = 0.75f * ft->tau;
      pa.ft_bias = g_tf32_ft_bias.load() >= 0.f ? g_tf32_ft_bias.load() : kFtBiasPerSlab;
    }
    if (chunked) {
      st = ensure_func_attributes((const void *)sgemm_3xtf32_pair_chunked_kernel, ctx->device, kChunkSmem);
      if (st != B2_OK) return st;
      const int clusters = tail_parts > 0 ? slots : (pairs < slots ? pairs : (slots > 0 ? slots : pairs));
      CUtensorMap map_c = maps[0], map_w = maps[0];
      if (N < 4) pa.vec_c = 0;
      if (pa.vec_c) {
        st = make_tmap_2d(&map_c, C, (uint64_t)(N & ~3), (uint64_t)M, (uint64_t)ldc, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != B2_OK) return st;
      }
      float *tail_ws = (float *)(w + 2 * align1k(a_elems * 4) + 2 * align1k(b_elems * 4) + align1k((size_t)srows * kp * 4));
      if (tail_parts > 0) {
        st = make_tmap_2d(&map_w, tail_ws, 256, (uint64_t)clusters * 256, 256, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != B2_OK) return st;
      }
      sgemm_3xtf32_pair_chunked_kernel<<<2 * clusters, kChunkThreads, kChunkSmem, s>>>(maps[0], maps[1], maps[2], maps[3], map_c, map_w, pa,
                                                                                       tail_first, tail_parts, pairs - tail_first, chunk);
      B2_CUDA(cudaGetLastError());
      if (tail_parts > 0) {
        const int nch = ((K + 31) / 32 + chunk - 1) / chunk;
        tf32_tail_fixup_kernel<<<dim3(64, pairs - tail_first), 256, 0, s>>>(pa, tail_ws, tail_first, tail_parts, pairs - tail_first, nch);
        B2_CUDA(cudaGetLastError());
      }
      return B2_OK;
    }
    if (g_tf32_persistent) {
      const void *fn = ftm ? (const void *)sgemm_3xtf32_pair_persistent_kernel<kFtCuda> : (const void *)sgemm_3xtf32_pair_persistent_kernel<0>;
      st = ensure_func_attributes(fn, ctx->device, ftm ? PersistCfg<kFtCuda>::kSmem : PersistCfg<0>::kSmem);
      if (st != B2_OK) return st;
      const int clusters = pairs < slots ? pairs : (slots > 0 ? slots : pairs);
      if (ftm == kFtCuda) {
        // the fault-tolerant form cuts a partial last round along K too, in units of one K-slab: every run is verified
        // and repaired against the checksums of its own k range before its sums go to the workspace
        int t_first = pairs, t_parts = 0, t_longest = 0;
        float *tail_ws = (float *)(w + 2 * align1k(a_elems * 4) + 2 * align1k(b_elems * 4) + align1k((size_t)srows * kp * 4));
        const bool cut = tail_slots && g_tf32_tail.load() != 0 && (size_t)slots <= kTailSlotsMax &&
                         tf32_tail_plan(pairs, slots, (K + 31) / 32, 1, &t_first, &t_parts, &t_longest);
        const int cl = cut ? slots : clusters;
        sgemm_3xtf32_pair_persistent_kernel<kFtCuda><<<2 * cl, PersistCfg<kFtCuda>::kThreads, PersistCfg<kFtCuda>::kSmem, s>>>(
            maps[0], maps[1], maps[2], maps[3], maps[4], pa, cut ? t_first : pairs, cut ? t_parts : 0, pairs - t_first, tail_ws);
        B2_CUDA(cudaGetLastError());
        if (cut) {
          tf32_tail_fixup_kernel<<<dim3(64, pairs - t_first), 256, 0, s>>>(pa, tail_ws, t_first, t_parts, pairs - t_first, (K + 31) / 32);
          B2_CUDA(cudaGetLastError());
        }
      } else {
        sgemm_3xtf32_pair_persistent_kernel<0><<<2 * clusters, PersistCfg<0>::kThreads, PersistCfg<0>::kSmem, s>>>(maps[0], maps[1], maps[2], maps[3], maps[4], pa, pairs, 0, 0, nullptr);
        B2_CUDA(cudaGetLastError());
      }
      return B2_OK;
    }
    st = ftm == kFtCuda ? ensure_func_attributes((const void *)sgemm_3xtf32_pair_kernel<kFtCuda>, ctx->device, PairCfg<kFtCuda>::kSmem)
                        : ensure_func_attributes((const void *)sgemm_3xtf32_pair_kernel<0>, ctx->device, PairCfg<0>::kSmem);
    if (st != B2_OK) return st;
    if (ftm == kFtCuda) sgemm_3xtf32_pair_kernel<kFtCuda><<<2 * pairs, 192, PairCfg<kFtCuda>::kSmem, s>>>(maps[0], maps[1], maps[2], maps[3], maps[4], pa);
    else sgemm_3xtf32_pair_kernel<0><<<2 * pairs, 192, PairCfg<0>::kSmem, s>>>(maps[0], maps[1], maps[2], maps[3], maps[4], pa);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
  }
  const int tbn = chunked ? 128 : g_tf32_tiles[chosen].tbn;
  st = make_tmap_2d(&maps[2], Bh, (uint64_t)K, (uint64_t)N, (uint64_t)kp, tbk, tbn, swz);
  if (st != B2_OK) return st;
  st = make_tmap_2d(&maps[3], Bl, (uint64_t)K, (uint64_t)N, (uint64_t)kp, tbk, tbn, swz);
  if (st != B2_OK) return st;

  if (ft) {
    st = make_tmap_2d(&maps[4], S, (uint64_t)K, (uint64_t)srows, (uint64_t)kp, tbk, 8, swz);
    if (st != B2_OK) return st;
  } else {
    maps[4] = maps[2];
  }

  Tf32Args args;
  memset(&args, 0, sizeof(args));
  args.C = C; args.M = M; args.N = N; args.K = K; args.ldc = ldc; args.alpha = alpha; args.beta = beta;
  args.vec_c = ((((uintptr_t)C) & 15) == 0 && (ldc % 4) == 0) ? 1 : 0;
  args.status = (int *)((char *)ctx->fixed + kFixedStatus);
  args.seq = next_launch_seq(ctx);
  const int grid = ((M + TBM - 1) / TBM) * ((N + tbn - 1) / tbn);
  if (ft) {
    args.ft = *ft;
    args.tau_elem = 0.75f * ft->tau;
    args.ft_bias = g_tf32_ft_bias.load() >= 0.f ? g_tf32_ft_bias.load() : kFtBiasPerSlab;
    return launch_tf32<256, 32, kFtCuda>(ctx, maps, args, grid, s);
  }
  if (chunked) {
    CUtensorMap map_c = maps[0];
    if (N < 4) args.vec_c = 0;
    if (args.vec_c) {
      st = make_tmap_2d(&map_c, C, (uint64_t)(N & ~3), (uint64_t)M, (uint64_t)ldc, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B);
      if (st != B2_OK) return st;
    }
    st = ensure_func_attributes((const void *)sgemm_3xtf32_chunked_kernel, ctx->device, kChunk1Smem);
    if (st != B2_OK) return st;
    sgemm_3xtf32_chunked_kernel<<<grid, 192, kChunk1Smem, s>>>(maps[0], maps[1], maps[2], maps[3], map_c, args, chunk);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
  }
  if (tbk == 32) return tbn == 128 ? launch_tf32<128, 32, 0>(ctx, maps, args, grid, s) : launch_tf32<256, 32, 0>(ctx, maps, args, grid, s);
  return tbn == 128 ? launch_tf32<128, 16, 0>(ctx, maps, args, grid, s) : launch_tf32<256, 16, 0>(ctx, maps, args, grid, s);
}

}  // namespace b2

using namespace b2;

extern "C" {

size_t b2_sgemm_workspace_bytes(int path, int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (path == B2_PATH_FFMA) return ffma_workspace_bytes(M, N, K);   // optional: used when there, never required
  if (path != B2_PATH_3XTF32) return 0;
  return tf32_workspace_bytes(M, N, K);
}

// Pins the 3xTF32 tile width (128 or 256 columns; 0 = automatic).  For benchmarking.
int b2_set_tf32_tile_n(int n) {
  B2_REQUIRE(n == 0 || n == 128 || n == 256, B2_ERR_INVALID_ARG, "b2_set_tf32_tile_n: %d is not 0, 128 or 256", n);
  b2::g_tf32_tile_n = n;
  return B2_OK;
}
// CTA pairs (256 x 256 tiles, tcgen05 cta_group::2) in the 3xTF32 SGEMM: 0 never, 1 automatic (default), 2 always.
int b2_set_tf32_pair(int on) {
  B2_REQUIRE(on >= 0 && on <= 2, B2_ERR_INVALID_ARG, "b2_set_tf32_pair: %d is not 0, 1 or 2", on);
  b2::g_tf32_pair = on;
  return B2_OK;
}
// 1 (default): the plain CTA-pair SGEMM is the persistent kernel; 0: one cluster per tile.
int b2_set_tf32_persistent(int on) {
  B2_REQUIRE(on == 0 || on == 1, B2_ERR_INVALID_ARG, "b2_set_tf32_persistent: %d is not 0 or 1", on);
  b2::g_tf32_persistent = on;
  return B2_OK;
}
// Fraction of its value that an accumulator is taken to lose per 32-deep K-slab to the tensor cores' truncating
// adds (CUDA-core checksums only); negative restores the built-in figure measured on B200.
int b2_set_tf32_abft_bias(float bias) {
  B2_REQUIRE(bias < 1e-3f, B2_ERR_INVALID_ARG, "b2_set_tf32_abft_bias: %g is not a plausible loss per K-slab", (double)bias);
  b2::g_tf32_ft_bias = bias;
  return B2_OK;
}
// Chunked accumulation of the plain CTA-pair 3xTF32 SGEMM: every `slabs` K-slabs (of 32) the tensor-memory
// accumulator is added to FP32 sums in registers and started again from zero, which bounds the tensor cores'
// truncation loss by that of one chunk.  0: one accumulation over all of K; negative: the default (16).
int b2_set_tf32_chunk(int slabs) {
  B2_REQUIRE(slabs <= 4096, B2_ERR_INVALID_ARG, "b2_set_tf32_chunk: %d is not in 0..4096 (or negative for the default)", slabs);
  b2::g_tf32_chunk = slabs < 0 ? b2::kDefaultChunk : slabs;
  return B2_OK;
}
// 1 (default): the last, partial round of the chunked CTA-pair kernel is shared out in chunks over all clusters
// (parts through the workspace, added in K order); 0: tile by tile.
int b2_set_tf32_tail_split(int on) {
  B2_REQUIRE(on == 0 || on == 1, B2_ERR_INVALID_ARG, "b2_set_tf32_tail_split: %d is not 0 or 1", on);
  b2::g_tf32_tail = on;
  return B2_OK;
}
// The cut of the last round for a given tile and cluster count (see b2_set_tf32_tail_split): returns 1 and the first
// cut tile, the runs per tile and the chunks of the longest run, or 0.  For tests and tools.
int b2_tf32_tail_plan(int tiles, int clusters, int K, int chunk_slabs, int *first, int *parts, int *longest) {
  int f = 0, p = 0, l = 0;
  const bool cut = K > 0 && b2::tf32_tail_plan(tiles, clusters, (K + 31) / 32, chunk_slabs, &f, &p, &l);
  if (first) *first = f;
  if (parts) *parts = p;
  if (longest) *longest = l;
  return cut ? 1 : 0;
}
// The hi/lo split inside the GEMM kernel: 0 never (always the two split kernels in front), 1 for very small plain
// products (one wave of 128 x 128 tiles, K <= 512; the default), 2 whenever A and B are 16-byte aligned.
int b2_set_tf32_fused_split(int mode) {
  B2_REQUIRE(mode >= 0 && mode <= 2, B2_ERR_INVALID_ARG, "b2_set_tf32_fused_split: %d is not 0, 1 or 2", mode);
  b2::g_tf32_fused = mode;
  return B2_OK;
}
// K-slab depth of the 3xTF32 kernel: 16 or 32.  For benchmarking.
int b2_set_tf32_slab_k(int k) {
  B2_REQUIRE(k == 16 || k == 32, B2_ERR_INVALID_ARG, "b2_set_tf32_slab_k: %d is not 16 or 32", k);
  b2::g_tf32_slab_k = k;
  return B2_OK;
}

}  // extern "C"
