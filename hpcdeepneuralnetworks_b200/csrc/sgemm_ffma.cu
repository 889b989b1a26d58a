// FP32 SIMT (FFMA) SGEMM and ABFT SGEMM for sm_100a: row-major C = alpha*A*B + beta*C, any
// M, N, K.
//
// Stands in for rung 14 of the reference series (kernel/sgemm/include/kernel_14.cuh:12:
// 128x128x32 block tile, 256 threads, 8x8 outputs per thread), for the plain and ABFT tile
// families of kernel/ft_sgemm (include_code_gen/{ft_}sgemm_{small..huge}.cuh:11, hand-written
// include/ft_sgemm_huge.cuh:21) and, through gen_ft_sgemm.py, for its code generator
// (code_gen/code_gen.py:4, code_gen/main.py:8-19).  What is different on Blackwell:
//   * A and B slabs are brought in by TMA (cp.async.bulk.tensor) into a 3-stage shared
//     ring guarded by full/empty mbarriers; no thread spends issue slots on global loads,
//     and out-of-range rows/columns/K are zero-filled by the copy engine, so any shape works.
//   * A stays K-contiguous in shared memory (TMA cannot transpose) under the 128-byte
//     swizzle; a thread reads a float4 ALONG K for each of its 4 rows, which costs the same
//     number of 128-bit shared loads as the reference's transposed store scheme
//     (kernel_9.cuh:37-40) and is bank-conflict free.
//   * BM/16 warps stacked along M, each spanning 16 rows x BN columns, lanes as 4 (M) x 8 (N),
//     4 x NR outputs per thread (NR = BN/8): the warp tiling idea of kernel_11.cuh:22-27 with
//     a shape chosen for the swizzled A reads and for the packed FMA below.
//   * The inner product uses the packed fma.rn.f32x2 instruction (two FP32 FMAs per issue
//     slot, pairs of adjacent columns); only the 4 A values per k have to be duplicated into
//     both halves of an operand.  Per output the arithmetic is still one FMA per k in
//     ascending k, so results are bit-identical to the scalar form (kept as a variant).
//     The K-slab body is fully unrolled: shorter unrolled bodies and register-free schemes
//     for the duplication (a per-warp shared region of (a,a) pairs) both measured slower.
// Each output element is accumulated by exactly one thread in ascending k with one FMA per
// k, and the epilogue is fma(alpha, acc, beta*c) (alpha*acc when beta == 0; C is then not
// read).
//
// The tile family (block tile BM x BN, BK = 32) is listed in ffma_tiles.inc, which
// gen_ft_sgemm.py writes; every entry is instantiated plain and with ABFT.
#include <math.h>
#include <stdlib.h>

#include <atomic>

#include "common.cuh"

namespace b2 {

constexpr int FBK = 32;
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
  int *status;  // device status words: [0] set to B2_ERR_TIMEOUT if a bounded wait runs out, [1] the number of that launch
  unsigned int seq;   // number of this launch on its handle
  int device;         // host side only: the device the launch goes to
  // split-K (plain SGEMM only): CTA (split s, tile t) sums K-slabs [s * slabs_per_split, (s + 1) * slabs_per_split) and
  // writes its raw sums to partial[s] (M x ldp); splitk_reduce_kernel adds the parts in ascending s and applies alpha/beta
  int k_splits, slabs_per_split, ldp;
  float *partial;
};

// ABFT.  Checksum algebra of kernel/ft_sgemm/README.md:4-14 at the granularity the accumulators are held:
// block (w, g) = the 16 rows of warp w x the NR columns of lane column g (64 blocks of 16 x 16 in a 128 x 128
// tile).  With Asum_w[k] = sum of A over the 16 rows of w (a column checksum e^T A of that row band) and
// Bsum_g[k] = sum of B[k][.] over the columns of g (a row checksum B e of that column set),
//     sum of the block's outputs = sum_k Asum_w[k] * Bsum_g[k].
// The reference encodes both operand checksums inside every CTA from the registers it prefetched
// (kernel/ft_sgemm/include/ft_sgemm_tall.cuh:178-267), so every CTA of a tile row re-encodes the same band of A
// and every CTA of a tile column the same panel of B.  Here (FT = 1) the operand checksums are encoded ONCE per
// product by two small pre-pass kernels (ft_encode_a_kernel, ft_encode_b_kernel: one more read of A and B, 1/16
// of their size written) into per-slab tables, and travel with each K-slab through the same TMA ring as the
// operand tiles (1 KB + 128 B per warp and stage); in the mainloop lane (g, r) adds
// sum_{8 k of r} Asum_w[k] * Bsum_g[k] to its running checksum: 4 shared loads and 4 packed FMAs per slab beside
// the 1024 packed FMAs of the product.  A corrupted operand tile in shared memory now disagrees with its checksum
// (with in-CTA encoding both would be wrong together).
// The epilogue folds the 4 k-ranges and the 4 x NR accumulators of the 4 lanes that share a block with two
// shuffles each and compares them in registers (the reference compares every 256 of K through shared memory,
// ft_sgemm_huge.cuh:143-271).  A block out of tolerance is recomputed element by element from A and B in global
// memory with the kernel's own arithmetic; every accumulator that differs is replaced, which both locates and
// corrects the fault exactly (the reference subtracts a rounded residual with the location left unfinished,
// ft_sgemm_huge.cuh:296-371).
template <int BM, int NR, int MR = 4, int NSTAGES = 3>
struct TileCfg {
  static constexpr int BN = 8 * NR;
  static constexpr int STAGES = NSTAGES;        // depth of the TMA ring
  static constexpr int BAND = 4 * MR;          // rows of a warp: 4 lanes along M x MR rows per thread
  static constexpr int WARPS = BM / BAND;
  static constexpr int THREADS = 32 * WARPS;
  static constexpr int kStageA = BM * FBK * 4;
  static constexpr int kStageB = FBK * BN * 4;
  static constexpr int kBarOff = STAGES * (kStageA + kStageB);   // full[STAGES], empty[STAGES]
  static constexpr int kCsOff = kBarOff + 128;                   // per stage: float Asum[WARPS][32], float Bsum[256]
  static constexpr int kStageCs = WARPS * 128 + 1024;
  static constexpr int kMiscOff = kCsOff + STAGES * kStageCs;    // int inj[8]; int nflag; int flagged[64]
  static constexpr int kSmem = 1024 + kMiscOff + 512;
  // resident CTAs per SM: 16 warps of 4 x NR thread tiles or 8 warps of 8 x NR thread tiles (twice the accumulators), as
  // far as 227 KB of shared memory hold that many rings (each CTA also takes 1 KB of system use)
  static constexpr int kByWarps = (MR == 4 ? 16 : 8) / WARPS;
  static constexpr int kBySmem = (227 * 1024) / (kSmem + 1024);
  static constexpr int MIN_BLOCKS = kByWarps < kBySmem ? kByWarps : (kBySmem > 0 ? kBySmem : 1);
  static_assert(MR == 4 || MR == 8, "MR is 4 or 8 rows per thread");
  static_assert(STAGES >= 2 && STAGES <= 8, "2 to 8 stages (the barriers share one 128-byte line)");
  static_assert(BM % BAND == 0 && BM >= 32 && BM <= 128, "BM is 32, 64 or 128 and a multiple of the warp's rows");
  static_assert(NR == 8 || NR == 16, "NR is 8 or 16 columns per thread");
};

// Accumulators of one thread: MR rows x NR columns.  Row i is tile row warp*4*MR + lm + 4*i
// (row-major A) or warp*4*MR + lm*MR + i (transposed A); column j is tile column
// ln*4 + 32*(j/4) + j%4, so one warp spans all BN columns of 4*MR rows.
template <bool PACKED, int NR, int MR>
struct Acc;
template <int NR, int MR>
struct Acc<false, NR, MR> {
  float v[MR][NR];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < MR; ++i)
#pragma unroll
      for (int j = 0; j < NR; ++j) v[i][j] = 0.f;
  }
  __device__ __forceinline__ void step(const float (&a)[MR], const float4 (&b)[NR / 4]) {
#pragma unroll
    for (int i = 0; i < MR; ++i)
#pragma unroll
      for (int q = 0; q < NR / 4; ++q) {
        v[i][4 * q + 0] = __fmaf_rn(a[i], b[q].x, v[i][4 * q + 0]);
        v[i][4 * q + 1] = __fmaf_rn(a[i], b[q].y, v[i][4 * q + 1]);
        v[i][4 * q + 2] = __fmaf_rn(a[i], b[q].z, v[i][4 * q + 2]);
        v[i][4 * q + 3] = __fmaf_rn(a[i], b[q].w, v[i][4 * q + 3]);
      }
  }
  __device__ __forceinline__ float get(int i, int j) const { return v[i][j]; }
  __device__ __forceinline__ void set(int i, int j, float x) { v[i][j] = x; }
  __device__ __forceinline__ float total() const {
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < MR; ++i)
#pragma unroll
      for (int j = 0; j < NR; ++j) s[i & 3] += v[i][j];
    return (s[0] + s[1]) + (s[2] + s[3]);
  }
};
template <int NR, int MR>
struct Acc<true, NR, MR> {
  uint64_t v[MR][NR / 2];  // pairs of adjacent columns
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < MR; ++i)
#pragma unroll
      for (int j = 0; j < NR / 2; ++j) v[i][j] = 0ull;
  }
  __device__ __forceinline__ void step(const float (&a)[MR], const float4 (&b)[NR / 4]) {
    uint64_t bp[NR / 2];
#pragma unroll
    for (int q = 0; q < NR / 4; ++q) {
      bp[2 * q] = pack2(b[q].x, b[q].y);
      bp[2 * q + 1] = pack2(b[q].z, b[q].w);
    }
#pragma unroll
    for (int i = 0; i < MR; ++i) {
      const uint64_t aa = pack2(a[i], a[i]);
#pragma unroll
      for (int j = 0; j < NR / 2; ++j) v[i][j] = ffma2(aa, bp[j], v[i][j]);
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
  __device__ __forceinline__ float total() const {
    uint64_t s[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s[i] = v[i][0];
#pragma unroll
      for (int j = 1; j < NR / 2; ++j) s[i] = fadd2(s[i], v[i][j]);
    }
#pragma unroll
    for (int i = 4; i < MR; ++i)
#pragma unroll
      for (int j = 0; j < NR / 2; ++j) s[i & 3] = fadd2(s[i & 3], v[i][j]);
    float lo, hi;
    unpack2(fadd2(fadd2(s[0], s[1]), fadd2(s[2], s[3])), lo, hi);
    return lo + hi;
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
template <bool TRANS_A, int MR>
__device__ __forceinline__ int acc_row(int warp, int lm, int i) {
  return TRANS_A ? (warp * (4 * MR) + lm * MR + i) : (warp * (4 * MR) + lm + 4 * i);
}
__device__ __forceinline__ int acc_col(int ln, int j) { return ln * 4 + 32 * (j >> 2) + (j & 3); }

// Thread-level encode (the idea of the reference's ft_sgemm_huge_thread, kernel/ft_sgemm/include/
// ft_sgemm_huge_thread.cuh:37): every thread keeps the checksum of its own 4 x NR outputs,
// chk += (sum of its 4 A values) * (sum of its NR B values) at every k, all in registers -- no
// shared-memory encoder, no extra barrier, but about 13 more instructions per k beside the 32
// packed FMAs.  Kept as a measured alternative to the block-level encoder (FT = 1).
template <int NR, int MR>
__device__ __forceinline__ float thread_checksum_step(const float (&a)[MR], const float4 (&b)[NR / 4], float chk) {
  uint64_t s2 = fadd2(pack2(b[0].x, b[0].y), pack2(b[0].z, b[0].w));
#pragma unroll
  for (int q = 1; q < NR / 4; ++q) s2 = fadd2(s2, fadd2(pack2(b[q].x, b[q].y), pack2(b[q].z, b[q].w)));
  float lo, hi;
  unpack2(s2, lo, hi);
  float as = (a[0] + a[1]) + (a[2] + a[3]);
  if (MR == 8) as += (a[4 % MR] + a[5 % MR]) + (a[6 % MR] + a[7 % MR]);
  return __fmaf_rn(as, lo + hi, chk);
}

template <int BM, int NR, int MR, int NSTAGES, bool PACKED, bool TRANS_A, int FT>
__global__ void __launch_bounds__(TileCfg<BM, NR, MR, NSTAGES>::THREADS, TileCfg<BM, NR, MR, NSTAGES>::MIN_BLOCKS)
sgemm_ffma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmSA, const __grid_constant__ CUtensorMap tmSB, const FfmaArgs p,
                  const FtArgs ft) {
  using Cfg = TileCfg<BM, NR, MR, NSTAGES>;
  constexpr int BN = Cfg::BN, WARPS = Cfg::WARPS, THREADS = Cfg::THREADS, BAND = Cfg::BAND, FSTAGES = Cfg::STAGES;
  constexpr int kStageA = Cfg::kStageA, kStageB = Cfg::kStageB, BROW = BN * 4;  // bytes per k row of the B stage
  extern __shared__ unsigned char smem_raw[];
  // round the dynamic shared window up to 1024 bytes without leaving the shared address space
  unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char *sA = smem;
  unsigned char *sB = smem + FSTAGES * kStageA;
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + Cfg::kBarOff);
  uint64_t *empty = full + FSTAGES;
  unsigned char *sCs = smem + Cfg::kCsOff;   // per stage: the slab's operand checksums, Asum[warp][32] then Bsum (1 KB)
  constexpr int kStageCs = Cfg::kStageCs;
  constexpr uint32_t kStageBytes = kStageA + kStageB + (FT == 1 ? kStageCs : 0);
  int *inj = reinterpret_cast<int *>(smem + Cfg::kMiscOff);
  int *nflag = inj + 8;
  int *flagged = inj + 9;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // Lanes of a warp: 4 (rows) x 8 (columns), the warp spanning all BN columns of 4*MR rows - or, for the plain K-major
  // kernel with 8 x 16 outputs per thread, 8 x 4 with the four warps in a 2 x 2 arrangement of 64 x 64 squares (what
  // the counters of cuBLAS's own SIMT SGEMM suggest it does).  Measured at 6144^3: FMA pipe 86.2 -> 88.0 % busy, 7.53 ->
  // 7.37 ms, with the same number of shared-memory wavefronts.
  constexpr bool SQUARE = (MR == 8 && TRANS_A && FT == 0 && BM == 128 && NR == 16);
  const int lm = SQUARE ? lane >> 2 : lane >> 3, ln = SQUARE ? lane & 3 : lane & 7;
  const int wm = warp >> 1, wn = warp & 1;   // SQUARE only
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  int tile_m, tile_n;
  const int split = p.k_splits > 1 ? (int)blockIdx.x / (tiles_m * tiles_n) : 0;
  tile_of_block((int)blockIdx.x - split * tiles_m * tiles_n, tiles_m, tiles_n, tile_m, tile_n);
  const int m0 = tile_m * BM, n0 = tile_n * BN;
  // this CTA's K-slabs: all of them, or one share of a split-K launch (possibly empty: it then writes zeros)
  const int kb0 = split * p.slabs_per_split;
  const int nkb_all = (p.K + FBK - 1) / FBK;
  const int nkb = p.k_splits > 1 ? max(0, min(p.slabs_per_split, nkb_all - kb0)) : nkb_all;

  {
    // an earlier CTA of this launch timed out: leave at once (one thread reads, so the whole CTA agrees)
    __shared__ int launch_aborted;
    if (threadIdx.x == 0) launch_aborted = b2::launch_aborted(p.status, p.seq) ? 1 : 0;
    __syncthreads();
    if (launch_aborted != 0) return;
  }
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < FSTAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], WARPS);
    }
    if (FT) *nflag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (FT == 1) {
      tma_prefetch_desc(&tmSA);
      tma_prefetch_desc(&tmSB);
    }
  }
  if (FT && warp == WARPS - 1) {
    // first planned fault that names this tile (a plan holds at most one per tile; tiles are
    // counted in units of this kernel's block tile)
    int found = 0x7fffffff;
    for (int f = lane; f < ft.n_faults; f += 32) {
      // the plan addresses 128 x 128 tiles; map its (row, col) into this kernel's tile grid
      const int gr = ft.plan[f].tile_m * 128 + ft.plan[f].row, gc = ft.plan[f].tile_n * 128 + ft.plan[f].col;
      if (gr / BM == tile_m && gc / BN == tile_n && f < found) found = f;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) found = min(found, __shfl_xor_sync(0xffffffffu, found, o));
    if (lane == 0) {
      inj[0] = (found != 0x7fffffff);
      if (inj[0]) {
        inj[1] = (ft.plan[found].tile_m * 128 + ft.plan[found].row) - m0;
        inj[2] = (ft.plan[found].tile_n * 128 + ft.plan[found].col) - n0;
        inj[3] = ft.plan[found].k_step;
        inj[4] = ft.plan[found].bit;
      }
    }
  }
  __syncthreads();
  uint32_t issued = 0;   // thread 0: stages it has filled so far
  if (tid == 0) {
    for (int s = 0; s < FSTAGES && s < nkb; ++s) {
      issued = (uint32_t)s + 1u;
      mbar_expect_tx(&full[s], kStageBytes);
      if (TRANS_A) tma_load_2d(sA + s * kStageA, &tmA, &full[s], m0, (kb0 + s) * FBK);
      else tma_load_2d(sA + s * kStageA, &tmA, &full[s], (kb0 + s) * FBK, m0);
      tma_load_2d(sB + s * kStageB, &tmB, &full[s], n0, (kb0 + s) * FBK);
      if (FT == 1) {
        tma_load_2d(sCs + s * kStageCs, &tmSA, &full[s], 0, (kb0 + s) * ft.nbands_pad + tile_m * WARPS);
        tma_load_2d(sCs + s * kStageCs + WARPS * 128, &tmSB, &full[s], 0, (kb0 + s) * tiles_n + tile_n);
      }
    }
  }

  // planned fault: the slab after which the owning thread flips a bit (-1: not this thread)
  int inj_kb = -1;
  if (FT && inj[0]) {
    const int r = inj[1], c = inj[2];
    const bool own = r >= 0 && r < BM && c >= 0 && c < BN && (r / BAND) == warp &&
                     (TRANS_A ? (((r % BAND) / MR) == lm) : ((r & 3) == lm)) && ((c & 31) >> 2) == ln;
    if (own) inj_kb = inj[3] < 0 ? 0 : (inj[3] >= nkb ? nkb - 1 : inj[3]);
  }

  Acc<PACKED, NR, MR> acc;
  acc.zero();
  // Byte offsets inside a stage.  A: row r at r*128, 16-byte chunk c of that row at
  // ((c ^ (r & 7)) << 4); rows of this thread are warp*16 + lm + 4*i, so r & 7 is lm for even
  // i and lm + 4 for odd i.  B: row k at k*BROW, column c at c*4.
  const uint32_t a_thread = SQUARE    ? (uint32_t)(wm * 64 + lm * MR) * 4u
                            : TRANS_A ? (uint32_t)(warp * BAND + lm * MR) * 4u
                                      : (uint32_t)(warp * BAND + lm) * 128u;
  const uint32_t a_swz = (uint32_t)lm << 4;
  const uint32_t b_thread = SQUARE ? (uint32_t)(wn * 64 + ln * 4) * 4u : (uint32_t)(ln * 4) * 4u;
  constexpr int BQ = SQUARE ? 64 : 128;   // bytes between a thread's groups of four columns
  uint64_t chk2[2] = {0ull, 0ull};  // running checksum of block (warp, ln) over this lane's k-range, packed
  float tchk = 0.f;                 // FT = 2: running checksum of this thread's own 4 x NR outputs
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
    // ---- ABFT (FT = 1): the slab's operand checksums came in with the stage; lane (g, r) = (ln, lm) folds
    // sum_{8 k of r} Asum_w[k] * Bsum_g[k] into its running checksum, issued from inside the unrolled FMA stream.
    // Bsum table: k = 8r + 4h + e of column set g at h*512 + (r*8 + g)*16 + e*4, so that the 32 lanes of a warp
    // read each half as one contiguous 512-byte row.
    auto fold = [&]() {
      const unsigned char *pw = sCs + s * kStageCs + warp * 128 + lm * 32;
      const unsigned char *pg = sCs + s * kStageCs + WARPS * 128 + (lm * 8 + ln) * 16;
      const ulonglong2 a01 = *reinterpret_cast<const ulonglong2 *>(pw);
      const ulonglong2 a23 = *reinterpret_cast<const ulonglong2 *>(pw + 16);
      const ulonglong2 g01 = *reinterpret_cast<const ulonglong2 *>(pg);
      const ulonglong2 g23 = *reinterpret_cast<const ulonglong2 *>(pg + 512);
      chk2[0] = ffma2(a01.x, g01.x, chk2[0]);
      chk2[1] = ffma2(a01.y, g01.y, chk2[1]);
      chk2[0] = ffma2(a23.x, g23.x, chk2[0]);
      chk2[1] = ffma2(a23.y, g23.y, chk2[1]);
    };
    const unsigned char *As = Ast + a_thread;
    const unsigned char *Bs = Bst + b_thread;
    if (TRANS_A) {
#pragma unroll
      for (int k = 0; k < FBK; ++k) {
        if (FT == 1 && k == 8) fold();
        float a[MR];
#pragma unroll
        for (int h = 0; h < MR / 4; ++h) {
          const float4 a4 = *reinterpret_cast<const float4 *>(As + k * (BM * 4) + h * 16);
          a[4 * h + 0] = a4.x; a[4 * h + 1] = a4.y; a[4 * h + 2] = a4.z; a[4 * h + 3] = a4.w;
        }
        float4 b[NR / 4];
#pragma unroll
        for (int q = 0; q < NR / 4; ++q) b[q] = *reinterpret_cast<const float4 *>(Bs + k * BROW + q * BQ);
        acc.step(a, b);
        if (FT == 2) tchk = thread_checksum_step<NR, MR>(a, b, tchk);
      }
    } else {
#pragma unroll
      for (int kc = 0; kc < FBK / 4; ++kc) {
        if (FT == 1 && kc == 2) fold();
        const uint32_t y0 = ((uint32_t)kc << 4) ^ a_swz, y1 = y0 ^ 64u;
        float4 a4[MR];
#pragma unroll
        for (int i = 0; i < MR; ++i)
          a4[i] = *reinterpret_cast<const float4 *>(As + ((i & 1) ? y1 : y0) + i * 512);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          float4 b[NR / 4];
#pragma unroll
          for (int q = 0; q < NR / 4; ++q) b[q] = *reinterpret_cast<const float4 *>(Bs + (kc * 4 + kk) * BROW + q * 128);
          float a[MR];
#pragma unroll
          for (int i = 0; i < MR; ++i) a[i] = (kk == 0) ? a4[i].x : (kk == 1) ? a4[i].y : (kk == 2) ? a4[i].z : a4[i].w;
          acc.step(a, b);
          if (FT == 2) tchk = thread_checksum_step<NR, MR>(a, b, tchk);
        }
      }
    }
    if (FT) {
      // ---- simulated soft error: flip one bit of one accumulator after this slab ----
      if (kb == inj_kb) {
        const int inj_i = TRANS_A ? (inj[1] % MR) : ((inj[1] % BAND) >> 2), inj_j = (inj[2] >> 5) * 4 + (inj[2] & 3);
        const uint32_t inj_mask = 1u << (inj[4] & 31);
#pragma unroll
        for (int i = 0; i < MR; ++i)
#pragma unroll
          for (int j = 0; j < NR; ++j)
            if (i == inj_i && j == inj_j) acc.set(i, j, __uint_as_float(__float_as_uint(acc.get(i, j)) ^ inj_mask));
        atomicAdd(&ft.report[1], 1);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
    // Refill, one slab behind: the stage that slab kb-1 used gets slab kb-1+FSTAGES once all
    // warps have released it.
    if (tid == 0 && kb >= 1) {
      const int kprev = kb - 1, knext = kprev + FSTAGES;
      if (knext < nkb) {
        const int sp = kprev % FSTAGES;
        if (!mbar_wait(&empty[sp], (uint32_t)(kprev / FSTAGES) & 1u)) {
          ok = false;
          break;
        }
        mbar_expect_tx(&full[sp], kStageBytes);
        issued = (uint32_t)knext + 1u;
        if (TRANS_A) tma_load_2d(sA + sp * kStageA, &tmA, &full[sp], m0, (kb0 + knext) * FBK);
        else tma_load_2d(sA + sp * kStageA, &tmA, &full[sp], (kb0 + knext) * FBK, m0);
        tma_load_2d(sB + sp * kStageB, &tmB, &full[sp], n0, (kb0 + knext) * FBK);
        if (FT == 1) {
          tma_load_2d(sCs + sp * kStageCs, &tmSA, &full[sp], 0, (kb0 + knext) * ft.nbands_pad + tile_m * WARPS);
          tma_load_2d(sCs + sp * kStageCs + WARPS * 128, &tmSB, &full[sp], 0, (kb0 + knext) * tiles_n + tile_n);
        }
      }
    }
  }
  if (!ok) {
    record_timeout(p.status, p.seq);
    if (tid == 0) ring_settle(full, FSTAGES, issued);   // no copy in flight into this CTA's shared memory when it leaves
    return;
  }

  if (FT) {
    // ---- verify in registers, then recompute the blocks that are out of tolerance ----
    float expect, actual = acc.total();
    if (FT == 2) {
      expect = tchk;
    } else {
      float c0, c1, c2, c3;
      unpack2(chk2[0], c0, c1);
      unpack2(chk2[1], c2, c3);
      expect = (c0 + c1) + (c2 + c3);
    }
    expect += __shfl_xor_sync(0xffffffffu, expect, 8);
    expect += __shfl_xor_sync(0xffffffffu, expect, 16);
    actual += __shfl_xor_sync(0xffffffffu, actual, 8);
    actual += __shfl_xor_sync(0xffffffffu, actual, 16);
    const float tau = ft.tau_scale ? ft.tau * __ldg(ft.tau_scale) : ft.tau;
    const bool bad = !(fabsf(actual - expect) <= tau);  // NaN-safe: a NaN difference is out of tolerance
    const int any_bad = __syncthreads_or(bad ? 1 : 0);      // also: the ring is idle from here on
    if (any_bad) {                                           // uniform over the block
      if (bad && lm == 0) flagged[atomicAdd(nflag, 1)] = warp * 8 + ln;
      __syncthreads();
      const int nf = *nflag;
      float *rec = reinterpret_cast<float *>(sA);  // [BAND rows][NR] recomputed outputs of one block
      for (int f = 0; f < nf; ++f) {
        const int bw = flagged[f] >> 3, bg = flagged[f] & 7;
        for (int e = tid; e < BAND * NR; e += THREADS) {
          const int er = e / NR, ec = e % NR;
          const int row = m0 + bw * BAND + er, col = n0 + acc_col(bg, ec);
          float v = 0.f;
          if (row < p.M && col < p.N) {
            const float *ap = TRANS_A ? ft.A + row : ft.A + (size_t)row * ft.lda;
            const size_t astep = TRANS_A ? (size_t)ft.lda : 1;
            const float *bp = ft.B + col;
            for (int k = 0; k < p.K; ++k) v = __fmaf_rn(ap[k * astep], bp[(size_t)k * ft.ldb], v);
          }
          rec[e] = v;
        }
        __syncthreads();
        if (warp == bw && ln == bg) {
          int fixed = 0;
#pragma unroll
          for (int i = 0; i < MR; ++i)
#pragma unroll
            for (int j = 0; j < NR; ++j) {
              const float want = rec[(acc_row<TRANS_A, MR>(0, lm, i)) * NR + j];
              if (__float_as_uint(want) != __float_as_uint(acc.get(i, j))) {
                acc.set(i, j, want);
                ++fixed;
              }
            }
          fixed += __shfl_xor_sync(0x01010101u << bg, fixed, 8);
          fixed += __shfl_xor_sync(0x01010101u << bg, fixed, 16);
          if (lm == 0) {
            if (fixed) {
              atomicAdd(&ft.report[2], 1);
              atomicAdd(&ft.report[3], fixed);
            } else {
              atomicAdd(&ft.report[5], 1);  // checksum out of tolerance but every output verified: false alarm
            }
          }
        }
        __syncthreads();
      }
    }
    if (tid == 0) atomicAdd(&ft.report[0], 1);
  }

  // Epilogue straight from registers: per row, 8 lanes x 16 bytes = 128 contiguous bytes per store.
  // (a split-K share goes to its own partial matrix unscaled: alpha = 1 is exact)
  const bool parts = p.k_splits > 1;
  float *const out_base = parts ? p.partial + (size_t)split * p.M * p.ldp : p.C;
  const int out_ld = parts ? p.ldp : p.ldc;
  const float alpha = parts ? 1.f : p.alpha, beta = parts ? 0.f : p.beta;
  const int vec_out = parts ? 1 : p.vec_c;
  const bool read_c = (beta != 0.f);
#pragma unroll
  for (int i = 0; i < MR; ++i) {
    const int row = m0 + (SQUARE ? wm * 64 + lm * MR + i : acc_row<TRANS_A, MR>(warp, lm, i));
    if (row >= p.M) continue;
    float *crow = out_base + (size_t)row * out_ld;
#pragma unroll
    for (int h = 0; h < NR / 4; ++h) {
      const int col = SQUARE ? n0 + wn * 64 + ln * 4 + 16 * h : n0 + ln * 4 + 32 * h;
      if (vec_out && col + 3 < p.N) {
        float4 o;
        if (read_c) {
          const float4 c = *reinterpret_cast<const float4 *>(crow + col);
          o.x = __fmaf_rn(alpha, acc.get(i, 4 * h + 0), __fmul_rn(beta, c.x));
          o.y = __fmaf_rn(alpha, acc.get(i, 4 * h + 1), __fmul_rn(beta, c.y));
          o.z = __fmaf_rn(alpha, acc.get(i, 4 * h + 2), __fmul_rn(beta, c.z));
          o.w = __fmaf_rn(alpha, acc.get(i, 4 * h + 3), __fmul_rn(beta, c.w));
        } else {
          o.x = __fmul_rn(alpha, acc.get(i, 4 * h + 0));
          o.y = __fmul_rn(alpha, acc.get(i, 4 * h + 1));
          o.z = __fmul_rn(alpha, acc.get(i, 4 * h + 2));
          o.w = __fmul_rn(alpha, acc.get(i, 4 * h + 3));
        }
        *reinterpret_cast<float4 *>(crow + col) = o;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (col + e < p.N) {
            const float a = acc.get(i, 4 * h + e);
            crow[col + e] = read_c ? __fmaf_rn(alpha, a, __fmul_rn(beta, crow[col + e])) : __fmul_rn(alpha, a);
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

static std::atomic<int> g_ffma_variant{-1};  // -1: pick from B2_FFMA_VARIANT (default packed)
static std::atomic<int> g_ffma_tile{-1};     // -1: automatic; otherwise an index into the tile table

// Sum of the split-K parts in ascending order of the split, then the usual epilogue: deterministic, one rounding per
// added part.  One thread per 4 consecutive columns.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ P, int S, int M, int N, int ldp, float alpha,
                                                            float beta, float *__restrict__ C, int ldc, int vec_c) {
  const int quads = (N + 3) / 4;
  const int64_t total = (int64_t)M * quads;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / quads), c = (int)(i - (int64_t)r * quads) * 4;
    const float *p0 = P + (size_t)r * ldp + c;
    float4 sum = *reinterpret_cast<const float4 *>(p0);
    for (int s = 1; s < S; ++s) {
      const float4 v = *reinterpret_cast<const float4 *>(p0 + (size_t)s * M * ldp);
      sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    float *cp = C + (size_t)r * ldc + c;
    const float in[4] = {sum.x, sum.y, sum.z, sum.w};
    if (vec_c && c + 3 < N) {
      float4 o;
      if (beta != 0.f) {
        const float4 cc = *reinterpret_cast<const float4 *>(cp);
        o.x = __fmaf_rn(alpha, sum.x, __fmul_rn(beta, cc.x)); o.y = __fmaf_rn(alpha, sum.y, __fmul_rn(beta, cc.y));
        o.z = __fmaf_rn(alpha, sum.z, __fmul_rn(beta, cc.z)); o.w = __fmaf_rn(alpha, sum.w, __fmul_rn(beta, cc.w));
      } else {
        o.x = __fmul_rn(alpha, sum.x); o.y = __fmul_rn(alpha, sum.y); o.z = __fmul_rn(alpha, sum.z); o.w = __fmul_rn(alpha, sum.w);
      }
      *reinterpret_cast<float4 *>(cp) = o;
    } else {
      for (int e = 0; e < 4 && c + e < N; ++e)
        cp[e] = beta != 0.f ? __fmaf_rn(alpha, in[e], __fmul_rn(beta, cp[e])) : __fmul_rn(alpha, in[e]);
    }
  }
}

static std::atomic<int> g_ffma_row_split{1};  // 1: a product may run as two launches on different tiles (rows split); 0: one launch
static std::atomic<int> g_ffma_split_k{0};  // 0: never (every output is one FMA chain over all of K); n > 1: n ways; -1: automatic

static int ffma_variant() {
  if (g_ffma_variant < 0) {
    const char *e = getenv("B2_FFMA_VARIANT");
    g_ffma_variant = e ? atoi(e) : 1;
    if (g_ffma_variant < 0 || g_ffma_variant > 1) g_ffma_variant = 1;
  }
  return g_ffma_variant;
}

// ---- ABFT pre-pass: the operand checksums of one product, one table entry per K-slab -------------------------
// Band checksums of A: out[(slab * nbands_pad + band) * 32 + k % 32] = sum over the band_rows rows of `band` of A(m, k)
// (rows past M, k past K and bands past the matrix count as zero).  trans = 0: A is M x K row-major; trans = 1:
// A is held K x M (the column-major operand of the kernel/ft_sgemm family, or the transposed copy in the
// workspace).  One block per (slab, 8 bands).
__global__ void __launch_bounds__(256) ft_encode_a_kernel(const float *__restrict__ A, int M, int K, int lda, int trans,
                                                          float *__restrict__ out, int nbands_pad, int band_rows) {
  const int slab = blockIdx.x, tid = threadIdx.x;
  float sum = 0.f;
  int kk, band;
  if (!trans) {
    kk = tid & 31;
    band = blockIdx.y * 8 + (tid >> 5);                  // a warp reads 32 consecutive k of one row at a time
    const int k = slab * FBK + kk;
    if (k < K) {
      const float *col = A + k;
#pragma unroll 4
      for (int i = 0; i < band_rows; ++i) {
        const int m = band * band_rows + i;
        if (m < M) sum += __ldg(col + (size_t)m * lda);
      }
    }
  } else {
    kk = tid >> 3;
    band = blockIdx.y * 8 + (tid & 7);                   // 8 lanes read 8 consecutive bands of one k
    const int k = slab * FBK + kk, m0 = band * band_rows;
    if (k < K && m0 < M) {
      const float *row = A + (size_t)k * lda + m0;
      if (m0 + band_rows - 1 < M && (((uintptr_t)row) & 15) == 0) {
        for (int q = 0; q < band_rows / 4; ++q) {
          const float4 v = __ldg(reinterpret_cast<const float4 *>(row) + q);
          sum += (v.x + v.y) + (v.z + v.w);
        }
      } else {
        for (int i = 0; i < band_rows && m0 + i < M; ++i) sum += __ldg(row + i);
      }
    }
  }
  if (band < nbands_pad) out[((size_t)slab * nbands_pad + band) * FBK + kk] = sum;
}

// Column-set checksums of B for tiles of BN = 8 * NR columns: per (slab, tile_n) a 1 KB block in which the entry of
// k (0..31) and column set g (0..7: tile columns g*4 + 32q + e, q < NR/4, e < 4) sits at float offset
// ((k >> 2) & 1) * 128 + ((k >> 3) * 8 + g) * 4 + (k & 3), the order in which the mainloop reads it.
template <int NR>
__global__ void __launch_bounds__(256) ft_encode_b_kernel(const float *__restrict__ B, int K, int N, int ldb,
                                                          float *__restrict__ out, int tiles_n) {
  const int slab = blockIdx.x, tile_n = blockIdx.y, tid = threadIdx.x;
  const int k = tid >> 3, g = tid & 7, row = slab * FBK + k;
  float sum = 0.f;
  if (row < K) {
    const float *r = B + (size_t)row * ldb;
#pragma unroll
    for (int q = 0; q < NR / 4; ++q) {
      const int col = tile_n * (8 * NR) + g * 4 + 32 * q;
      if (col + 3 < N && (((uintptr_t)(r + col)) & 15) == 0) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(r + col));
        sum += (v.x + v.y) + (v.z + v.w);
      } else {
        for (int e = 0; e < 4; ++e)
          if (col + e < N) sum += __ldg(r + col + e);
      }
    }
  }
  out[((size_t)slab * tiles_n + tile_n) * 256 + ((k >> 2) & 1) * 128 + ((k >> 3) * 8 + g) * 4 + (k & 3)] = sum;
}

// Upper bound, for any tile of the family, of the bytes the two tables of an M x N x K product take.
size_t ft_tables_bytes(int M, int N, int K) {
  const size_t slabs = ((size_t)K + FBK - 1) / FBK;
  return slabs * (((size_t)M / 16 + 9) * 128 + ((size_t)N / 64 + 1) * 1024) + 4096;
}

template <int BM, int NR, int MR, int NSTAGES, bool PACKED, bool TRANS_A, int FT>
static int launch_ffma(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tsa, const CUtensorMap &tsb,
                       const FfmaArgs &args, int grid, cudaStream_t s, const FtArgs &ft) {
  using Cfg = TileCfg<BM, NR, MR, NSTAGES>;
  int st = ensure_func_attributes((const void *)sgemm_ffma_kernel<BM, NR, MR, NSTAGES, PACKED, TRANS_A, FT>, args.device, Cfg::kSmem, 100);
  if (st != B2_OK) return st;
  sgemm_ffma_kernel<BM, NR, MR, NSTAGES, PACKED, TRANS_A, FT><<<grid, Cfg::THREADS, Cfg::kSmem, s>>>(ta, tb, tsa, tsb, args, ft);
  B2_CUDA(cudaGetLastError());
  return B2_OK;
}

// One row per generated tile: the launcher for each (packed?, transposed A?, ABFT?) combination.
typedef int (*FfmaLauncher)(const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const CUtensorMap &, const FfmaArgs &, int,
                            cudaStream_t, const FtArgs &);
struct FfmaTile {
  const char *name;
  int bm, bn, mr, stages, threads, ctas_per_sm;
  float efficiency;  // measured throughput at large sizes relative to the 128 x 128 tile of 4 x 16 thread tiles, used by the picker
  int min_waves;     // the picker considers the tile only for problems of at least this many waves of CTAs
  FfmaLauncher fn[2][2][2];  // [packed][trans_a][ft]
};

#define B2_FFMA_TILE(NAME, BM, NR, MR, ST, EFF, MIN_WAVES)                                                         \
  {NAME, BM, 8 * NR, MR, ST, TileCfg<BM, NR, MR, ST>::THREADS, TileCfg<BM, NR, MR, ST>::MIN_BLOCKS, EFF, MIN_WAVES, \
   {{{launch_ffma<BM, NR, MR, ST, false, false, false>, launch_ffma<BM, NR, MR, ST, false, false, true>},          \
     {launch_ffma<BM, NR, MR, ST, false, true, false>, launch_ffma<BM, NR, MR, ST, false, true, true>}},           \
    {{launch_ffma<BM, NR, MR, ST, true, false, false>, launch_ffma<BM, NR, MR, ST, true, false, true>},            \
     {launch_ffma<BM, NR, MR, ST, true, true, false>, launch_ffma<BM, NR, MR, ST, true, true, true>}}}},
static const FfmaTile g_tiles[] = {
#include "ffma_tiles.inc"
};
constexpr int kNumTiles = sizeof(g_tiles) / sizeof(g_tiles[0]);

// Picks the tile with the best predicted throughput: its measured efficiency times how well its
// CTA count fills whole waves of the CTAs that are co-resident on an SM.  The fill term matters
// less the more waves there are (the hardware back-fills), hence the 1/waves exponent.
// Ways of an automatic split-K for a tile whose grid has `ctas` CTAs: as many as fill the CTAs the GPU holds, at most 8,
// at least two K-slabs each.
static int auto_split_ways(const Context *ctx, const FfmaTile &tl, double ctas, int K) {
  int ways = (int)((double)ctx->sm_count * tl.ctas_per_sm / ctas);
  const int slabs = (K + FBK - 1) / FBK;
  if (ways > 8) ways = 8;
  if (ways > slabs / 2) ways = slabs / 2;
  return ways < 1 ? 1 : ways;
}

// Time model of one launch: the CTAs are dealt out over the SMs, and the CTAs resident on one SM share its FMA
// pipes, so the launch lasts as long as the SM with the most CTAs needs for them: ceil(CTAs / SMs) tiles of bm x bn
// outputs at the tile's measured efficiency.  (Counting whole waves of resident CTAs instead overrates large tiles
// whenever the last wave is partly filled: 2816^3 runs 8.6 % faster on 64 x 128 tiles than on 128 x 128, 2048^3 4.4 %
// faster on 64 x 64; this model ranks the seven tiles as measured from 1024^3 to 8192^3.)  Unit: outputs of one
// SM-round; a negative value: the tile is not considered for this shape.
static double tile_time(int sm_count, const FfmaTile &tl, int M, int N) {
  const double ctas = (double)((M + tl.bm - 1) / tl.bm) * ((N + tl.bn - 1) / tl.bn);
  // the 8-row thread tiles run 8 warps per SM: below two waves of resident CTAs they lose to the 16-warp tiles
  const double slots = (double)sm_count * ((tl.mr == 4 ? 512 : 256) / tl.threads);
  if (ctas / slots < (double)tl.min_waves) return -1.0;
  const double per_sm = ceil(ctas / (double)sm_count);
  double time = per_sm * (double)(tl.bm * tl.bn) / tl.efficiency;
  // an SM needs two warps per scheduler to keep its FMA pipes busy: a launch that leaves fewer resident runs
  // slower than the efficiency measured on full SMs says (1024^3: 128 CTAs of 4 warps, 32.8 TFLOP/s against 36.4)
  const double max_resident = (double)((tl.mr == 4 ? 512 : 256) / tl.threads);
  const double warps = (per_sm < max_resident ? per_sm : max_resident) * (tl.threads / 32);
  if (warps < 8.0) time *= sqrt(8.0 / warps);
  return time;
}
static int pick_tile_for(int sm_count, int M, int N, double *time_out = nullptr) {
  int best = 0;
  double best_time = 1e300;
  for (int t = 0; t < kNumTiles; ++t) {
    const double time = tile_time(sm_count, g_tiles[t], M, N);
    if (time >= 0.0 && time < best_time) {
      best_time = time;
      best = t;
    }
  }
  if (time_out) *time_out = best_time;
  return best;
}
// Two launches instead of one: the first `rows1` rows on tile t1, as many whole SM-rounds of it as fit, the rest on
// whatever tile suits the remainder best.  Every output is still one FMA chain over all of K whatever its tile, so
// the result is bit-identical; the split is taken when the model gives it 3 % or more over the best single launch
// (3840^3: 29 of 30 tile rows on 128 x 128 tiles and the last 128 rows on 32 x 64 tiles, measured +3.8 %).
struct RowSplit {
  int rows1 = 0, t1 = -1, t2 = -1;
};
static RowSplit plan_row_split(int sm_count, int M, int N) {
  RowSplit best;
  double single = 0.0;
  (void)pick_tile_for(sm_count, M, N, &single);
  double best_time = 0.97 * single;
  for (int t1 = 0; t1 < kNumTiles; ++t1) {
    const FfmaTile &tl = g_tiles[t1];
    const long long per_row = (N + tl.bn - 1) / tl.bn, tile_rows = (M + tl.bm - 1) / tl.bm;
    const long long rounds = tile_rows * per_row / sm_count;          // whole SM-rounds in the launch
    if (rounds < 1) continue;
    const long long rows_t = rounds * sm_count / per_row;              // tile rows that fit into them
    if (rows_t < 1 || rows_t >= tile_rows) continue;
    const int rows1 = (int)(rows_t * tl.bm);
    const double time1 = tile_time(sm_count, tl, rows1, N);
    if (time1 < 0.0) continue;
    double time2 = 0.0;
    const int t2 = pick_tile_for(sm_count, M - rows1, N, &time2);
    const double launch = 0.01 * (double)(128 * 128);                  // a second launch: a hundredth of a 128 x 128 SM-round
    if (time1 + time2 + launch < best_time) {
      best_time = time1 + time2 + launch;
      best.rows1 = rows1;
      best.t1 = t1;
      best.t2 = t2;
    }
  }
  return best;
}
static int pick_tile(const Context *ctx, int M, int N) {
  if (g_ffma_tile >= 0 && g_ffma_tile < kNumTiles) return g_ffma_tile;
  return pick_tile_for(ctx->sm_count, M, N);
}

int sgemm_ffma_dispatch_ft(Context *ctx, int trans_a, int M, int N, int K, float alpha, const float *A, int lda,
                           const float *B, int ldb, float beta, float *C, int ldc, const FtArgs *ft, cudaStream_t s);

// Y[c][r] = X[r][c] for a rows x cols matrix X (pitch ld) into Y (pitch ldy): 64 x 64 tiles through
// shared memory, both sides coalesced.
__global__ void __launch_bounds__(256) transpose_kernel(const float *__restrict__ X, int rows, int cols, int ld,
                                                        float *__restrict__ Y, int ldy) {
  __shared__ float t[64][65];
  const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64, tid = threadIdx.x;
#pragma unroll 4
  for (int e = tid; e < 64 * 64; e += 256) {
    const int rr = e >> 6, cc = e & 63;
    t[rr][cc] = (r0 + rr < rows && c0 + cc < cols) ? __ldcs(X + (size_t)(r0 + rr) * ld + c0 + cc) : 0.f;
  }
  __syncthreads();
#pragma unroll 4
  for (int e = tid; e < 64 * 64; e += 256) {
    const int cc = e >> 6, rr = e & 63;
    if (c0 + cc < cols && r0 + rr < ldy) Y[(size_t)(c0 + cc) * ldy + r0 + rr] = t[rr][cc];
  }
}

// The FFMA kernels run about 3.5 % faster with the A tile K-major in shared memory (one 128-bit load
// fetches four rows of one k instead of four k of one row, which frees the inner loop of the
// component selects).  A row-major A is therefore transposed into the workspace first when the
// pass pays for itself (it moves 8*M*K bytes; the gain grows with N) and scratch can be had.
static std::atomic<int> g_ft_level{1};   // ABFT encode granularity of the FFMA path: 1 block (16 x NR per warp slice), 2 thread
static std::atomic<int> g_ffma_transpose_a{1};
size_t ffma_workspace_bytes(int M, int N, int K) {
  if (!g_ffma_transpose_a || N < 2048 || M < 128 || K < 32) return 0;
  const size_t bytes = (size_t)K * (((size_t)M + 3) & ~(size_t)3) * sizeof(float) + 2048;
  // an optional speed-up does not take gigabytes: beyond 1 GiB (a 16384 x 16384 A) the row-major kernel runs
  return bytes <= ((size_t)1 << 30) + 2048 ? bytes : 0;
}

// trans_a = 0: A is M x K row-major (lda >= K).  trans_a = 1: A is given as K x M row-major
// (lda >= M), i.e. the column-major M x K operand of the kernel/ft_sgemm family.
int sgemm_ffma_dispatch(Context *ctx, int trans_a, int M, int N, int K, float alpha, const float *A, int lda,
                        const float *B, int ldb, float beta, float *C, int ldc, cudaStream_t s) {
  return sgemm_ffma_dispatch_ft(ctx, trans_a, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, nullptr, s);
}

// ft == nullptr: plain SGEMM.  Otherwise the ABFT kernel (operands must be describable to TMA,
// i.e. 16-byte aligned with leading dimensions that are multiples of 4).
static int ffma_dispatch_impl(Context *ctx, int trans_a, int M, int N, int K, float alpha, const float *A, int lda, const float *B,
                              int ldb, float beta, float *C, int ldc, const FtArgs *ft, cudaStream_t s, size_t ws_front,
                              int force_tile = -1);

int sgemm_ffma_dispatch_ft(Context *ctx, int trans_a, int M, int N, int K, float alpha, const float *A, int lda,
                           const float *B, int ldb, float beta, float *C, int ldc, const FtArgs *ft, cudaStream_t s) {
  return ffma_dispatch_impl(ctx, trans_a, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, ft, s, 0);
}

// ws_front: bytes at the front of the workspace that are in use (the transposed copy of A).
static int ffma_dispatch_impl(Context *ctx, int trans_a, int M, int N, int K, float alpha, const float *A, int lda, const float *B,
                              int ldb, float beta, float *C, int ldc, const FtArgs *ft, cudaStream_t s, size_t ws_front,
                              int force_tile) {
  if (M == 0 || N == 0) return B2_OK;
  if (K == 0 || alpha == 0.f) {
    if (beta == 1.f) return B2_OK;
    scale_c_kernel<<<ctx->sm_count * 4, 256, 0, s>>>(M, N, beta, C, ldc);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
  }
  const bool tma_ok = ((((uintptr_t)A | (uintptr_t)B) & 15) == 0) && (lda % 4 == 0) && (ldb % 4 == 0);
  if (ft) {
    B2_REQUIRE(tma_ok, B2_ERR_UNSUPPORTED,
               "ft_sgemm: A and B must be 16-byte aligned with lda, ldb multiples of 4 (lda=%d ldb=%d)", lda, ldb);
  }
  if (!tma_ok) {
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    sgemm_generic_kernel<<<grid, 256, 0, s>>>(M, N, K, alpha, A, trans_a ? 1 : lda, trans_a ? lda : 1, B, ldb, beta, C, ldc);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
  }
  // block-level ABFT keeps the two operand-checksum tables of this product in the workspace, behind the transposed
  // copy of A if there is one
  const bool tables = ft != nullptr && g_ft_level == 1;
  if (!trans_a) {
    const size_t want_t = ffma_workspace_bytes(M, N, K);
    const size_t want = want_t + (tables ? ft_tables_bytes(M, N, K) : 0);
    const bool fixed_too_small = ctx->ws != nullptr && !ctx->ws_owned && ctx->ws_bytes < want;
    if (want_t != 0 && !fixed_too_small) {
      if (ensure_workspace(ctx, want, s) == B2_OK) {
        const int mp = (M + 3) & ~3;
        float *AT = (float *)(((uintptr_t)ctx->ws + 1023) & ~(uintptr_t)1023);
        dim3 g((K + 63) / 64, (M + 63) / 64);
        transpose_kernel<<<g, 256, 0, s>>>(A, M, K, lda, AT, mp);
        B2_CUDA(cudaGetLastError());
        const size_t used = (((size_t)K * mp * sizeof(float)) + 2047) & ~(size_t)1023;
        if (ft) {
          FtArgs ft2 = *ft;
          ft2.A = AT;     // the recomputation reads the operand the kernel used
          ft2.lda = mp;
          return ffma_dispatch_impl(ctx, 1, M, N, K, alpha, AT, mp, B, ldb, beta, C, ldc, &ft2, s, used);
        }
        return ffma_dispatch_impl(ctx, 1, M, N, K, alpha, AT, mp, B, ldb, beta, C, ldc, nullptr, s, used);
      }
      set_error("");   // no scratch to be had: the row-major kernel needs none
    }
  }
  if (force_tile < 0 && ft == nullptr && g_ffma_tile < 0 && g_ffma_split_k == 0 && g_ffma_row_split != 0) {
    const RowSplit rs = plan_row_split(ctx->sm_count, M, N);
    if (rs.rows1 > 0) {
      int st1 = ffma_dispatch_impl(ctx, trans_a, rs.rows1, N, K, alpha, A, lda, B, ldb, beta, C, ldc, nullptr, s, ws_front, rs.t1);
      if (st1 != B2_OK) return st1;
      const float *A2 = trans_a ? A + rs.rows1 : A + (size_t)rs.rows1 * lda;
      return ffma_dispatch_impl(ctx, trans_a, M - rs.rows1, N, K, alpha, A2, lda, B, ldb, beta, C + (size_t)rs.rows1 * ldc, ldc, nullptr, s,
                                ws_front, rs.t2);
    }
  }
  const FfmaTile &tl = g_tiles[force_tile >= 0 ? force_tile : pick_tile(ctx, M, N)];
  CUtensorMap ta, tb, tsa, tsb;
  int st = trans_a ? make_tmap_2d(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, tl.bm, FBK, CU_TENSOR_MAP_SWIZZLE_NONE)
                   : make_tmap_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, FBK, tl.bm, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != B2_OK) return st;
  st = make_tmap_2d(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, tl.bn, FBK, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (st != B2_OK) return st;
  tsa = ta;
  tsb = tb;
  FfmaArgs args;
  args.C = C; args.M = M; args.N = N; args.K = K; args.ldc = ldc; args.alpha = alpha; args.beta = beta;
  args.vec_c = ((((uintptr_t)C) & 15) == 0 && (ldc % 4) == 0) ? 1 : 0;
  args.status = (int *)((char *)ctx->fixed + kFixedStatus);
  args.seq = next_launch_seq(ctx);
  args.device = ctx->device;
  const int tiles_m = (M + tl.bm - 1) / tl.bm, tiles_n = (N + tl.bn - 1) / tl.bn;
  int grid = tiles_m * tiles_n;
  args.k_splits = 1;
  args.slabs_per_split = 0;
  args.ldp = 0;
  args.partial = nullptr;
  // Split-K, opt-in (b2_set_ffma_split_k) and for the plain product only: with fewer CTAs than the GPU holds, the K loop of
  // every tile is cut into `ways` shares computed side by side and summed by a second kernel.  Each output is then a sum
  // of `ways` FMA chains instead of one, so the result differs in the last bits from the default's.
  if (!ft) {
    const int knob = g_ffma_split_k, slabs = (K + FBK - 1) / FBK;
    int ways = 1;
    if (knob > 1) ways = knob;
    else if (knob < 0) ways = auto_split_ways(ctx, tl, (double)grid, K);
    if (ways > 8) ways = 8;
    if (ways > slabs / 2) ways = slabs / 2;          // at least two K-slabs per share
    if (ways > 1) {
      const int ldp = (N + 3) & ~3;
      const size_t need = ws_front + (size_t)ways * M * ldp * sizeof(float) + 2048;
      if (ensure_workspace(ctx, need, s) == B2_OK) {
        args.k_splits = ways;
        args.slabs_per_split = (slabs + ways - 1) / ways;
        args.ldp = ldp;
        args.partial = (float *)((char *)(((uintptr_t)ctx->ws + 1023) & ~(uintptr_t)1023) + ws_front);
        grid *= ways;
      } else {
        set_error("");   // no scratch for the parts: one chain per output, as by default
      }
    }
  }
  FtArgs ftl = {nullptr, 0, 0.f, nullptr, nullptr, nullptr, nullptr, 0, 0, 0};
  if (ft) ftl = *ft;
  const bool thread_level = ft && g_ft_level == 2 && tl.bm == 128 && tl.bn == 128 && tl.mr == 4 && tl.stages == 3;   // built for that tile only
  if (ft && !thread_level) {
    // operand checksums of this product, one entry per K-slab, encoded once and brought in by TMA with each slab
    const int slabs = (K + FBK - 1) / FBK, band_rows = 4 * tl.mr, warps = tl.bm / band_rows;
    const int nbands_pad = tiles_m * warps;
    const size_t bytes_a = (size_t)slabs * nbands_pad * 128, bytes_b = (size_t)slabs * tiles_n * 1024;
    const size_t need = ws_front + bytes_a + bytes_b + 4096;
    st = ensure_workspace(ctx, need, s);
    if (st != B2_OK) {
      set_error("ft_sgemm: the operand-checksum tables need %zu bytes of workspace (b2_ft_sgemm_workspace_bytes); the handle has %zu",
                need, ctx->ws_bytes);
      return B2_ERR_WORKSPACE;
    }
    char *base = (char *)(((uintptr_t)ctx->ws + 1023) & ~(uintptr_t)1023) + ws_front;
    float *TA = (float *)base, *TB = (float *)(base + ((bytes_a + 1023) & ~(size_t)1023));
    ft_encode_a_kernel<<<dim3(slabs, (nbands_pad + 7) / 8), 256, 0, s>>>(A, M, K, lda, trans_a ? 1 : 0, TA, nbands_pad, band_rows);
    if (tl.bn == 128) ft_encode_b_kernel<16><<<dim3(slabs, tiles_n), 256, 0, s>>>(B, K, N, ldb, TB, tiles_n);
    else ft_encode_b_kernel<8><<<dim3(slabs, tiles_n), 256, 0, s>>>(B, K, N, ldb, TB, tiles_n);
    B2_CUDA(cudaGetLastError());
    st = make_tmap_2d(&tsa, TA, 32, (uint64_t)slabs * nbands_pad, 32, 32, warps, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st != B2_OK) return st;
    st = make_tmap_2d(&tsb, TB, 256, (uint64_t)slabs * tiles_n, 256, 256, 1, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st != B2_OK) return st;
    ftl.nbands_pad = nbands_pad;
  }
  const int packed = (ft != nullptr || ffma_variant() != 0) ? 1 : 0;
  if (thread_level)
    return trans_a ? launch_ffma<128, 16, 4, 3, true, true, 2>(ta, tb, tsa, tsb, args, grid, s, ftl)
                   : launch_ffma<128, 16, 4, 3, true, false, 2>(ta, tb, tsa, tsb, args, grid, s, ftl);
  st = tl.fn[packed][trans_a ? 1 : 0][ft ? 1 : 0](ta, tb, tsa, tsb, args, grid, s, ftl);
  if (st != B2_OK || args.k_splits <= 1) return st;
  const int64_t quads = (int64_t)M * ((N + 3) / 4);
  int64_t blocks = (quads + 255) / 256;
  if (blocks > (int64_t)ctx->sm_count * 8) blocks = (int64_t)ctx->sm_count * 8;
  splitk_reduce_kernel<<<(int)blocks, 256, 0, s>>>(args.partial, args.k_splits, M, N, args.ldp, alpha, beta, C, ldc, args.vec_c);
  B2_CUDA(cudaGetLastError());
  return B2_OK;
}

}  // namespace b2

using namespace b2;

namespace b2 {
int sgemm_3xtf32_dispatch(Context *ctx, int M, int N, int K, float alpha, const float *A, int lda, const float *B, int ldb,
                          float beta, float *C, int ldc, const FtArgs *ft, cudaStream_t s);
// knobs of the FFMA path that other translation units set
void set_ft_level_knob(int level) { g_ft_level = level; }
void set_ffma_transpose_a_knob(int on) { g_ffma_transpose_a = on; }
}

extern "C" {

// Selects the inner-loop variant of the FFMA kernel (0 scalar FFMA, 1 packed f32x2).  For
// benchmarking; results are bit-identical.
int b2_set_ffma_variant(int v) {
  B2_REQUIRE(v >= 0 && v <= 1, B2_ERR_INVALID_ARG, "b2_set_ffma_variant: %d not in 0..1", v);
  b2::g_ffma_variant = v;
  return B2_OK;
}

// Split-K of the plain FFMA SGEMM: 0 never (default), n > 1 n ways (at most 8, at least two K-slabs each), -1 as many
// ways as fill the GPU.
int b2_set_ffma_split_k(int ways) {
  B2_REQUIRE(ways >= -1 && ways != 1 && ways <= 8, B2_ERR_INVALID_ARG, "b2_set_ffma_split_k: %d is not -1, 0 or 2..8", ways);
  b2::g_ffma_split_k = ways;
  return B2_OK;
}

// Tile family (ffma_tiles.inc): number of tiles, description of tile i, and a pin for the
// picker (-1 = automatic).
int b2_ffma_tile_count(void) { return b2::kNumTiles; }
int b2_ffma_tile_info(int i, int *bm, int *bn, int *threads, const char **name) {
  B2_REQUIRE(i >= 0 && i < b2::kNumTiles, B2_ERR_INVALID_ARG, "b2_ffma_tile_info: tile %d not in 0..%d", i, b2::kNumTiles - 1);
  if (bm) *bm = b2::g_tiles[i].bm;
  if (bn) *bn = b2::g_tiles[i].bn;
  if (threads) *threads = b2::g_tiles[i].threads;
  if (name) *name = b2::g_tiles[i].name;
  return B2_OK;
}
// The tile the picker takes for an M x N output on a device of `sm_count` SMs (no pin, no device needed).
int b2_ffma_pick_tile(int M, int N, int sm_count) {
  B2_REQUIRE(M > 0 && N > 0 && sm_count > 0, B2_ERR_INVALID_ARG, "b2_ffma_pick_tile: M = %d, N = %d, sm_count = %d must be positive", M, N, sm_count);
  return b2::pick_tile_for(sm_count, M, N);
}
// 1 (default): the plain FFMA SGEMM may run as two launches, the first rows on one tile in whole SM-rounds and the rest
// on another, when the time model gives that 3 % or more (bit-identical results); 0: always one launch.
int b2_set_ffma_row_split(int on) {
  B2_REQUIRE(on == 0 || on == 1, B2_ERR_INVALID_ARG, "b2_set_ffma_row_split: %d is not 0 or 1", on);
  b2::g_ffma_row_split = on;
  return B2_OK;
}
// The split b2_set_ffma_row_split(1) would make for an M x N output on `sm_count` SMs: returns 1 and the rows of the
// first launch with the two tiles' indices, or 0 (one launch).  Host-side model, no device needed.
int b2_ffma_row_split_plan(int M, int N, int sm_count, int *rows1, int *tile1, int *tile2) {
  B2_REQUIRE(M > 0 && N > 0 && sm_count > 0, B2_ERR_INVALID_ARG, "b2_ffma_row_split_plan: M = %d, N = %d, sm_count = %d must be positive", M, N, sm_count);
  const b2::RowSplit rs = b2::plan_row_split(sm_count, M, N);
  if (rows1) *rows1 = rs.rows1;
  if (tile1) *tile1 = rs.t1;
  if (tile2) *tile2 = rs.t2;
  return rs.rows1 > 0 ? 1 : 0;
}
int b2_set_ffma_tile(int i) {
  B2_REQUIRE(i >= -1 && i < b2::kNumTiles, B2_ERR_INVALID_ARG, "b2_set_ffma_tile: tile %d not in -1..%d", i, b2::kNumTiles - 1);
  b2::g_ffma_tile = i;
  return B2_OK;
}

// Reads and clears the device status word that bounded waits set; synchronises the stream.
int b2_check_status(b2_handle h, void *stream) {
  B2_CONTEXT(ctx, h, "b2_check_status");
  int v = 0;
  int *dev = (int *)((char *)ctx->fixed + kFixedStatus);
  B2_CUDA(cudaMemcpyAsync(&v, dev, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  B2_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  if (v != 0) {
    B2_CUDA(cudaMemsetAsync(dev, 0, 8, (cudaStream_t)stream));   // the status word and the aborted launch's number
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
  B2_CONTEXT(ctx, h, "b2_sgemm");
  if (path == B2_PATH_3XTF32)
    return sgemm_3xtf32_dispatch(ctx, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, nullptr, (cudaStream_t)stream);
  return sgemm_ffma_dispatch(ctx, 0, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, (cudaStream_t)stream);
}

int sgemm(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C) {
  return b2_sgemm(nullptr, B2_PATH_FFMA, M, N, K, alpha, A, K, B, N, beta, C, N, nullptr);
}

int ref_sgemm_rowmajor(int N, float *A, float *B, float *C, float alpha, float beta) {
  return b2_sgemm(nullptr, B2_PATH_FFMA, N, N, N, alpha, A, N, B, N, beta, C, N, nullptr);
}

}  // extern "C"
