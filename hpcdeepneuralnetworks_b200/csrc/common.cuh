// Shared host/device helpers of the b2blas kernels: status plumbing, the seeded input
// hash, and thin inline-PTX wrappers for the sm_100a features the kernels use
// (mbarrier, TMA tiled loads, tcgen05/TMEM).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/b2blas.h"

namespace b2 {

// ---- host-side status plumbing -------------------------------------------------------
void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what, const char *file, int line);

#define B2_CUDA(call)                                                        \
  do {                                                                       \
    cudaError_t e__ = (call);                                                \
    if (e__ != cudaSuccess) return ::b2::cuda_fail(e__, #call, __FILE__, __LINE__); \
  } while (0)

#define B2_REQUIRE(cond, status, ...)        \
  do {                                       \
    if (!(cond)) {                           \
      ::b2::set_error(__VA_ARGS__);          \
      return (status);                       \
    }                                        \
  } while (0)

// Scratch owner behind b2_handle.
struct Context {
  int device = -1;
  void *fixed = nullptr;      // small scratch allocated at create (SDOT partials, counters, status)
  size_t fixed_bytes = 0;
  void *ws = nullptr;         // large workspace (3xTF32 planes)
  size_t ws_bytes = 0;
  bool ws_owned = false;
  int sm_count = 0;
  int max_pairs = -1;         // CTA pairs of the 3xTF32 kernels this device holds at once (-1: not asked yet)
  unsigned int launch_seq = 0;  // number of the last SGEMM launch made on this handle (see next_launch_seq)
};
Context *default_context();           // process-wide, created on first use for the current device
// The context behind a handle (NULL: the current device's default handle), or nullptr with the error text set when
// there is none or when the handle belongs to another device than the current one.
Context *resolve_context(b2_handle h, const char *who);
// cudaFuncSetAttribute acts on the current device only: sets the dynamic shared-memory limit (and, when
// carveout >= 0, the preferred carve-out) of `func` once per device.
int ensure_func_attributes(const void *func, int device, int dynamic_smem_bytes, int carveout = -1);
// Every SGEMM launch on a handle gets a number.  A CTA whose bounded wait runs out stores that number in the
// handle's abort word (and B2_ERR_TIMEOUT in the sticky status word); CTAs of the same launch that start later
// see their own number there and leave at once, launches made afterwards carry another number and run normally.
unsigned int next_launch_seq(Context *ctx);
#define B2_CONTEXT(ctx, h, who)                                   \
  ::b2::Context *ctx = ::b2::resolve_context((h), (who));         \
  if (!ctx) return (h) ? B2_ERR_INVALID_ARG : B2_ERR_CUDA
int ensure_workspace(Context *ctx, size_t bytes, cudaStream_t s);
// Enqueues the reduction that leaves 3 * rms(X1) * rms(X2) in the context's scratch (1 for operands uniform in
// [-1, 1)) and returns the device address of that float: the factor by which rounding noise, and so an ABFT
// threshold, grows with the operands' scale.
int ft_data_scale(Context *ctx, const float *X1, int rows1, int cols1, int ld1, const float *X2, int rows2, int cols2,
                  int ld2, cudaStream_t s, const float **scale_dev);

// Layout of Context::fixed (all offsets 256-byte aligned).
constexpr size_t kSdotMaxBlocks = 4096;
constexpr size_t kFixedSdotPartials = 0;                                  // double[kSdotMaxBlocks]
constexpr size_t kFixedSdotTicket = kSdotMaxBlocks * sizeof(double);      // unsigned int
constexpr size_t kFixedStatus = kFixedSdotTicket + 256;                   // int status word of bounded waits (sticky), then the abort word
constexpr size_t kFixedVerify = kFixedStatus + 256;                       // verify_matrix result {uint fails, uint maxbits}
constexpr size_t kFixedFtReport = kFixedVerify + 256;                     // b2_ft_report scratch
constexpr size_t kFixedFtScale = kFixedFtReport + 256;                    // double ssA, ssB; float scale (ABFT threshold scaling)
constexpr size_t kFixedBytes = kFixedFtScale + 256;

// cuTensorMapEncodeTiled fetched through the runtime (no link-time libcuda dependency, so
// the shared object still loads on a machine without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();
// 2-D fp32 tensor map: `inner` contiguous elements, `outer` rows of pitch `ld` elements.
int make_tmap_2d(CUtensorMap *out, const float *base, uint64_t inner, uint64_t outer, uint64_t ld,
                 uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz);

// ---- seeded input hash (bit-identical to oracle.c o_uniform_at) -------------------------
__host__ __device__ inline uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__host__ __device__ inline float uniform_at(uint64_t mixed_seed, uint64_t i) {
  uint64_t h = mix64(mixed_seed ^ (i * 0xD1342543DE82EF95ull));
  uint32_t u = (uint32_t)(h >> 40);
  return (float)u * (1.0f / 8388608.0f) - 1.0f;
}

// What an ABFT launch needs beyond the plain SGEMM arguments (both math paths).
struct FtArgs {
  const b2_fault *plan;
  int n_faults;
  float tau;                // threshold for operands of unit scale (uniform in [-1, 1))
  const float *tau_scale;   // device float that multiplies tau and follows the operands' scale, or NULL
  int *report;  // b2_ft_report as ints: tiles, injected, detected, corrected, uncorrectable, false alarms, max residual bits
  const float *A, *B;
  int lda, ldb;
  int nbands_pad;   // FFMA path: 16-row bands of A per K-slab in the table of A's band checksums
};

#ifdef __CUDACC__
// ---- device: mbarrier --------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: polls the barrier and gives up about one second after the first failed poll
// (wall clock of the device's global timer, checked every 256 polls) or after `limit` polls,
// whichever comes first; returns false, the caller records B2_ERR_TIMEOUT and leaves.
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = (1u << 22),
                                          uint64_t limit_ns = 1000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 1; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 0 && global_timer_ns() - t0 > limit_ns) return false;
  }
  return false;
}

// After a wait has run out somewhere in the CTA: the thread that issued the ring's TMA loads waits, with a short
// bound, for the (at most `stages`) loads that may still be in flight to land, so that nothing is being written
// into the CTA's shared memory when it leaves.  `issued` counts the stages that thread has filled so far.
__device__ __forceinline__ void ring_settle(uint64_t *full, int stages, uint32_t issued) {
  const uint32_t first = issued > (uint32_t)stages ? issued - (uint32_t)stages : 0u;
  for (uint32_t j = first; j < issued; ++j) (void)mbar_wait(&full[j % stages], (j / stages) & 1u, 1u << 18, 100000000ull);
}

// A bounded wait ran out in the launch numbered `seq`: record it (status[0] sticky for b2_check_status, status[1]
// the number of the launch, which lets the launch's remaining CTAs leave at once).
__device__ __forceinline__ void record_timeout(int *status, unsigned int seq) {
  atomicExch(status, (int)B2_ERR_TIMEOUT);
  atomicExch(reinterpret_cast<unsigned int *>(status) + 1, seq);
}
__device__ __forceinline__ bool launch_aborted(const int *status, unsigned int seq) {
  return *(reinterpret_cast<const volatile unsigned int *>(status) + 1) == seq;
}

// ---- device: TMA -----------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)m) : "memory");
}
// 2-D tiled load global -> shared::cta, completion on an mbarrier.  x (inner coordinate)
// times 4 bytes must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *m, uint64_t *bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"((uint64_t)m), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// 2-D tiled store shared::cta -> global (elements outside the tensor are not written); x as above, and the
// coordinates are never negative.  The store belongs to the issuing thread's bulk group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *m, const void *smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"((uint64_t)m),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the issuing thread's bulk stores have read their shared-memory source / have completed
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- device: tcgen05 / TMEM --------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem desc] * B[smem desc], TF32 inputs, FP32 accumulate; one thread issues.
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// mbarrier arrives once every previously issued tcgen05.mma of this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// ---- device: CTA pairs (cluster of two, tcgen05 cta_group::2) ------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t cta_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
  return r;
}
// one arrival on an mbarrier of another CTA of the cluster, given by its shared::cluster address (no release:
// a releasing arrive from the MMA-issuing thread stalled it for about a microsecond per K-slab)
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ uint32_t ld_shared_cluster_u32(uint32_t cluster_addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
  return v;
}
// A bounded wait of a CTA pair ran out: raise the abort flag of BOTH CTAs (same shared-memory offset in each), so that
// the peer's roles leave their polling loops at once instead of sitting out their own limit.  Both CTAs stay resident
// until the kernel's final cluster barrier, so the remote word exists whenever this runs.
__device__ __forceinline__ void pair_abort(volatile int *flag) {
  *flag = 1;
  const uint32_t peer = mapa_u32(smem_u32(const_cast<const int *>(flag)), cluster_ctarank() ^ 1u);
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer), "r"(1) : "memory");
}
// every thread of both CTAs arrives and waits (release/acquire)
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 2-D tiled load into this CTA's shared memory whose completion is signalled on an mbarrier given
// by its shared::cluster address (the pair leader's barrier).  No multicast: each CTA fetches
// its own tile.
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *m, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"((uint64_t)m), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// One MMA over both CTAs of the pair: M = 256 (128 rows from each CTA's A tile), B halves from each
// CTA's shared memory at the same offsets, accumulator rows in each CTA's own TMEM.
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The barrier at this offset in every CTA of `cta_mask` gets one arrival once all earlier MMAs of
// this thread have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(cta_mask)
               : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base_lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 1 column.
__device__ __forceinline__ uint32_t tmem_ld_32x1(uint32_t taddr) {
  uint32_t v;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v) : "r"(taddr) : "memory");
  return v;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of tcgen05.mma (sm_100 format): start address, leading and
// stride byte offsets in 16-byte units, descriptor version 1, swizzle mode in bits 61..63
// (0 none, 2 = 128-byte, 4 = 64-byte, 6 = 32-byte).
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout_type) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(layout_type & 7) << 61;
  return d;
}
// Instruction descriptor of kind::tf32, FP32 accumulator, dense.  a_mn/b_mn: 0 = K-major
// operand, 1 = MN-major operand.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int M, int N, int a_mn, int b_mn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
#endif  // __CUDACC__

}  // namespace b2
