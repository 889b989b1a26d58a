/*
 * b2blas.h -- C ABI of the B200 (sm_100a) FP32 BLAS-kernel library.
 *
 * The reference project (shixun404/HPCDeepNeuralNetworks) has no library API: its
 * "interface" is the __global__ signature of each kernel plus the launch geometry that
 * each driver main() hard-codes.  Every entry point below replaces one such
 * kernel-plus-launch pair; the comment above it cites the reference file:line it stands
 * in for.  All pointers named *_dev / A / B / C / x / y are caller-owned DEVICE pointers.
 * Every function returns a b2_status (0 = ok, negative = error) and never exits the
 * process; b2_last_error() gives a thread-local human-readable message.
 *
 * `stream` arguments are cudaStream_t values passed as void* so that this header needs
 * no CUDA header; NULL is the default stream.  Work is enqueued, not synchronised,
 * unless stated otherwise.
 */
#ifndef B2BLAS_H
#define B2BLAS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  B2_OK = 0,
  B2_ERR_INVALID_ARG = -1,   /* null pointer, negative size, bad leading dimension */
  B2_ERR_UNSUPPORTED = -2,   /* shape the selected kernel cannot run (e.g. N not a tile multiple) */
  B2_ERR_CUDA = -3,          /* a CUDA runtime/driver call failed; see b2_last_error() */
  B2_ERR_TIMEOUT = -4,       /* a bounded device-side wait ran out (status word set by the kernel) */
  B2_ERR_UNCORRECTABLE = -5, /* ABFT found a fault it could not locate or correct */
  B2_ERR_WORKSPACE = -6      /* scratch workspace missing or too small */
} b2_status;

/* SGEMM math paths (north-star: two paths behind one launcher). */
enum { B2_PATH_FFMA = 0, B2_PATH_3XTF32 = 1 };

typedef struct b2_context *b2_handle;

/* ---- library / handle ------------------------------------------------------------- */

const char *b2_status_string(int status);
const char *b2_last_error(void);
/* Version as major*10000 + minor*100 + patch. */
int b2_version(void);

/* A handle owns per-device scratch (SDOT block partials, 3xTF32 split planes, ABFT
 * report words).  b2_create allocates a small fixed scratch with cudaMalloc on the
 * current device; larger scratch is either grown on demand (cudaMalloc, synchronising)
 * or supplied by the caller with b2_set_workspace (no allocation inside the library).
 * The scratch is shared by every call made on the handle: calls on one handle must be ordered
 * on one stream (or otherwise serialised); work on several streams takes one handle per stream.
 * A NULL handle means a default handle per device, with the same rule.  A handle belongs to the device that was
 * current in b2_create; calls that pass it while another device is current return B2_ERR_INVALID_ARG. */
int b2_create(b2_handle *out);
int b2_destroy(b2_handle h);
int b2_set_workspace(b2_handle h, void *dev_ptr, size_t bytes);
/* Bytes of workspace an MxNxK problem uses.  path = B2_PATH_3XTF32: the hi/lo planes of A and B are required; for
 * K >= 1024 the figure includes 20 MB of slots that let a partial last round of tiles be cut along K (see
 * b2_set_tf32_tail_split), and a caller-supplied workspace without them is accepted.
 * path = B2_PATH_FFMA: optional; when that much scratch is there (or the handle may grow its own) a
 * row-major A is transposed into it first, which makes large products about 3 % faster; 0 when the
 * pass would not pay or would need more than 1 GiB.  Results are bit-identical either way. */
size_t b2_sgemm_workspace_bytes(int path, int M, int N, int K);

/* ---- SGEMM: row-major C = alpha*A*B + beta*C --------------------------------------- */

/* North-star launcher `sgemm(M,N,K,alpha,A,B,beta,C)`: row-major NN, lda=K, ldb=N, ldc=N,
 * FFMA path, default stream, process-wide default handle.  Stands in for
 * kernel/sgemm/sgemm.cu:135-141 (sgemm_14<<<grid,256,64KB>>>) generalised to M,N,K. */
int sgemm(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);

/* Full form.  path = B2_PATH_FFMA | B2_PATH_3XTF32.  Any M,N,K >= 0, any lda>=K, ldb>=N,
 * ldc>=N.  beta == 0 means C is not read (BLAS convention; the reference kernels read it,
 * kernel/sgemm/include/kernel_14.cuh:5-9).  Replaces the `if (kernel_number == k)` launch
 * ladder of kernel/sgemm/sgemm.cu:70-144. */
int b2_sgemm(b2_handle h, int path, int M, int N, int K, float alpha, const float *A, int lda,
             const float *B, int ldb, float beta, float *C, int ldc, void *stream);

/* The reference's optimisation series sgemm_1..sgemm_14 as sm_100a kernels, square N only,
 * N a multiple of the rung's block tile (else B2_ERR_UNSUPPORTED), argument order exactly
 * as the reference kernels: (N, A, B, C, alpha, beta)
 * (kernel/sgemm/include/kernel_1.cuh:2 ... kernel_14.cuh:12; launches kernel/sgemm/sgemm.cu:70-141).
 * `threads_x` is the reference driver's 4th argv (tile edge t of rungs 1-5; ignored >= 6). */
int b2_sgemm_series(int kernel_id, int threads_x, int N, const float *A, const float *B, float *C,
                    float alpha, float beta, void *stream);
/* Reference-shaped shim, kernel/sgemm semantics: best kernel, default stream
 * (kernel/sgemm/include/kernel_14.cuh:12). */
int ref_sgemm_rowmajor(int N, float *A, float *B, float *C, float alpha, float beta);
/* Reference-shaped shim, kernel/ft_sgemm semantics: column-major A (MxK, lda=M),
 * B stored NxK (ldb=N), C MxN (ldc=M); C = alpha*A*B^T + beta*C
 * (kernel/ft_sgemm/include_code_gen/sgemm_huge.cuh:11, oracle call kernel/ft_sgemm/sgemm.cu:111). */
int ref_sgemm_colmajor_nt(int M, int N, int K, float *A, float *B, float *C, float alpha, float beta);

/* ---- ABFT (fault-tolerant) SGEMM --------------------------------------------------- */

/* One simulated soft error: after K-slab `k_step` (slab = 32 of K), bit `bit` of the FP32
 * accumulator of output element (tile_m*128 + row, tile_n*128 + col) is flipped in registers.
 * A plan holds at most one fault per 128x128 tile.  A simulated fault never faults the GPU.
 * On the 3xTF32 path the accumulators live in tensor memory for the whole K loop, so the bit is
 * flipped as the accumulator is read back after the last slab and `k_step` is ignored. */
typedef struct {
  int32_t tile_m, tile_n;
  int32_t row, col;     /* 0..127 inside the tile */
  int32_t k_step;       /* K-slab index (slab = 32 of K); clamped to the last slab */
  int32_t bit;          /* 0..31 */
} b2_fault;

typedef struct {
  int32_t tiles;          /* output tiles verified */
  int32_t injected;       /* faults applied from the plan */
  int32_t detected;       /* 16 x 16 blocks whose checksum was out of tolerance and held a wrong output */
  int32_t corrected;      /* accumulators found wrong by recomputation and replaced */
  int32_t uncorrectable;  /* always 0 with recompute-based correction; kept for callers that test it */
  int32_t false_alarms;   /* blocks out of tolerance whose outputs all verified */
  int32_t max_residual_bits; /* 3xTF32 path: bit pattern of the largest in-tolerance |sum - checksum| (a float >= 0) */
  int32_t reserved;
} b2_ft_report;

/* North-star launcher `ft_sgemm`: as sgemm() with checksum encode in the mainloop and
 * verify/locate/correct in the epilogue, no injection.  Stands in for
 * kernel/ft_sgemm/sgemm.cu:144-151 (ft_sgemm_huge launch) and
 * kernel/ft_sgemm/include/ft_sgemm_huge.cuh:21. */
int ft_sgemm(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);

/* Full form.  `plan_dev`/`n_faults`: optional device array of faults to inject (NULL/0 =
 * clean run).  `tau` > 0 is an absolute threshold; `tau` == 0 selects the default 2e-6*K, right for
 * operands of unit scale (uniform in [-1, 1)); `tau` < 0 selects the same default multiplied by
 * 3*rms(A)*rms(B), measured by one extra pass over A and B, for operands of any scale.  The
 * reference uses a fixed 0.1 (kernel/ft_sgemm/include/ft_sgemm_huge.cuh:30).
 * `report_dev`: optional device b2_ft_report that this call ADDS to (caller zeroes it).
 * path = B2_PATH_3XTF32: one checksum per output row and group of 32 columns, formed on the CUDA cores beside
 * the MMAs and corrected for what the tensor cores' truncating accumulation takes from a group over the K loop
 * (see b2_set_tf32_abft_bias); a group out of tolerance is recomputed in FP32 from A and B and every output further
 * than 0.75*tau from its recomputed value is replaced.  Default tau there is 2.5e-6*K: five times the largest
 * residual of clean products (4.7e-7*K for K = 256..8192) and half the path's accuracy bound of
 * 2e-5*sum_k|a||b| (5e-6*K for operands uniform in [-1, 1)), so a fault that would break that bound is always
 * found and repaired.  Operands that are all of one sign make the tensor cores' loss coherent; the plain 3xTF32
 * product bounds it with chunked accumulation (b2_set_tf32_chunk), this form accumulates over all of K in one go
 * and raises alarms on such data at K beyond about 2000 (every alarmed group is then recomputed in FP32: correct,
 * slow): use the FFMA path's ABFT for it.
 * Needs the workspace of b2_sgemm_workspace_bytes(B2_PATH_3XTF32, ...). */
int b2_ft_sgemm(b2_handle h, int path, int M, int N, int K, float alpha, const float *A, int lda,
                const float *B, int ldb, float beta, float *C, int ldc, const b2_fault *plan_dev,
                int n_faults, float tau, b2_ft_report *report_dev, void *stream);

/* Bytes of workspace the fault-tolerant product uses.  path = B2_PATH_FFMA: the operand-checksum tables (one entry
 * per K-slab of 32: about (M + 2N) * K / 8 bytes) are REQUIRED, the transposed copy of A of b2_sgemm_workspace_bytes
 * stays optional; a handle that owns its workspace grows it on demand (synchronising), a caller-supplied workspace
 * that is too small makes b2_ft_sgemm return B2_ERR_WORKSPACE.  path = B2_PATH_3XTF32: as b2_sgemm_workspace_bytes. */
size_t b2_ft_sgemm_workspace_bytes(int path, int M, int N, int K);

/* The same in the reference's own ABFT layout, column-major NT (A MxK lda=M, B NxK ldb=N, C MxN
 * ldc=M): ft_sgemm_<tile>(M, N, K, A, B, C, alpha, beta) of kernel/ft_sgemm/include/ft_sgemm_huge.cuh:21
 * and include_code_gen/ft_sgemm_wide.cuh:11.  The product is computed as C^T = B * A^T, so a planned
 * fault's (row, col) address C^T (row along N, col along M). */
int b2_ft_sgemm_colmajor_nt(b2_handle h, int M, int N, int K, float alpha, const float *A, const float *B,
                            float beta, float *C, const b2_fault *plan_dev, int n_faults, float tau,
                            b2_ft_report *report_dev, void *stream);
int ref_ft_sgemm_colmajor_nt(int M, int N, int K, float *A, float *B, float *C, float alpha, float beta);

/* ---- SAXPY / SDOT ----------------------------------------------------------------- */

/* y <- alpha*x + y, one fused multiply-add per element (bit-exact with fmaf on the host).
 * Replaces saxpy<<<ceil(n/4/tpb),tpb>>> / saxpy3 / _saxpy (kernel/saxpy/saxpy.cu:15-48,
 * launches :109-126). */
int saxpy(int n, float alpha, const float *x, float *y);
int b2_saxpy(b2_handle h, int64_t n, float alpha, const float *x, float *y, void *stream);

/* *result_dev <- sum_i x[i]*y[i].  OVERWRITES the result (the reference's _sdot
 * atomically adds into it, kernel/sdot/sdot.cu:32-33) and is deterministic run to run.
 * Replaces _sdot / sdot+reduction (kernel/sdot/sdot.cu:9-67, launches :156,:172-195). */
int sdot(int n, const float *x, const float *y, float *result_dev);
int b2_sdot(b2_handle h, int64_t n, const float *x, const float *y, float *result_dev, void *stream);
/* As b2_sdot, but also leaves the double-precision partial sum in *partial_dev (used by
 * the multi-GPU finish, which all-reduces the double). */
int b2_sdot_partial(b2_handle h, int64_t n, const float *x, const float *y, float *result_dev,
                    double *partial_dev, void *stream);

/* SDOT fused with its sum over GPUs (one process per GPU; no library collective).  Every rank owns a
 * 512-byte, 256-byte aligned, zero-initialised mailbox that every rank can address (peer memory over
 * NVLink, e.g. symmetric memory); `mailboxes` is this rank's host array of the `world` device addresses.
 * The kernel's last block stores this GPU's partial sum into every mailbox, flags it with `seq`, waits
 * (at most one second: then B2_ERR_TIMEOUT is recorded for b2_check_status and the local sum is returned)
 * for the other ranks' flags and adds the slots in rank order: *result_dev and *sum_dev (double, may be
 * NULL) hold the same bits on every rank.  All ranks call it the same number of times with seq = 1, 2, 3...
 * Stands in for the reference's single-GPU _sdot (kernel/sdot/sdot.cu:9) at world > 1; world <= 16. */
int b2_sdot_fused(b2_handle h, int64_t n, const float *x, const float *y, float *result_dev, double *sum_dev,
                  void *const *mailboxes, int rank, int world, uint64_t seq, void *stream);

/* SDOT for callers that must not allocate.  This entry point has no counterpart in the
 * reference.  It is meant for code that cannot call cudaMalloc at the point where it needs a dot
 * product: a plugin running under a host framework that has already handed all device memory to its
 * own pool, a callback on a latency-critical path where cudaMalloc's implicit device
 * synchronisation is not acceptable, or a process whose memory budget is fixed at start-up.  It
 * creates no handle and calls no cudaMalloc, cudaFree or other allocating routine: its scratch (one
 * double per block and a ticket word, 16.25 KB) is a static device array inside the library, which
 * every GPU that loads the library holds until the process exits.  Same arithmetic, same result
 * and same determinism as b2_sdot; *result_dev is overwritten.
 * Limits and rules:
 *  - n may be at most 2^30 elements; larger n returns B2_ERR_UNSUPPORTED (use b2_sdot).
 *  - The first call on each device looks up the device address of the scratch array (with that
 *    device current); make that first call before starting any stream capture.
 *  - All calls on a device share the one scratch array, so two calls that can overlap on the GPU
 *    (different streams, no dependency) race with each other; serialise them. */
int b2_sdot_static(int64_t n, const float *x, const float *y, float *result_dev, void *stream);

/* ---- SGEMM on host arrays --------------------------------------------------------------- */

/* The reference drivers hold their matrices on the host and move them with blocking cudaMemcpy calls around the
 * launch (kernel/sgemm/sgemm.cu:50-63, kernel/ft_sgemm/sgemm.cu:60-66).  A host plan does the same for one problem
 * shape with the transfers overlapped with the kernels: it owns device copies of A (M x K), B (K x N) and C (M x N),
 * three streams and their events.  first_panel_rows / panel_rows / panel_cols / panel_k = 0 select the defaults (half of
 * M / one wave of 128 x 128 tiles, 768 rows at N = 6144 / 768 / all of K); they are rounded to multiples of 128.  The first row panel of C is computed in column tiles
 * of panel_cols while the column panels of B arrive, the following row panels of panel_rows full width as their rows of A
 * and C land.  The plan computes on its own stream with the handle's scratch: do not use the handle elsewhere while
 * b2_sgemm_host runs. */
typedef struct b2_host_plan_s *b2_host_plan;
int b2_host_plan_create(b2_host_plan *out, b2_handle h, int path, int M, int N, int K, int first_panel_rows, int panel_rows,
                        int panel_cols, int panel_k);
int b2_host_plan_destroy(b2_host_plan p);
/* C <- alpha*A*B + beta*C on HOST arrays (row-major, leading dimensions in floats); returns when C is complete on
 * the host.  With one K panel (the default) every output sums all of K inside one kernel, so the FFMA result is
 * bit-identical to b2_sgemm on device copies; with panel_k < K block (p, q) accumulates into C with beta on the
 * first K panel and 1 afterwards.  Host memory from b2_host_alloc (or registered with cudaHostRegister) lets the
 * copies run asynchronously; pageable memory works but serialises them.  abft != 0 runs the fault-tolerant kernels
 * (default threshold, no injection) and, if report_host is not NULL, leaves the summed report there. */
int b2_sgemm_host(b2_host_plan p, float alpha, const float *A, int lda, const float *B, int ldb, float beta, float *C,
                  int ldc, int abft, b2_ft_report *report_host);
/* Page-locked host memory for the arrays above (cudaMallocHost / cudaFreeHost). */
int b2_host_alloc(void **out, size_t bytes);
int b2_host_free(void *p);

/* ---- multi-GPU: one process (or host thread) per GPU --------------------------------------- */

/* The reference is single-GPU.  Large products are sharded the way its row-major layout suggests: A and C by
 * contiguous row blocks, one per rank; B lives on `root` and is broadcast once per product in K panels (contiguous
 * row blocks of the row-major B) on a communication stream while the compute stream consumes the panels that have
 * landed: C_r = beta*C_r + alpha * sum_p A_r[:, panel p] * B[panel p, :].  There is no result exchange.  SDOT: every
 * rank reduces its slice to a double, then one all-reduce of that scalar.  The collectives are NCCL's, looked up at
 * run time in libnccl.so.2 (the copy already loaded in the process, else the system's): the library has no
 * link-time dependency on NCCL, and world = 1 needs none at all. */
typedef struct b2_mg_context *b2_mg_handle;
#define B2_MG_ID_BYTES 128
/* Rank 0 calls this and hands the 128 bytes to every rank by its own means (a file, MPI, a key-value store). */
int b2_mg_unique_id(void *id_out);
/* Collective over all ranks, each with its own GPU current: joins the communicator.  `h` is the handle whose
 * scratch the rank's kernels use (NULL: the device's default handle).  world = 1: `id` may be NULL. */
int b2_mg_create(b2_mg_handle *out, b2_handle h, int rank, int world, const void *id);
int b2_mg_destroy(b2_mg_handle mg);
/* Partition helpers (host only, no device needed): rank's contiguous block of M rows (block sizes differ by at most
 * one), and K panel `index` of width `panel` (the last may be narrower); b2_mg_k_panel returns the number of panels. */
int b2_mg_row_block(int64_t M, int rank, int world, int64_t *start, int64_t *rows);
int b2_mg_k_panel(int K, int panel, int index, int *k0, int *width);
/* Sharded row-major SGEMM (abft != 0: the fault-tolerant kernels; report_dev as in b2_ft_sgemm, may be NULL).
 * A_local (rows_r x K, lda) and C_local (rows_r x N, ldc) are this rank's row blocks of b2_mg_row_block(M, ...);
 * B (K x N, ldb) is a device buffer on every rank whose contents are valid on `root` at entry and on every rank once
 * the call's work has completed.  panel_k = 0 selects 4096.  Work is enqueued on `stream` and on the handle's own
 * communication stream; every rank must make the same sequence of b2_mg_* calls. */
int b2_mg_sgemm(b2_mg_handle mg, int path, int abft, int M, int N, int K, float alpha, const float *A_local, int lda,
                float *B, int ldb, float beta, float *C_local, int ldc, int root, int panel_k, b2_ft_report *report_dev,
                void *stream);
/* Sum over all ranks of x_local . y_local: *sum_dev (double) and *result_dev (float, may be NULL) hold the same value
 * on every rank once the stream has completed.  b2_sdot_fused is the form without any collective call. */
int b2_mg_sdot(b2_mg_handle mg, int64_t n_local, const float *x_local, const float *y_local, float *result_dev,
               double *sum_dev, void *stream);

/* ---- harness (rebuild of utils/utils.cu around CUDA events) ----------------------- */

/* Element i of the stream `seed` is a counter-based hash of (seed, i) mapped to a
 * multiple of 2^-23 in [-1,1); identical bits on host and device.  Replaces
 * generate_random_vector/matrix (utils/utils.cu:28-44), whose rand() grid cannot be
 * reproduced on the device. */
int b2_fill_uniform(float *dev, int64_t n, uint64_t seed, void *stream);
int b2_fill_uniform_host(float *host, int64_t n, uint64_t seed);
/* fill_vector (utils/utils.cu:15-19) on the device. */
int b2_fill_const(float *dev, int64_t n, float value, void *stream);
/* copy_matrix (utils/utils.cu:46-54) between host and device for a rectangular piece of a pitched matrix:
 * `rows` rows of `cols` floats, source pitch `ld_src` and destination pitch `ld_dst` in floats.
 * direction: 1 host -> device, 2 device -> host.  Asynchronous on `stream` when the host side is pinned.
 * The drivers copy whole matrices with cudaMemcpy (kernel/sgemm/sgemm.cu:60-63); the host-buffer pipeline
 * needs column panels. */
int b2_copy_matrix_async(float *dst, int64_t ld_dst, const float *src, int64_t ld_src, int64_t rows, int64_t cols,
                         int direction, void *stream);

/* verify_matrix (utils/utils.cu:75-91): first element with |ref-got| > abs_tol fails.
 * Device-side compare; returns 0 if all pass, 1 if any fail, <0 on error, and writes the
 * max |ref-got| to *max_abs_host when non-NULL.  Synchronises the stream.  Like the FFMA peak probes below it takes
 * no handle and keeps its two result words in the scratch of the device's default handle: calls on one device must
 * not overlap (different streams without ordering), nor overlap other work on the default handle. */
int b2_verify_matrix(const float *ref_dev, const float *got_dev, int64_t rows, int64_t cols,
                     int64_t ld, float abs_tol, float *max_abs_host, void *stream);

/* CUDA-event timer replacing saxpy_timer (utils/utils.cuh:56-77, host chrono). */
typedef struct b2_timer_s *b2_timer;
int b2_timer_create(b2_timer *out);
int b2_timer_destroy(b2_timer t);
int b2_timer_start(b2_timer t, void *stream);
int b2_timer_stop(b2_timer t, void *stream);
/* Synchronises on the stop event; milliseconds between start and stop. */
int b2_timer_elapsed_ms(b2_timer t, float *ms_out);

/* Register-only FFMA throughput microbenchmark: enqueues `launches` launches of a kernel
 * that performs `ffma_per_thread` dependent-chain-free FMAs per thread on every SM and
 * returns the total flop count (2 per FMA) in *flops_out.  Used to measure the FP32 SIMT
 * peak that SGEMM's roofline fraction is quoted against. */
int b2_ffma_peak_probe(int launches, int64_t ffma_per_thread, double *flops_out, void *stream);
/* The same probe issued as packed fma.rn.f32x2 (two FMAs per instruction). */
int b2_ffma2_peak_probe(int launches, int64_t ffma_per_thread, double *flops_out, void *stream);
/* Inner-loop variant of the FFMA SGEMM kernel (0 scalar FFMA, 1 packed f32x2, the default);
 * results are bit-identical, used for benchmarking only. */
int b2_set_ffma_variant(int v);
/* ABFT encode granularity of the FFMA path: 1 (default) block-level, the checksums of a warp's 16 x 16 blocks formed
 * through shared memory beside the FMAs; 2 thread-level, every thread keeps the checksum of its own outputs in
 * registers (kernel/ft_sgemm/include/ft_sgemm_huge_thread.cuh:37; 128x128 tile only).  Detection, location and
 * correction are the same. */
int b2_set_ft_level(int level);
/* 1 (default): the FFMA path may transpose a row-major A into the workspace first (see
 * b2_sgemm_workspace_bytes); 0: never. */
int b2_set_ffma_transpose_a(int on);
/* Split-K of the plain FFMA SGEMM, for products with fewer tiles than the GPU holds CTAs: 0 (default) never -- every
 * output is one FMA chain over all of K, the arithmetic the path is pinned on bit for bit; n = 2..8: the K loop of every
 * tile is cut into n shares computed side by side (partial sums in the handle's workspace, grown on demand) and added in
 * ascending order by a second kernel, deterministic but different in the last bits; -1: as many ways as fill the GPU.
 * The role of the reference generator's small tiles (kernel/ft_sgemm/code_gen/main.py:8-9) on a 148-SM GPU. */
int b2_set_ffma_split_k(int ways);
/* FFMA tile family (generated table): count, description of tile i, and a pin for the automatic
 * picker (-1 = automatic).  Stands in for the positional kernel ids of kernel/ft_sgemm/sgemm.cu:114-157. */
int b2_ffma_tile_count(void);
int b2_ffma_tile_info(int i, int *bm, int *bn, int *threads, const char **name);
int b2_set_ffma_tile(int i);
/* The index of the tile the picker takes for an M x N output on a device of `sm_count` SMs (148 on B200) when nothing is
 * pinned: a host-side time model, no device needed.  Negative status on invalid arguments. */
int b2_ffma_pick_tile(int M, int N, int sm_count);
/* 1 (default): the plain FFMA SGEMM may run as two launches, the first rows on one tile in whole SM-rounds and the remaining
 * rows on the tile that suits them best, when the time model gives that 3 % or more over the best single launch.  Every
 * output is one FMA chain over all of K on any tile, so results are bit-identical.  0: always one launch.
 * b2_ffma_row_split_plan returns 1 and the rows of the first launch with the two tile indices, or 0. */
int b2_set_ffma_row_split(int on);
int b2_ffma_row_split_plan(int M, int N, int sm_count, int *rows1, int *tile1, int *tile2);
/* Pins the tile width of the 3xTF32 kernel (128 or 256 output columns per CTA; 0 = automatic). */
int b2_set_tf32_tile_n(int n);
/* K-slab depth of the 3xTF32 kernel: 16 (64-byte swizzle, 4-6 stages) or 32 (128-byte swizzle, 2-3 stages). */
int b2_set_tf32_slab_k(int k);
/* 256x256 tiles on pairs of CTAs (tcgen05 cta_group::2, a cluster of two) in the 3xTF32 SGEMM: 0 never, 1 chosen
 * against 128x128 single-CTA tiles by whole waves (default), 2 always.  A width pinned with b2_set_tf32_tile_n
 * selects the single-CTA kernel of that width. */
int b2_set_tf32_pair(int on);
/* 1 (default): the CTA-pair kernels, plain and ABFT with CUDA-core checksums, are persistent (as many clusters as
 * the device holds, each walking several tiles, accumulator double-buffered in tensor memory so that a tile's
 * epilogue overlaps the next tile's MMAs); 0: one cluster per tile. */
int b2_set_tf32_persistent(int on);
/* Chunked accumulation of the plain 3xTF32 SGEMM.  The tensor cores add every MMA's products to the accumulator
 * with truncation, a loss per K-slab of 32 proportional to what the accumulator holds; over a long K loop it grows
 * with K and, for operands of one sign, adds up coherently (9e-5 of sum|a||b| at K = 8192).  With chunks, every
 * `slabs` K-slabs the tensor-memory accumulator is added to FP32 sums that the epilogue warps hold in registers and
 * started again from zero while the MMAs go on in a second buffer: the loss is bounded by that of one chunk whatever
 * K is (5.6e-6 for operands of one sign at the default 16, 2.5e-7 for signed operands at K = 8192) at no
 * measurable cost in time.  Applies to plain calls (not ABFT) whose K spans more than two chunks (K > 1024 at the
 * default) and no pinned tile width; 0: one accumulation over all of K; negative: the default.  No counterpart in
 * the reference. */
int b2_set_tf32_chunk(int slabs);
/* The hi/lo split of the 3xTF32 path inside the GEMM kernel (raw tiles of A and B by TMA, converted in shared memory
 * between the loads and the MMAs; no workspace, one launch instead of three; identical results): 0 never, 1 for very
 * small plain products where the saved launches outweigh the slower K-slabs (one wave of 128 x 128 tiles, K <= 512;
 * the default, and only while the kernel form is left to the library), 2 whenever A and B are 16-byte aligned with
 * lda, ldb multiples of 4 (accumulates over all of K in one go).  No counterpart in the reference. */
int b2_set_tf32_fused_split(int mode);
/* 1 (default): when the tiles of a chunked CTA-pair call (or of the fault-tolerant CTA-pair kernel, which cuts in units
 * of one K-slab and verifies every run against the checksums of its own k range) leave at least half of the clusters
 * idle in the last round,
 * each tile of that round is cut along K into runs of whole chunks on different clusters; the runs' sums go through
 * the workspace and a second kernel adds them in K order and applies alpha and beta (deterministic for a given shape
 * and device; identical to the uncut result when every run is one chunk, else different in the last bits).  A
 * caller-supplied workspace smaller than b2_sgemm_workspace_bytes() but large enough for the operand planes is
 * accepted, and the last round then runs tile by tile.  0: every tile on one cluster.  No counterpart in the
 * reference. */
int b2_set_tf32_tail_split(int on);
/* The cut that b2_set_tf32_tail_split(1) makes for `tiles` 256 x 256 tiles on `clusters` clusters and a K loop of K in
 * chunks of `chunk_slabs` K-slabs: returns 1 and the first cut tile, the runs per tile and the chunks of the longest
 * run (any of the three pointers may be NULL), or 0 when the last round is left whole.  For tests and tools. */
int b2_tf32_tail_plan(int tiles, int clusters, int K, int chunk_slabs, int *first, int *parts, int *longest);
/* The tensor cores add each MMA's products to the accumulator with truncation, which costs an accumulator a
 * fraction of its value per K-slab of 32 (about 4e-7 on B200, the built-in figure; the same for uniform and normal
 * operands of any scale).  The CUDA-core checksums keep, beside each checksum, its sum over the K-slabs, and the
 * verification expects the group sum to fall short of the checksum by `bias` times that sum.  bias < 0 restores the
 * built-in figure; 0 switches the correction off (the clean residual is then 15 times larger). */
int b2_set_tf32_abft_bias(float bias);
/* Reads and clears the device status word that bounded waits set; synchronises the stream.
 * Returns 0 or the recorded negative status.  The word is sticky until it is read here, but it does not stop later
 * work: a wait that runs out ends only the launch it happened in (that launch's output is then incomplete), and
 * launches made afterwards on the handle run normally. */
int b2_check_status(b2_handle h, void *stream);

/* Self-test of the bounded-wait path: one block waits `timeout_us` (1..100000) on a barrier that
 * nothing completes, gives up and records B2_ERR_TIMEOUT in the handle's status word, which
 * b2_check_status then returns.  The GPU context stays usable; nothing faults or hangs. */
int b2_selftest_wait_timeout(b2_handle h, int timeout_us, void *stream);

/* getDetails (utils/utils.cu:21-26): SM count and clock of the current device. */
int b2_device_info(int *sm_count, int *sm_clock_khz, size_t *global_mem_bytes);

#ifdef __cplusplus
}
#endif
#endif /* B2BLAS_H */
