// SGEMM on HOST arrays: the situation of the reference drivers before their cudaMemcpy calls
// (kernel/sgemm/sgemm.cu:50-63: malloc, fill, cudaMemcpy in, launch, cudaMemcpy out), as one entry point that
// overlaps the transfers with the kernels.  A plan owns the device copies of A, B and C, three streams and the
// events between them; b2_sgemm_host runs one product through it and returns when C is back on the host.
//
// Default schedule (one K panel; every output sums all of K in one kernel, so the FFMA result is bit-identical
// to a single device call): C is cut into row panels.  B has to be on the device before a full-width row panel
// can be computed, so the FIRST row panel is cut further into column panels and computed tile by tile while the
// column panels of B (and of C) arrive as pitched copies; the following row panels are one full-width GEMM each,
// issued as soon as their rows of A and C have landed; a row panel of C travels back on a third stream when it
// is done.  With panel_k > 0 the second cut is along K instead (rows of B, contiguous): row panels and K panels
// are sent alternately and block (p, q) accumulates into C_p with beta on the first K panel and 1 afterwards.
#include <vector>

#include "common.cuh"

namespace b2 {
int sgemm_dispatch(Context *ctx, int path, bool abft, int M, int N, int K, float alpha, const float *A, int lda, const float *B,
                   int ldb, float beta, float *C, int ldc, b2_ft_report *report_dev, cudaStream_t s);
}
using namespace b2;

struct b2_host_plan_s {
  Context *ctx = nullptr;
  int path = 0, M = 0, N = 0, K = 0;
  int pr0 = 0, pr = 0, pc = 0, pk = 0;   // panel sizes: rows of the first row panel, of the others, columns of the first panel's tiles, K (== K: one panel)
  float *dA = nullptr, *dB = nullptr, *dC = nullptr;
  b2_ft_report *report = nullptr;   // device
  cudaStream_t compute = nullptr, h2d = nullptr, d2h = nullptr;
  std::vector<cudaEvent_t> events;
  size_t next_event = 0;
};

static int round_panel(int want, int extent, int floor_at) {
  if (extent < floor_at) return extent;
  int p = want < extent ? want : extent;
  p = (p + 127) / 128 * 128;
  return p < 128 ? 128 : p;
}

static int plan_event(b2_host_plan_s *p, cudaEvent_t *out) {
  if (p->next_event == p->events.size()) {
    cudaEvent_t e;
    B2_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    p->events.push_back(e);
  }
  *out = p->events[p->next_event++];
  return B2_OK;
}

// records an event on `from` and makes `to` wait for it
static int chain(b2_host_plan_s *p, cudaStream_t from, cudaStream_t to) {
  cudaEvent_t e;
  int st = plan_event(p, &e);
  if (st != B2_OK) return st;
  B2_CUDA(cudaEventRecord(e, from));
  B2_CUDA(cudaStreamWaitEvent(to, e, 0));
  return B2_OK;
}

static int copy2d(float *dst, size_t ld_dst, const float *src, size_t ld_src, int rows, int cols, cudaMemcpyKind kind, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return B2_OK;
  B2_CUDA(cudaMemcpy2DAsync(dst, ld_dst * sizeof(float), src, ld_src * sizeof(float), (size_t)cols * sizeof(float), (size_t)rows, kind, s));
  return B2_OK;
}

#define B2_TRY(call)                 \
  do {                               \
    int st__ = (call);               \
    if (st__ != B2_OK) return st__;  \
  } while (0)

extern "C" {

int b2_host_alloc(void **out, size_t bytes) {
  B2_REQUIRE(out != nullptr, B2_ERR_INVALID_ARG, "b2_host_alloc: out is NULL");
  B2_CUDA(cudaMallocHost(out, bytes ? bytes : 1));
  return B2_OK;
}

int b2_host_free(void *p) {
  if (p) B2_CUDA(cudaFreeHost(p));
  return B2_OK;
}

int b2_host_plan_destroy(b2_host_plan p) {
  if (!p) return B2_OK;
  if (p->compute) cudaStreamSynchronize(p->compute);
  if (p->h2d) cudaStreamSynchronize(p->h2d);
  if (p->d2h) cudaStreamSynchronize(p->d2h);
  for (cudaEvent_t e : p->events) cudaEventDestroy(e);
  if (p->compute) cudaStreamDestroy(p->compute);
  if (p->h2d) cudaStreamDestroy(p->h2d);
  if (p->d2h) cudaStreamDestroy(p->d2h);
  cudaFree(p->dA);
  cudaFree(p->dB);
  cudaFree(p->dC);
  cudaFree(p->report);
  delete p;
  return B2_OK;
}

int b2_host_plan_create(b2_host_plan *out, b2_handle h, int path, int M, int N, int K, int first_panel_rows, int panel_rows,
                        int panel_cols, int panel_k) {
  B2_REQUIRE(out != nullptr, B2_ERR_INVALID_ARG, "b2_host_plan_create: out is NULL");
  B2_REQUIRE(path == B2_PATH_FFMA || path == B2_PATH_3XTF32, B2_ERR_INVALID_ARG, "b2_host_plan_create: unknown path %d", path);
  B2_REQUIRE(M >= 0 && N >= 0 && K >= 0, B2_ERR_INVALID_ARG, "b2_host_plan_create: negative dimension (M=%d N=%d K=%d)", M, N, K);
  B2_REQUIRE(first_panel_rows >= 0 && panel_rows >= 0 && panel_cols >= 0 && panel_k >= 0, B2_ERR_INVALID_ARG,
             "b2_host_plan_create: negative panel size");
  B2_CONTEXT(ctx, h, "b2_host_plan_create");
  b2_host_plan_s *p = new b2_host_plan_s();
  p->ctx = ctx;
  p->path = path;
  p->M = M; p->N = N; p->K = K;
  // Defaults.  The first row panel is half of C, computed in column tiles of 768 behind the column panels of B: a
  // 3072 x 768 tile of a 6144^3 product takes about as long as its share of B and C takes to arrive, so the kernels keep
  // pace with the link while B streams in.  The other half follows in row panels that are one wave of 128 x 128 tiles
  // each (768 rows at N = 6144: 288 tiles for the 296 CTAs a B200 holds), short enough that the last kernel and the last
  // copy back add little after the last byte has gone in.  Measured at 6144^3: 12.5 ms with four panels of 1536, 11.05 ms so.
  int wave_rows = 128 * ((2 * ctx->sm_count) / ((N + 127) / 128 > 0 ? (N + 127) / 128 : 1));
  if (wave_rows < 128) wave_rows = 128;
  if (wave_rows > 1536) wave_rows = 1536;
  p->pr0 = round_panel(first_panel_rows > 0 ? first_panel_rows : (M + 1) / 2, M, 128);
  p->pr = round_panel(panel_rows > 0 ? panel_rows : wave_rows, M, 128);
  p->pc = round_panel(panel_cols > 0 ? panel_cols : 768, N, 256);
  p->pk = panel_k > 0 ? round_panel(panel_k, K, 128) : K;
  auto fail = [&](int st) {
    b2_host_plan_destroy(p);
    return st;
  };
  const size_t one = 1;
  if (cudaMalloc(&p->dA, sizeof(float) * ((size_t)M * K > 0 ? (size_t)M * K : one)) != cudaSuccess ||
      cudaMalloc(&p->dB, sizeof(float) * ((size_t)K * N > 0 ? (size_t)K * N : one)) != cudaSuccess ||
      cudaMalloc(&p->dC, sizeof(float) * ((size_t)M * N > 0 ? (size_t)M * N : one)) != cudaSuccess ||
      cudaMalloc(&p->report, sizeof(b2_ft_report)) != cudaSuccess ||
      cudaStreamCreateWithFlags(&p->compute, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&p->h2d, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&p->d2h, cudaStreamNonBlocking) != cudaSuccess)
    return fail(cuda_fail(cudaGetLastError(), "b2_host_plan_create (device buffers and streams)", __FILE__, __LINE__));
  // scratch sized once, outside the pipeline (growing it later would synchronise the device)
  size_t ws = 0;
  const int rows_big = p->pr0 > p->pr ? p->pr0 : p->pr;
  const int rows_max = rows_big < M ? rows_big : M, k_max = p->pk < K ? p->pk : K;
  if (M > 0 && N > 0 && K > 0) {
    ws = b2_ft_sgemm_workspace_bytes(path, rows_max, N, k_max);
    const size_t ws_first = b2_ft_sgemm_workspace_bytes(path, rows_max, p->pc < N ? p->pc : N, k_max);
    if (ws_first > ws) ws = ws_first;
  }
  if (ws > ctx->ws_bytes && (ctx->ws == nullptr || ctx->ws_owned)) {
    int st = ensure_workspace(ctx, ws, nullptr);
    if (st != B2_OK) return fail(st);
  }
  *out = p;
  return B2_OK;
}

int b2_sgemm_host(b2_host_plan p, float alpha, const float *A, int lda, const float *B, int ldb, float beta, float *C, int ldc,
                  int abft, b2_ft_report *report_host) {
  B2_REQUIRE(p != nullptr, B2_ERR_INVALID_ARG, "b2_sgemm_host: plan is NULL");
  const int M = p->M, N = p->N, K = p->K;
  if (M == 0 || N == 0) return B2_OK;
  B2_REQUIRE(C != nullptr && ldc >= N, B2_ERR_INVALID_ARG, "b2_sgemm_host: C is NULL or ldc = %d < N = %d", ldc, N);
  B2_REQUIRE(K == 0 || (A != nullptr && B != nullptr && lda >= K && ldb >= N), B2_ERR_INVALID_ARG,
             "b2_sgemm_host: A or B is NULL, or lda = %d < K = %d, or ldb = %d < N = %d", lda, K, ldb, N);
  int dev = -1;
  B2_CUDA(cudaGetDevice(&dev));
  B2_REQUIRE(dev == p->ctx->device, B2_ERR_INVALID_ARG, "b2_sgemm_host: the plan belongs to device %d but device %d is current",
             p->ctx->device, dev);
  p->next_event = 0;
  if (abft) B2_CUDA(cudaMemsetAsync(p->report, 0, sizeof(b2_ft_report), p->compute));
  const bool use_c = beta != 0.f;
  struct Span { int a, b; };
  std::vector<Span> rows, cols, kps;
  for (int r0 = 0; r0 < M;) {
    // with several K panels every row panel has the regular height
    const int h = (r0 == 0 && p->pk >= K) ? p->pr0 : p->pr;
    rows.push_back({r0, r0 + h < M ? r0 + h : M});
    r0 += h;
  }
  for (int c0 = 0; c0 < N; c0 += p->pc) cols.push_back({c0, c0 + p->pc < N ? c0 + p->pc : N});
  for (int k0 = 0; k0 < K; k0 += (p->pk > 0 ? p->pk : 1)) kps.push_back({k0, k0 + p->pk < K ? k0 + p->pk : K});
  auto gemm = [&](int m, int n, int k, const float *a, const float *b, float bt, float *c) {
    return sgemm_dispatch(p->ctx, p->path, abft != 0, m, n, k, alpha, a, K > 0 ? K : 1, b, N, bt, c, N, abft ? p->report : nullptr,
                          p->compute);
  };
  auto back = [&](const Span &r) -> int {
    B2_TRY(chain(p, p->compute, p->d2h));
    return copy2d(C + (size_t)r.a * ldc, ldc, p->dC + (size_t)r.a * N, N, r.b - r.a, N, cudaMemcpyDeviceToHost, p->d2h);
  };
  auto send_rows = [&](const Span &r, bool with_c) -> int {
    B2_TRY(copy2d(p->dA + (size_t)r.a * K, K, A + (size_t)r.a * lda, lda, r.b - r.a, K, cudaMemcpyHostToDevice, p->h2d));
    if (with_c && use_c)
      B2_TRY(copy2d(p->dC + (size_t)r.a * N, N, C + (size_t)r.a * ldc, ldc, r.b - r.a, N, cudaMemcpyHostToDevice, p->h2d));
    return B2_OK;
  };

  if (kps.size() <= 1) {
    // ---- one K panel (or K == 0: C <- beta * C through the same schedule): first row panel in column tiles behind the column panels of B, the others full width ----
    B2_TRY(send_rows(rows[0], false));
    for (const Span &c : cols) {
      B2_TRY(copy2d(p->dB + c.a, N, B + c.a, ldb, K, c.b - c.a, cudaMemcpyHostToDevice, p->h2d));
      if (use_c)
        B2_TRY(copy2d(p->dC + (size_t)rows[0].a * N + c.a, N, C + (size_t)rows[0].a * ldc + c.a, ldc, rows[0].b - rows[0].a,
                      c.b - c.a, cudaMemcpyHostToDevice, p->h2d));
      B2_TRY(chain(p, p->h2d, p->compute));
      B2_TRY(gemm(rows[0].b - rows[0].a, c.b - c.a, K, p->dA + (size_t)rows[0].a * K, p->dB + c.a, beta,
                  p->dC + (size_t)rows[0].a * N + c.a));
    }
    B2_TRY(back(rows[0]));
    for (size_t i = 1; i < rows.size(); ++i) {
      B2_TRY(send_rows(rows[i], true));
      B2_TRY(chain(p, p->h2d, p->compute));
      B2_TRY(gemm(rows[i].b - rows[i].a, N, K, p->dA + (size_t)rows[i].a * K, p->dB, beta, p->dC + (size_t)rows[i].a * N));
      B2_TRY(back(rows[i]));
    }
  } else {
    // ---- several K panels: row panels and K panels sent alternately; block (p, q) as soon as both are there ----
    std::vector<cudaEvent_t> row_ev(rows.size(), nullptr), k_ev(kps.size(), nullptr);
    std::vector<size_t> done(rows.size(), 0);
    auto compute_ready = [&]() -> int {
      for (size_t i = 0; i < rows.size(); ++i) {
        if (!row_ev[i]) continue;
        while (done[i] < kps.size() && k_ev[done[i]]) {
          const size_t q = done[i];
          B2_CUDA(cudaStreamWaitEvent(p->compute, row_ev[i], 0));
          B2_CUDA(cudaStreamWaitEvent(p->compute, k_ev[q], 0));
          B2_TRY(gemm(rows[i].b - rows[i].a, N, kps[q].b - kps[q].a, p->dA + (size_t)rows[i].a * K + kps[q].a,
                      p->dB + (size_t)kps[q].a * N, q == 0 ? beta : 1.f, p->dC + (size_t)rows[i].a * N));
          done[i] = q + 1;
          if (done[i] == kps.size()) B2_TRY(back(rows[i]));
        }
      }
      return B2_OK;
    };
    const size_t steps = rows.size() > kps.size() ? rows.size() : kps.size();
    for (size_t i = 0; i < steps; ++i) {
      if (i < rows.size()) {
        B2_TRY(send_rows(rows[i], true));
        B2_TRY(plan_event(p, &row_ev[i]));
        B2_CUDA(cudaEventRecord(row_ev[i], p->h2d));
        B2_TRY(compute_ready());
      }
      if (i < kps.size()) {
        B2_TRY(copy2d(p->dB + (size_t)kps[i].a * N, N, B + (size_t)kps[i].a * ldb, ldb, kps[i].b - kps[i].a, N,
                      cudaMemcpyHostToDevice, p->h2d));
        B2_TRY(plan_event(p, &k_ev[i]));
        B2_CUDA(cudaEventRecord(k_ev[i], p->h2d));
        B2_TRY(compute_ready());
      }
    }
  }
  if (abft && report_host)
    B2_CUDA(cudaMemcpyAsync(report_host, p->report, sizeof(b2_ft_report), cudaMemcpyDeviceToHost, p->compute));
  B2_CUDA(cudaStreamSynchronize(p->d2h));
  B2_CUDA(cudaStreamSynchronize(p->compute));
  return B2_OK;
}

}  // extern "C"
