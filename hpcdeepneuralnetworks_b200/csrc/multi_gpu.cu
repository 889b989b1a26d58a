// Multi-GPU forms of the path, one process (or host thread) per GPU: row-block sharded SGEMM / ABFT SGEMM with B
// broadcast in K panels behind the compute, and sharded SDOT with a scalar all-reduce.  The reference is
// single-GPU (no NCCL or MPI call anywhere in it); these entry points have no counterpart there.
//
// NCCL is used through its public C API, looked up at run time (dlopen of libnccl.so.2: the copy already in
// the process if there is one, else the system's), so that the library loads on machines without NCCL and
// single-GPU users never touch it.
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "common.cuh"

namespace b2 {
int sgemm_dispatch(Context *ctx, int path, bool abft, int M, int N, int K, float alpha, const float *A, int lda, const float *B,
                   int ldb, float beta, float *C, int ldc, b2_ft_report *report_dev, cudaStream_t s);
size_t tf32_workspace_bytes(int M, int N, int K);

// The slice of NCCL's public API that is used (nccl.h: ncclUniqueId is 128 opaque bytes passed by value;
// ncclFloat32 = 7, ncclFloat64 = 8, ncclSum = 0; every call returns ncclResult_t, 0 = success).
struct NcclId {
  char bytes[B2_MG_ID_BYTES];
};
struct NcclApi {
  void *lib = nullptr;
  int (*GetUniqueId)(NcclId *) = nullptr;
  int (*CommInitRank)(void **comm, int nranks, NcclId id, int rank) = nullptr;
  int (*CommDestroy)(void *comm) = nullptr;
  int (*Broadcast)(const void *send, void *recv, size_t count, int dtype, int root, void *comm, cudaStream_t s) = nullptr;
  int (*AllReduce)(const void *send, void *recv, size_t count, int dtype, int op, void *comm, cudaStream_t s) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
};
static NcclApi g_nccl;
static std::mutex g_nccl_mu;

static int nccl_api(const NcclApi **out) {
  std::lock_guard<std::mutex> lk(g_nccl_mu);
  if (!g_nccl.lib) {
    const char *override_path = getenv("B2_NCCL_LIB");
    void *lib = nullptr;
    if (override_path && *override_path) lib = dlopen(override_path, RTLD_NOW | RTLD_LOCAL);
    if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL | RTLD_NOLOAD);   // the copy the process already uses
    if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    B2_REQUIRE(lib != nullptr, B2_ERR_UNSUPPORTED, "multi-GPU entry points need NCCL: libnccl.so.2 could not be loaded (%s)", dlerror());
    NcclApi a;
    a.lib = lib;
    *(void **)&a.GetUniqueId = dlsym(lib, "ncclGetUniqueId");
    *(void **)&a.CommInitRank = dlsym(lib, "ncclCommInitRank");
    *(void **)&a.CommDestroy = dlsym(lib, "ncclCommDestroy");
    *(void **)&a.Broadcast = dlsym(lib, "ncclBroadcast");
    *(void **)&a.AllReduce = dlsym(lib, "ncclAllReduce");
    *(void **)&a.GetErrorString = dlsym(lib, "ncclGetErrorString");
    B2_REQUIRE(a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.Broadcast && a.AllReduce, B2_ERR_UNSUPPORTED,
               "the NCCL library that was found lacks a required entry point");
    g_nccl = a;
  }
  *out = &g_nccl;
  return B2_OK;
}

static int nccl_fail(const NcclApi *api, int r, const char *what) {
  set_error("NCCL error %d (%s) in %s", r, api->GetErrorString ? api->GetErrorString(r) : "?", what);
  return B2_ERR_CUDA;
}
#define B2_NCCL(api, call)                                   \
  do {                                                       \
    int r__ = (call);                                        \
    if (r__ != 0) return nccl_fail((api), r__, #call);       \
  } while (0)

void row_block(int64_t M, int rank, int world, int64_t *start, int64_t *rows) {
  const int64_t base = M / world, rem = M % world;
  *rows = base + (rank < rem ? 1 : 0);
  *start = (int64_t)rank * base + (rank < rem ? rank : rem);
}
}  // namespace b2

using namespace b2;

struct b2_mg_context {
  Context *ctx = nullptr;
  int rank = 0, world = 1;
  void *comm = nullptr;            // ncclComm_t
  const NcclApi *api = nullptr;
  cudaStream_t comm_stream = nullptr;
  std::vector<cudaEvent_t> events;
  double *partial = nullptr;       // device: this rank's SDOT partial / the reduced sum
  float *scratch_f = nullptr;      // device: float result when the caller wants none
};

extern "C" {

int b2_mg_row_block(int64_t M, int rank, int world, int64_t *start, int64_t *rows) {
  B2_REQUIRE(M >= 0 && world >= 1 && rank >= 0 && rank < world && start && rows, B2_ERR_INVALID_ARG,
             "b2_mg_row_block: bad arguments (M=%lld rank=%d world=%d)", (long long)M, rank, world);
  row_block(M, rank, world, start, rows);
  return B2_OK;
}

int b2_mg_k_panel(int K, int panel, int index, int *k0, int *width) {
  B2_REQUIRE(K >= 0 && index >= 0, B2_ERR_INVALID_ARG, "b2_mg_k_panel: bad arguments (K=%d index=%d)", K, index);
  if (panel < 1) panel = 1;
  const int count = (K + panel - 1) / panel;
  if (index < count) {
    if (k0) *k0 = index * panel;
    if (width) *width = (K - index * panel < panel) ? K - index * panel : panel;
  }
  return count;
}

int b2_mg_unique_id(void *id_out) {
  B2_REQUIRE(id_out != nullptr, B2_ERR_INVALID_ARG, "b2_mg_unique_id: id_out is NULL");
  const NcclApi *api = nullptr;
  int st = nccl_api(&api);
  if (st != B2_OK) return st;
  NcclId id;
  memset(&id, 0, sizeof(id));
  B2_NCCL(api, api->GetUniqueId(&id));
  memcpy(id_out, &id, sizeof(id));
  return B2_OK;
}

int b2_mg_destroy(b2_mg_handle mg) {
  if (!mg) return B2_OK;
  if (mg->comm_stream) cudaStreamSynchronize(mg->comm_stream);
  if (mg->comm && mg->api) mg->api->CommDestroy(mg->comm);
  for (cudaEvent_t e : mg->events) cudaEventDestroy(e);
  if (mg->comm_stream) cudaStreamDestroy(mg->comm_stream);
  cudaFree(mg->partial);
  delete mg;
  return B2_OK;
}

int b2_mg_create(b2_mg_handle *out, b2_handle h, int rank, int world, const void *id) {
  B2_REQUIRE(out != nullptr, B2_ERR_INVALID_ARG, "b2_mg_create: out is NULL");
  B2_REQUIRE(world >= 1 && rank >= 0 && rank < world, B2_ERR_INVALID_ARG, "b2_mg_create: rank %d of %d", rank, world);
  B2_REQUIRE(world == 1 || id != nullptr, B2_ERR_INVALID_ARG, "b2_mg_create: more than one rank needs the id of b2_mg_unique_id");
  B2_CONTEXT(ctx, h, "b2_mg_create");
  b2_mg_context *mg = new b2_mg_context();
  mg->ctx = ctx;
  mg->rank = rank;
  mg->world = world;
  auto fail = [&](int st) {
    b2_mg_destroy(mg);
    return st;
  };
  if (cudaStreamCreateWithFlags(&mg->comm_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaMalloc(&mg->partial, 256) != cudaSuccess)
    return fail(cuda_fail(cudaGetLastError(), "b2_mg_create (stream and scratch)", __FILE__, __LINE__));
  mg->scratch_f = reinterpret_cast<float *>(mg->partial + 8);
  if (world > 1) {
    int st = nccl_api(&mg->api);
    if (st != B2_OK) return fail(st);
    NcclId nid;
    memcpy(&nid, id, sizeof(nid));
    int r = mg->api->CommInitRank(&mg->comm, world, nid, rank);
    if (r != 0) return fail(nccl_fail(mg->api, r, "ncclCommInitRank"));
  }
  *out = mg;
  return B2_OK;
}

int b2_mg_sgemm(b2_mg_handle mg, int path, int abft, int M, int N, int K, float alpha, const float *A_local, int lda, float *B,
                int ldb, float beta, float *C_local, int ldc, int root, int panel_k, b2_ft_report *report_dev, void *stream) {
  B2_REQUIRE(mg != nullptr, B2_ERR_INVALID_ARG, "b2_mg_sgemm: handle is NULL");
  B2_REQUIRE(path == B2_PATH_FFMA || path == B2_PATH_3XTF32, B2_ERR_INVALID_ARG, "b2_mg_sgemm: unknown path %d", path);
  B2_REQUIRE(M >= 0 && N >= 0 && K >= 0, B2_ERR_INVALID_ARG, "b2_mg_sgemm: negative dimension (M=%d N=%d K=%d)", M, N, K);
  B2_REQUIRE(root >= 0 && root < mg->world, B2_ERR_INVALID_ARG, "b2_mg_sgemm: root %d of %d ranks", root, mg->world);
  int64_t start = 0, rows64 = 0;
  row_block(M, mg->rank, mg->world, &start, &rows64);
  const int rows = (int)rows64;
  B2_REQUIRE(ldb >= N && (rows == 0 || N == 0 || (C_local != nullptr && ldc >= N)), B2_ERR_INVALID_ARG,
             "b2_mg_sgemm: C_local is NULL, or ldb = %d or ldc = %d is below N = %d", ldb, ldc, N);
  B2_REQUIRE(K == 0 || N == 0 || (B != nullptr && (rows == 0 || (A_local != nullptr && lda >= K))), B2_ERR_INVALID_ARG,
             "b2_mg_sgemm: A_local or B is NULL, or lda = %d < K = %d", lda, K);
  int dev = -1;
  B2_CUDA(cudaGetDevice(&dev));
  B2_REQUIRE(dev == mg->ctx->device, B2_ERR_INVALID_ARG, "b2_mg_sgemm: the handle belongs to device %d but device %d is current",
             mg->ctx->device, dev);
  cudaStream_t s = (cudaStream_t)stream;
  if (N == 0) return B2_OK;
  const int panel = panel_k > 0 ? panel_k : 4096;
  const int count = b2_mg_k_panel(K, panel, 0, nullptr, nullptr);
  if (count == 0)   // K == 0: C <- beta * C on every rank's block
    return sgemm_dispatch(mg->ctx, path, abft != 0, rows, N, 0, alpha, A_local, lda > 0 ? lda : 1, B, ldb, beta, C_local, ldc, report_dev, s);
  // scratch for the largest panel product up front: growing it between panels would synchronise the device
  if (rows > 0 && (mg->ctx->ws == nullptr || mg->ctx->ws_owned)) {
    const size_t need = b2_ft_sgemm_workspace_bytes(path, rows, N, panel < K ? panel : K);
    if (need > mg->ctx->ws_bytes) {
      int st = ensure_workspace(mg->ctx, need, s);
      if (st != B2_OK && path == B2_PATH_3XTF32) return st;
    }
  }
  while ((int)mg->events.size() < count + 1) {
    cudaEvent_t e;
    B2_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    mg->events.push_back(e);
  }
  if (mg->world > 1) {
    // B may still be being written by earlier work of the compute stream
    B2_CUDA(cudaEventRecord(mg->events[count], s));
    B2_CUDA(cudaStreamWaitEvent(mg->comm_stream, mg->events[count], 0));
    for (int i = 0; i < count; ++i) {
      int k0 = 0, kw = 0;
      b2_mg_k_panel(K, panel, i, &k0, &kw);
      float *bp = B + (size_t)k0 * ldb;
      const size_t span = (size_t)(kw - 1) * ldb + (size_t)N;   // the panel's rows with their pitch; same layout on every rank
      B2_NCCL(mg->api, mg->api->Broadcast(bp, bp, span, 7 /* ncclFloat32 */, root, mg->comm, mg->comm_stream));
      B2_CUDA(cudaEventRecord(mg->events[i], mg->comm_stream));
    }
  }
  for (int i = 0; i < count; ++i) {
    int k0 = 0, kw = 0;
    b2_mg_k_panel(K, panel, i, &k0, &kw);
    if (mg->world > 1) B2_CUDA(cudaStreamWaitEvent(s, mg->events[i], 0));   // the compute stream waits for panel i only
    if (rows > 0) {
      int st = sgemm_dispatch(mg->ctx, path, abft != 0, rows, N, kw, alpha, A_local + k0, lda, B + (size_t)k0 * ldb, ldb,
                              i == 0 ? beta : 1.f, C_local, ldc, report_dev, s);
      if (st != B2_OK) return st;
    }
  }
  return B2_OK;
}

int b2_mg_sdot(b2_mg_handle mg, int64_t n_local, const float *x_local, const float *y_local, float *result_dev, double *sum_dev,
               void *stream);

}  // extern "C"

namespace b2 {
__global__ void mg_sdot_finish_kernel(const double *sum, float *result) { *result = (float)*sum; }
}

extern "C" int b2_mg_sdot(b2_mg_handle mg, int64_t n_local, const float *x_local, const float *y_local, float *result_dev,
                          double *sum_dev, void *stream) {
  B2_REQUIRE(mg != nullptr, B2_ERR_INVALID_ARG, "b2_mg_sdot: handle is NULL");
  B2_REQUIRE(sum_dev != nullptr || result_dev != nullptr, B2_ERR_INVALID_ARG, "b2_mg_sdot: no result pointer");
  cudaStream_t s = (cudaStream_t)stream;
  double *sum = sum_dev ? sum_dev : mg->partial;
  float *res = result_dev ? result_dev : mg->scratch_f;
  int st = b2_sdot_partial(reinterpret_cast<b2_handle>(mg->ctx), n_local, x_local, y_local, res, sum, s);
  if (st != B2_OK) return st;
  if (mg->world > 1) {
    B2_NCCL(mg->api, mg->api->AllReduce(sum, sum, 1, 8 /* ncclFloat64 */, 0 /* ncclSum */, mg->comm, s));
    mg_sdot_finish_kernel<<<1, 1, 0, s>>>(sum, res);
    B2_CUDA(cudaGetLastError());
  }
  return B2_OK;
}
