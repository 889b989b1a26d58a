// Library core: status strings, thread-local error text, the scratch-owning handle,
// tensor-map encoding, the CUDA-event timer and device info.
#include <stdarg.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "common.cuh"

namespace b2 {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what, const char *file, int line) {
  set_error("CUDA error %d (%s) in %s at %s:%d", (int)e, cudaGetErrorString(e), what, file, line);
  return B2_ERR_CUDA;
}

static std::mutex g_mu;
static Context *g_default[64] = {nullptr};

static int context_init(Context *c) {
  B2_CUDA(cudaGetDevice(&c->device));
  B2_CUDA(cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, c->device));
  B2_CUDA(cudaMalloc(&c->fixed, kFixedBytes));
  c->fixed_bytes = kFixedBytes;
  B2_CUDA(cudaMemset(c->fixed, 0, kFixedBytes));
  return B2_OK;
}

Context *default_context() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("no usable CUDA device for the default handle");
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_default[dev]) {
    Context *c = new Context();
    if (context_init(c) != B2_OK) {
      delete c;
      return nullptr;
    }
    g_default[dev] = c;
  }
  return g_default[dev];
}

Context *resolve_context(b2_handle h, const char *who) {
  if (!h) {
    Context *c = default_context();
    if (!c) {
      char why[512];
      snprintf(why, sizeof(why), "%s", g_err);
      set_error("%s: no context (%s)", who, why);
    }
    return c;
  }
  Context *c = reinterpret_cast<Context *>(h);
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != c->device) {
    set_error("%s: the handle belongs to device %d but device %d is current", who, c->device, dev);
    return nullptr;
  }
  return c;
}

unsigned int next_launch_seq(Context *ctx) {
  std::lock_guard<std::mutex> lk(g_mu);
  ctx->launch_seq += 1;
  if (ctx->launch_seq == 0) ctx->launch_seq = 1;   // 0 is what a cleared abort word holds
  return ctx->launch_seq;
}

struct FuncOnDevice {
  const void *func;
  int device;
};
static std::vector<FuncOnDevice> g_configured;

int ensure_func_attributes(const void *func, int device, int dynamic_smem_bytes, int carveout) {
  std::lock_guard<std::mutex> lk(g_mu);
  for (const FuncOnDevice &f : g_configured)
    if (f.func == func && f.device == device) return B2_OK;
  B2_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, dynamic_smem_bytes));
  if (carveout >= 0) B2_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributePreferredSharedMemoryCarveout, carveout));
  g_configured.push_back({func, device});
  return B2_OK;
}

int ensure_workspace(Context *ctx, size_t bytes, cudaStream_t s) {
  if (bytes <= ctx->ws_bytes) return B2_OK;
  if (ctx->ws && !ctx->ws_owned) {
    set_error("caller-supplied workspace of %zu bytes is too small: %zu needed", ctx->ws_bytes, bytes);
    return B2_ERR_WORKSPACE;
  }
  // Growing a library-owned workspace: earlier work on any stream may still read the old block.
  B2_CUDA(cudaDeviceSynchronize());
  if (ctx->ws) B2_CUDA(cudaFree(ctx->ws));
  ctx->ws = nullptr;
  ctx->ws_bytes = 0;
  size_t want = bytes + (bytes >> 3);
  B2_CUDA(cudaMalloc(&ctx->ws, want));
  ctx->ws_bytes = want;
  ctx->ws_owned = true;
  (void)s;
  return B2_OK;
}

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!tried) {
    tried = true;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

int make_tmap_2d(CUtensorMap *out, const float *base, uint64_t inner, uint64_t outer, uint64_t ld,
                 uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_tiled_fn();
  B2_REQUIRE(fn != nullptr, B2_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * sizeof(float)};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B2_REQUIRE(r == CUDA_SUCCESS, B2_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (inner=%llu outer=%llu ld=%llu)",
             (int)r, (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)ld);
  return B2_OK;
}

}  // namespace b2

namespace b2 {
// One block waits on an mbarrier that nothing will ever arrive on, with a short time limit, and
// reports the timeout through the status word: the path every bounded wait of the GEMM kernels
// takes when a copy or a peer never shows up.  The context stays usable.
__global__ void wait_timeout_selftest_kernel(uint64_t limit_ns, int *status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !mbar_wait(&bar, 0, 1u << 22, limit_ns)) atomicExch(status, (int)B2_ERR_TIMEOUT);
}
}  // namespace b2

using namespace b2;

struct b2_context : public Context {};
struct b2_timer_s {
  cudaEvent_t beg, end;
};

extern "C" {

const char *b2_status_string(int s) {
  switch (s) {
    case B2_OK: return "ok";
    case B2_ERR_INVALID_ARG: return "invalid argument";
    case B2_ERR_UNSUPPORTED: return "unsupported shape for this kernel";
    case B2_ERR_CUDA: return "CUDA call failed";
    case B2_ERR_TIMEOUT: return "bounded device wait ran out";
    case B2_ERR_UNCORRECTABLE: return "ABFT fault could not be corrected";
    case B2_ERR_WORKSPACE: return "workspace missing or too small";
    default: return "unknown status";
  }
}

const char *b2_last_error(void) { return g_err; }
int b2_version(void) { return 100; }

int b2_create(b2_handle *out) {
  B2_REQUIRE(out != nullptr, B2_ERR_INVALID_ARG, "b2_create: out is NULL");
  b2_context *c = new b2_context();
  int st = context_init(c);
  if (st != B2_OK) {
    delete c;
    return st;
  }
  *out = c;
  return B2_OK;
}

int b2_destroy(b2_handle h) {
  if (!h) return B2_OK;
  if (h->ws && h->ws_owned) cudaFree(h->ws);
  if (h->fixed) cudaFree(h->fixed);
  delete h;
  return B2_OK;
}

int b2_set_workspace(b2_handle h, void *dev_ptr, size_t bytes) {
  B2_CONTEXT(c, h, "b2_set_workspace");
  B2_REQUIRE(((uintptr_t)dev_ptr & 1023) == 0, B2_ERR_INVALID_ARG, "workspace must be 1024-byte aligned");
  if (c->ws && c->ws_owned) {
    B2_CUDA(cudaDeviceSynchronize());
    B2_CUDA(cudaFree(c->ws));
  }
  c->ws = dev_ptr;
  c->ws_bytes = dev_ptr ? bytes : 0;
  c->ws_owned = false;
  return B2_OK;
}

int b2_timer_create(b2_timer *out) {
  B2_REQUIRE(out != nullptr, B2_ERR_INVALID_ARG, "b2_timer_create: out is NULL");
  b2_timer_s *t = new b2_timer_s();
  if (cudaEventCreate(&t->beg) != cudaSuccess || cudaEventCreate(&t->end) != cudaSuccess) {
    delete t;
    return cuda_fail(cudaGetLastError(), "cudaEventCreate", __FILE__, __LINE__);
  }
  *out = t;
  return B2_OK;
}
int b2_timer_destroy(b2_timer t) {
  if (!t) return B2_OK;
  cudaEventDestroy(t->beg);
  cudaEventDestroy(t->end);
  delete t;
  return B2_OK;
}
int b2_timer_start(b2_timer t, void *stream) {
  B2_REQUIRE(t != nullptr, B2_ERR_INVALID_ARG, "timer is NULL");
  B2_CUDA(cudaEventRecord(t->beg, (cudaStream_t)stream));
  return B2_OK;
}
int b2_timer_stop(b2_timer t, void *stream) {
  B2_REQUIRE(t != nullptr, B2_ERR_INVALID_ARG, "timer is NULL");
  B2_CUDA(cudaEventRecord(t->end, (cudaStream_t)stream));
  return B2_OK;
}
int b2_timer_elapsed_ms(b2_timer t, float *ms_out) {
  B2_REQUIRE(t != nullptr && ms_out != nullptr, B2_ERR_INVALID_ARG, "timer or output is NULL");
  B2_CUDA(cudaEventSynchronize(t->end));
  B2_CUDA(cudaEventElapsedTime(ms_out, t->beg, t->end));
  return B2_OK;
}

int b2_selftest_wait_timeout(b2_handle h, int timeout_us, void *stream) {
  B2_CONTEXT(c, h, "b2_selftest_wait_timeout");
  B2_REQUIRE(timeout_us >= 1 && timeout_us <= 100000, B2_ERR_INVALID_ARG, "b2_selftest_wait_timeout: %d us not in 1..100000", timeout_us);
  wait_timeout_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((uint64_t)timeout_us * 1000ull,
                                                                    (int *)((char *)c->fixed + kFixedStatus));
  B2_CUDA(cudaGetLastError());
  return B2_OK;
}

int b2_device_info(int *sm_count, int *sm_clock_khz, size_t *global_mem_bytes) {
  int dev = 0;
  B2_CUDA(cudaGetDevice(&dev));
  if (sm_count) B2_CUDA(cudaDeviceGetAttribute(sm_count, cudaDevAttrMultiProcessorCount, dev));
  if (sm_clock_khz) B2_CUDA(cudaDeviceGetAttribute(sm_clock_khz, cudaDevAttrClockRate, dev));
  if (global_mem_bytes) {
    size_t fr = 0, tot = 0;
    B2_CUDA(cudaMemGetInfo(&fr, &tot));
    *global_mem_bytes = tot;
  }
  return B2_OK;
}

}  // extern "C"
