// placeholder replaced below
#include "common.cuh"
namespace b2 {
int sgemm_ffma_dispatch(Context *ctx, int trans_a, int M, int N, int K, float alpha, const float *A, int lda,
                        const float *B, int ldb, float beta, float *C, int ldc, cudaStream_t s);
}
using namespace b2;
extern "C" int ref_sgemm_colmajor_nt(int M, int N, int K, float *A, float *B, float *C, float alpha, float beta) {
  Context *ctx = default_context();
  B2_REQUIRE(ctx != nullptr, B2_ERR_CUDA, "no context");
  return sgemm_ffma_dispatch(ctx, 1, N, M, K, alpha, B, N, A, M, beta, C, M, nullptr);
}
extern "C" int b2_ft_sgemm(b2_handle h, int path, int M, int N, int K, float alpha, const float *A, int lda,
                const float *B, int ldb, float beta, float *C, int ldc, const b2_fault *plan_dev,
                int n_faults, float tau, b2_ft_report *report_dev, void *stream) {
  set_error("b2_ft_sgemm: not built yet");
  return B2_ERR_UNSUPPORTED;
}
extern "C" int ft_sgemm(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C) {
  return b2_ft_sgemm(nullptr, 0, M, N, K, alpha, A, K, B, N, beta, C, N, nullptr, 0, 0.f, nullptr, nullptr);
}
