// Reference-shaped shim for the column-major NT layout of kernel/ft_sgemm.
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
