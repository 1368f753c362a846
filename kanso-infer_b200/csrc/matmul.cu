// Chooses the kernel behind LinearWeight::forward (src/weights.rs:43-45) by the number
// of activation rows, and exposes the pointer-level GEMM entry points.
#include "ctx.h"

namespace kanso {
int32_t stream_matmul(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x, float* y,
                      int64_t M, int64_t N, int64_t K, int32_t act_mode);

int32_t matmul_dispatch(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x,
                        float* y, int64_t M, int64_t N, int64_t K, int32_t act_mode) {
  return stream_matmul(ctx, dtype, w, x, y, M, N, K, act_mode);
}
}  // namespace kanso

using namespace kanso;

extern "C" {
int32_t kanso_cuda_gemm_q8_0(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                             int64_t M, int64_t N, int64_t K, int32_t act_mode) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "gemm_q8_0: ctx is NULL");
  return matmul_dispatch(ctx, KANSO_DTYPE_Q8_0, w, x, y, M, N, K, act_mode);
}
int32_t kanso_cuda_gemm_q4_k(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                             int64_t M, int64_t N, int64_t K, int32_t act_mode) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "gemm_q4_k: ctx is NULL");
  return matmul_dispatch(ctx, KANSO_DTYPE_Q4_K, w, x, y, M, N, K, act_mode);
}
}
