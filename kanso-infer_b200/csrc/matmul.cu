// Chooses the kernel behind LinearWeight::forward (src/weights.rs:43-45) by the number
// of activation rows, and exposes the pointer-level GEMM entry points.
#include "ctx.h"

namespace kanso {
int32_t stream_matmul(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x, float* y,
                      int64_t M, int64_t N, int64_t K, int32_t act_mode);

int32_t tc_matmul(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x, float* y,
                  int64_t M, int64_t N, int64_t K, bool* handled);
int32_t q4k_direct_matmul(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y, int64_t M,
                          int64_t N, int64_t K, bool* handled);

int32_t q8_mma_matmul(kanso_cuda_ctx* ctx, int nseg, const void* const* w, float* const* y,
                      const int64_t* rows, const float* x, const float* x2, const float* norm_w,
                      float eps, const float* resid, int64_t K, int M, int32_t act_mode,
                      bool decode_chain, bool* handled);

int32_t tma_matmul(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x, float* y,
                   int64_t M, int64_t N, int64_t K, bool* handled);
int32_t i8_matmul(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y, int64_t M,
                  int64_t N, int64_t K, bool* handled);

int32_t matmul_dispatch(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x,
                        float* y, int64_t M, int64_t N, int64_t K, int32_t act_mode) {
  // More than 8 activation rows on a matrix whose rows start on 16-byte boundaries: the
  // TMA-staged tcgen05 GEMM, up to 512 rows per pass over the weights. Q8_0 takes it from two
  // rows on: measured on 14336 x 4096 / 4096 x 4096 / 4096 x 14336 it needs 31.8 / 11.9 / 30.0 us
  // at up to 16 rows, the int8-MMA GEMV 30.8 / 14.1 / 40.6 us at two rows and 37.5 / 15.3 /
  // 50.4 us at eight (one row stays with the GEMV: 23.8 / 10.0 / 26.4 us).
  const bool tma_rows = M > 8 || (M >= 2 && dtype == KANSO_DTYPE_Q8_0);
  if (tma_rows && act_mode == KANSO_ACT_F32 && N > 0 && K > 0 && w && x && y) {
    bool all = true;
    for (int64_t m0 = 0; m0 < M && all; m0 += 512) {
      bool handled = false;
      // a tail of fewer than 9 rows rides with the chunk before it
      int64_t mc = M - m0 < 512 ? M - m0 : 512;
      if (M - m0 - mc > 0 && M - m0 - mc < 9) mc -= 16;
      int32_t st = tma_matmul(ctx, dtype, w, x + m0 * K, y + m0 * N, mc, N, K, &handled);
      if (st != KANSO_OK) return st;
      if (!handled) all = false;
      m0 -= 512 - mc;
    }
    if (all) return KANSO_OK;
  }
  // More than 8 activation rows: the tcgen05 GEMM, at most 128 rows per pass over the weights
  // (the A/B tiles of two stages plus the raw-byte ring fill one SM's shared memory).
  if (M > 8 && act_mode == KANSO_ACT_F32 && (dtype == KANSO_DTYPE_Q8_0 || dtype == KANSO_DTYPE_Q4_K) &&
      N > 0 && K > 0 && w && x && y && aligned16(x)) {
    bool all = true;
    for (int64_t m0 = 0; m0 < M && all; m0 += 128) {
      bool handled = false;
      int32_t st = tc_matmul(ctx, dtype, w, x + m0 * K, y + m0 * N, M - m0 < 128 ? M - m0 : 128, N,
                             K, &handled);
      if (st != KANSO_OK) return st;
      if (!handled) all = false;
    }
    if (all) return KANSO_OK;
  }
  // Q8_0 weights with Q8 activations and more than 8 rows: int8 tensor-core GEMM with exact
  // int32 block sums, 128 rows per pass over the weights
  if (M > 8 && act_mode == KANSO_ACT_Q8 && dtype == KANSO_DTYPE_Q8_0 && N > 0 && K > 0 && w && x &&
      y) {
    bool all = true;
    for (int64_t m0 = 0; m0 < M && all;) {
      int64_t mc = M - m0 < 128 ? M - m0 : 128;
      if (M - m0 - mc > 0 && M - m0 - mc < 9) mc -= 16;  // a short tail rides with this chunk
      bool handled = false;
      int32_t st = i8_matmul(ctx, w, x + m0 * K, y + m0 * N, mc, N, K, &handled);
      if (st != KANSO_OK) return st;
      if (!handled) all = false;
      m0 += mc;
    }
    if (all) return KANSO_OK;
  }
  if (dtype == KANSO_DTYPE_Q4_K && act_mode == KANSO_ACT_F32 && K > 0 && K % 256 == 0 && M > 0 &&
      N > 0 && w && x && y && aligned16(w) && aligned16(x)) {
    // int8 tensor-core GEMV. Up to 6 activation rows go in one pass over the weights; from 7
    // rows on, passes of 4 are faster than the kernel's 7- and 8-row forms (which spill
    // registers): 22.6 us against 36.5 us for 8 rows of a 14336 x 4096 matrix. Fewer rows per
    // pass also when the activation planes of a long K do not fit in shared memory.
    const int64_t mp0 = M > 6 ? 4 : 8;
    for (int64_t mp = mp0; mp >= 1; mp /= 2) {
      if (mp < mp0 && M <= mp) continue;  // the same single pass as the attempt before
      bool all = true;
      for (int64_t m0 = 0; m0 < M && all; m0 += mp) {
        bool handled = false;
        int32_t st = q4k_direct_matmul(ctx, w, x + m0 * K, y + m0 * N, M - m0 < mp ? M - m0 : mp,
                                       N, K, &handled);
        if (st != KANSO_OK) return st;
        if (!handled) all = false;  // decided by the shape of the largest (first) pass
      }
      if (all) return KANSO_OK;
    }
  }
  if (dtype == KANSO_DTYPE_Q8_0 && (act_mode == KANSO_ACT_F32 || act_mode == KANSO_ACT_Q8) &&
      K > 0 && M > 0 && N > 0 && w && x && y) {
    // int8 tensor-core GEMV, at most 8 activation rows per pass over the weights
    bool all = true;
    for (int64_t m0 = 0; m0 < M && all; m0 += 8) {
      bool handled = false;
      const void* w1[1] = {w};
      float* y1[1] = {y + m0 * N};
      const int64_t r1[1] = {N};
      int32_t st = q8_mma_matmul(ctx, 1, w1, y1, r1, x + m0 * K, nullptr, nullptr, 0.f, nullptr, K,
                                 (int)(M - m0 < 8 ? M - m0 : 8), act_mode, false, &handled);
      if (st != KANSO_OK) return st;
      if (!handled) all = false;
    }
    if (all) return KANSO_OK;
  }
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
