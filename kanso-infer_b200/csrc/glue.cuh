// Small device helpers and the launchers the decode step shares.
#pragma once
#include "ctx.h"

namespace kanso {

// Sum over the CTA; `red` is 32 floats of shared memory. Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  v = lane < nw ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  v = lane < nw ? red[lane] : -INFINITY;
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

int32_t launch_rmsnorm(kanso_cuda_ctx* ctx, const float* x, const float* w, float* out,
                       int64_t rows, int64_t hidden, float eps);
int32_t launch_rope(kanso_cuda_ctx* ctx, float* x, const uint32_t* positions, int64_t T,
                    int64_t heads, int64_t head_dim, float theta, const float* cos_t,
                    const float* sin_t, int table_len);
struct KvGeom;
// Inputs of the decode step's attention fusion: un-rotated q goes in as the attention's q; the
// newest token's K and V, their positions and pool slots, and the RoPE tables.
struct PaDecodeFusion {
  const float* k_new;
  const float* v_new;
  const uint32_t* positions;
  const uint32_t* slots;
  const float* cos_t;
  const float* sin_t;
  int table_len;
  // Optional (batched decode): when not null the attention also writes its output as the packed
  // f16 hi/lo activation tile of the o-projection's tensor-core GEMM and returns the tile here;
  // it returns nullptr when it could not (the caller then packs the f32 output as usual).
  const void** packed_out;
};

int32_t launch_silu_mul(kanso_cuda_ctx* ctx, const float* g, const float* u, float* out,
                        int64_t n);
int32_t launch_residual_add(kanso_cuda_ctx* ctx, float* h, const float* p, int64_t n);
int32_t stream_fused_q8_0(kanso_cuda_ctx* ctx, int nseg, const void* const* w, float* const* y,
                          const int64_t* rows, const float* x, const float* x2,
                          const float* norm_w, float eps, const float* resid, int64_t K, int M,
                          int32_t act_mode);
int32_t matmul_dispatch(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x,
                        float* y, int64_t M, int64_t N, int64_t K, int32_t act_mode);

}  // namespace kanso
