// Element-wise pieces of the decode step: RMSNorm, rotate-half RoPE, SiLU*up,
// residual add, greedy argmax (src/model.rs:653-737,367-382; src/sampler.rs:7-17).
#include <cmath>

#include "ctx.h"
#include "glue.cuh"
#include "kv_pool.h"

namespace kanso {

// x / sqrt(mean(x^2) + eps) * w, one CTA per row (src/model.rs:653-659).
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               float* __restrict__ out, int hidden, float eps) {
  __shared__ float red[32];
  const float* xr = x + (int64_t)blockIdx.x * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) ss += xr[i] * xr[i];
  ss = block_sum(ss, red);
  float rms = sqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    out[(int64_t)blockIdx.x * hidden + i] = xr[i] / rms * w[i];
}

// Rotate-half RoPE in place (src/model.rs:721-737). With a table: cos/sin rows of
// build_rope_table (src/model.rs:698-719); without: computed on the fly.
constexpr int ROPE_MAX_HALF = 128;  // head_dim <= 256
struct RopeFreq {
  float f[ROPE_MAX_HALF];
};
__global__ void rope_kernel(float* __restrict__ x, const uint32_t* __restrict__ positions,
                            int heads, int head_dim, const RopeFreq freq,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            int table_len, int* status) {
  int t = blockIdx.x;
  int half = head_dim / 2;
  uint32_t pos = positions[t];
  if (cos_t && pos >= (uint32_t)table_len) {
    if (threadIdx.x == 0) atomicOr(status, DEV_BAD_INDEX);
    return;
  }
  for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
    int h = i / half, j = i - h * half;
    float c, s;
    if (cos_t) {
      c = cos_t[(int64_t)pos * half + j];
      s = sin_t[(int64_t)pos * half + j];
    } else {
      float ang = __fmul_rn((float)pos, freq.f[j]);
      c = cosf(ang);
      s = sinf(ang);
    }
    float* v = x + ((int64_t)t * heads + h) * head_dim;
    float a = v[j], b = v[j + half];
    v[j] = a * c - b * s;
    v[j + half] = a * s + b * c;
  }
}

__global__ void silu_mul_kernel(const float* __restrict__ g, const float* __restrict__ u,
                                float* __restrict__ out, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = g[i] / (1.0f + expf(-g[i])) * u[i];
}

__global__ void residual_add_kernel(float* __restrict__ h, const float* __restrict__ p,
                                    int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) h[i] = h[i] + p[i];
}

// First maximum wins (src/sampler.rs:7-17). One CTA per row.
__global__ void greedy_token_kernel(const float* __restrict__ logits, uint32_t* __restrict__ out,
                                    int64_t vocab) {
  __shared__ float bv[32];
  __shared__ int64_t bi[32];
  const float* row = logits + (int64_t)blockIdx.x * vocab;
  float best = -INFINITY;
  int64_t idx = 0x7FFFFFFFFFFFFFFFll;
  for (int64_t i = threadIdx.x; i < vocab; i += blockDim.x)
    if (row[i] > best) {
      best = row[i];
      idx = i;
    }
  auto better = [](float v1, int64_t i1, float v2, int64_t i2) {
    return v1 > v2 || (v1 == v2 && i1 < i2);
  };
  for (int o = 16; o; o >>= 1) {
    float v = __shfl_xor_sync(0xFFFFFFFFu, best, o);
    int64_t i = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
    if (better(v, i, best, idx)) {
      best = v;
      idx = i;
    }
  }
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    bv[warp] = best;
    bi[warp] = idx;
  }
  __syncthreads();
  if (warp == 0) {
    int nw = blockDim.x >> 5;
    best = lane < nw ? bv[lane] : -INFINITY;
    idx = lane < nw ? bi[lane] : 0x7FFFFFFFFFFFFFFFll;
    for (int o = 16; o; o >>= 1) {
      float v = __shfl_xor_sync(0xFFFFFFFFu, best, o);
      int64_t i = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
      if (better(v, i, best, idx)) {
        best = v;
        idx = i;
      }
    }
    // all -inf / NaN rows keep index 0, as the reference's loop does
    if (lane == 0) out[blockIdx.x] = idx == 0x7FFFFFFFFFFFFFFFll ? 0u : (uint32_t)idx;
  }
}

int32_t launch_rmsnorm(kanso_cuda_ctx* ctx, const float* x, const float* w, float* out,
                       int64_t rows, int64_t hidden, float eps) {
  rmsnorm_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(x, w, out, (int)hidden, eps);
  return after_launch(ctx, "rmsnorm");
}

int32_t launch_rope(kanso_cuda_ctx* ctx, float* x, const uint32_t* positions, int64_t T,
                    int64_t heads, int64_t head_dim, float theta, const float* cos_t,
                    const float* sin_t, int table_len) {
  RopeFreq freq;
  if (!cos_t)  // theta^(-2j/head_dim) with the host's powf, as build_rope_table (src/model.rs:700-707)
    for (int j = 0; j < head_dim / 2; ++j)
      freq.f[j] = std::pow(theta, -2.0f * (float)j / (float)head_dim);
  rope_kernel<<<(unsigned)T, 128, 0, ctx->stream>>>(x, positions, (int)heads, (int)head_dim, freq,
                                                    cos_t, sin_t, table_len, ctx->dev_status);
  return after_launch(ctx, "rope");
}

int32_t launch_silu_mul(kanso_cuda_ctx* ctx, const float* g, const float* u, float* out,
                        int64_t n) {
  silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(g, u, out, n);
  return after_launch(ctx, "silu_mul");
}

int32_t launch_residual_add(kanso_cuda_ctx* ctx, float* h, const float* p, int64_t n) {
  residual_add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(h, p, n);
  return after_launch(ctx, "residual_add");
}

}  // namespace kanso

using namespace kanso;

extern "C" {

int32_t kanso_cuda_rmsnorm(kanso_cuda_ctx* ctx, const float* x, const float* weight, float* out,
                           int64_t rows, int64_t hidden, float eps) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "rmsnorm: ctx is NULL");
  if (rows < 0 || hidden <= 0) return fail(ctx, KANSO_ERR_SHAPE, "rmsnorm: bad shape");
  if (rows == 0) return KANSO_OK;
  return launch_rmsnorm(ctx, x, weight, out, rows, hidden, eps);
}

int32_t kanso_cuda_rope(kanso_cuda_ctx* ctx, float* x, const uint32_t* positions, int64_t T,
                        int64_t heads, int64_t head_dim, float theta) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "rope: ctx is NULL");
  if (T < 0 || heads <= 0 || head_dim <= 0 || head_dim % 2 || head_dim > 2 * ROPE_MAX_HALF)
    return fail(ctx, KANSO_ERR_SHAPE, "rope: head_dim %lld must be even, positive and <= %d",
                (long long)head_dim, 2 * ROPE_MAX_HALF);
  if (T == 0) return KANSO_OK;
  return launch_rope(ctx, x, positions, T, heads, head_dim, theta, nullptr, nullptr, 0);
}

int32_t kanso_cuda_silu_mul(kanso_cuda_ctx* ctx, const float* gate, const float* up, float* out,
                            int64_t n) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "silu_mul: ctx is NULL");
  if (n < 0) return fail(ctx, KANSO_ERR_SHAPE, "silu_mul: n < 0");
  if (n == 0) return KANSO_OK;
  return launch_silu_mul(ctx, gate, up, out, n);
}

int32_t kanso_cuda_residual_add(kanso_cuda_ctx* ctx, float* hidden, const float* proj, int64_t n) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "residual_add: ctx is NULL");
  if (n < 0) return fail(ctx, KANSO_ERR_SHAPE, "residual_add: n < 0");
  if (n == 0) return KANSO_OK;
  return launch_residual_add(ctx, hidden, proj, n);
}

int32_t kanso_cuda_greedy_token(kanso_cuda_ctx* ctx, const float* logits, uint32_t* out,
                                int64_t B, int64_t vocab) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "greedy_token: ctx is NULL");
  if (B < 0 || vocab <= 0) return fail(ctx, KANSO_ERR_SHAPE, "greedy_token: bad shape");
  if (B == 0) return KANSO_OK;
  greedy_token_kernel<<<(unsigned)B, 256, 0, ctx->stream>>>(logits, out, vocab);
  return after_launch(ctx, "greedy_token");
}

}  // extern "C"
