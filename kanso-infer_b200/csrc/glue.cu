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

// Decode-step glue in one launch (src/model.rs:1164-1171): rotate-half RoPE of the query
// heads in place, RoPE of the key heads, and the int8 quantising write of the roped K and of
// V into the pool (quantize_head_slice, src/kv_cache/quantized_storage.rs:452-469).
// One warp per (token, slot): slots [0, H) = query heads, [H, H+KH) = key heads, the rest = V.
// Multiplies and adds round separately, as the reference's tensor ops do, so the stored
// bytes equal the CPU path's.
__global__ void rope_kv_write_kernel(float* __restrict__ q, const float* __restrict__ k,
                                     const float* __restrict__ v,
                                     const uint32_t* __restrict__ positions,
                                     const uint32_t* __restrict__ slots, int64_t T, int H,
                                     const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, int table_len, KvGeom g,
                                     uint32_t layer, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int KH = (int)g.kv_heads, hd = (int)g.head_dim, half = hd / 2;
  const int nslot = H + 2 * KH;
  if (wid >= T * nslot) return;
  const int64_t t = wid / nslot;
  const int slot = (int)(wid - t * nslot);
  const uint32_t pos = positions[t];
  if (pos >= (uint32_t)table_len) {
    if (lane == 0) atomicOr(status, DEV_BAD_INDEX);
    return;
  }
  constexpr int MAXP = 4;  // head_dim <= 256: at most 4 (first, second) pairs per lane
  float a[MAXP], b[MAXP];
  const bool is_q = slot < H, is_k = !is_q && slot < H + KH;
  const int head = is_q ? slot : (is_k ? slot - H : slot - H - KH);
  const float* src = is_q ? q + (t * H + head) * hd
                          : (is_k ? k : v) + (t * KH + head) * hd;
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    const int j = lane + 32 * i;
    a[i] = b[i] = 0.f;
    if (j < half) {
      float x0 = src[j], x1 = src[j + half];
      if (is_q || is_k) {
        const float c = cos_t[(int64_t)pos * half + j], s = sin_t[(int64_t)pos * half + j];
        const float r0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        const float r1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
        x0 = r0;
        x1 = r1;
      }
      a[i] = x0;
      b[i] = x1;
      amax = fmaxf(amax, fmaxf(fabsf(x0), fabsf(x1)));
    }
  }
  if (is_q) {
    float* dst = q + (t * H + head) * hd;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int j = lane + 32 * i;
      if (j < half) {
        dst[j] = a[i];
        dst[j + half] = b[i];
      }
    }
    return;
  }
  const uint32_t sl = slots[t];
  const uint32_t block = sl / g.block_size, off = sl % g.block_size;
  if (block >= g.num_blocks) {
    if (lane == 0) atomicOr(status, DEV_BAD_INDEX);
    return;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  const float scale = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
  const float inv = __fdiv_rn(1.0f, scale);
  uint8_t* rec = g.pool + g.rec_offset(layer, block, head);
  int8_t* dst =
      reinterpret_cast<int8_t*>(rec + (is_k ? g.k_off() : g.v_off())) + (size_t)off * hd;
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    const int j = lane + 32 * i;
    if (j < half) {
      dst[j] = (int8_t)fminf(fmaxf(roundf(__fmul_rn(a[i], inv)), -127.f), 127.f);
      dst[j + half] = (int8_t)fminf(fmaxf(roundf(__fmul_rn(b[i], inv)), -127.f), 127.f);
    }
  }
  if (lane == 0) reinterpret_cast<float*>(rec + (is_k ? g.ks_off() : g.vs_off()))[off] = scale;
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

int32_t launch_rope_kv_write(kanso_cuda_ctx* ctx, float* q, const float* k, const float* v,
                             const uint32_t* positions, const uint32_t* slots, int64_t T, int H,
                             const float* cos_t, const float* sin_t, int table_len,
                             const KvGeom& g, uint32_t layer) {
  const int64_t warps = T * (H + 2 * (int64_t)g.kv_heads);
  cudaError_t e = launch_dependent(ctx, rope_kv_write_kernel,
                                   dim3((unsigned)((warps * 32 + 127) / 128)), dim3(128), 0, q, k,
                                   v, positions, slots, T, H, cos_t, sin_t, table_len, g, layer,
                                   ctx->dev_status);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "rope_kv_write launch");
  return after_launch(ctx, "rope_kv_write");
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
