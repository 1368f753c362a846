// int8 / fp8 KV pool: creation, quantising writes, block reset, token read-back
// (src/kv_cache/quantized_storage.rs; seam src/kv_cache/kind.rs:176-494).
#include <cuda_fp8.h>

#include "kv_pool.h"

namespace kanso {

// reset: quants 0, scales 1.0 (quantized_storage.rs:24-40)
__global__ void kv_reset_kernel(KvGeom g, uint32_t block_first, uint32_t block_count) {
  // one CTA per (layer, block, head) record
  uint32_t rec = blockIdx.x;
  uint32_t head = rec % g.kv_heads;
  uint32_t b = (rec / g.kv_heads) % block_count + block_first;
  uint32_t layer = rec / (g.kv_heads * block_count);
  uint8_t* p = g.pool + g.rec_offset(layer, b, head);
  uint32_t* w = reinterpret_cast<uint32_t*>(p);
  for (uint32_t i = threadIdx.x; i < 2 * g.q_bytes / 4; i += blockDim.x) w[i] = 0u;
  float* s = reinterpret_cast<float*>(p + g.ks_off());
  for (uint32_t i = threadIdx.x; i < 2 * g.block_size; i += blockDim.x) s[i] = 1.0f;
}

// quantize_head_slice (quantized_storage.rs:452-484) + write_quantized_kv_token
// (quantized_storage.rs:143-204). One warp per (token, head, K|V).
__global__ void kv_write_kernel(KvGeom g, uint32_t layer, const uint32_t* __restrict__ slots,
                                const float* __restrict__ k, const float* __restrict__ v,
                                int64_t T, int64_t k_stride, int64_t v_stride, int* status) {
  int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  int64_t total = T * g.kv_heads * 2;
  if (wid >= total) return;
  int which = (int)(wid & 1);
  uint32_t head = (uint32_t)((wid >> 1) % g.kv_heads);
  int64_t t = (wid >> 1) / g.kv_heads;
  uint32_t slot = slots[t];
  uint32_t block = slot / g.block_size, off = slot % g.block_size;
  if (block >= g.num_blocks) {
    if (lane == 0) atomicOr(status, DEV_BAD_INDEX);
    return;
  }
  const float* src = (which ? v + t * v_stride : k + t * k_stride) + (int64_t)head * g.head_dim;
  float amax = 0.f;
  for (uint32_t d = lane; d < g.head_dim; d += 32) amax = fmaxf(amax, fabsf(src[d]));
#pragma unroll
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  float scale = kv_scale_of(amax, g.fp8 != 0);
  float inv = __fdiv_rn(1.0f, scale);
  uint8_t* rec = g.pool + g.rec_offset(layer, block, head);
  int8_t* dst = reinterpret_cast<int8_t*>(rec + (which ? g.v_off() : g.k_off())) +
                (size_t)off * g.head_dim;
  for (uint32_t d = lane; d < g.head_dim; d += 32) {
    const float scaled = __fmul_rn(src[d], inv);
    if (g.fp8) {
      // F8E4M3::from_f32: round to nearest even onto the E4M3 grid (quantized_storage.rs:477-482)
      dst[d] = (int8_t)__nv_cvt_float_to_fp8(scaled, __NV_SATFINITE, __NV_E4M3);
    } else {
      dst[d] = (int8_t)fminf(fmaxf(roundf(scaled), -127.f), 127.f);
    }
  }
  if (lane == 0)
    reinterpret_cast<float*>(rec + (which ? g.vs_off() : g.ks_off()))[off] = scale;
}

// The value of an E4M3 bit pattern (sign, 4 exponent bits with bias 7, 3 mantissa bits; no
// infinities, S.1111.111 is NaN): what float8::F8E4M3::to_f32 returns (quantized_storage.rs:440-449).
static float e4m3_to_f32(uint8_t b) {
  const int e = (b >> 3) & 15, m = b & 7;
  float v;
  if (e == 15 && m == 7)
    v = NAN;
  else if (e == 0)
    v = ldexpf((float)m, -9);
  else
    v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  return (b & 0x80) ? -v : v;
}

int32_t launch_kv_write(kanso_cuda_ctx* ctx, kanso_cuda_kv* kv, uint32_t layer,
                        const uint32_t* slots, const float* k, const float* v, int64_t T,
                        int64_t k_stride, int64_t v_stride) {
  KvGeom g = kv_geom(kv);
  int64_t warps = T * g.kv_heads * 2;
  kv_write_kernel<<<(unsigned)((warps * 32 + 127) / 128), 128, 0, ctx->stream>>>(
      g, layer, slots, k, v, T, k_stride, v_stride, ctx->dev_status);
  return after_launch(ctx, "kv_write_slots");
}

}  // namespace kanso

using namespace kanso;

extern "C" {

int32_t kanso_cuda_kv_create(kanso_cuda_ctx* ctx, uint32_t num_layers, uint32_t num_blocks,
                             uint32_t block_size, uint32_t num_kv_heads, uint32_t head_dim,
                             int32_t kv_type, kanso_cuda_kv** out) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "kv_create: ctx is NULL");
  if (!out) return fail(ctx, KANSO_ERR_CONFIG, "kv_create: out is NULL");
  *out = nullptr;
  if (kv_type == KANSO_KV_F32)
    return fail(ctx, KANSO_ERR_UNSUPPORTED,
                "kv type 'f32' is not available on backend 'cuda': its decode attention reads "
                "the quantised pool (expected: int8 or fp8)");
  if (kv_type != KANSO_KV_INT8 && kv_type != KANSO_KV_FP8)
    return fail(ctx, KANSO_ERR_CONFIG, "unknown kv type %d (expected one of: f32, int8, fp8)",
                kv_type);
  if (!num_layers || !num_blocks || !block_size || !num_kv_heads || !head_dim)
    return fail(ctx, KANSO_ERR_CONFIG, "kv_create: every dimension must be non-zero");
  auto* kv = new kanso_cuda_kv;
  kv->ctx = ctx;
  kv->layers = num_layers;
  kv->num_blocks = num_blocks;
  kv->block_size = block_size;
  kv->kv_heads = num_kv_heads;
  kv->head_dim = head_dim;
  kv->kv_type = kv_type;
  KvGeom g = kv_geom(kv);
  kv->pool_bytes = (size_t)num_layers * num_blocks * num_kv_heads * g.rec_bytes;
  cudaError_t e = cudaMalloc((void**)&kv->pool, kv->pool_bytes);
  if (e != cudaSuccess) {
    delete kv;
    // an allocation failure at start-up is a Config error (src/kv_cache/storage.rs:29-68)
    return fail(ctx, KANSO_ERR_CONFIG, "kv_create: cannot allocate %zu bytes of KV pool: %s",
                (size_t)num_layers * num_blocks * num_kv_heads * g.rec_bytes,
                cudaGetErrorString(e));
  }
  g.pool = kv->pool;
  kv_reset_kernel<<<num_layers * num_blocks * num_kv_heads, 128, 0, ctx->stream>>>(g, 0,
                                                                                  num_blocks);
  int32_t st = after_launch(ctx, "kv_create reset");
  if (st) {
    cudaFree(kv->pool);
    delete kv;
    return st;
  }
  *out = kv;
  return KANSO_OK;
}

int32_t kanso_cuda_kv_destroy(kanso_cuda_kv* kv) {
  if (!kv) return KANSO_OK;
  cudaDeviceSynchronize();  // the context may already be destroyed
  cudaFree(kv->pool);
  delete kv;
  return KANSO_OK;
}

int32_t kanso_cuda_kv_write_slots(kanso_cuda_ctx* ctx, kanso_cuda_kv* kv, uint32_t layer,
                                  const uint32_t* slots, const float* k, const float* v,
                                  int64_t T, const uint32_t* host_slots) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "kv_write_slots: ctx is NULL");
  if (!kv) return fail(ctx, KANSO_ERR_SHAPE, "kv_write_slots: pool is NULL");
  if (layer >= kv->layers)
    return fail(ctx, KANSO_ERR_SHAPE, "Layer index %u out of bounds (%u)", layer, kv->layers);
  if (T < 0) return fail(ctx, KANSO_ERR_SHAPE, "kv_write_slots: T < 0");
  if (T == 0) return KANSO_OK;
  if (host_slots) {
    uint64_t n = (uint64_t)kv->num_blocks * kv->block_size;
    for (int64_t t = 0; t < T; ++t)
      if (host_slots[t] >= n)
        return fail(ctx, KANSO_ERR_SHAPE, "Slot %u out of bounds for %u blocks of size %u",
                    host_slots[t], kv->num_blocks, kv->block_size);
  }
  int64_t stride = (int64_t)kv->kv_heads * kv->head_dim;
  return launch_kv_write(ctx, kv, layer, slots, k, v, T, stride, stride);
}

int32_t kanso_cuda_kv_reset_block(kanso_cuda_ctx* ctx, kanso_cuda_kv* kv, uint32_t block) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "kv_reset_block: ctx is NULL");
  if (!kv) return fail(ctx, KANSO_ERR_SHAPE, "kv_reset_block: pool is NULL");
  if (block >= kv->num_blocks) return KANSO_OK;  // the reference ignores it (quantized_storage.rs:135)
  KvGeom g = kv_geom(kv);
  kv_reset_kernel<<<kv->layers * kv->kv_heads, 128, 0, ctx->stream>>>(g, block, 1);
  return after_launch(ctx, "kv_reset_block");
}

int32_t kanso_cuda_kv_read_token(kanso_cuda_ctx* ctx, const kanso_cuda_kv* kv, uint32_t layer,
                                 uint32_t block, uint32_t offset, int8_t* k_q, int8_t* v_q,
                                 float* k_scale, float* v_scale, float* k_deq, float* v_deq) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "kv_read_token: ctx is NULL");
  if (!kv) return fail(ctx, KANSO_ERR_SHAPE, "kv_read_token: pool is NULL");
  if (layer >= kv->layers)
    return fail(ctx, KANSO_ERR_SHAPE, "Layer index %u out of bounds (%u)", layer, kv->layers);
  if (block >= kv->num_blocks)
    return fail(ctx, KANSO_ERR_SHAPE, "Block index %u out of bounds (%u)", block, kv->num_blocks);
  if (offset >= kv->block_size)
    return fail(ctx, KANSO_ERR_SHAPE, "Offset %u out of bounds for block size %u", offset,
                kv->block_size);
  KvGeom g = kv_geom(kv);
  KANSO_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream), "kv_read_token: sync");
  std::vector<int8_t> kq(kv->head_dim), vq(kv->head_dim);
  for (uint32_t h = 0; h < kv->kv_heads; ++h) {
    const uint8_t* rec = kv->pool + g.rec_offset(layer, block, h);
    float ks, vs;
    KANSO_CUDA_TRY(ctx,
                   cudaMemcpy(kq.data(), rec + g.k_off() + (size_t)offset * kv->head_dim,
                              kv->head_dim, cudaMemcpyDeviceToHost),
                   "kv_read_token");
    KANSO_CUDA_TRY(ctx,
                   cudaMemcpy(vq.data(), rec + g.v_off() + (size_t)offset * kv->head_dim,
                              kv->head_dim, cudaMemcpyDeviceToHost),
                   "kv_read_token");
    KANSO_CUDA_TRY(ctx, cudaMemcpy(&ks, rec + g.ks_off() + 4 * offset, 4, cudaMemcpyDeviceToHost),
                   "kv_read_token");
    KANSO_CUDA_TRY(ctx, cudaMemcpy(&vs, rec + g.vs_off() + 4 * offset, 4, cudaMemcpyDeviceToHost),
                   "kv_read_token");
    if (k_scale) k_scale[h] = ks;
    if (v_scale) v_scale[h] = vs;
    for (uint32_t d = 0; d < kv->head_dim; ++d) {
      size_t i = (size_t)h * kv->head_dim + d;
      if (k_q) k_q[i] = kq[d];
      if (v_q) v_q[i] = vq[d];
      // (src as f32) * scale, or fp8_to_f32(src as u8) * scale (quantized_storage.rs:352-366):
      // exact on any IEEE host
      if (k_deq) k_deq[i] = (g.fp8 ? e4m3_to_f32((uint8_t)kq[d]) : (float)kq[d]) * ks;
      if (v_deq) v_deq[i] = (g.fp8 ? e4m3_to_f32((uint8_t)vq[d]) : (float)vq[d]) * vs;
    }
  }
  return KANSO_OK;
}

uint64_t kanso_cuda_kv_bytes_per_token(const kanso_cuda_kv* kv) {
  if (!kv) return 0;
  // memory_bytes_per_token, quantized_storage.rs:414-419
  return 2ull * kv->kv_heads * kv->head_dim + 2ull * kv->kv_heads * sizeof(float);
}

}  // extern "C"
