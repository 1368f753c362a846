// Device layout of the quantised (int8 or fp8) KV pool.
//
// The reference keeps, per (layer, block), four host vectors: quants
// [offset][head][dim] and scales [offset][head] for K and for V
// (src/kv_cache/quantized_storage.rs:16-21). On the device one record per
// (layer, block, kv head) holds everything decode attention reads for that head:
//
//   [ K bytes block_size x head_dim ][ V bytes block_size x head_dim ]   (int8, or E4M3 bits)
//   [ k_scale f32 block_size ][ v_scale f32 block_size ]
//
// so that one (sequence, kv head) walk touches one contiguous record per block
// (2176 bytes at block_size 16, head_dim 64). Records are 16-byte multiples.
#pragma once
#include "ctx.h"

struct kanso_cuda_kv {
  kanso_cuda_ctx* ctx = nullptr;
  uint32_t layers = 0, num_blocks = 0, block_size = 0, kv_heads = 0, head_dim = 0;
  int32_t kv_type = 0;
  uint8_t* pool = nullptr;
  size_t pool_bytes = 0;
};

namespace kanso {

struct KvGeom {
  uint32_t layers, num_blocks, block_size, kv_heads, head_dim;
  uint32_t q_bytes;    // block_size * head_dim rounded up to 16
  uint32_t rec_bytes;  // 2*q_bytes + 8*block_size rounded up to 16
  uint32_t fp8;        // 1: the bytes are E4M3 bit patterns with power-of-two scales
  uint8_t* pool;
  __host__ __device__ size_t rec_offset(uint32_t layer, uint32_t block, uint32_t head) const {
    return (((size_t)layer * num_blocks + block) * kv_heads + head) * rec_bytes;
  }
  __host__ __device__ uint32_t k_off() const { return 0; }
  __host__ __device__ uint32_t v_off() const { return q_bytes; }
  __host__ __device__ uint32_t ks_off() const { return 2 * q_bytes; }
  __host__ __device__ uint32_t vs_off() const { return 2 * q_bytes + 4 * block_size; }
};

inline KvGeom kv_geom(const kanso_cuda_kv* kv) {
  KvGeom g;
  g.layers = kv->layers;
  g.num_blocks = kv->num_blocks;
  g.block_size = kv->block_size;
  g.kv_heads = kv->kv_heads;
  g.head_dim = kv->head_dim;
  g.q_bytes = (kv->block_size * kv->head_dim + 15u) & ~15u;
  g.rec_bytes = (2 * g.q_bytes + 8 * kv->block_size + 15u) & ~15u;
  g.fp8 = kv->kv_type == KANSO_KV_FP8 ? 1u : 0u;
  g.pool = kv->pool;
  return g;
}

int32_t launch_kv_write(kanso_cuda_ctx* ctx, kanso_cuda_kv* kv, uint32_t layer,
                        const uint32_t* slots, const float* k, const float* v, int64_t T,
                        int64_t k_stride, int64_t v_stride);

// quantize_head_slice's scale (src/kv_cache/quantized_storage.rs:452-484).
// Int8: amax / 127. Fp8: the smallest power of two that is >= amax / 64, i.e.
// 2^ceil(log2(amax / 64)), taken from the exponent so that no logarithm is rounded.
__host__ __device__ inline float kv_scale_of(float amax, bool fp8) {
  if (!(amax > 0.f)) return 1.0f;
#ifdef __CUDA_ARCH__
  if (!fp8) return __fdiv_rn(amax, 127.0f);
#else
  if (!fp8) return amax / 127.0f;
#endif
  int e;
  const float m = frexpf(amax * 0.015625f, &e);  // amax / 64 = m * 2^e, m in [0.5, 1)
  return ldexpf(1.0f, m == 0.5f ? e - 1 : e);
}

}  // namespace kanso
