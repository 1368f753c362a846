// Block-level kernels of src/quant: dequantise, unpack, quantise, int32 block sums.
// These are the bit-exact statements the parity tests pin; the streaming GEMV uses the
// same device helpers. Multiplies and subtracts that must round separately use the
// __fmul_rn/__fsub_rn/__fdiv_rn intrinsics so the compiler cannot contract them.
#include "ctx.h"

namespace kanso {

// BlockQ8_0::dequantize (src/quant/q8_0.rs:35-39): out = d * (f32)q
__global__ void dequantize_q8_0_kernel(const uint8_t* __restrict__ w, float* __restrict__ out,
                                       int64_t nblocks) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one element per thread
  if (i >= nblocks * 32) return;
  int64_t b = i >> 5;
  int k = (int)(i & 31);
  const uint8_t* blk = w + b * Q8_BYTES;
  float d = f16_bits_to_f32(blk[0] | (blk[1] << 8));
  out[i] = __fmul_rn(d, (float)(int8_t)blk[2 + k]);
}

// BlockQ4_K::dequantize (src/quant/q4_k.rs:30-55): (d*sc)*q - (dmin*m), each step rounded.
__global__ void dequantize_q4_k_kernel(const uint8_t* __restrict__ w, float* __restrict__ out,
                                       int64_t nblocks) {
  int64_t b = blockIdx.x;
  if (b >= nblocks) return;
  const uint8_t* blk = w + b * Q4K_BYTES;
  const uint32_t* hw = reinterpret_cast<const uint32_t*>(blk);
  uint32_t h0 = hw[0];
  float d = f16_bits_to_f32(h0), dmin = f16_bits_to_f32(h0 >> 16);
  uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
  unpack_scales_k4(hw[1], hw[2], hw[3], sc_lo, sc_hi, mn_lo, mn_hi);
  int i = threadIdx.x;       // 256 threads: one weight each
  int g = i >> 6;            // 64-weight group
  int hi = (i >> 5) & 1;     // 0: low nibbles (sub-block 2g), 1: high nibbles (2g+1)
  int j = 2 * g + hi;        // sub-block
  uint32_t scw = j < 4 ? sc_lo : sc_hi, mnw = j < 4 ? mn_lo : mn_hi;
  float sc = (float)((scw >> (8 * (j & 3))) & 0xFF);
  float mn = (float)((mnw >> (8 * (j & 3))) & 0xFF);
  uint8_t byte = blk[16 + 32 * g + (i & 31)];
  float q = (float)(hi ? (byte >> 4) : (byte & 0xF));
  float d1 = __fmul_rn(d, sc), m1 = __fmul_rn(dmin, mn);
  out[b * 256 + i] = __fsub_rn(__fmul_rn(d1, q), m1);
}

// get_scale_min_k4 (src/quant/q4_k.rs:16-26): 8 scales then 8 mins per super-block.
__global__ void unpack_scales_q4_k_kernel(const uint8_t* __restrict__ w, uint8_t* __restrict__ out,
                                          int64_t nblocks) {
  int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  const uint32_t* hw = reinterpret_cast<const uint32_t*>(w + b * Q4K_BYTES);
  uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
  unpack_scales_k4(hw[1], hw[2], hw[3], sc_lo, sc_hi, mn_lo, mn_hi);
  uint32_t* o = reinterpret_cast<uint32_t*>(out + b * 16);
  o[0] = sc_lo;
  o[1] = sc_hi;
  o[2] = mn_lo;
  o[3] = mn_hi;
}

// quantize_row_q8_0 (src/quant/q8_0.rs:13-32,43-48): one warp per block of 32.
__global__ void quantize_row_q8_0_kernel(const float* __restrict__ x, float* __restrict__ d_out,
                                         int8_t* __restrict__ qs_out, int64_t nblocks) {
  int64_t b = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  if (b >= nblocks) return;
  float v = x[b * 32 + lane];
  float amax = fabsf(v);
#pragma unroll
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  float d = __fdiv_rn(amax, 127.0f);
  float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
  float r = roundf(__fmul_rn(v, id));  // half away from zero, as f32::round
  r = fminf(fmaxf(r, -128.0f), 127.0f);
  qs_out[b * 32 + lane] = (int8_t)r;
  if (lane == 0) d_out[b] = d;
}

// The int32 sums of scalar_dot_q8_0_q8_0 (src/quant/q8_0.rs:60-66), one per (row, block).
__global__ void block_isums_q8_0_kernel(const uint8_t* __restrict__ w,
                                        const int8_t* __restrict__ x_qs,
                                        int32_t* __restrict__ isums, int64_t rows, int64_t bpr) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * bpr) return;
  int64_t b = i % bpr;
  const uint8_t* blk = w + i * Q8_BYTES + 2;  // 2-byte aligned: read as 16-bit pairs
  const int8_t* xq = x_qs + b * 32;
  int32_t s = 0;
#pragma unroll
  for (int k = 0; k < 32; k += 4) {
    uint32_t lo = *reinterpret_cast<const uint16_t*>(blk + k);
    uint32_t hi = *reinterpret_cast<const uint16_t*>(blk + k + 2);
    int xw = *reinterpret_cast<const int*>(xq + k);
    s = dp4a_ss((int)(lo | (hi << 16)), xw, s);
  }
  isums[i] = s;
}

}  // namespace kanso

using namespace kanso;

extern "C" {

int32_t kanso_cuda_dequantize_q8_0(kanso_cuda_ctx* ctx, const void* w, float* out,
                                   int64_t nblocks) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "dequantize_q8_0: ctx is NULL");
  if (nblocks < 0 || !w || !out) return fail(ctx, KANSO_ERR_SHAPE, "dequantize_q8_0: bad args");
  if (nblocks == 0) return KANSO_OK;
  int64_t n = nblocks * 32;
  dequantize_q8_0_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(
      (const uint8_t*)w, out, nblocks);
  return after_launch(ctx, "dequantize_q8_0");
}

int32_t kanso_cuda_dequantize_q4_k(kanso_cuda_ctx* ctx, const void* w, float* out,
                                   int64_t nblocks) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "dequantize_q4_k: ctx is NULL");
  if (nblocks < 0 || !w || !out) return fail(ctx, KANSO_ERR_SHAPE, "dequantize_q4_k: bad args");
  if (!aligned16(w)) return fail(ctx, KANSO_ERR_SHAPE, "dequantize_q4_k: w not 16-byte aligned");
  if (nblocks == 0) return KANSO_OK;
  dequantize_q4_k_kernel<<<(unsigned)nblocks, 256, 0, ctx->stream>>>((const uint8_t*)w, out,
                                                                     nblocks);
  return after_launch(ctx, "dequantize_q4_k");
}

int32_t kanso_cuda_unpack_scales_q4_k(kanso_cuda_ctx* ctx, const void* w, uint8_t* out,
                                      int64_t nblocks) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "unpack_scales_q4_k: ctx is NULL");
  if (nblocks < 0 || !w || !out) return fail(ctx, KANSO_ERR_SHAPE, "unpack_scales_q4_k: bad args");
  if (!aligned16(w) || !aligned16(out))
    return fail(ctx, KANSO_ERR_SHAPE, "unpack_scales_q4_k: pointers not 16-byte aligned");
  if (nblocks == 0) return KANSO_OK;
  unpack_scales_q4_k_kernel<<<(unsigned)((nblocks + 127) / 128), 128, 0, ctx->stream>>>(
      (const uint8_t*)w, out, nblocks);
  return after_launch(ctx, "unpack_scales_q4_k");
}

int32_t kanso_cuda_quantize_row_q8_0(kanso_cuda_ctx* ctx, const float* x, float* d_out,
                                     int8_t* qs_out, int64_t cols) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "quantize_row_q8_0: ctx is NULL");
  if (cols < 0 || cols % 32 != 0)
    return fail(ctx, KANSO_ERR_SHAPE, "quantize_row_q8_0: cols %lld is not a multiple of 32",
                (long long)cols);
  if (cols == 0) return KANSO_OK;
  int64_t nb = cols / 32;
  quantize_row_q8_0_kernel<<<(unsigned)((nb * 32 + 255) / 256), 256, 0, ctx->stream>>>(
      x, d_out, qs_out, nb);
  return after_launch(ctx, "quantize_row_q8_0");
}

int32_t kanso_cuda_block_isums_q8_0(kanso_cuda_ctx* ctx, const void* w, const int8_t* x_qs,
                                    int32_t* isums, int64_t rows, int64_t cols) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "block_isums_q8_0: ctx is NULL");
  if (rows < 0 || cols < 0 || cols % 32 != 0)
    return fail(ctx, KANSO_ERR_SHAPE, "block_isums_q8_0: cols %lld is not a multiple of 32",
                (long long)cols);
  if ((reinterpret_cast<uintptr_t>(x_qs) & 3) != 0)
    return fail(ctx, KANSO_ERR_SHAPE, "block_isums_q8_0: x_qs not 4-byte aligned");
  int64_t n = rows * (cols / 32);
  if (n == 0) return KANSO_OK;
  block_isums_q8_0_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(
      (const uint8_t*)w, x_qs, isums, rows, cols / 32);
  return after_launch(ctx, "block_isums_q8_0");
}

}  // extern "C"
