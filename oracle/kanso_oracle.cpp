// CPU restatement of kanso-infer's quantized hot path. TEST INFRASTRUCTURE ONLY:
// the checker for the CUDA kernels, never part of the product path. See
// kanso_oracle.h for the parity status and the layout conventions. Compile with
// -ffp-contract=off: every multiply and add below must round separately, as the
// reference's scalar Rust does.
#include "kanso_oracle.h"

#include <cmath>
#include <cstring>
#include <limits>
#include <vector>

namespace {

constexpr int QK8_0 = 32;      // src/quant/q8_0.rs:1
constexpr int Q8_BYTES = 34;   // f16 d + 32 int8
constexpr int QK_K = 256;      // src/quant/q4_k.rs:1
constexpr int Q4K_BYTES = 144; // f16 d, f16 dmin, 12 B scales, 128 B qs

constexpr int ST_OK = 0, ST_SHAPE = 2, ST_UNSUPPORTED = 3;

inline uint32_t f32_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}
inline float bits_f32(uint32_t u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

inline uint16_t load_u16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
inline void store_u16(uint8_t* p, uint16_t v) {
  p[0] = (uint8_t)(v & 0xFF);
  p[1] = (uint8_t)(v >> 8);
}

// f32::round is half away from zero; the `as i8` cast after clamp is exact.
inline int8_t round_clamp_i8(float v, float lo, float hi) {
  float r = std::round(v);
  if (r < lo) r = lo;
  if (r > hi) r = hi;
  return (int8_t)r;
}

// src/quant/q8_0.rs:13-32 on one chunk of 32 floats.
inline float quantize_block_q8_0(const float* x, int8_t* qs) {
  float amax = 0.0f;
  for (int i = 0; i < QK8_0; ++i) {
    float ax = std::fabs(x[i]);
    if (ax > amax) amax = ax;
  }
  float d = amax / 127.0f;
  float id = d != 0.0f ? 1.0f / d : 0.0f;
  for (int i = 0; i < QK8_0; ++i) qs[i] = round_clamp_i8(x[i] * id, -128.0f, 127.0f);
  return d;
}

// src/quant/q8_0.rs:51-57
inline float dot_q8_0(float d, const int8_t* qs, const float* x) {
  float sum = 0.0f;
  for (int i = 0; i < QK8_0; ++i) sum += (float)qs[i] * x[i];
  return d * sum;
}

// src/quant/q8_0.rs:60-66
inline float dot_q8_0_q8_0(float wd, const int8_t* wqs, float xd, const int8_t* xqs,
                           int32_t* isum_out) {
  int32_t s = 0;
  for (int i = 0; i < QK8_0; ++i) s += (int32_t)wqs[i] * (int32_t)xqs[i];
  if (isum_out) *isum_out = s;
  return wd * xd * (float)s;
}

// src/quant/q4_k.rs:16-26
inline void scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
  if (j < 4) {
    *sc = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

// src/quant/q4_k.rs:30-55
inline void dequant_q4_k(float d, float dmin, const uint8_t* scales, const uint8_t* qs,
                         float* out) {
  int is = 0, y = 0;
  for (int j = 0; j < QK_K; j += 64) {
    const uint8_t* q = qs + j / 2;
    uint8_t sc1, m1, sc2, m2;
    scale_min_k4(is, scales, &sc1, &m1);
    float d1 = d * (float)sc1;
    float min1 = dmin * (float)m1;
    scale_min_k4(is + 1, scales, &sc2, &m2);
    float d2 = d * (float)sc2;
    float min2 = dmin * (float)m2;
    for (int i = 0; i < 32; ++i) out[y++] = d1 * (float)(q[i] & 0xF) - min1;
    for (int i = 0; i < 32; ++i) out[y++] = d2 * (float)(q[i] >> 4) - min2;
    is += 2;
  }
}

// src/quant/q4_k.rs:58-66
inline float dot_q4_k(float d, float dmin, const uint8_t* scales, const uint8_t* qs,
                      const float* x) {
  float w[QK_K];
  dequant_q4_k(d, dmin, scales, qs, w);
  float sum = 0.0f;
  for (int i = 0; i < QK_K; ++i) sum += w[i] * x[i];
  return sum;
}

// One (sequence, head) of cpu_paged_attention (src/metal/paged_attention.rs:117-175) over
// rows fetched by `row(t)`.
template <class RowK, class RowV>
void attend_one(const float* q, uint32_t ctx, uint32_t hd, float scale, RowK krow,
                       RowV vrow, float* out) {
  std::vector<float> scores(ctx);
  for (uint32_t t = 0; t < ctx; ++t) {
    const float* k = krow(t);
    float dot = 0.0f;
    for (uint32_t d = 0; d < hd; ++d) dot += q[d] * k[d];
    scores[t] = dot * scale;
  }
  float mx = -INFINITY;
  for (uint32_t t = 0; t < ctx; ++t)
    if (scores[t] > mx) mx = scores[t];
  float sum = 0.0f;
  for (uint32_t t = 0; t < ctx; ++t) {
    scores[t] = std::exp(scores[t] - mx);
    sum += scores[t];
  }
  float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
  for (uint32_t t = 0; t < ctx; ++t) {
    float wgt = scores[t] * inv;
    const float* v = vrow(t);
    for (uint32_t d = 0; d < hd; ++d) out[d] += wgt * v[d];
  }
}

}  // namespace

extern "C" {

uint16_t kanso_ref_f32_to_f16(float f) {
  uint32_t x = f32_bits(f);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t mant = x & 0x007FFFFFu;
  int32_t exp = (int32_t)((x >> 23) & 0xFF);
  if (exp == 0xFF) return (uint16_t)(sign | 0x7C00u | (mant ? 0x200u | (mant >> 13) : 0));
  int32_t e = exp - 127 + 15;
  if (e >= 31) return (uint16_t)(sign | 0x7C00u);
  if (e <= 0) {
    if (e < -10) return (uint16_t)sign;
    mant |= 0x00800000u;
    uint32_t shift = (uint32_t)(14 - e);
    uint32_t half = mant >> shift;
    uint32_t rem = mant & ((1u << shift) - 1);
    uint32_t mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) half++;
    return (uint16_t)(sign | half);
  }
  uint32_t half = ((uint32_t)e << 10) | (mant >> 13);
  uint32_t rem = mant & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++;
  return (uint16_t)(sign | half);
}

float kanso_ref_f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1F;
  uint32_t mant = h & 0x3FFu;
  if (exp == 0) {
    if (mant == 0) return bits_f32(sign);
    int e = -1;
    do {
      mant <<= 1;
      e++;
    } while (!(mant & 0x400u));
    mant &= 0x3FFu;
    return bits_f32(sign | ((uint32_t)(127 - 15 - e) << 23) | (mant << 13));
  }
  if (exp == 31) return bits_f32(sign | 0x7F800000u | (mant << 13));
  return bits_f32(sign | ((exp + 112) << 23) | (mant << 13));
}

/* ------------------------------ Q8_0 ------------------------------ */

void kanso_ref_quantize_row_q8_0(const float* x, int64_t cols, float* d_out, int8_t* qs_out) {
  for (int64_t b = 0; b < cols / QK8_0; ++b)
    d_out[b] = quantize_block_q8_0(x + b * QK8_0, qs_out + b * QK8_0);
}

void kanso_ref_quantize_weights_q8_0(const float* w, int64_t rows, int64_t cols,
                                     uint8_t* gguf_out) {
  int64_t nb = rows * (cols / QK8_0);
  for (int64_t b = 0; b < nb; ++b) {
    int8_t qs[QK8_0];
    float d = quantize_block_q8_0(w + b * QK8_0, qs);
    uint8_t* o = gguf_out + b * Q8_BYTES;
    store_u16(o, kanso_ref_f32_to_f16(d));
    std::memcpy(o + 2, qs, QK8_0);
  }
}

void kanso_ref_dequantize_q8_0(const uint8_t* gguf, int64_t nblocks, float* out) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t* blk = gguf + b * Q8_BYTES;
    float d = kanso_ref_f16_to_f32(load_u16(blk));
    const int8_t* qs = (const int8_t*)(blk + 2);
    for (int i = 0; i < QK8_0; ++i) out[b * QK8_0 + i] = d * (float)qs[i];
  }
}

float kanso_ref_dot_q8_0_ref(float d, const int8_t* qs, const float* x) {
  return dot_q8_0(d, qs, x);
}

float kanso_ref_dot_q8_0_q8_0_ref(float wd, const int8_t* wqs, float xd, const int8_t* xqs,
                                  int32_t* isum) {
  return dot_q8_0_q8_0(wd, wqs, xd, xqs, isum);
}

void kanso_ref_gemv_q8_0(const uint8_t* w, const float* x, float* out, int64_t rows,
                         int64_t cols) {
  int64_t bpr = cols / QK8_0;
  for (int64_t r = 0; r < rows; ++r) {
    const uint8_t* row = w + r * bpr * Q8_BYTES;
    float sum = 0.0f;
    for (int64_t b = 0; b < bpr; ++b) {
      const uint8_t* blk = row + b * Q8_BYTES;
      sum += dot_q8_0(kanso_ref_f16_to_f32(load_u16(blk)), (const int8_t*)(blk + 2),
                      x + b * QK8_0);
    }
    out[r] = sum;
  }
}

void kanso_ref_gemv_q8_0_ref(const float* d, const int8_t* qs, const float* x, float* out,
                             int64_t rows, int64_t cols) {
  int64_t bpr = cols / QK8_0;
  for (int64_t r = 0; r < rows; ++r) {
    float sum = 0.0f;
    for (int64_t b = 0; b < bpr; ++b)
      sum += dot_q8_0(d[r * bpr + b], qs + (r * bpr + b) * QK8_0, x + b * QK8_0);
    out[r] = sum;
  }
}

static void gemv_q8_0_q8_prequant(const uint8_t* w, const float* xd, const int8_t* xq, float* out,
                                  int64_t rows, int64_t cols) {
  int64_t bpr = cols / QK8_0;
  for (int64_t r = 0; r < rows; ++r) {
    const uint8_t* row = w + r * bpr * Q8_BYTES;
    float sum = 0.0f;
    for (int64_t b = 0; b < bpr; ++b) {
      const uint8_t* blk = row + b * Q8_BYTES;
      sum += dot_q8_0_q8_0(kanso_ref_f16_to_f32(load_u16(blk)), (const int8_t*)(blk + 2), xd[b],
                           xq + b * QK8_0, nullptr);
    }
    out[r] = sum;
  }
}

void kanso_ref_gemv_q8_0_q8(const uint8_t* w, const float* x, float* out, int64_t rows,
                            int64_t cols) {
  std::vector<float> xd(cols / QK8_0);
  std::vector<int8_t> xq(cols);
  kanso_ref_quantize_row_q8_0(x, cols, xd.data(), xq.data());
  gemv_q8_0_q8_prequant(w, xd.data(), xq.data(), out, rows, cols);
}

void kanso_ref_block_isums_q8_0(const uint8_t* w, const int8_t* x_qs, int32_t* isums,
                                int64_t rows, int64_t cols) {
  int64_t bpr = cols / QK8_0;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t b = 0; b < bpr; ++b) {
      const int8_t* wq = (const int8_t*)(w + (r * bpr + b) * Q8_BYTES + 2);
      int32_t s = 0;
      for (int i = 0; i < QK8_0; ++i) s += (int32_t)wq[i] * (int32_t)x_qs[b * QK8_0 + i];
      isums[r * bpr + b] = s;
    }
}

void kanso_ref_gemm_q8_0(const uint8_t* w, const float* x, float* y, int64_t M, int64_t N,
                         int64_t K, int32_t act_mode) {
  for (int64_t m = 0; m < M; ++m) {
    if (act_mode == 1)
      kanso_ref_gemv_q8_0_q8(w, x + m * K, y + m * N, N, K);
    else
      kanso_ref_gemv_q8_0(w, x + m * K, y + m * N, N, K);
  }
}

/* ------------------------------ Q4_K ------------------------------ */

void kanso_ref_get_scale_min_k4(int32_t j, const uint8_t* scales12, uint8_t* sc, uint8_t* m) {
  scale_min_k4(j, scales12, sc, m);
}

void kanso_ref_unpack_scales_q4_k(const uint8_t* gguf, int64_t nblocks, uint8_t* out) {
  for (int64_t b = 0; b < nblocks; ++b)
    for (int j = 0; j < 8; ++j)
      scale_min_k4(j, gguf + b * Q4K_BYTES + 4, out + b * 16 + j, out + b * 16 + 8 + j);
}

void kanso_ref_dequantize_q4_k_ref(float d, float dmin, const uint8_t* scales12,
                                   const uint8_t* qs128, float* out256) {
  dequant_q4_k(d, dmin, scales12, qs128, out256);
}

void kanso_ref_dequantize_q4_k(const uint8_t* gguf, int64_t nblocks, float* out) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t* blk = gguf + b * Q4K_BYTES;
    dequant_q4_k(kanso_ref_f16_to_f32(load_u16(blk)), kanso_ref_f16_to_f32(load_u16(blk + 2)),
                 blk + 4, blk + 16, out + b * QK_K);
  }
}

float kanso_ref_dot_q4_k_ref(float d, float dmin, const uint8_t* scales12, const uint8_t* qs128,
                             const float* x256) {
  return dot_q4_k(d, dmin, scales12, qs128, x256);
}

void kanso_ref_gemv_q4_k(const uint8_t* w, const float* x, float* out, int64_t rows,
                         int64_t cols) {
  int64_t bpr = cols / QK_K;
  for (int64_t r = 0; r < rows; ++r) {
    float sum = 0.0f;
    for (int64_t b = 0; b < bpr; ++b) {
      const uint8_t* blk = w + (r * bpr + b) * Q4K_BYTES;
      sum += dot_q4_k(kanso_ref_f16_to_f32(load_u16(blk)),
                      kanso_ref_f16_to_f32(load_u16(blk + 2)), blk + 4, blk + 16, x + b * QK_K);
    }
    out[r] = sum;
  }
}

void kanso_ref_gemm_q4_k(const uint8_t* w, const float* x, float* y, int64_t M, int64_t N,
                         int64_t K) {
  for (int64_t m = 0; m < M; ++m) kanso_ref_gemv_q4_k(w, x + m * K, y + m * N, N, K);
}

void kanso_ref_quantize_weights_q4_k(const float* w, int64_t rows, int64_t cols,
                                     uint8_t* gguf_out) {
  int64_t nsb = rows * (cols / QK_K);
  for (int64_t b = 0; b < nsb; ++b) {
    const float* x = w + b * QK_K;
    uint8_t* o = gguf_out + b * Q4K_BYTES;
    float sub_scale[8], sub_min[8];
    float max_scale = 0.0f, max_min = 0.0f;
    for (int s = 0; s < 8; ++s) {
      float lo = 0.0f, hi = 0.0f;  // the grid always contains 0 on its low side
      for (int i = 0; i < 32; ++i) {
        float v = x[s * 32 + i];
        if (v < lo) lo = v;
        if (v > hi) hi = v;
      }
      sub_scale[s] = (hi - lo) / 15.0f;
      sub_min[s] = -lo;
      if (sub_scale[s] > max_scale) max_scale = sub_scale[s];
      if (sub_min[s] > max_min) max_min = sub_min[s];
    }
    uint16_t dh = kanso_ref_f32_to_f16(max_scale / 63.0f);
    uint16_t dmh = kanso_ref_f32_to_f16(max_min / 63.0f);
    float d = kanso_ref_f16_to_f32(dh), dmin = kanso_ref_f16_to_f32(dmh);
    uint8_t sc[8], mn[8];
    for (int s = 0; s < 8; ++s) {
      float a = d > 0.0f ? std::round(sub_scale[s] / d) : 0.0f;
      float m = dmin > 0.0f ? std::round(sub_min[s] / dmin) : 0.0f;
      sc[s] = (uint8_t)(a > 63.0f ? 63.0f : a);
      mn[s] = (uint8_t)(m > 63.0f ? 63.0f : m);
    }
    store_u16(o, dh);
    store_u16(o + 2, dmh);
    uint8_t* ps = o + 4;
    for (int j = 0; j < 4; ++j) {
      ps[j] = (uint8_t)(sc[j] | ((sc[j + 4] >> 4) << 6));
      ps[j + 4] = (uint8_t)(mn[j] | ((mn[j + 4] >> 4) << 6));
      ps[j + 8] = (uint8_t)((sc[j + 4] & 0xF) | ((mn[j + 4] & 0xF) << 4));
    }
    uint8_t q[QK_K];
    for (int s = 0; s < 8; ++s) {
      float es = d * (float)sc[s], em = dmin * (float)mn[s];
      for (int i = 0; i < 32; ++i) {
        float v = es > 0.0f ? std::round((x[s * 32 + i] + em) / es) : 0.0f;
        if (v < 0.0f) v = 0.0f;
        if (v > 15.0f) v = 15.0f;
        q[s * 32 + i] = (uint8_t)v;
      }
    }
    uint8_t* pq = o + 16;
    for (int g = 0; g < 4; ++g)
      for (int i = 0; i < 32; ++i)
        pq[g * 32 + i] = (uint8_t)(q[g * 64 + i] | (q[g * 64 + 32 + i] << 4));
  }
}

/* --------------------------- int8 / fp8 KV pool --------------------------- */

struct kanso_ref_kv {
  uint32_t layers, num_blocks, block_size, kv_heads, head_dim;
  // [layer][block] -> planes in the reference's order: quants [offset][head][dim],
  // scales [offset][head] (src/kv_cache/quantized_storage.rs:16-21).
  std::vector<int8_t> kq, vq;
  std::vector<float> ks, vs;
  int32_t fp8 = 0;  // QuantMode::Fp8: the bytes are E4M3 bit patterns (quantized_storage.rs:7-10)
  size_t q_per_block() const { return (size_t)block_size * kv_heads * head_dim; }
  size_t s_per_block() const { return (size_t)block_size * kv_heads; }
  size_t blk(uint32_t layer, uint32_t block) const { return (size_t)layer * num_blocks + block; }
};

float kanso_ref_kv_quantize_head(const float* x, int32_t n, int8_t* q) {
  float amax = 0.0f;
  for (int i = 0; i < n; ++i) {
    float ax = std::fabs(x[i]);
    if (ax > amax) amax = ax;
  }
  float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
  float inv = 1.0f / scale;
  for (int i = 0; i < n; ++i) q[i] = round_clamp_i8(x[i] * inv, -127.0f, 127.0f);
  return scale;
}

/* float8::F8E4M3 (crate float8 0.7.0, not vendored in the reference tree): the OCP E4M3 format,
 * 1 sign, 4 exponent bits with bias 7, 3 mantissa bits, no infinities, S.1111.111 = NaN, largest
 * finite value 448. Restated from the published format; conversion from f32 rounds to nearest,
 * ties to even, subnormals (multiples of 2^-9) included. The quantiser below never produces a
 * magnitude above 64, so the overflow rule of the crate is not exercised. */
float kanso_ref_fp8_e4m3_to_f32(uint8_t b) {
  const int e = (b >> 3) & 15, m = b & 7;
  float v;
  if (e == 15 && m == 7)
    v = std::numeric_limits<float>::quiet_NaN();
  else if (e == 0)
    v = std::ldexp((float)m, -9);
  else
    v = std::ldexp(1.0f + (float)m / 8.0f, e - 7);
  return (b & 0x80) ? -v : v;
}

uint8_t kanso_ref_fp8_e4m3_from_f32(float x) {
  const uint8_t sign = std::signbit(x) ? 0x80 : 0;
  if (std::isnan(x)) return sign | 0x7F;
  const float a = std::fabs(x);
  if (a >= 464.0f) return sign | 0x7E;  // beyond the midpoint above 448: saturate
  if (a < 0.015625f) {                   // below 2^-6: subnormal grid of 2^-9
    const int q = (int)std::nearbyint(std::ldexp(a, 9));  // ties to even; 8 becomes the first normal
    return sign | (uint8_t)q;
  }
  int e;
  std::frexp(a, &e);  // a = m * 2^e, m in [0.5, 1): exponent of the leading bit is e - 1
  int ex = e - 1;
  int q = (int)std::nearbyint(std::ldexp(a, 3 - ex));  // 8..16
  if (q == 16) {
    q = 8;
    ++ex;
  }
  if (ex > 8) return sign | 0x7E;
  uint8_t bits = (uint8_t)(((ex + 7) << 3) | (q - 8));
  if (bits == 0x7F) bits = 0x7E;
  return sign | bits;
}

/* quantize_head_slice, Fp8 arm (quantized_storage.rs:470-484), written as the reference writes
 * it: scale = 2^ceil(log2(amax / 64)) through the platform's f32 log2. */
float kanso_ref_kv_quantize_head_fp8(const float* x, int32_t n, int8_t* q) {
  float amax = 0.0f;
  for (int i = 0; i < n; ++i) {
    float ax = std::fabs(x[i]);
    if (ax > amax) amax = ax;
  }
  float scale = 1.0f;
  if (amax > 0.0f) {
    const int exp = (int)std::ceil(std::log2(amax / 64.0f));
    scale = std::ldexp(1.0f, exp);  // 2.0f32.powi(exp)
  }
  const float inv = 1.0f / scale;
  for (int i = 0; i < n; ++i) q[i] = (int8_t)kanso_ref_fp8_e4m3_from_f32(x[i] * inv);
  return scale;
}

kanso_ref_kv* kanso_ref_kv_create_typed(uint32_t layers, uint32_t num_blocks, uint32_t block_size,
                                        uint32_t kv_heads, uint32_t head_dim, int32_t fp8) {
  kanso_ref_kv* kv = kanso_ref_kv_create(layers, num_blocks, block_size, kv_heads, head_dim);
  kv->fp8 = fp8 ? 1 : 0;
  return kv;
}

kanso_ref_kv* kanso_ref_kv_create(uint32_t layers, uint32_t num_blocks, uint32_t block_size,
                                  uint32_t kv_heads, uint32_t head_dim) {
  auto* kv = new kanso_ref_kv{layers, num_blocks, block_size, kv_heads, head_dim, {}, {}, {}, {}};
  size_t nq = (size_t)layers * num_blocks * kv->q_per_block();
  size_t ns = (size_t)layers * num_blocks * kv->s_per_block();
  kv->kq.assign(nq, 0);
  kv->vq.assign(nq, 0);
  kv->ks.assign(ns, 1.0f);
  kv->vs.assign(ns, 1.0f);
  return kv;
}

void kanso_ref_kv_destroy(kanso_ref_kv* kv) { delete kv; }

int32_t kanso_ref_kv_write_token(kanso_ref_kv* kv, uint32_t layer, uint32_t block,
                                 uint32_t offset, const float* k, const float* v) {
  if (layer >= kv->layers || block >= kv->num_blocks || offset >= kv->block_size)
    return ST_SHAPE;
  size_t b = kv->blk(layer, block);
  uint32_t hd = kv->head_dim, H = kv->kv_heads;
  for (uint32_t h = 0; h < H; ++h) {
    size_t si = b * kv->s_per_block() + (size_t)offset * H + h;
    size_t qi = b * kv->q_per_block() + (size_t)offset * H * hd + (size_t)h * hd;
    if (kv->fp8) {
      kv->ks[si] = kanso_ref_kv_quantize_head_fp8(k + h * hd, (int32_t)hd, &kv->kq[qi]);
      kv->vs[si] = kanso_ref_kv_quantize_head_fp8(v + h * hd, (int32_t)hd, &kv->vq[qi]);
    } else {
      kv->ks[si] = kanso_ref_kv_quantize_head(k + h * hd, (int32_t)hd, &kv->kq[qi]);
      kv->vs[si] = kanso_ref_kv_quantize_head(v + h * hd, (int32_t)hd, &kv->vq[qi]);
    }
  }
  return ST_OK;
}

int32_t kanso_ref_kv_write_slots(kanso_ref_kv* kv, uint32_t layer, const uint32_t* slots,
                                 const float* k, const float* v, int64_t T) {
  const size_t row = (size_t)kv->kv_heads * kv->head_dim;
  for (int64_t t = 0; t < T; ++t) {
    int32_t st = kanso_ref_kv_write_token(kv, layer, slots[t] / kv->block_size,
                                          slots[t] % kv->block_size, k + t * row, v + t * row);
    if (st != ST_OK) return st;
  }
  return ST_OK;
}

void kanso_ref_kv_reset_block(kanso_ref_kv* kv, uint32_t block) {
  if (block >= kv->num_blocks) return;
  for (uint32_t l = 0; l < kv->layers; ++l) {
    size_t b = kv->blk(l, block);
    std::memset(&kv->kq[b * kv->q_per_block()], 0, kv->q_per_block());
    std::memset(&kv->vq[b * kv->q_per_block()], 0, kv->q_per_block());
    for (size_t i = 0; i < kv->s_per_block(); ++i) {
      kv->ks[b * kv->s_per_block() + i] = 1.0f;
      kv->vs[b * kv->s_per_block() + i] = 1.0f;
    }
  }
}

/* (src as f32), or fp8_to_f32(src as u8) (quantized_storage.rs:352-366) */
static inline float kv_value(const kanso_ref_kv* kv, int8_t b) {
  return kv->fp8 ? kanso_ref_fp8_e4m3_to_f32((uint8_t)b) : (float)b;
}

int32_t kanso_ref_kv_read_token(const kanso_ref_kv* kv, uint32_t layer, uint32_t block,
                                uint32_t offset, int8_t* k_q, int8_t* v_q, float* k_scale,
                                float* v_scale, float* k_deq, float* v_deq) {
  if (layer >= kv->layers || block >= kv->num_blocks || offset >= kv->block_size)
    return ST_SHAPE;
  size_t b = kv->blk(layer, block);
  uint32_t hd = kv->head_dim, H = kv->kv_heads;
  for (uint32_t h = 0; h < H; ++h) {
    size_t si = b * kv->s_per_block() + (size_t)offset * H + h;
    size_t qi = b * kv->q_per_block() + (size_t)offset * H * hd + (size_t)h * hd;
    if (k_scale) k_scale[h] = kv->ks[si];
    if (v_scale) v_scale[h] = kv->vs[si];
    for (uint32_t d = 0; d < hd; ++d) {
      if (k_q) k_q[h * hd + d] = kv->kq[qi + d];
      if (v_q) v_q[h * hd + d] = kv->vq[qi + d];
      if (k_deq) k_deq[h * hd + d] = kv_value(kv, kv->kq[qi + d]) * kv->ks[si];
      if (v_deq) v_deq[h * hd + d] = kv_value(kv, kv->vq[qi + d]) * kv->vs[si];
    }
  }
  return ST_OK;
}

int32_t kanso_ref_kv_gather(const kanso_ref_kv* kv, uint32_t layer, const uint32_t* blocks,
                            uint32_t nblocks, uint32_t num_tokens, float* k_out, float* v_out) {
  if (layer >= kv->layers) return ST_SHAPE;
  uint32_t hd = kv->head_dim, H = kv->kv_heads;
  for (uint32_t t = 0; t < num_tokens; ++t) {
    uint32_t bi = t / kv->block_size, off = t % kv->block_size;
    if (bi >= nblocks) return ST_SHAPE;
    if (blocks[bi] >= kv->num_blocks) return ST_SHAPE;
    size_t b = kv->blk(layer, blocks[bi]);
    for (uint32_t h = 0; h < H; ++h) {
      size_t si = b * kv->s_per_block() + (size_t)off * H + h;
      size_t qi = b * kv->q_per_block() + (size_t)off * H * hd + (size_t)h * hd;
      float ksc = kv->ks[si], vsc = kv->vs[si];
      float* kd = k_out + ((size_t)t * H + h) * hd;
      float* vd = v_out + ((size_t)t * H + h) * hd;
      for (uint32_t d = 0; d < hd; ++d) {
        kd[d] = kv_value(kv, kv->kq[qi + d]) * ksc;
        vd[d] = kv_value(kv, kv->vq[qi + d]) * vsc;
      }
    }
  }
  return ST_OK;
}

/* ------------------------------ paged attention ------------------------------ */

uint32_t kanso_ref_pa_num_partitions(const kanso_ref_pa_params* p) {
  uint64_t cap = (uint64_t)p->max_num_blocks_per_seq * p->block_size;
  if (cap > 0xFFFFFFFFull) cap = 0xFFFFFFFFull;  // saturating_mul
  uint64_t parts = (cap + 255) / 256;
  return (uint32_t)(parts < 1 ? 1 : parts);
}

int32_t kanso_ref_validate_pa_params(const kanso_ref_pa_params* p) {
  if (p->num_seqs == 0 || p->num_heads == 0 || p->num_kv_heads == 0) return ST_UNSUPPORTED;
  if (p->num_heads % p->num_kv_heads != 0) return ST_UNSUPPORTED;
  if (p->num_heads / p->num_kv_heads > 8) return ST_UNSUPPORTED;
  if (p->head_dim == 0 || p->head_dim > 256) return ST_UNSUPPORTED;
  if (p->block_size == 0 || p->max_num_blocks_per_seq == 0) return ST_UNSUPPORTED;
  uint64_t partial = (uint64_t)p->num_seqs * p->num_heads * kanso_ref_pa_num_partitions(p) *
                     p->head_dim;
  if (partial > (1ull << 31)) return ST_UNSUPPORTED;
  return ST_OK;
}

void kanso_ref_paged_attention_f32(const float* q, const float* k_cache, const float* v_cache,
                                   const uint32_t* block_tables, const uint32_t* context_lens,
                                   const kanso_ref_pa_params* p, float* out) {
  uint32_t H = p->num_heads, KH = p->num_kv_heads, hd = p->head_dim, bs = p->block_size;
  uint32_t group = H / KH;
  std::memset(out, 0, sizeof(float) * (size_t)p->num_seqs * H * hd);
  for (uint32_t s = 0; s < p->num_seqs; ++s) {
    uint32_t ctx = context_lens[s];
    if (ctx == 0) continue;
    const uint32_t* table = block_tables + (size_t)s * p->max_num_blocks_per_seq;
    for (uint32_t h = 0; h < H; ++h) {
      uint32_t kvh = h / group;
      auto off = [&](uint32_t t) {
        return (size_t)table[t / bs] * ((size_t)bs * KH * hd) + (size_t)(t % bs) * (KH * hd) +
               (size_t)kvh * hd;
      };
      attend_one(
          q + ((size_t)s * H + h) * hd, ctx, hd, p->scale,
          [&](uint32_t t) { return k_cache + off(t); },
          [&](uint32_t t) { return v_cache + off(t); }, out + ((size_t)s * H + h) * hd);
    }
  }
}

int32_t kanso_ref_paged_attention_int8(const kanso_ref_kv* kv, uint32_t layer, const float* q,
                                       const uint32_t* block_tables,
                                       const uint32_t* context_lens,
                                       const kanso_ref_pa_params* p, float* out) {
  uint32_t H = p->num_heads, KH = p->num_kv_heads, hd = p->head_dim;
  if (KH != kv->kv_heads || hd != kv->head_dim || p->block_size != kv->block_size)
    return ST_SHAPE;
  uint32_t group = H / KH;
  std::memset(out, 0, sizeof(float) * (size_t)p->num_seqs * H * hd);
  for (uint32_t s = 0; s < p->num_seqs; ++s) {
    uint32_t ctx = context_lens[s];
    if (ctx == 0) continue;
    std::vector<float> kd((size_t)ctx * KH * hd), vd((size_t)ctx * KH * hd);
    int32_t st = kanso_ref_kv_gather(kv, layer, block_tables + (size_t)s * p->max_num_blocks_per_seq,
                                     p->max_num_blocks_per_seq, ctx, kd.data(), vd.data());
    if (st != ST_OK) return st;
    for (uint32_t h = 0; h < H; ++h) {
      uint32_t kvh = h / group;
      attend_one(
          q + ((size_t)s * H + h) * hd, ctx, hd, p->scale,
          [&](uint32_t t) { return kd.data() + ((size_t)t * KH + kvh) * hd; },
          [&](uint32_t t) { return vd.data() + ((size_t)t * KH + kvh) * hd; },
          out + ((size_t)s * H + h) * hd);
    }
  }
  return ST_OK;
}

// Chunked-prefill attention of one sequence, as Model::forward_prefill does it
// (src/model.rs:1027-1085 with gqa_attention, src/model.rs:764-795): gather the whole prefix
// 0..start_pos+chunk_len from the pool (the chunk's own tokens were written just before), form
// the score matrix [chunk_len, total_len] scaled by `scale`, ADD the offset causal mask (-1e9
// where key j > start_pos + i), softmax over the row (max-subtracted), then P.V.
int32_t kanso_ref_prefill_attention_int8(const kanso_ref_kv* kv, uint32_t layer, const float* q,
                                         const uint32_t* blocks, uint32_t nblocks,
                                         uint32_t start_pos, uint32_t chunk_len,
                                         uint32_t num_heads, float scale, float* out) {
  const uint32_t KH = kv->kv_heads, hd = kv->head_dim;
  if (num_heads % KH != 0 || chunk_len == 0) return ST_SHAPE;
  const uint32_t group = num_heads / KH, total = start_pos + chunk_len;
  std::vector<float> kd((size_t)total * KH * hd), vd((size_t)total * KH * hd);
  int32_t st = kanso_ref_kv_gather(kv, layer, blocks, nblocks, total, kd.data(), vd.data());
  if (st != ST_OK) return st;
  std::vector<float> sc(total);
  for (uint32_t i = 0; i < chunk_len; ++i) {
    for (uint32_t h = 0; h < num_heads; ++h) {
      const uint32_t kvh = h / group;
      const float* qv = q + ((size_t)i * num_heads + h) * hd;
      float mx = -INFINITY;
      for (uint32_t j = 0; j < total; ++j) {
        const float* kr = kd.data() + ((size_t)j * KH + kvh) * hd;
        float dot = 0.0f;
        for (uint32_t d = 0; d < hd; ++d) dot += qv[d] * kr[d];
        float v = dot * scale;
        if (j > start_pos + i) v = v + -1e9f;
        sc[j] = v;
        mx = std::max(mx, v);
      }
      float sum = 0.0f;
      for (uint32_t j = 0; j < total; ++j) {
        sc[j] = std::exp(sc[j] - mx);
        sum += sc[j];
      }
      float* o = out + ((size_t)i * num_heads + h) * hd;
      for (uint32_t d = 0; d < hd; ++d) o[d] = 0.0f;
      for (uint32_t j = 0; j < total; ++j) {
        const float pj = sc[j] / sum;
        const float* vr = vd.data() + ((size_t)j * KH + kvh) * hd;
        for (uint32_t d = 0; d < hd; ++d) o[d] += pj * vr[d];
      }
    }
  }
  return ST_OK;
}

/* ------------------------------ glue ------------------------------ */

// src/model.rs:653-659: x / sqrt(mean(x^2) + eps) * w
void kanso_ref_rmsnorm(const float* x, const float* w, float* out, int64_t rows, int64_t hidden,
                       float eps) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * hidden;
    float ss = 0.0f;
    for (int64_t i = 0; i < hidden; ++i) ss += xr[i] * xr[i];
    float rms = std::sqrt(ss / (float)hidden + eps);
    for (int64_t i = 0; i < hidden; ++i) out[r * hidden + i] = xr[i] / rms * w[i];
  }
}

// src/model.rs:698-719
void kanso_ref_rope_table(float theta, int64_t len, int64_t head_dim, float* cos_out,
                          float* sin_out) {
  int64_t half = head_dim / 2;
  std::vector<float> freq(half);
  for (int64_t j = 0; j < half; ++j)
    freq[j] = std::pow(theta, -2.0f * (float)j / (float)head_dim);
  for (int64_t p = 0; p < len; ++p)
    for (int64_t j = 0; j < half; ++j) {
      float a = (float)p * freq[j];
      cos_out[p * half + j] = std::cos(a);
      sin_out[p * half + j] = std::sin(a);
    }
}

// src/model.rs:721-737
void kanso_ref_rope(float* x, const uint32_t* positions, int64_t T, int64_t heads,
                    int64_t head_dim, float theta) {
  int64_t half = head_dim / 2;
  std::vector<float> c(half), s(half);
  for (int64_t t = 0; t < T; ++t) {
    for (int64_t j = 0; j < half; ++j) {
      float a = (float)positions[t] * std::pow(theta, -2.0f * (float)j / (float)head_dim);
      c[j] = std::cos(a);
      s[j] = std::sin(a);
    }
    for (int64_t h = 0; h < heads; ++h) {
      float* v = x + (t * heads + h) * head_dim;
      for (int64_t j = 0; j < half; ++j) {
        float a = v[j], b = v[j + half];
        v[j] = a * c[j] - b * s[j];
        v[j + half] = a * s[j] + b * c[j];
      }
    }
  }
}

// src/model.rs:367-382 with candle_nn::ops::silu = g / (1 + exp(-g))
void kanso_ref_silu_mul(const float* gate, const float* up, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = gate[i] / (1.0f + std::exp(-gate[i])) * up[i];
}

// src/sampler.rs:7-17
uint32_t kanso_ref_greedy_token(const float* logits, int64_t n) {
  int64_t best = 0;
  float bv = -INFINITY;
  for (int64_t i = 0; i < n; ++i)
    if (logits[i] > bv) {
      bv = logits[i];
      best = i;
    }
  return (uint32_t)best;
}

// src/model.rs:64-116
uint32_t kanso_ref_padded_decode_tables(uint32_t block_size, const uint32_t* tables,
                                        const uint32_t* table_lens, const uint32_t* context_lens,
                                        uint32_t num_seqs, uint32_t* out, uint32_t out_capacity,
                                        int32_t* status) {
  *status = ST_OK;
  uint32_t max_blocks = 1;
  for (uint32_t s = 0; s < num_seqs; ++s) {
    uint32_t need = (context_lens[s] + block_size - 1) / block_size;
    if (need < 1) need = 1;
    if (need > max_blocks) max_blocks = need;
  }
  if ((uint64_t)num_seqs * max_blocks > out_capacity) {
    *status = ST_SHAPE;
    return 0;
  }
  size_t base = 0;
  for (uint32_t s = 0; s < num_seqs; ++s) {
    uint32_t need = (context_lens[s] + block_size - 1) / block_size;
    if (need < 1) need = 1;
    if (table_lens[s] < need) {
      *status = ST_SHAPE;
      return 0;
    }
    for (uint32_t b = 0; b < max_blocks; ++b)
      out[(size_t)s * max_blocks + b] = tables[base + (b < need - 1 ? b : need - 1)];
    base += table_lens[s];
  }
  return max_blocks;
}

/* ------------------------------ decode step ------------------------------ */

struct kanso_ref_model {
  kanso_ref_model_config cfg;
  struct Lin {
    const uint8_t* w = nullptr;
    int64_t rows = 0, cols = 0;
  };
  struct Layer {
    Lin w[7];
    std::vector<float> attn_norm, ffn_norm;
  };
  std::vector<Layer> layers;
  Lin token_embd, output;
  std::vector<float> final_norm;
};

kanso_ref_model* kanso_ref_model_create(const kanso_ref_model_config* cfg) {
  auto* m = new kanso_ref_model;
  m->cfg = *cfg;
  m->layers.resize(cfg->num_hidden_layers);
  return m;
}
void kanso_ref_model_destroy(kanso_ref_model* m) { delete m; }

int32_t kanso_ref_model_set_weight(kanso_ref_model* m, uint32_t layer, int32_t which,
                                   const uint8_t* gguf, int64_t rows, int64_t cols) {
  kanso_ref_model::Lin l;
  l.w = gguf;
  l.rows = rows;
  l.cols = cols;
  if (cols % QK8_0) return ST_SHAPE;
  if (which == 7) {
    m->token_embd = l;
    return ST_OK;
  }
  if (which == 8) {
    m->output = l;
    return ST_OK;
  }
  if (which < 0 || which > 8 || layer >= m->layers.size()) return ST_SHAPE;
  m->layers[layer].w[which] = l;
  return ST_OK;
}

int32_t kanso_ref_model_set_norm(kanso_ref_model* m, uint32_t layer, int32_t which,
                                 const float* w, int64_t n) {
  if (n != (int64_t)m->cfg.hidden_size) return ST_SHAPE;
  if (which == 2) {
    m->final_norm.assign(w, w + n);
    return ST_OK;
  }
  if (layer >= m->layers.size() || which < 0 || which > 2) return ST_SHAPE;
  (which == 0 ? m->layers[layer].attn_norm : m->layers[layer].ffn_norm).assign(w, w + n);
  return ST_OK;
}

static void linear(const kanso_ref_model::Lin& l, const float* x, float* y, int32_t act_mode) {
  if (act_mode == 1)
    kanso_ref_gemv_q8_0_q8(l.w, x, y, l.rows, l.cols);
  else
    kanso_ref_gemv_q8_0(l.w, x, y, l.rows, l.cols);
}

int32_t kanso_ref_decode_step(const kanso_ref_model* m, kanso_ref_kv* kv, const uint32_t* tokens,
                              const uint32_t* positions, const uint32_t* slots,
                              const uint32_t* block_tables, const uint32_t* context_lens,
                              uint32_t B, uint32_t max_blocks, int32_t act_mode,
                              uint32_t num_layers_to_run, float* logits_out) {
  const auto& c = m->cfg;
  uint32_t hidden = c.hidden_size, H = c.num_attention_heads, KH = c.num_key_value_heads;
  uint32_t hd = hidden / H, inter = c.intermediate_size, bs = kv->block_size;
  uint32_t L = num_layers_to_run ? num_layers_to_run : c.num_hidden_layers;
  if (L > c.num_hidden_layers) return ST_SHAPE;
  std::vector<float> h(hidden), normed(hidden), qv(H * hd), kvec(KH * hd), vvec(KH * hd),
      attn(H * hd), proj(hidden), gate(inter), up(inter), act(inter);
  kanso_ref_pa_params pa{1, H, KH, hd, bs, max_blocks, 1.0f / std::sqrt((float)hd)};
  for (uint32_t s = 0; s < B; ++s) {
    if (tokens[s] >= (uint32_t)m->token_embd.rows) return ST_SHAPE;
    uint32_t pos = positions[s], slot = slots[s];
    uint32_t block = slot / bs, offset = slot % bs;
    // embed: dequantise the selected row (src/weights.rs:50-57)
    kanso_ref_dequantize_q8_0(m->token_embd.w + (size_t)tokens[s] * (hidden / QK8_0) * Q8_BYTES,
                              hidden / QK8_0, h.data());
    for (uint32_t l = 0; l < L; ++l) {
      const auto& ly = m->layers[l];
      kanso_ref_rmsnorm(h.data(), ly.attn_norm.data(), normed.data(), 1, hidden, c.rms_norm_eps);
      linear(ly.w[0], normed.data(), qv.data(), act_mode);
      linear(ly.w[1], normed.data(), kvec.data(), act_mode);
      linear(ly.w[2], normed.data(), vvec.data(), act_mode);
      kanso_ref_rope(qv.data(), &pos, 1, H, hd, c.rope_theta);
      kanso_ref_rope(kvec.data(), &pos, 1, KH, hd, c.rope_theta);
      int32_t st = kanso_ref_kv_write_token(kv, l, block, offset, kvec.data(), vvec.data());
      if (st != ST_OK) return st;
      st = kanso_ref_paged_attention_int8(kv, l, qv.data(), block_tables + (size_t)s * max_blocks,
                                          context_lens + s, &pa, attn.data());
      if (st != ST_OK) return st;
      linear(ly.w[3], attn.data(), proj.data(), act_mode);
      for (uint32_t i = 0; i < hidden; ++i) h[i] = h[i] + proj[i];
      kanso_ref_rmsnorm(h.data(), ly.ffn_norm.data(), normed.data(), 1, hidden, c.rms_norm_eps);
      linear(ly.w[4], normed.data(), gate.data(), act_mode);
      linear(ly.w[5], normed.data(), up.data(), act_mode);
      kanso_ref_silu_mul(gate.data(), up.data(), act.data(), inter);
      linear(ly.w[6], act.data(), proj.data(), act_mode);
      for (uint32_t i = 0; i < hidden; ++i) h[i] = h[i] + proj[i];
    }
    kanso_ref_rmsnorm(h.data(), m->final_norm.data(), normed.data(), 1, hidden, c.rms_norm_eps);
    const auto& head = m->output.w ? m->output : m->token_embd;
    linear(head, normed.data(), logits_out + (size_t)s * c.vocab_size, act_mode);
  }
  return ST_OK;
}

}  // extern "C"
