// Batched quantized GEMM on the 5th-generation tensor cores (tcgen05 + TMEM):
// LinearWeight::forward for many activation rows (src/weights.rs:43-45; continuous-batching
// and chunked-prefill rows of forward_batch_rows, src/model.rs:1418-1740).
//
//   y[M,N] = x[M,K] @ W[N,K]^T,  W in GGUF Q8_0 / Q4_K blocks, x and y f32.
//
// This is the three-product form used by the decode step's chain of matmuls (more than 8
// sequences) and by shapes whose rows do not start on 16-byte boundaries; single matmuls of 9..512
// rows with aligned rows take the TMA-staged kernel in gemm_tma.cu, KANSO_ACT_Q8 batches the
// kind::i8 kernel in gemm_i8.cu.
//
// Mapping. The weight matrix is the 128-row operand of the MMA (A, K-major) and the
// activations are the narrow operand (B, K-major, 16..128 rows), so one CTA owns 128 weight
// rows x one K range and streams its weight bytes from HBM exactly once:
//   * a pack kernel converts x to f16 hi/lo planes in the canonical K-major core-matrix layout,
//     one contiguous tile per 64-wide K stage (it can fold in rmsnorm or the SwiGLU product and
//     clears the outputs of a split-K launch);
//   * 16 producer warps copy the raw block bytes of the CTA's 128 rows into a shared-memory ring
//     with cp.async (three stages ahead), dequantise 16 weights per thread and stage (Q8_0: exact
//     int8 -> f16 by byte permute; Q4_K: (d*sc)*q - dmin*m in f32) into f16 hi/lo terms and store
//     16-byte core-matrix rows (no swizzle: 8 rows x 16 bytes per core matrix, K-adjacent matrices
//     2 KB apart), double-buffered;
//   * one thread of a 19th warp fetches the activation tile of every stage with one
//     cp.async.bulk; the elected lanes of a 17th and an 18th warp issue the tcgen05.mma
//     instructions (M=128, N=Mt, K=16, kind::f16, f32 accumulate in TMEM) of the even and of the
//     odd stages, each into an accumulator of its own (the instruction is bound by its issuing
//     thread at these widths), and commit them to the stage's mbarrier, which frees its buffers;
//   * after the last stage the producer warps read both accumulators with tcgen05.ld (lane =
//     weight row, column = activation row), add them and write y (optionally adding a
//     residual); with split-K the partial sums are added with atomics (y is cleared by the pack
//     kernel).
// Several matrices that share their activations (Q/K/V, gate/up) run as one launch.
// Every mbarrier wait is bounded; on a timeout the CTA records DEV_WAIT_TIMEOUT, frees its
// TMEM columns and returns.
//
// Numerics: a single f16 rounding of each operand (2^-12 on average) keeps one matmul inside
// the 1e-3 bound but drifts past the 1e-2 logit bound over a stack of layers, so both
// operands are split in two f16 terms, w = wh + wl and x = xh + xl (the remainders are exact
// or near-exact), and each 16-wide K step issues three MMAs: wh*xh + wl*xh + wh*xl. Only the
// wl*xl term (2^-22) is dropped; products accumulate in f32 in TMEM.
#include <cstdlib>

#include "ctx.h"
#include "tc05.cuh"

namespace kanso {

constexpr int TC_PRODUCERS = 512;           // threads that copy, dequantise and run the epilogue
constexpr int TC_THREADS = TC_PRODUCERS + 96;  // plus two warps that issue the MMAs and one that loads B
constexpr int TC_MAX_SEGS = 3;   // matrices of one launch that share the activations (Q, K, V)
constexpr int TC_KC = 64;        // K values per stage
constexpr int TC_TILE_N = 128;   // weight rows per CTA = MMA M
constexpr int TC_A_PLANE = TC_TILE_N * TC_KC * 2;  // bytes of one f16 A term per stage (16 KB)
constexpr int TC_A_STAGE = 2 * TC_A_PLANE;         // hi and lo terms

struct TcArgs {
  const uint8_t* w[TC_MAX_SEGS];
  float* y[TC_MAX_SEGS];          // [M, N] each
  int64_t N[TC_MAX_SEGS];
  int tile_begin[TC_MAX_SEGS];    // first CTA (along x) of each matrix
  int nseg;
  const __half* xp;  // packed activations [K/64][8][Mt][8]
  const float* resid;  // ksplit == 1: y = resid + W.x (may alias y); nullptr: plain store
  int K, M, Mt;      // Mt = M rounded up to 16
  int bpr;           // blocks (Q8_0) or super-blocks (Q4_K) per row
  int ksplit;        // CTAs along K; > 1: partial sums are added into y with atomics
  int stages_total;  // K / 64
  int nstage_smem;   // shared-memory stages of the A/B tiles (2 or 3)
  int* status;
};


// Result buffers the pack kernels clear on the way (a split-K GEMM adds into them).
struct TcZero {
  float* p[TC_MAX_SEGS];
  int64_t n[TC_MAX_SEGS];
};
__device__ __forceinline__ void tc_zero_fill(const TcZero& z, int64_t tid, int64_t nthreads) {
#pragma unroll
  for (int i = 0; i < TC_MAX_SEGS; ++i)
    for (int64_t j = tid; j < z.n[i]; j += nthreads) z.p[i][j] = 0.f;
}

// x f32 [M,K] -> two f16 terms xh + xl, layout [stage][term][chunk of 8 k][row m][8 values];
// rows >= M are zero.
__global__ void tc_pack_activations_kernel(const float* __restrict__ x,
                                           const float* __restrict__ x2,
                                           __half* __restrict__ xp, int M, int Mt, int K,
                                           const TcZero zero) {
  pdl_launch_dependents();
  pdl_wait();  // x (and the readers of the buffers cleared here) belong to earlier kernels
  tc_zero_fill(zero, (int64_t)blockIdx.x * blockDim.x + threadIdx.x,
               (int64_t)gridDim.x * blockDim.x);
  const int64_t total = (int64_t)(K / 8) * Mt;  // one thread per (chunk, row)
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int m = (int)(i % Mt);
    const int chunk = (int)(i / Mt);  // global chunk index = k / 8
    __align__(16) __half hi[8], lo[8];
    if (m < M) {
      const float4* src = reinterpret_cast<const float4*>(x + (int64_t)m * K + chunk * 8);
      const float4 a = src[0], b = src[1];
      float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      if (x2) {  // the SwiGLU product feeding ffn_down: silu(x) * x2 (src/model.rs:367-382)
        const float4* up = reinterpret_cast<const float4*>(x2 + (int64_t)m * K + chunk * 8);
        const float4 c = up[0], d = up[1];
        const float u[8] = {c.x, c.y, c.z, c.w, d.x, d.y, d.z, d.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = f[j] / (1.0f + expf(-f[j])) * u[j];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        hi[j] = __float2half_rn(f[j]);
        lo[j] = __float2half_rn(f[j] - __half2float(hi[j]));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) hi[j] = lo[j] = __float2half_rn(0.f);
    }
    const int stage = chunk >> 3, c = chunk & 7;
    __half* base = xp + (int64_t)stage * (2 * 8 * Mt * 8);
    *reinterpret_cast<uint4*>(base + ((int64_t)c * Mt + m) * 8) = *reinterpret_cast<uint4*>(hi);
    *reinterpret_cast<uint4*>(base + ((int64_t)(8 + c) * Mt + m) * 8) =
        *reinterpret_cast<uint4*>(lo);
  }
}

// The same pack with rmsnorm folded in (src/model.rs:653-659): one CTA per activation row
// computes 1 / sqrt(mean(x^2) + eps), then packs x * r * norm_w. Rows >= M of the tile are
// zeroed by the CTAs of rows M .. Mt-1.
__global__ void tc_pack_norm_kernel(const float* __restrict__ x, const float* __restrict__ norm_w,
                                    float eps, __half* __restrict__ xp, int M, int Mt, int K,
                                    const TcZero zero) {
  __shared__ float s_red[32];
  pdl_launch_dependents();
  pdl_wait();
  tc_zero_fill(zero, (int64_t)blockIdx.x * blockDim.x + threadIdx.x,
               (int64_t)gridDim.x * blockDim.x);
  const int m = blockIdx.x;
  float r = 0.f;
  if (m < M) {
    const float4* row = reinterpret_cast<const float4*>(x + (int64_t)m * K);
    float ss = 0.f;
    for (int i = threadIdx.x; i < K / 4; i += blockDim.x) {
      const float4 t = row[i];
      ss += (t.x * t.x + t.y * t.y) + (t.z * t.z + t.w * t.w);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float t = threadIdx.x < (blockDim.x >> 5) ? s_red[threadIdx.x] : 0.f;
    if (threadIdx.x < 32) {
#pragma unroll
      for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
      if (threadIdx.x == 0) s_red[0] = 1.0f / sqrtf(t / (float)K + eps);
    }
    __syncthreads();
    r = s_red[0];
  }
  for (int chunk = threadIdx.x; chunk < K / 8; chunk += blockDim.x) {
    __align__(16) __half hi[8], lo[8];
    if (m < M) {
      const float4* src = reinterpret_cast<const float4*>(x + (int64_t)m * K + chunk * 8);
      const float4* nw = reinterpret_cast<const float4*>(norm_w + chunk * 8);
      const float4 a = src[0], b = src[1], c = __ldg(nw), d = __ldg(nw + 1);
      const float f[8] = {a.x * r * c.x, a.y * r * c.y, a.z * r * c.z, a.w * r * c.w,
                          b.x * r * d.x, b.y * r * d.y, b.z * r * d.z, b.w * r * d.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        hi[j] = __float2half_rn(f[j]);
        lo[j] = __float2half_rn(f[j] - __half2float(hi[j]));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) hi[j] = lo[j] = __float2half_rn(0.f);
    }
    const int stage = chunk >> 3, c8 = chunk & 7;
    __half* base = xp + (int64_t)stage * (2 * 8 * Mt * 8);
    *reinterpret_cast<uint4*>(base + ((int64_t)c8 * Mt + m) * 8) = *reinterpret_cast<uint4*>(hi);
    *reinterpret_cast<uint4*>(base + ((int64_t)(8 + c8) * Mt + m) * 8) =
        *reinterpret_cast<uint4*>(lo);
  }
}

constexpr int TC_FMT_Q8_0 = 0;
constexpr int TC_FMT_Q4_K = 1;

// Raw weight bytes travel through a ring of TC_RAW_DEPTH shared-memory stages filled with
// cp.async copies issued three stages ahead of their use, so the HBM latency is hidden
// without holding registers. A raw stage keeps, per weight row, the bytes of that row's
// 64 K-values: Q8_0 two blocks = 68 bytes (row stride 68: odd word stride, conflict-free);
// Q4_K header + 32 nibble bytes = 48 bytes (row stride 80 for conflict-free 128-bit loads).
constexpr int TC_RAW_DEPTH = 4;  // raw stages in flight: three ahead of the one in use
constexpr int TC_RAW_ROW_Q8 = 68;
constexpr int TC_RAW_ROW_Q4 = 80;
constexpr int TC_RAW_STAGE = TC_TILE_N * TC_RAW_ROW_Q4;  // the larger of the two

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16_cg(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// Per-thread source and destination offsets of the raw-byte copies, fixed for the whole K loop.
// Q8_0: the stage's 128 rows x 17 words are dealt to the threads in flat order, so the lanes
// of a warp copy consecutive words of two or three rows (few memory lines per instruction).
// Q4_K: threads 0..383 = (row tid / 3, part tid % 3): header, nibble bytes 0..15, 16..31.
template <int FMT>
struct TcRawCopy {
  static constexpr int kPerThread =
      FMT == TC_FMT_Q8_0 ? (TC_TILE_N * 17 + TC_PRODUCERS - 1) / TC_PRODUCERS : 1;
  const uint8_t* src[kPerThread];
  uint32_t dst[kPerThread];
  bool on[kPerThread];
  int part;

  __device__ __forceinline__ void init(const TcArgs& a, const uint8_t* w, int64_t N, int64_t n0,
                                       int tid) {
    if (FMT == TC_FMT_Q8_0) {
#pragma unroll
      for (int k = 0; k < kPerThread; ++k) {
        const int idx = tid + k * TC_PRODUCERS;
        on[k] = idx < TC_TILE_N * 17;
        const int row = min(idx / 17, TC_TILE_N - 1), word = idx - 17 * (idx / 17);
        const int64_t n = min(n0 + row, N - 1);  // rows past N re-read the last row
        src[k] = w + n * a.bpr * Q8_BYTES + 4 * word;
        dst[k] = row * TC_RAW_ROW_Q8 + 4 * word;
      }
    } else {
      on[0] = tid < 3 * TC_TILE_N;
      const int row = min(tid / 3, TC_TILE_N - 1);
      part = tid - 3 * (tid / 3);
      src[0] = w + min(n0 + row, N - 1) * a.bpr * Q4K_BYTES;
      dst[0] = row * TC_RAW_ROW_Q4 + 16 * part;
    }
  }
  __device__ __forceinline__ void issue(int s, uint32_t raw_stage) const {
    if (FMT == TC_FMT_Q8_0) {
#pragma unroll
      for (int k = 0; k < kPerThread; ++k)
        if (on[k]) cp_async4(raw_stage + dst[k], src[k] + (int64_t)s * (2 * Q8_BYTES));
    } else if (on[0]) {
      const uint8_t* p = src[0] + (int64_t)(s >> 2) * Q4K_BYTES;
      cp_async16_cg(raw_stage + dst[0], part == 0 ? p : p + 32 * (s & 3) + 16 * part);
    }
  }
};

// Dequantise this thread's 16 weights of the stage into the A tile (core-matrix layout):
// two chunks of 8 k-values, each one 16-byte row of a core matrix, in a hi and a lo plane.
// Q8_0: thread = (block tid / 256 of the two in the stage, half block (tid / 128) % 2, row).
__device__ __forceinline__ void tc_dequant_q8_0(const uint8_t* raw_stage, int tid, uint8_t* As) {
  const int blk = tid >> 8, hb = (tid >> 7) & 1, row = tid & 127;
  const uint32_t off = row * TC_RAW_ROW_Q8 + blk * Q8_BYTES;  // of the block; 2-byte aligned
  const __half d = *reinterpret_cast<const __half*>(raw_stage + off);
  const uint32_t qoff = off + 2 + 16 * hb;  // 16 int8 values, 2-byte aligned
  const uint32_t* al = reinterpret_cast<const uint32_t*>(raw_stage + (qoff & ~3u));
  const uint32_t sh = (qoff & 3u) * 8;  // 0 or 16, the same for the whole warp
  uint32_t r[5];
#pragma unroll
  for (int k = 0; k < 4; ++k) r[k] = al[k];
  r[4] = sh ? al[4] : 0u;
  const __half2 d2 = __half2half2(d);
  const __half2 bias = __floats2half2_rn(1152.f, 1152.f);  // 1024 + 128, exact in f16
#pragma unroll
  for (int c = 0; c < 2; ++c) {  // chunk of 8 weights = two words of int8
    uint32_t out[4], rem[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t q = __funnelshift_r(r[2 * c + h], r[2 * c + h + 1], sh) ^ 0x80808080u;
      // 0x6400 | byte = 1024 + (q + 128) as f16, exactly
      uint32_t p01 = __byte_perm(q, 0x64646464u, 0x4140);
      uint32_t p23 = __byte_perm(q, 0x64646464u, 0x4342);
      const __half2 q01 = __hsub2(*reinterpret_cast<__half2*>(&p01), bias);
      const __half2 q23 = __hsub2(*reinterpret_cast<__half2*>(&p23), bias);
      __half2 h01 = __hmul2(q01, d2), h23 = __hmul2(q23, d2);
      // d*q - round(d*q): the fused multiply-add forms the product exactly
      __half2 l01 = __hfma2(q01, d2, __hneg2(h01)), l23 = __hfma2(q23, d2, __hneg2(h23));
      out[2 * h] = *reinterpret_cast<uint32_t*>(&h01);
      out[2 * h + 1] = *reinterpret_cast<uint32_t*>(&h23);
      rem[2 * h] = *reinterpret_cast<uint32_t*>(&l01);
      rem[2 * h + 1] = *reinterpret_cast<uint32_t*>(&l23);
    }
    const int kc = blk * 4 + hb * 2 + c;  // chunk of 8 k-values within the stage
    *reinterpret_cast<uint4*>(As + kc * (TC_TILE_N * 16) + row * 16) =
        make_uint4(out[0], out[1], out[2], out[3]);
    *reinterpret_cast<uint4*>(As + TC_A_PLANE + kc * (TC_TILE_N * 16) + row * 16) =
        make_uint4(rem[0], rem[1], rem[2], rem[3]);
  }
}

// Q4_K: stage s = 64-weight group g = s % 4 of super-block s / 4; thread = (nibble half
// tid / 256 -> sub-block 2g + half, byte half (tid / 128) % 2 -> 16 of the 32 nibble bytes, row).
// (d*sc)*q - dmin*m as src/quant/q4_k.rs:30-55, then split into two f16 terms.
__device__ __forceinline__ void tc_dequant_q4_k(const uint8_t* raw_stage, int s, int tid,
                                                uint8_t* As) {
  const int half = tid >> 8, part = (tid >> 7) & 1, row = tid & 127;
  const int g = s & 3;
  const uint4* p = reinterpret_cast<const uint4*>(raw_stage + row * TC_RAW_ROW_Q4);
  const uint4 hdr = p[0], qv = p[1 + part];
  const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
  uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
  unpack_scales_k4(hdr.y, hdr.z, hdr.w, sc_lo, sc_hi, mn_lo, mn_hi);
  const int j = 2 * g + half;
  const uint32_t scw = j < 4 ? sc_lo : sc_hi, mnw = j < 4 ? mn_lo : mn_hi;
  const float d1 = __fmul_rn(d, (float)((scw >> (8 * (j & 3))) & 0xFF));
  const float m1 = __fmul_rn(dmin, (float)((mnw >> (8 * (j & 3))) & 0xFF));
  const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
  const int sh0 = 4 * half;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t out[4], rem[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t w = qw[2 * c + h] >> sh0;
      float f[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const float q = __uint_as_float(0x4B000000u | ((w >> (8 * b)) & 0xFu)) - 8388608.0f;
        f[b] = __fsub_rn(__fmul_rn(d1, q), m1);
      }
      __half2 h01 = __floats2half2_rn(f[0], f[1]);
      __half2 h23 = __floats2half2_rn(f[2], f[3]);
      const float2 g01 = __half22float2(h01), g23 = __half22float2(h23);
      __half2 l01 = __floats2half2_rn(f[0] - g01.x, f[1] - g01.y);
      __half2 l23 = __floats2half2_rn(f[2] - g23.x, f[3] - g23.y);
      out[2 * h] = *reinterpret_cast<uint32_t*>(&h01);
      out[2 * h + 1] = *reinterpret_cast<uint32_t*>(&h23);
      rem[2 * h] = *reinterpret_cast<uint32_t*>(&l01);
      rem[2 * h + 1] = *reinterpret_cast<uint32_t*>(&l23);
    }
    // low nibbles: k 0..31 of the group, high nibbles: 32..63
    const int kc = half * 4 + part * 2 + c;
    *reinterpret_cast<uint4*>(As + kc * (TC_TILE_N * 16) + row * 16) =
        make_uint4(out[0], out[1], out[2], out[3]);
    *reinterpret_cast<uint4*>(As + TC_A_PLANE + kc * (TC_TILE_N * 16) + row * 16) =
        make_uint4(rem[0], rem[1], rem[2], rem[3]);
  }
}

// Warps 0-15 produce the A tiles (raw-byte copies, dequantisation) and run the epilogue; warp 16
// fetches the B tiles with one bulk copy per stage and issues the MMAs, so building descriptors
// and issuing never delays the next stage's dequantisation. Buffer indices and mbarrier
// parities are carried as counters (no division in the loop).
template <int FMT>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const TcArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t b_plane = 8u * a.Mt * 16u;  // bytes of one term of the B tile of a stage
  const uint32_t b_stage = 2u * b_plane;
  const int NS = a.nstage_smem;  // shared-memory stages of the A/B tiles (2 or 3)
  uint8_t* As = smem;
  uint8_t* Bs = smem + NS * TC_A_STAGE;
  uint64_t* done = reinterpret_cast<uint64_t*>(Bs + NS * b_stage);  // [3] MMAs of a buffer retired
  uint64_t* full = done + 3;                                        // [3] A tile of a buffer ready
  uint64_t* bfull = full + 3;                                       // [3] B tile of a buffer landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bfull + 3);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint8_t* Raw = reinterpret_cast<uint8_t*>(done) + 96;  // 16-byte aligned

  int sg = 0;
#pragma unroll
  for (int i = 1; i < TC_MAX_SEGS; ++i)
    if (i < a.nseg && (int)blockIdx.x >= a.tile_begin[i]) sg = i;
  const int64_t n0 = (int64_t)((int)blockIdx.x - a.tile_begin[sg]) * TC_TILE_N;
  const int64_t N = a.N[sg];
  const int s0 = (int)((int64_t)a.stages_total * blockIdx.y / a.ksplit);
  const int s1 = (int)((int64_t)a.stages_total * (blockIdx.y + 1) / a.ksplit);
  // Two issuing threads with an accumulator each take the stages in turn (even / odd) and the
  // epilogue adds the accumulators: a tcgen05.mma of this width is bound by its issuing thread
  // (about 86 cycles each, whatever a second thread does beside it), and a stage has twelve.
  uint32_t acc_cols = 32;
  while (acc_cols < (uint32_t)a.Mt) acc_cols <<= 1;  // Mt <= 128
  const uint32_t ncols = 2 * acc_cols;

  if (warp == 0) tmem_alloc(tmem_slot, ncols);
  if (tid == 0) {
    for (int i = 0; i < 3; ++i) {
      mbar_init(&done[i], 1);  // the commit of the issuer that owns the stage
      mbar_init(&full[i], TC_PRODUCERS / 32);  // one arrival per producer warp
      mbar_init(&bfull[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Dependent launch: the weights never depend on the kernel before this one (the activation
  // pack), so the producers start fetching them at once; the MMA warp waits for the pack
  // before it touches the packed activations, and every store to y comes after MMAs that
  // consumed them.
  pdl_launch_dependents();

  if (warp < TC_PRODUCERS / 32) {
    TcRawCopy<FMT> raw_copy;
    raw_copy.init(a, a.w[sg], N, n0, tid);
    const uint32_t raw_base = smem_u32(Raw);
    // one commit group per call, also when there is nothing left to copy, so that the
    // wait_group arithmetic below holds at the end of the K range
    auto copy_raw = [&](int s, int slot) {
      if (s < s1) raw_copy.issue(s, raw_base + slot * TC_RAW_STAGE);
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    copy_raw(s0, 0);
    copy_raw(s0 + 1, 1);
    copy_raw(s0 + 2, 2);
    int buf = 0;             // A buffer of this stage
    uint32_t reuse_par = 1;  // parity of done[buf] for the previous use of the buffer
    for (int s = s0; s < s1; ++s) {
      const int it = s - s0;
      copy_raw(s + 3, (it + 3) & (TC_RAW_DEPTH - 1));
      // the A buffer of this stage was last read by the MMAs of stage s - NS
      if (it >= NS && !mbar_wait_bounded(&done[buf], reuse_par)) *abort_flag = 1;
      // all but the three newest groups have landed: raw(s) is in shared memory
      asm volatile("cp.async.wait_group 3;" ::: "memory");
      // producers' barrier: every producer's copies of this stage are visible to all
      asm volatile("bar.sync 1, %0;" ::"n"(TC_PRODUCERS) : "memory");
      if (*abort_flag) break;
      uint8_t* Ab = As + buf * TC_A_STAGE;
      const uint8_t* rs = Raw + (it & (TC_RAW_DEPTH - 1)) * TC_RAW_STAGE;
      if (FMT == TC_FMT_Q8_0)
        tc_dequant_q8_0(rs, tid, Ab);
      else
        tc_dequant_q4_k(rs, s, tid, Ab);
      fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(&full[buf]);
      if (++buf == NS) {
        buf = 0;
        reuse_par ^= 1;
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (warp == TC_PRODUCERS / 32 + 2) {
    if (lane == 0) {
      // ---- B tiles (packed activations) by bulk copy, one stage per shared-memory buffer; a
      // buffer is refilled once the MMAs of the stage that used it last have retired
      const uint8_t* bsrc = reinterpret_cast<const uint8_t*>(a.xp);
      pdl_wait();  // the pack kernel has written the activations
      int buf = 0;
      uint32_t reuse_par = 1;
      for (int s = s0; s < s1; ++s) {
        const int it = s - s0;
        if ((it >= NS && !mbar_wait_bounded(&done[buf], reuse_par)) || *abort_flag) {
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&bfull[buf], b_stage);
        bulk_g2s(Bs + buf * b_stage, bsrc + (size_t)s * b_stage, b_stage, &bfull[buf]);
        if (++buf == NS) {
          buf = 0;
          reuse_par ^= 1;
        }
      }
    }
    __syncwarp();
  } else {
    // ---- MMA issuers: thread `me` owns the stages it = me, me + 2, ... and the accumulator
    // columns [me * acc_cols, me * acc_cols + Mt); the two never read the same tile at once
    const int me = warp - TC_PRODUCERS / 32;
    if (lane == 0) {
      const uint32_t idesc = tc_idesc_f16(TC_TILE_N, a.Mt);
      const uint32_t a_k = (2 * (TC_TILE_N * 16)) >> 4, b_k = (2 * (a.Mt * 16)) >> 4;  // per 16 k
      const uint32_t acc = tmem_base + (uint32_t)me * acc_cols;
      for (int it = me; it < s1 - s0; it += 2) {
        const int buf = it % NS;
        const uint32_t par = (uint32_t)(it / NS) & 1u;
        if (!mbar_wait_bounded(&full[buf], par) || !mbar_wait_bounded(&bfull[buf], par)) {
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(As + buf * TC_A_STAGE);
        const uint32_t b_addr = smem_u32(Bs + buf * b_stage);
        const uint64_t ah0 = tc_smem_desc(a_addr, TC_TILE_N * 16, 128);
        const uint64_t al0 = tc_smem_desc(a_addr + TC_A_PLANE, TC_TILE_N * 16, 128);
        const uint64_t bh0 = tc_smem_desc(b_addr, a.Mt * 16, 128);
        const uint64_t bl0 = tc_smem_desc(b_addr + b_plane, a.Mt * 16, 128);
#pragma unroll
        for (int j = 0; j < TC_KC / 16; ++j) {  // one MMA = 16 k-values = two core matrices in K
          const uint64_t ah = ah0 + (uint64_t)(j * a_k), al = al0 + (uint64_t)(j * a_k);
          const uint64_t bh = bh0 + (uint64_t)(j * b_k), bl = bl0 + (uint64_t)(j * b_k);
          tc_mma_f16(acc, ah, bh, idesc, (it > me || j > 0) ? 1u : 0u);  // wh * xh
          tc_mma_f16(acc, al, bh, idesc, 1u);                            // wl * xh
          tc_mma_f16(acc, ah, bl, idesc, 1u);                            // wh * xl
        }
        tc_commit(&done[buf]);  // frees the A and the B tile of the stage
      }
    }
    __syncwarp();
  }
  __syncthreads();
  int failed = *abort_flag != 0;
  if (!failed && s1 > s0) {
    const int last = s1 - s0 - 1;
    failed = !mbar_wait_bounded(&done[last % NS], (uint32_t)(last / NS) & 1);
    // the other issuer's last stage is the one before (its commits retire in its own order)
    if (!failed && last >= 1)
      failed = !mbar_wait_bounded(&done[(last - 1) % NS], (uint32_t)((last - 1) / NS) & 1);
  }
  failed = __syncthreads_or(failed);
  tc_fence_after();
  if (!failed && s1 > s0 && warp < TC_PRODUCERS / 32) {
    // lane = weight row inside the tile, column = activation row
    const int q = warp & 3;
    const int64_t n = n0 + q * 32 + lane;
    for (int c16 = warp >> 2; c16 < a.Mt / 16; c16 += TC_PRODUCERS / 128) {
      uint32_t r[16], r1[16];
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c16 * 16);
      tmem_ld16(taddr, r);
      if (s1 - s0 > 1) {
        tmem_ld16(taddr + acc_cols, r1);  // the odd stages
      } else {
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) r1[jj] = 0u;
      }
      if (n < N) {
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
          const int m = c16 * 16 + jj;
          if (m < a.M) {
            float* dst = a.y[sg] + (int64_t)m * N + n;
            const float v = __uint_as_float(r[jj]) + __uint_as_float(r1[jj]);
            if (a.ksplit == 1)
              *dst = a.resid ? a.resid[(int64_t)m * N + n] + v : v;
            else
              atomicAdd(dst, v);  // y holds zeros or the residual
          }
        }
      }
    }
  } else if (failed && tid == 0) {
    atomicOr(a.status, DEV_WAIT_TIMEOUT);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, ncols);
}

// y_i[M,N_i] = x[M,K] @ W_i^T on the tensor cores for up to three matrices that share x, M up
// to 128 per call (larger M is chunked by the caller). Optional fusions of the decode step:
// x2 (activations are silu(x) * x2), norm_w (activations are rmsnorm(x) * norm_w) and resid
// (y = resid + W.x, one matrix; may alias y).
// Sets *handled = false (and launches nothing) when the shape is outside this kernel's range.
int32_t tc_matmul_multi(kanso_cuda_ctx* ctx, int32_t dtype, int nseg, const void* const* w,
                        float* const* y, const int64_t* rows, const float* x, const float* x2,
                        const float* norm_w, float eps, const float* resid, int64_t M, int64_t K,
                        bool* handled, const void* prepacked) {
  // prepacked: x is already in the packed f16 hi/lo layout (written by the kernel before this
  // one, e.g. the attention's merge); the pack launch is skipped. Only for a launch that has
  // nothing else for the pack kernel to do (no norm, no SwiGLU, no output to clear).
  *handled = false;
  if (prepacked && (x2 || norm_w)) return KANSO_OK;
  const int blk = dtype == KANSO_DTYPE_Q8_0 ? 32 : 256;
  if (nseg < 1 || nseg > TC_MAX_SEGS || (resid && nseg != 1)) return KANSO_OK;
  if (M < 1 || M > 128 || K < TC_KC || K % TC_KC != 0 || K % blk != 0) return KANSO_OK;
  if (!aligned16(x) || (x2 && !aligned16(x2)) || (norm_w && (!aligned16(norm_w) || x2)))
    return KANSO_OK;
  int tiles_n = 0;
  TcArgs a;
  for (int i = 0; i < nseg; ++i) {
    if (!w[i] || !y[i] || rows[i] < 1) return KANSO_OK;
    if (dtype == KANSO_DTYPE_Q8_0 && (reinterpret_cast<uintptr_t>(w[i]) & 3) != 0) return KANSO_OK;
    if (dtype == KANSO_DTYPE_Q4_K && !aligned16(w[i])) return KANSO_OK;
    a.w[i] = (const uint8_t*)w[i];
    a.y[i] = y[i];
    a.N[i] = rows[i];
    a.tile_begin[i] = tiles_n;
    tiles_n += (int)((rows[i] + TC_TILE_N - 1) / TC_TILE_N);
  }
  for (int i = nseg; i < TC_MAX_SEGS; ++i) {
    a.w[i] = a.w[0];
    a.y[i] = a.y[0];
    a.N[i] = a.N[0];
    a.tile_begin[i] = tiles_n;
  }
  a.nseg = nseg;
  const int Mt = (int)((M + 15) / 16 * 16);
  const int stages_total = (int)(K / TC_KC);
  // Split K while the grid stays within about one wave of CTAs (one CTA per SM): the decode
  // step's matrices have 8 to 40 row tiles and would otherwise leave most SMs idle. Large
  // matrices are not split: a second partial wave costs more than it gains, and the partial
  // sums of a split are added with atomics (onto the residual, or after a clear of y). At
  // least 2 stages stay in every CTA.
  int ksplit = 1;
  while (tiles_n * ksplit * 2 <= ctx->sm_count + ctx->sm_count / 4 &&
         stages_total / (ksplit * 2) >= 2)
    ksplit *= 2;
  if (prepacked && ksplit > 1 && !(resid && resid == y[0])) return KANSO_OK;  // y needs a clear
  const size_t xp_bytes = 2 * (size_t)(K / 8) * Mt * 16;
  uint8_t* scratch =
      prepacked ? (uint8_t*)const_cast<void*>(prepacked) : (uint8_t*)ctx_scratch(ctx, xp_bytes + 256);
  if (!scratch) return KANSO_ERR_DEVICE;
  *handled = true;

  a.resid = resid;
  TcZero zero = {};
  if (ksplit > 1) {
    // the K slices add into y: y must hold the residual (in place) or zeros (cleared by the
    // pack kernel below)
    a.resid = nullptr;
    for (int i = 0; i < nseg; ++i) {
      if (resid && resid == y[i]) continue;
      if (resid) {
        KANSO_CUDA_TRY(ctx,
                       cudaMemcpyAsync(y[i], resid, sizeof(float) * (size_t)M * rows[i],
                                       cudaMemcpyDeviceToDevice, ctx->stream),
                       "gemm_tc: residual copy");
      } else {
        zero.p[i] = y[i];
        zero.n[i] = M * rows[i];
      }
    }
  }
  const int64_t chunks = (K / 8) * Mt;
  cudaError_t le = cudaSuccess;
  if (prepacked)
    ;  // nothing to pack
  else if (norm_w)
    le = launch_dependent(ctx, tc_pack_norm_kernel, dim3(Mt), dim3(256), 0, x, norm_w, eps,
                          reinterpret_cast<__half*>(scratch), (int)M, Mt, (int)K, zero);
  else
    le = launch_dependent(ctx, tc_pack_activations_kernel,
                          dim3((unsigned)((chunks + 255) / 256)), dim3(256), 0, x, x2,
                          reinterpret_cast<__half*>(scratch), (int)M, Mt, (int)K, zero);
  if (le != cudaSuccess) return cuda_fail(ctx, le, "gemm_tc pack launch");
  int32_t st = prepacked ? KANSO_OK : after_launch(ctx, "gemm_tc pack activations");
  if (st) return st;
  a.xp = reinterpret_cast<const __half*>(scratch);
  a.K = (int)K;
  a.M = (int)M;
  a.Mt = Mt;
  a.bpr = (int)(K / blk);
  a.ksplit = ksplit;
  a.stages_total = stages_total;
  a.status = ctx->dev_status;
  const size_t per_stage = TC_A_STAGE + (size_t)(2 * 8 * Mt * 16);
  const size_t fixed = 96 + (size_t)TC_RAW_DEPTH * TC_RAW_STAGE;
  // Three A/B stages if they fit, else two, and one CTA per SM (the request is padded past half
  // of the SM's shared memory where the stages alone would let two CTAs in): with two issuing
  // threads per CTA a second CTA on the SM did not make the decode step faster (2209 us with two
  // stages and two CTAs against 2177 us with three stages and one, 32 sequences).
  const size_t half_sm = ((size_t)ctx->smem_optin - 2048) / 2;
  a.nstage_smem = 3 * per_stage + fixed <= (size_t)ctx->smem_optin ? 3 : 2;
  size_t smem = a.nstage_smem * per_stage + fixed;
  if (smem <= half_sm + 1024) smem = half_sm + 2048;
  auto kern = dtype == KANSO_DTYPE_Q8_0 ? gemm_tc_kernel<TC_FMT_Q8_0> : gemm_tc_kernel<TC_FMT_Q4_K>;
  static bool attr_set[2][16] = {};
  bool& done = attr_set[dtype == KANSO_DTYPE_Q8_0 ? 0 : 1][ctx->device & 15];
  if (!done) {
    KANSO_CUDA_TRY(ctx,
                   cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        ctx->smem_optin),
                   "gemm_tc: shared memory opt-in");
    done = true;
  }
  le = launch_dependent(ctx, kern, dim3(tiles_n, ksplit), dim3(TC_THREADS), smem, a);
  if (le != cudaSuccess) return cuda_fail(ctx, le, "gemm_tc launch");
  return after_launch(ctx, "gemm_tc");
}

int32_t tc_matmul(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x, float* y,
                  int64_t M, int64_t N, int64_t K, bool* handled) {
  const void* w1[1] = {w};
  float* y1[1] = {y};
  const int64_t r1[1] = {N};
  return tc_matmul_multi(ctx, dtype, 1, w1, y1, r1, x, nullptr, nullptr, 0.f, nullptr, M, K,
                         handled, nullptr);
}

}  // namespace kanso
