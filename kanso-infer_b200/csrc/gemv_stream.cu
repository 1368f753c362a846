// Streaming quantized GEMV / few-row GEMM for GGUF Q8_0 and Q4_K weights.
//
// Replaces scalar_gemv_q8_0 / scalar_gemv_q4_k (src/quant/q8_0.rs:69-93,
// src/quant/q4_k.rs:69-93) and, for a handful of activation rows,
// LinearWeight::forward (src/weights.rs:43-45).
//
// Shape of the kernel (HBM-bound byte work, no tensor cores):
//   * one persistent CTA per SM owns a contiguous range of weight rows;
//   * every warp runs its own ring of shared-memory stages: lane 0 issues
//     cp.async.bulk copies (the TMA engine's untiled form) of whole-row tiles
//     straight from the GGUF byte stream, completion is signalled on an
//     mbarrier, the warp decodes the blocks out of shared memory. Copies start
//     and end on 16-byte boundaries of the stream, so the 34-byte Q8_0 blocks
//     (2-byte aligned) need no re-layout in HBM;
//   * one lane decodes one block (Q8_0) or one super-block (Q4_K); the lane
//     stride in shared memory (34 B / 144 B) and the padded activation layout
//     (48 B / 272 B per item) keep 128-bit shared loads free of bank conflicts;
//   * activations are converted once per CTA into int8 planes so that the inner
//     product is dp4a on packed bytes (Q4_K nibbles are masked in place, never
//     widened). KANSO_ACT_Q8 keeps the one plane of quantize_row_q8_0; the
//     default KANSO_ACT_F32 adds a second plane holding the quantisation
//     residual (x ~= d*(hi + lo/254), max error d/508), which keeps the result
//     within ~3e-5 of the f32 reference while staying on the integer pipe;
//   * per-row sums finish with a (segmented) warp shuffle reduction.
#include "ctx.h"

namespace kanso {

constexpr int FMT_Q8_0 = 0;
constexpr int FMT_Q4_K = 1;

template <int FMT>
struct Fmt;
template <>
struct Fmt<FMT_Q8_0> {
  static constexpr int ITEM_BYTES = 34, ITEM_ELEMS = 32, XSTRIDE = 48;
};
template <>
struct Fmt<FMT_Q4_K> {
  static constexpr int ITEM_BYTES = 144, ITEM_ELEMS = 256, XSTRIDE = 272;
};

constexpr int MAX_STAGES = 4;
constexpr int MAX_WARPS = 16;

constexpr int MAX_SEGS = 3;
// One weight matrix of a launch. A launch may carry up to three matrices that share the
// activations (Q, K, V or gate, up): CTAs [cta_begin, next cta_begin) work on segment i.
struct StreamSeg {
  const uint8_t* w;
  float* y;
  int64_t rows;         // weight rows (N)
  int64_t total_bytes;  // rows * row_bytes
  int64_t ldy;          // elements between activation rows in y
  int cta_begin;
};

struct StreamArgs {
  StreamSeg seg[MAX_SEGS];
  int nseg;
  const float* x;
  // optional fusions of the decode step (src/model.rs:1141-1207):
  const float* x2;      // activations are silu(x) * x2 (the SwiGLU product feeding ffn_down)
  const float* norm_w;  // activations are rmsnorm(x) * norm_w (attn_norm / ffn_norm / final norm)
  float eps;
  const float* resid;   // result is resid + W.x (residual add); may alias y
  int64_t ldr;
  int64_t ldx;          // elements between activation rows in x
  int K, bpr, row_bytes;
  int M;                // activation rows handled by this launch
  int tile_rows;        // rows per bulk copy (multiple of rows-per-warp-iteration)
  int stage_bytes;      // bytes reserved per stage (16-byte multiple, with slack)
  int nstage;
  int* status;
};

// Shared-memory carve-up, computed the same way on host and device.
struct StreamLayout {
  int off_scale, off_sum, off_planes, off_stages, plane_bytes, total;
};
template <int FMT, int PLANES>
__host__ __device__ inline StreamLayout stream_layout(int K, int bpr, int M, int nwarps,
                                                      int nstage, int stage_bytes) {
  StreamLayout L;
  int nblk = K / 32;
  int off = MAX_WARPS * MAX_STAGES * 8;  // mbarriers
  L.off_scale = off;
  off += M * nblk * 4;
  L.off_sum = off;
  if (FMT == FMT_Q4_K) off += M * nblk * 4;
  off = (off + 15) & ~15;
  L.off_planes = off;
  L.plane_bytes = bpr * Fmt<FMT>::XSTRIDE;
  off += M * PLANES * L.plane_bytes;
  off = (off + 127) & ~127;
  L.off_stages = off;
  off += nwarps * nstage * stage_bytes;
  L.total = off;
  return L;
}

__device__ __forceinline__ uint32_t pack4(float a, float b, float c, float d) {
  return ((uint32_t)(int)a & 0xFF) | (((uint32_t)(int)b & 0xFF) << 8) |
         (((uint32_t)(int)c & 0xFF) << 16) | (((uint32_t)(int)d & 0xFF) << 24);
}

// Converts the activations into the int8 planes. Eight consecutive threads own one
// block of 32 (a float4 each). Plane 0 is exactly quantize_row_q8_0
// (src/quant/q8_0.rs:13-32); plane 1 is the residual in units of d/254.
template <int FMT, int PLANES>
__device__ __forceinline__ void stage_activations(const StreamArgs& a, const StreamLayout& L,
                                                  uint8_t* smem) {
  const int nblk = a.K / 32;
  const int per_row = a.K / 4;  // float4s per activation row
  const int total = a.M * per_row;
  float* xscale = reinterpret_cast<float*>(smem + L.off_scale);
  float* xsum = reinterpret_cast<float*>(smem + L.off_sum);
  // rmsnorm fold (src/model.rs:653-659): 1 / sqrt(mean(x^2) + eps) per activation row
  __shared__ float s_inv_rms[8];
  __shared__ float s_red[32];
  if (a.norm_w) {
    for (int m = 0; m < a.M; ++m) {
      const float4* xr = reinterpret_cast<const float4*>(a.x + (int64_t)m * a.ldx);
      float ss = 0.f;
      for (int c = threadIdx.x; c < per_row; c += blockDim.x) {
        const float4 t = xr[c];
        ss += (t.x * t.x + t.y * t.y) + (t.z * t.z + t.w * t.w);
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
      __syncthreads();
      if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
      __syncthreads();
      if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? s_red[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
        if (threadIdx.x == 0) s_inv_rms[m] = 1.0f / sqrtf(t / (float)a.K + a.eps);
      }
    }
    __syncthreads();
  }
  for (int base = 0; base < total; base += blockDim.x) {
    int i = base + threadIdx.x;
    bool on = i < total;
    int m = on ? i / per_row : 0;
    int c4 = on ? i - m * per_row : 0;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (on) {
      // plain loads: with dependent launch the producer kernel has just finished
      v = reinterpret_cast<const float4*>(a.x + (int64_t)m * a.ldx)[c4];
      if (a.x2) {  // silu(g) * u with silu(g) = g / (1 + e^-g), src/model.rs:367-382
        const float4 u = reinterpret_cast<const float4*>(a.x2 + (int64_t)m * a.ldx)[c4];
        v.x = v.x / (1.0f + expf(-v.x)) * u.x;
        v.y = v.y / (1.0f + expf(-v.y)) * u.y;
        v.z = v.z / (1.0f + expf(-v.z)) * u.z;
        v.w = v.w / (1.0f + expf(-v.w)) * u.w;
      }
      if (a.norm_w) {
        const float4 nw = __ldg(reinterpret_cast<const float4*>(a.norm_w) + c4);
        const float r = s_inv_rms[m];
        v.x = v.x * r * nw.x;
        v.y = v.y * r * nw.y;
        v.z = v.z * r * nw.z;
        v.w = v.w * r * nw.w;
      }
    }
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    float sum = (v.x + v.y) + (v.z + v.w);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
      amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    }
    float d = __fdiv_rn(amax, 127.0f);
    float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    float h0 = fminf(fmaxf(roundf(__fmul_rn(v.x, id)), -128.f), 127.f);
    float h1 = fminf(fmaxf(roundf(__fmul_rn(v.y, id)), -128.f), 127.f);
    float h2 = fminf(fmaxf(roundf(__fmul_rn(v.z, id)), -128.f), 127.f);
    float h3 = fminf(fmaxf(roundf(__fmul_rn(v.w, id)), -128.f), 127.f);
    if (!on) continue;
    int e = c4 * 4;  // element index inside the row
    int item = e / Fmt<FMT>::ITEM_ELEMS, within = e % Fmt<FMT>::ITEM_ELEMS;
    uint8_t* plane0 = smem + L.off_planes + (m * PLANES) * L.plane_bytes;
    *reinterpret_cast<uint32_t*>(plane0 + item * Fmt<FMT>::XSTRIDE + within) =
        pack4(h0, h1, h2, h3);
    if (PLANES == 2) {
      float il = 254.0f * id;
      float l0 = fminf(fmaxf(rintf(fmaf(-d, h0, v.x) * il), -127.f), 127.f);
      float l1 = fminf(fmaxf(rintf(fmaf(-d, h1, v.y) * il), -127.f), 127.f);
      float l2 = fminf(fmaxf(rintf(fmaf(-d, h2, v.z) * il), -127.f), 127.f);
      float l3 = fminf(fmaxf(rintf(fmaf(-d, h3, v.w) * il), -127.f), 127.f);
      *reinterpret_cast<uint32_t*>(plane0 + L.plane_bytes + item * Fmt<FMT>::XSTRIDE + within) =
          pack4(l0, l1, l2, l3);
    }
    if ((threadIdx.x & 7) == 0) {
      int blk = e / 32;
      xscale[m * nblk + blk] = PLANES == 2 ? d * (1.0f / 254.0f) : d;
      if (FMT == FMT_Q4_K) xsum[m * nblk + blk] = sum;
    }
  }
}

// One Q8_0 block against the staged activations of every row m < M.
template <int MT, int PLANES>
__device__ __forceinline__ void item_dot_q8_0(const uint8_t* p, int col, const StreamLayout& L,
                                              const uint8_t* smem, int M, int nblk,
                                              float (&acc)[MT]) {
  float wd = __half2float(*reinterpret_cast<const __half*>(p));
  uintptr_t q = reinterpret_cast<uintptr_t>(p) + 2;
  const uint32_t* al = reinterpret_cast<const uint32_t*>(q & ~uintptr_t(3));
  uint32_t sh = (uint32_t)(q & 3) * 8;  // 0 or 16
  uint32_t r[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) r[k] = al[k];
  int w[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) w[k] = (int)__funnelshift_r(r[k], r[k + 1], sh);
  const float* xscale = reinterpret_cast<const float*>(smem + L.off_scale);
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    if (m >= M) break;
    const uint8_t* xp = smem + L.off_planes + (m * PLANES) * L.plane_bytes + col * 48;
    const uint4 a0 = *reinterpret_cast<const uint4*>(xp);
    const uint4 a1 = *reinterpret_cast<const uint4*>(xp + 16);
    int ih = 0;
    ih = dp4a_ss(w[0], (int)a0.x, ih);
    ih = dp4a_ss(w[1], (int)a0.y, ih);
    ih = dp4a_ss(w[2], (int)a0.z, ih);
    ih = dp4a_ss(w[3], (int)a0.w, ih);
    ih = dp4a_ss(w[4], (int)a1.x, ih);
    ih = dp4a_ss(w[5], (int)a1.y, ih);
    ih = dp4a_ss(w[6], (int)a1.z, ih);
    ih = dp4a_ss(w[7], (int)a1.w, ih);
    float xs = xscale[m * nblk + col];
    if (PLANES == 2) {
      const uint4 b0 = *reinterpret_cast<const uint4*>(xp + L.plane_bytes);
      const uint4 b1 = *reinterpret_cast<const uint4*>(xp + L.plane_bytes + 16);
      int il = 0;
      il = dp4a_ss(w[0], (int)b0.x, il);
      il = dp4a_ss(w[1], (int)b0.y, il);
      il = dp4a_ss(w[2], (int)b0.z, il);
      il = dp4a_ss(w[3], (int)b0.w, il);
      il = dp4a_ss(w[4], (int)b1.x, il);
      il = dp4a_ss(w[5], (int)b1.y, il);
      il = dp4a_ss(w[6], (int)b1.z, il);
      il = dp4a_ss(w[7], (int)b1.w, il);
      acc[m] = fmaf(wd * xs, (float)(ih * 254 + il), acc[m]);
    } else {
      // w.d * x.d * (sum_i as f32), src/quant/q8_0.rs:65
      acc[m] += wd * xs * (float)ih;
    }
  }
}

// One Q4_K super-block against the staged activations of every row m < M.
// value = (d*sc)*q - dmin*m (src/quant/q4_k.rs:30-55), regrouped per 32-weight
// sub-block as (d*sc) * sum(q*x) - (dmin*m) * sum(x).
template <int MT, int PLANES>
__device__ __forceinline__ void item_dot_q4_k(const uint8_t* p, int col, const StreamLayout& L,
                                              const uint8_t* smem, int M, int nblk,
                                              float (&acc)[MT]) {
  const uint4 hdr = *reinterpret_cast<const uint4*>(p);
  const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
  uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
  unpack_scales_k4(hdr.y, hdr.z, hdr.w, sc_lo, sc_hi, mn_lo, mn_hi);
  const float* xscale = reinterpret_cast<const float*>(smem + L.off_scale);
  const float* xsum = reinterpret_cast<const float*>(smem + L.off_sum);
  const uint4* q4 = reinterpret_cast<const uint4*>(p + 16);
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const uint4 qa = q4[2 * g], qb = q4[2 * g + 1];
    const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    // sub-blocks 2g (low nibbles) and 2g+1 (high nibbles)
    const uint32_t scw = g < 2 ? sc_lo : sc_hi, mnw = g < 2 ? mn_lo : mn_hi;
    const int sh = 16 * (g & 1);
    const float ds_a = d * (float)((scw >> sh) & 0xFF);
    // the high nibbles are used in place (16*q), hence the 1/16
    const float ds_b = d * (float)((scw >> (sh + 8)) & 0xFF) * 0.0625f;
    const float dm_a = dmin * (float)((mnw >> sh) & 0xFF);
    const float dm_b = dmin * (float)((mnw >> (sh + 8)) & 0xFF);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m >= M) break;
      const uint8_t* xp = smem + L.off_planes + (m * PLANES) * L.plane_bytes + col * 272 + 64 * g;
      int ia = 0, ib = 0;
      {
        const uint4 x0 = *reinterpret_cast<const uint4*>(xp);
        const uint4 x1 = *reinterpret_cast<const uint4*>(xp + 16);
        const uint4 x2 = *reinterpret_cast<const uint4*>(xp + 32);
        const uint4 x3 = *reinterpret_cast<const uint4*>(xp + 48);
        const int xl[8] = {(int)x0.x, (int)x0.y, (int)x0.z, (int)x0.w,
                           (int)x1.x, (int)x1.y, (int)x1.z, (int)x1.w};
        const int xh[8] = {(int)x2.x, (int)x2.y, (int)x2.z, (int)x2.w,
                           (int)x3.x, (int)x3.y, (int)x3.z, (int)x3.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          ia = dp4a_ss((int)(qw[k] & 0x0F0F0F0Fu), xl[k], ia);
          ib = dp4a_us(qw[k] & 0xF0F0F0F0u, xh[k], ib);
        }
      }
      if (PLANES == 2) {
        int ja = 0, jb = 0;
        const uint8_t* xq = xp + L.plane_bytes;
        const uint4 x0 = *reinterpret_cast<const uint4*>(xq);
        const uint4 x1 = *reinterpret_cast<const uint4*>(xq + 16);
        const uint4 x2 = *reinterpret_cast<const uint4*>(xq + 32);
        const uint4 x3 = *reinterpret_cast<const uint4*>(xq + 48);
        const int xl[8] = {(int)x0.x, (int)x0.y, (int)x0.z, (int)x0.w,
                           (int)x1.x, (int)x1.y, (int)x1.z, (int)x1.w};
        const int xh[8] = {(int)x2.x, (int)x2.y, (int)x2.z, (int)x2.w,
                           (int)x3.x, (int)x3.y, (int)x3.z, (int)x3.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          ja = dp4a_ss((int)(qw[k] & 0x0F0F0F0Fu), xl[k], ja);
          jb = dp4a_us(qw[k] & 0xF0F0F0F0u, xh[k], jb);
        }
        ia = ia * 254 + ja;
        ib = ib * 254 + jb;
      }
      const int sb = m * nblk + col * 8 + 2 * g;
      const float2 xs = *reinterpret_cast<const float2*>(xscale + sb);
      const float2 xm = *reinterpret_cast<const float2*>(xsum + sb);
      float t = acc[m];
      t = fmaf(ds_a * xs.x, (float)ia, t);
      t = fmaf(ds_b * xs.y, (float)ib, t);
      t = fmaf(-dm_a, xm.x, t);
      t = fmaf(-dm_b, xm.y, t);
      acc[m] = t;
    }
  }
}

template <int FMT, int MT, int PLANES>
__global__ void __launch_bounds__(MAX_WARPS * 32)
    gemv_stream_kernel(const StreamArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const StreamLayout L =
      stream_layout<FMT, PLANES>(a.K, a.bpr, a.M, nwarps, a.nstage, a.stage_bytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem) + warp * MAX_STAGES;
  uint8_t* my_stages = smem + L.off_stages + warp * a.nstage * a.stage_bytes;
  const int nblk = a.K / 32;

  // the matrix this CTA works on, then its rows there and the tiles of this warp within them
  int sg = 0;
  while (sg + 1 < a.nseg && (int)blockIdx.x >= a.seg[sg + 1].cta_begin) ++sg;
  const StreamSeg& S = a.seg[sg];
  const int cta = (int)blockIdx.x - S.cta_begin;
  const int nctas = (sg + 1 < a.nseg ? a.seg[sg + 1].cta_begin : (int)gridDim.x) - S.cta_begin;
  const int64_t rb = S.rows * cta / nctas;
  const int64_t re = S.rows * (cta + 1) / nctas;
  const int TR = a.tile_rows;
  const int ntiles_cta = (int)((re - rb + TR - 1) / TR);
  const int n_my = warp < ntiles_cta ? (ntiles_cta - warp + nwarps - 1) / nwarps : 0;
  const int64_t total16 = S.total_bytes & ~int64_t(15);

  if (lane == 0)
    for (int s = 0; s < a.nstage; ++s) mbar_init(&bars[s], 1);
  mbar_fence_init();
  __syncwarp();

  // lane 0: start the bulk copy of this warp's i-th tile into stage i % nstage
  auto issue = [&](int i) {
    const int64_t r0 = rb + (int64_t)(warp + i * nwarps) * TR;
    const int nr = (int)min((int64_t)TR, re - r0);
    const int64_t b0 = r0 * a.row_bytes, b1 = b0 + (int64_t)nr * a.row_bytes;
    const int64_t a0 = b0 & ~int64_t(15);
    int64_t a1 = (b1 + 15) & ~int64_t(15);
    const int s = i % a.nstage;
    uint8_t* dst = my_stages + s * a.stage_bytes;
    if (a1 > total16) {
      // the stream ends inside a 16-byte unit: fetch that ragged end with plain loads
      a1 = total16;
      for (int64_t t = a1; t < b1; ++t) dst[t - a0] = S.w[t];
    }
    const uint32_t bytes = (uint32_t)(a1 - a0);
    mbar_arrive_expect_tx(&bars[s], bytes);
    bulk_g2s(dst, S.w + a0, bytes, &bars[s]);
  };
  int issued = 0;
  if (lane == 0)
    for (; issued < n_my && issued < a.nstage; ++issued) issue(issued);
  issued = __shfl_sync(0xFFFFFFFFu, issued, 0);

  // Programmatic dependent launch: the weight copies above never depend on the kernel before
  // this one; the activations (and the residual) may, so everything below waits for it.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  stage_activations<FMT, PLANES>(a, L, smem);
  __syncthreads();

  // lane -> (row within the warp's pass, block column); several short rows share a pass
  const int bpr = a.bpr;
  const int R = bpr <= 32 ? 32 / bpr : 1;  // rows per pass
  const int lrow = bpr <= 32 ? lane / bpr : 0;
  const int lcol = bpr <= 32 ? lane - lrow * bpr : lane;
  const bool lane_on = bpr <= 32 ? lane < R * bpr : true;

  int fail_at = -1;
  for (int i = 0; i < n_my; ++i) {
    const int s = i % a.nstage;
    if (!mbar_wait_bounded(&bars[s], (uint32_t)(i / a.nstage) & 1)) {
      fail_at = i;
      break;
    }
    const int64_t r0 = rb + (int64_t)(warp + i * nwarps) * TR;
    const int nr = (int)min((int64_t)TR, re - r0);
    const int64_t b0 = r0 * a.row_bytes;
    const uint8_t* tile = my_stages + s * a.stage_bytes + (int)(b0 & 15);

    for (int rr = 0; rr < nr; rr += R) {
      float acc[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[m] = 0.f;
      const int row = rr + lrow;
      if (lane_on && row < nr) {
        const uint8_t* rowp = tile + row * a.row_bytes;
        for (int col = lcol; col < bpr; col += 32) {
          const uint8_t* p = rowp + col * Fmt<FMT>::ITEM_BYTES;
          if (FMT == FMT_Q8_0)
            item_dot_q8_0<MT, PLANES>(p, col, L, smem, a.M, nblk, acc);
          else
            item_dot_q4_k<MT, PLANES>(p, col, L, smem, a.M, nblk, acc);
        }
      }
      // segmented reduction over the lanes of one row
      const int seg = bpr <= 32 ? bpr : 32;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m >= a.M) break;
        float v = acc[m];
#pragma unroll
        for (int o = 16; o; o >>= 1) {
          float u = __shfl_down_sync(0xFFFFFFFFu, v, o);
          if (lcol + o < seg) v += u;
        }
        if (lane_on && lcol == 0 && row < nr) {
          if (a.resid) v += a.resid[(int64_t)m * a.ldr + r0 + row];
          S.y[(int64_t)m * S.ldy + r0 + row] = v;
        }
      }
    }
    __syncwarp();
    if (i + a.nstage < n_my) {
      if (lane == 0) issue(i + a.nstage);
      issued = i + a.nstage + 1;
    }
  }
  if (fail_at >= 0) {
    if (lane == 0) atomicOr(a.status, DEV_WAIT_TIMEOUT);
    // do not leave while copies of this warp may still land in shared memory
    for (int i = fail_at; i < issued; ++i)
      mbar_wait_bounded(&bars[i % a.nstage], (uint32_t)(i / a.nstage) & 1);
  }
}

// What one launch computes: up to three matrices over shared activations, with the optional
// fusions of the decode step.
struct StreamCall {
  int nseg = 1;
  const void* w[MAX_SEGS] = {nullptr, nullptr, nullptr};
  float* y[MAX_SEGS] = {nullptr, nullptr, nullptr};
  int64_t rows[MAX_SEGS] = {0, 0, 0};
  const float* x = nullptr;
  const float* x2 = nullptr;
  const float* norm_w = nullptr;
  float eps = 0.f;
  const float* resid = nullptr;
  int64_t K = 0;
  int M = 1;
};

template <int FMT, int MT, int PLANES>
static int32_t launch_stream(kanso_cuda_ctx* ctx, const StreamCall& c) {
  using F = Fmt<FMT>;
  StreamArgs a;
  a.K = (int)c.K;
  a.bpr = (int)(c.K / F::ITEM_ELEMS);
  a.row_bytes = a.bpr * F::ITEM_BYTES;
  a.nseg = c.nseg;
  a.x = c.x;
  a.x2 = c.x2;
  a.norm_w = c.norm_w;
  a.eps = c.eps;
  a.resid = c.resid;
  a.ldx = c.K;
  a.M = c.M;
  a.status = ctx->dev_status;
  int64_t total_rows = 0, max_rows = 0;
  for (int i = 0; i < c.nseg; ++i) {
    total_rows += c.rows[i];
    if (c.rows[i] > max_rows) max_rows = c.rows[i];
  }
  // CTAs are dealt to the matrices in proportion to their rows
  int grid = ctx->sm_count;
  if (total_rows < grid) grid = (int)total_rows;
  if (grid < c.nseg) grid = c.nseg;
  int cta = 0;
  int64_t rows_per_cta = 1;
  for (int i = 0; i < MAX_SEGS; ++i) {
    StreamSeg& sgm = a.seg[i];
    if (i < c.nseg) {
      sgm.w = (const uint8_t*)c.w[i];
      sgm.y = c.y[i];
      sgm.rows = c.rows[i];
      sgm.total_bytes = c.rows[i] * a.row_bytes;
      sgm.ldy = c.rows[i];
      sgm.cta_begin = cta;
      int n = i + 1 == c.nseg ? grid - cta
                              : (int)((c.rows[i] * grid + total_rows / 2) / total_rows);
      if (n < 1) n = 1;
      if (n > grid - cta - (c.nseg - 1 - i)) n = grid - cta - (c.nseg - 1 - i);
      const int64_t rpc = (c.rows[i] + n - 1) / n;
      if (rpc > rows_per_cta) rows_per_cta = rpc;
      cta += n;
    } else {
      sgm = StreamSeg{nullptr, nullptr, 0, 0, 0, grid};
    }
  }
  a.ldr = c.rows[0];  // the residual has the shape of the (single) result

  const int R = a.bpr <= 32 ? 32 / a.bpr : 1;
  // Pick warps, tile rows and stages so the rings fit in shared memory.
  const int smem_max = ctx->smem_optin - 1024;  // the kernel also has a little static shared memory
  int best_w = 0, best_s = 0, best_tr = 0, best_sb = 0;
  for (int nw : {8, 4, 2, 1}) {
    // tile: about 4 KB, whole passes of R rows, no more than this warp's share of the CTA's rows
    int tr = (int)((4096 + a.row_bytes - 1) / a.row_bytes);
    tr = ((tr + R - 1) / R) * R;
    int64_t share = (rows_per_cta + nw - 1) / nw;
    share = ((share + R - 1) / R) * R;
    if (tr > share) tr = (int)share;
    if (tr < R) tr = R;
    int sb = ((tr * a.row_bytes + 15) & ~15) + 32;
    // no more stages than this warp has tiles: a small launch then leaves shared memory for
    // the CTAs of the launches after it, which prefetch their weights while this one runs
    const int tiles = (int)((share + tr - 1) / tr);
    for (int st = tiles < MAX_STAGES ? (tiles < 1 ? 1 : tiles) : MAX_STAGES; st >= 1; --st) {
      StreamLayout L = stream_layout<FMT, PLANES>(a.K, a.bpr, c.M, nw, st, sb);
      if (L.total <= smem_max) {
        best_w = nw;
        best_s = st;
        best_tr = tr;
        best_sb = sb;
        break;
      }
    }
    if (best_w) break;
  }
  if (!best_w)
    return fail(ctx, KANSO_ERR_UNSUPPORTED,
                "gemv: K=%lld with %d activation rows does not fit the %d-byte shared memory of "
                "one SM",
                (long long)c.K, c.M, smem_max);
  a.tile_rows = best_tr;
  a.stage_bytes = best_sb;
  a.nstage = best_s;
  StreamLayout L = stream_layout<FMT, PLANES>(a.K, a.bpr, c.M, best_w, best_s, best_sb);
  auto kern = gemv_stream_kernel<FMT, MT, PLANES>;
  static int smem_set[16] = {0};  // per device: largest opt-in already made for this kernel
  if (L.total > smem_set[ctx->device & 15]) {
    KANSO_CUDA_TRY(ctx,
                   cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        smem_max),
                   "gemv: shared memory opt-in");
    smem_set[ctx->device & 15] = smem_max;
  }
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(grid);
  lc.blockDim = dim3(best_w * 32);
  lc.dynamicSmemBytes = L.total;
  lc.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = ctx->overlap_weight_prefetch ? 1 : 0;
  lc.attrs = attr;
  lc.numAttrs = 1;
  KANSO_CUDA_TRY(ctx, cudaLaunchKernelEx(&lc, kern, a), "gemv_stream launch");
  return after_launch(ctx, "gemv_stream");
}

template <int FMT, int PLANES>
static int32_t dispatch_call(kanso_cuda_ctx* ctx, const StreamCall& c) {
  switch (c.M) {
    case 1: return launch_stream<FMT, 1, PLANES>(ctx, c);
    case 2: return launch_stream<FMT, 2, PLANES>(ctx, c);
    case 3:
    case 4: return launch_stream<FMT, 4, PLANES>(ctx, c);
    default: return launch_stream<FMT, 8, PLANES>(ctx, c);
  }
}

template <int FMT, int PLANES>
static int32_t dispatch_m(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                          int64_t rows, int64_t K, int M, int64_t ldx, int64_t ldy) {
  (void)ldx;
  (void)ldy;
  StreamCall c;
  c.w[0] = w;
  c.y[0] = y;
  c.rows[0] = rows;
  c.x = x;
  c.K = K;
  c.M = M;
  return dispatch_call<FMT, PLANES>(ctx, c);
}

// Fused decode-step matmul on Q8_0 weights, at most 8 activation rows: up to three matrices
// over the same activations, rmsnorm folded into the activation staging, silu(x)*x2 as the
// activations, residual added to the result. Declared in glue.cuh.
int32_t q8_mma_matmul(kanso_cuda_ctx* ctx, int nseg, const void* const* w, float* const* y,
                      const int64_t* rows, const float* x, const float* x2, const float* norm_w,
                      float eps, const float* resid, int64_t K, int M, int32_t act_mode,
                      bool decode_chain, bool* handled);

int32_t stream_fused_q8_0(kanso_cuda_ctx* ctx, int nseg, const void* const* w, float* const* y,
                          const int64_t* rows, const float* x, const float* x2,
                          const float* norm_w, float eps, const float* resid, int64_t K, int M,
                          int32_t act_mode) {
  if (nseg < 1 || nseg > MAX_SEGS || M < 1 || M > 8 || K <= 0 || K % 32 != 0)
    return fail(ctx, KANSO_ERR_SHAPE, "fused matmul: bad shape (nseg %d, M %d, K %lld)", nseg, M,
                (long long)K);
  if (resid && nseg != 1)
    return fail(ctx, KANSO_ERR_SHAPE, "fused matmul: a residual needs a single matrix");
  {
    // the tensor-core kernel takes the shapes it covers (K a multiple of 64, at most 4096)
    bool handled = false;
    int32_t st = q8_mma_matmul(ctx, nseg, w, y, rows, x, x2, norm_w, eps, resid, K, M, act_mode,
                               true, &handled);
    if (st != KANSO_OK || handled) return st;
  }
  StreamCall c;
  c.nseg = nseg;
  for (int i = 0; i < nseg; ++i) {
    if (!w[i] || !y[i] || rows[i] < 1 || !aligned16(w[i]))
      return fail(ctx, KANSO_ERR_SHAPE, "fused matmul: matrix %d is missing or misaligned", i);
    c.w[i] = w[i];
    c.y[i] = y[i];
    c.rows[i] = rows[i];
  }
  c.x = x;
  c.x2 = x2;
  c.norm_w = norm_w;
  c.eps = eps;
  c.resid = resid;
  c.K = K;
  c.M = M;
  return act_mode == KANSO_ACT_Q8 ? dispatch_call<FMT_Q8_0, 1>(ctx, c)
                                  : dispatch_call<FMT_Q8_0, 2>(ctx, c);
}

// y[M,N] = x[M,K] @ W[N,K]^T with the streaming kernel, at most 8 activation rows per pass.
int32_t stream_matmul(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x, float* y,
                      int64_t M, int64_t N, int64_t K, int32_t act_mode) {
  if (M < 0 || N < 0 || K < 0) return fail(ctx, KANSO_ERR_SHAPE, "matmul: negative dimension");
  const int blk = dtype == KANSO_DTYPE_Q8_0 ? 32 : 256;
  if (dtype != KANSO_DTYPE_Q8_0 && dtype != KANSO_DTYPE_Q4_K)
    return fail(ctx, KANSO_ERR_UNSUPPORTED, "matmul: dtype %d is neither Q8_0 nor Q4_K", dtype);
  if (K % blk != 0)
    return fail(ctx, KANSO_ERR_SHAPE, "matmul: cols %lld is not a multiple of the %d-weight block",
                (long long)K, blk);
  if (act_mode != KANSO_ACT_F32 && act_mode != KANSO_ACT_Q8)
    return fail(ctx, KANSO_ERR_CONFIG, "matmul: unknown activation mode %d", act_mode);
  if (dtype == KANSO_DTYPE_Q4_K && act_mode == KANSO_ACT_Q8)
    return fail(ctx, KANSO_ERR_UNSUPPORTED,
                "matmul: Q4_K has no Q8-activation dot in the reference; use KANSO_ACT_F32");
  if (M == 0 || N == 0) return KANSO_OK;
  if (K == 0) {
    KANSO_CUDA_TRY(ctx, cudaMemsetAsync(y, 0, sizeof(float) * M * N, ctx->stream), "matmul: K=0");
    return KANSO_OK;
  }
  if (!w || !x || !y) return fail(ctx, KANSO_ERR_SHAPE, "matmul: NULL pointer");
  if (!aligned16(w) || !aligned16(x))
    return fail(ctx, KANSO_ERR_SHAPE, "matmul: w and x must be 16-byte aligned");
  if (K > (1 << 20) || N > (int64_t(1) << 31))
    return fail(ctx, KANSO_ERR_UNSUPPORTED, "matmul: dimension too large");
  for (int64_t m0 = 0; m0 < M; m0 += 8) {
    int mc = (int)(M - m0 < 8 ? M - m0 : 8);
    int32_t st;
    const float* xp = x + m0 * K;
    float* yp = y + m0 * N;
    if (dtype == KANSO_DTYPE_Q8_0)
      st = act_mode == KANSO_ACT_Q8
               ? dispatch_m<FMT_Q8_0, 1>(ctx, w, xp, yp, N, K, mc, K, N)
               : dispatch_m<FMT_Q8_0, 2>(ctx, w, xp, yp, N, K, mc, K, N);
    else
      st = dispatch_m<FMT_Q4_K, 2>(ctx, w, xp, yp, N, K, mc, K, N);
    if (st != KANSO_OK) return st;
  }
  return KANSO_OK;
}

}  // namespace kanso

using namespace kanso;

namespace kanso {
int32_t matmul_dispatch(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x,
                        float* y, int64_t M, int64_t N, int64_t K, int32_t act_mode);
}

extern "C" {

int32_t kanso_cuda_gemv_q8_0(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                             int64_t rows, int64_t cols) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "gemv_q8_0: ctx is NULL");
  return matmul_dispatch(ctx, KANSO_DTYPE_Q8_0, w, x, y, 1, rows, cols, KANSO_ACT_F32);
}

int32_t kanso_cuda_gemv_q4_k(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                             int64_t rows, int64_t cols) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "gemv_q4_k: ctx is NULL");
  return matmul_dispatch(ctx, KANSO_DTYPE_Q4_K, w, x, y, 1, rows, cols, KANSO_ACT_F32);
}

}  // extern "C"
