// Q8_0 GEMV / few-row GEMM (1..8 activation rows) on the int8 tensor-core path.
//
// Math: src/quant/q8_0.rs (block = f16 d + 32 int8; dot = sum over blocks of d_w * d_x * isum).
// The activations are quantised per block of 32 exactly as quantize_row_q8_0
// (src/quant/q8_0.rs:13-32) into an int8 plane; KANSO_ACT_F32 adds a second plane with the
// quantisation residual in units of d/254, so x ~= d * (hi + lo/254) to ~2^-15 of the block
// maximum. One mma.sync m16n8k32 (s8 x s8 -> s32) then forms the int32 block sums of 16 weight
// rows against up to 8 columns (activation rows, or activation rows x planes) at once, so the
// cost per weight byte does not grow with the number of activation rows.
//
// Work split: a CTA owns a run of 16-row groups; its warps split K, warp w owning the same
// (at most two) blocks of every row, so the activation fragments of a warp's K slice stay in
// registers for the whole kernel and the weights of two row groups are in flight per warp.
// Rows longer than 32 blocks are split across CTAs (grid y); those CTAs add their sums into
// the output with atomics, on top of the residual the output already holds (the decode step's
// in-place "hidden += W.x") or of zeros written by a memset before the launch.
// Weight bytes go straight from global memory into the A fragments (no shared-memory staging):
// the lane of MMA row g and k-word t reads three aligned 32-bit words of rows g and g+8. A
// Q8_0 block is 34 bytes, so every other block starts half-way into a word; instead of
// shifting, those blocks feed the MMA with their k-values rotated by two (k-word 7 = q30 q31 q0
// q1), and the activation fragment is built in the same order. The warps' partial sums meet in
// shared memory once per pair of row groups.
#include "common.cuh"
#include "ctx.h"

namespace kanso {

constexpr int Q8M_WARPS = 16;
constexpr int Q8M_THREADS = Q8M_WARPS * 32;
constexpr int Q8M_NB = 2;        // blocks of a row per warp
constexpr int Q8M_MAX_SEGS = 3;

// column use of the MMA's 8 columns
constexpr int Q8M_MODE_A = 0;  // two planes, M <= 4: column = 2 * m + plane, one MMA per block
constexpr int Q8M_MODE_B = 1;  // two planes, M <= 8: column = m, one MMA per plane
constexpr int Q8M_MODE_C = 2;  // one plane (KANSO_ACT_Q8), M <= 8: column = m

struct Q8mSeg {
  const uint8_t* w;
  float* y;
  int64_t rows;
  int64_t ldy;
  int group_begin;  // first 16-row group of this matrix in the launch's group numbering
};

struct Q8mArgs {
  Q8mSeg seg[Q8M_MAX_SEGS];
  int nseg;
  int total_groups;
  const float* x;
  const float* x2;      // activations are silu(x) * x2 (src/model.rs:367-382)
  const float* norm_w;  // activations are rmsnorm(x) * norm_w (src/model.rs:653-659)
  float eps;
  const float* resid;   // result is resid + W.x; may alias y
  int64_t ldr, ldx;
  int K, bpr, M;
  int accumulate;       // 1: add into y with atomics (y holds the residual or zeros)
};

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ uint32_t q8m_pack4(const float (&v)[4]) {
  return ((uint32_t)(int)v[0] & 0xFF) | (((uint32_t)(int)v[1] & 0xFF) << 8) |
         (((uint32_t)(int)v[2] & 0xFF) << 16) | (((uint32_t)(int)v[3] & 0xFF) << 24);
}

// The three words a lane needs of one row's block: P[0] (scale half + two bytes), P[1 + t],
// P[5 + t], with P the block's address rounded down to a word.
struct Q8mRaw {
  uint32_t w0, wa, wb;
};

// NBT = blocks per warp slice, PD = row groups whose weights are in flight per warp = row
// groups between two reductions.
template <int MODE, bool COOP>
__global__ void __launch_bounds__(Q8M_THREADS, 2) gemv_q8_mma_kernel(const Q8mArgs a) {
  constexpr int NBT = Q8M_NB;
  constexpr int PLANES = MODE == Q8M_MODE_C ? 1 : 2;
  constexpr int NCOL = MODE == Q8M_MODE_A ? 1 : 2;  // activation rows per lane in C
  constexpr int MC = MODE == Q8M_MODE_A ? 4 : 8;    // activation rows kept per weight row
  constexpr int BATCH = 2, PD = 2;
  __shared__ float s_part[BATCH][Q8M_WARPS][16][MC];
  __shared__ float s_ss[Q8M_WARPS][8];
  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);
  const int g = lane >> 2, t = lane & 3;

  // this CTA's run of row groups and K slice, this warp's blocks
  const int g_begin = (int)((int64_t)a.total_groups * blockIdx.x / gridDim.x);
  const int g_end = (int)((int64_t)a.total_groups * (blockIdx.x + 1) / gridDim.x);
  const int wg = blockIdx.y * Q8M_WARPS + warp, WG = gridDim.y * Q8M_WARPS;
  const int kb0 = (int)((int64_t)a.bpr * wg / WG);
  const int nb = (int)((int64_t)a.bpr * (wg + 1) / WG) - kb0;  // <= NBT by the host's choice

  // loads this lane's words of group `grp`: rows g and g + 8 (clamped to the matrix).
  // bpr is even, so block kb starts on a word when kb is even and half-way into one when odd
  auto load_group = [&](int grp, Q8mRaw (&raw)[NBT][2]) {
    int s = 0;
#pragma unroll
    for (int i = 1; i < Q8M_MAX_SEGS; ++i)
      if (i < a.nseg && grp >= a.seg[i].group_begin) s = i;
    const int64_t n0 = (int64_t)(grp - a.seg[s].group_begin) * 16 + g;
    const int64_t last = a.seg[s].rows - 1;
    const uint8_t* r0 = a.seg[s].w + min(n0, last) * a.bpr * Q8_BYTES;
    const uint8_t* r1 = a.seg[s].w + min(n0 + 8, last) * a.bpr * Q8_BYTES;
#pragma unroll
    for (int j = 0; j < NBT; ++j) {
      if (j < nb) {
        const int kb = kb0 + j;
        const int off = kb * Q8_BYTES - ((kb & 1) ? 2 : 0);
        const uint32_t* p0 = reinterpret_cast<const uint32_t*>(r0 + off);
        const uint32_t* p1 = reinterpret_cast<const uint32_t*>(r1 + off);
        raw[j][0].w0 = __ldg(p0);
        raw[j][0].wa = __ldg(p0 + 1 + t);
        raw[j][0].wb = __ldg(p0 + 5 + t);
        raw[j][1].w0 = __ldg(p1);
        raw[j][1].wa = __ldg(p1 + 1 + t);
        raw[j][1].wb = __ldg(p1 + 5 + t);
      }
    }
  };

  // weights of the first groups are on their way before the activations are touched: with a
  // dependent launch they overlap the tail of the kernel that produces the activations
  Q8mRaw raw[PD][NBT][2];
#pragma unroll
  for (int p = 0; p < PD; ++p)
    if (g_begin + p < g_end) load_group(g_begin + p, raw[p]);
  // B column g of the MMA: activation row mcol (and plane, in mode A)
  const int mcol = MODE == Q8M_MODE_A ? g >> 1 : g;
  const int plane = MODE == Q8M_MODE_A ? g & 1 : 0;
  constexpr int MROWS = MODE == Q8M_MODE_A ? 4 : 8;  // activation rows a launch may carry
  uint32_t bh[NBT][2];  // activation fragments: plane used by the first (or only) MMA
  uint32_t bl[MODE == Q8M_MODE_B ? NBT : 1][2];
  float dx[NBT][NCOL];  // activation scale per block for this lane's C columns
  // Few activation rows (COOP): the warp's lanes share the quantisation of every (row, block)
  // pair. More rows: each lane quantises the k-words of its own MMA column.
  float nwv[NBT];
  if (COOP) {
    // The norm weights are weights: read before the wait. Lane = element of the block.
#pragma unroll
    for (int j = 0; j < NBT; ++j)
      nwv[j] = (a.norm_w && j < nb) ? __ldg(a.norm_w + 32 * (kb0 + j) + lane) : 1.0f;
  }
  pdl_launch_dependents();
  pdl_wait();
  if (COOP) {
    // ---- activation fragments of this warp's K slice. The 32 lanes quantise the 32 values of
    // one (activation row, block) pair together, one value each; the bytes are then gathered
    // into 32-bit words inside each quad of lanes and handed to the lanes that own the matching
    // MMA column with shuffles. Every load is issued before any arithmetic.
    float xv[MROWS][NBT], uv[MROWS][NBT];
#pragma unroll
    for (int m = 0; m < MROWS; ++m)
#pragma unroll
      for (int j = 0; j < NBT; ++j) {
        xv[m][j] = 0.f;
        uv[m][j] = 1.f;
        if (m < a.M && j < nb) {
          const int64_t at = (int64_t)m * a.ldx + 32 * (kb0 + j) + lane;
          xv[m][j] = a.x[at];
          if (a.x2) uv[m][j] = a.x2[at];
        }
      }
#pragma unroll
    for (int j = 0; j < NBT; ++j) {
      bh[j][0] = bh[j][1] = 0u;
      if (MODE == Q8M_MODE_B) bl[j][0] = bl[j][1] = 0u;
#pragma unroll
      for (int cidx = 0; cidx < NCOL; ++cidx) dx[j][cidx] = 0.f;
    }
    float ss[MROWS];  // per activation row: this lane's share of the sum of squares
#pragma unroll
    for (int m = 0; m < MROWS; ++m) {
      ss[m] = 0.f;
      if (m < a.M) {
#pragma unroll
        for (int j = 0; j < NBT; ++j) {
          float x = xv[m][j];
          if (a.x2) x = x / (1.0f + expf(-x)) * uv[m][j];  // silu(g) * u
          if (a.norm_w) {
            ss[m] = fmaf(x, x, ss[m]);
            x *= nwv[j];
          }
          float amax = fabsf(x);
#pragma unroll
          for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
          float d, id;
          if (PLANES == 1) {  // exactly quantize_row_q8_0
            d = __fdiv_rn(amax, 127.0f);
            id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
          } else {  // the second plane absorbs the last-bit differences of the fast forms
            d = amax * (1.0f / 127.0f);
            id = d != 0.0f ? __frcp_rn(d) : 0.0f;
          }
          const float scaled = __fmul_rn(x, id);
          const float hq = fminf(fmaxf(PLANES == 1 ? roundf(scaled) : rintf(scaled), -128.f), 127.f);
          float lq = 0.f;
          if (PLANES == 2)
            lq = fminf(fmaxf(rintf(fmaf(-d, hq, x) * (254.0f * id)), -127.f), 127.f);
          // words of four consecutive elements, complete in every lane of the quad
          const int sh8 = 8 * (lane & 3);
          uint32_t hw = ((uint32_t)(int)hq & 0xFFu) << sh8, lw = ((uint32_t)(int)lq & 0xFFu) << sh8;
          hw |= __shfl_xor_sync(0xFFFFFFFFu, hw, 1);
          hw |= __shfl_xor_sync(0xFFFFFFFFu, hw, 2);
          if (PLANES == 2) {
            lw |= __shfl_xor_sync(0xFFFFFFFFu, lw, 1);
            lw |= __shfl_xor_sync(0xFFFFFFFFu, lw, 2);
          }
          // k-word kw of the block in the order its weights feed the MMA: the natural word, or
          // (block starting on a word) the bytes 4kw+2 .. 4kw+5, wrapping at 32
          const bool rotated = ((kb0 + j) & 1) == 0;
          auto kword = [&](uint32_t w, int kw) {
            const uint32_t lo = __shfl_sync(0xFFFFFFFFu, w, 4 * kw);
            const uint32_t hi = __shfl_sync(0xFFFFFFFFu, w, 4 * ((kw + 1) & 7));
            return rotated ? __funnelshift_r(lo, hi, 16) : lo;
          };
          const float dsc = PLANES == 2 ? d * (1.0f / 254.0f) : d;
          if (MODE == Q8M_MODE_A) {
            // odd lanes of a quad offer the low plane, even lanes the high plane
            const uint32_t offer = (lane & 1) ? lw : hw;
            const uint32_t lo0 = __shfl_sync(0xFFFFFFFFu, offer, 4 * t + plane);
            const uint32_t hi0 = __shfl_sync(0xFFFFFFFFu, offer, 4 * ((t + 1) & 7) + plane);
            const uint32_t lo1 = __shfl_sync(0xFFFFFFFFu, offer, 4 * (4 + t) + plane);
            const uint32_t hi1 = __shfl_sync(0xFFFFFFFFu, offer, 4 * ((5 + t) & 7) + plane);
            if (mcol == m) {
              bh[j][0] = rotated ? __funnelshift_r(lo0, hi0, 16) : lo0;
              bh[j][1] = rotated ? __funnelshift_r(lo1, hi1, 16) : lo1;
            }
            if (t == m) dx[j][0] = dsc;
          } else {
            const uint32_t h0 = kword(hw, t), h1 = kword(hw, 4 + t);
            if (mcol == m) {
              bh[j][0] = h0;
              bh[j][1] = h1;
            }
            if (MODE == Q8M_MODE_B) {
              const uint32_t l0 = kword(lw, t), l1 = kword(lw, 4 + t);
              if (mcol == m) {
                bl[j][0] = l0;
                bl[j][1] = l1;
              }
            }
            if (2 * t == m) dx[j][0] = dsc;
            if (2 * t + 1 == m) dx[j][NCOL - 1] = dsc;
          }
        }
      }
    }
    if (a.norm_w) {
      // 1 / rms of every activation row: this warp's slice, then all warps (the host does not
      // split K across CTAs when a norm is folded in, so the CTA sees the whole row)
#pragma unroll
      for (int m = 0; m < MROWS; ++m) {
        if (m < a.M) {
          float v = ss[m];
#pragma unroll
          for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
          if (lane == 0) s_ss[warp][m] = v;
        }
      }
      __syncthreads();
#pragma unroll
      for (int cidx = 0; cidx < NCOL; ++cidx) {
        const int m = MODE == Q8M_MODE_A ? t : 2 * t + cidx;
        float tot = 0.f;
        if (m < a.M)
          for (int w = 0; w < Q8M_WARPS; ++w) tot += s_ss[w][m];
        const float r = 1.0f / sqrtf(tot / (float)a.K + a.eps);
#pragma unroll
        for (int j = 0; j < NBT; ++j) dx[j][cidx] *= r;
      }
    }
  } else {
    float ss = 0.f;  // sum of squares of row mcol over this warp's slice
#pragma unroll
    for (int j = 0; j < NBT; ++j) {
      float v[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int e = 0; e < 4; ++e) v[h][e] = 0.f;
      const int kb = kb0 + j;
      if (j < nb && mcol < a.M) {
        // k-words t and 4 + t of the block, in the order the weights feed the MMA
        const float* xb = a.x + (int64_t)mcol * a.ldx + 32 * kb;
        const float* x2b = a.x2 ? a.x2 + (int64_t)mcol * a.ldx + 32 * kb : nullptr;
        const float* nwb = a.norm_w ? a.norm_w + 32 * kb : nullptr;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int kw = 4 * h + t;
          int k0, k1;  // first element of the two halves of the k-word
          if (kb & 1) {
            k0 = 4 * kw;
            k1 = 4 * kw + 2;
          } else {
            k0 = (4 * kw + 2) & 31;
            k1 = (4 * kw + 4) & 31;
          }
          const float2 p0 = *reinterpret_cast<const float2*>(xb + k0);
          const float2 p1 = *reinterpret_cast<const float2*>(xb + k1);
          v[h][0] = p0.x; v[h][1] = p0.y; v[h][2] = p1.x; v[h][3] = p1.y;
          if (x2b) {  // silu(g) * u with silu(g) = g / (1 + e^-g)
            const float2 u0 = *reinterpret_cast<const float2*>(x2b + k0);
            const float2 u1 = *reinterpret_cast<const float2*>(x2b + k1);
            v[h][0] = v[h][0] / (1.0f + expf(-v[h][0])) * u0.x;
            v[h][1] = v[h][1] / (1.0f + expf(-v[h][1])) * u0.y;
            v[h][2] = v[h][2] / (1.0f + expf(-v[h][2])) * u1.x;
            v[h][3] = v[h][3] / (1.0f + expf(-v[h][3])) * u1.y;
          }
          if (nwb) {
            const float2 n0 = __ldg(reinterpret_cast<const float2*>(nwb + k0));
            const float2 n1 = __ldg(reinterpret_cast<const float2*>(nwb + k1));
#pragma unroll
            for (int e = 0; e < 4; ++e) ss = fmaf(v[h][e], v[h][e], ss);
            v[h][0] *= n0.x; v[h][1] *= n0.y; v[h][2] *= n1.x; v[h][3] *= n1.y;
          }
        }
      }
      float amax = 0.f;
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int e = 0; e < 4; ++e) amax = fmaxf(amax, fabsf(v[h][e]));
      amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
      float d, id;
      if (PLANES == 1) {  // exactly quantize_row_q8_0
        d = __fdiv_rn(amax, 127.0f);
        id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
      } else {  // the second plane absorbs the last-bit differences of the fast forms
        d = amax * (1.0f / 127.0f);
        id = d != 0.0f ? __frcp_rn(d) : 0.0f;
      }
      float hq[2][4], lq[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float scaled = __fmul_rn(v[h][e], id);
          hq[h][e] = fminf(fmaxf(PLANES == 1 ? roundf(scaled) : rintf(scaled), -128.f), 127.f);
          if (PLANES == 2)
            lq[h][e] =
                fminf(fmaxf(rintf(fmaf(-d, hq[h][e], v[h][e]) * (254.0f * id)), -127.f), 127.f);
        }
      if (MODE == Q8M_MODE_A) {
        bh[j][0] = plane ? q8m_pack4(lq[0]) : q8m_pack4(hq[0]);
        bh[j][1] = plane ? q8m_pack4(lq[1]) : q8m_pack4(hq[1]);
      } else {
        bh[j][0] = q8m_pack4(hq[0]);
        bh[j][1] = q8m_pack4(hq[1]);
        if (MODE == Q8M_MODE_B) {
          bl[j][0] = q8m_pack4(lq[0]);
          bl[j][1] = q8m_pack4(lq[1]);
        }
      }
      // scales of the activation rows this lane's C columns belong to
      const float dsc = PLANES == 2 ? d * (1.0f / 254.0f) : d;
      dx[j][0] = __shfl_sync(0xFFFFFFFFu, dsc, 8 * t);  // column 2t (mode A: row t, plane 0)
      if (NCOL == 2) dx[j][NCOL - 1] = __shfl_sync(0xFFFFFFFFu, dsc, 8 * t + 4);  // column 2t + 1
    }
    if (a.norm_w) {
      // 1 / rms of every activation row: this warp's slice, then all warps (the host does not
      // split K across CTAs when a norm is folded in, so the CTA sees the whole row)
      ss += __shfl_xor_sync(0xFFFFFFFFu, ss, 1);
      ss += __shfl_xor_sync(0xFFFFFFFFu, ss, 2);
      if (t == 0 && plane == 0) s_ss[warp][mcol] = ss;
      __syncthreads();
#pragma unroll
      for (int cidx = 0; cidx < NCOL; ++cidx) {
        const int m = MODE == Q8M_MODE_A ? t : 2 * t + cidx;
        float tot = 0.f;
        if (m < a.M)
          for (int w = 0; w < Q8M_WARPS; ++w) tot += s_ss[w][m];
        const float r = 1.0f / sqrtf(tot / (float)a.K + a.eps);
#pragma unroll
        for (int j = 0; j < NBT; ++j) dx[j][cidx] *= r;
      }
    }
  }

  // ---- row groups, BATCH at a time
  for (int gb = g_begin; gb < g_end; gb += BATCH) {
#pragma unroll
    for (int gi = 0; gi < BATCH; ++gi) {
      const int grp = gb + gi;
      if (grp < g_end) {
        Q8mRaw(&cur)[NBT][2] = raw[gi % PD];
        float acc[2][NCOL];  // [row g / row g + 8][column]
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int cidx = 0; cidx < NCOL; ++cidx) acc[r][cidx] = 0.f;
#pragma unroll
        for (int j = 0; j < NBT; ++j) {
          if (j < nb) {
            const bool word_start = ((kb0 + j) & 1) == 0;
            uint32_t afr[2][2];
            float wd[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              const Q8mRaw& q = cur[j][r];
              wd[r] = f16_bits_to_f32(word_start ? (q.w0 & 0xFFFFu) : (q.w0 >> 16));
              afr[r][0] = q.wa;
              // k-word 7 of a block that starts on a word: q30 q31 from P[8], q0 q1 from P[0]
              afr[r][1] = (word_start && t == 3) ? __byte_perm(q.wb, q.w0, 0x7610) : q.wb;
            }
            int c[4];
            mma_s8(c, afr[0][0], afr[1][0], afr[0][1], afr[1][1], bh[j][0], bh[j][1]);
            if (MODE == Q8M_MODE_A) {
              acc[0][0] = fmaf(wd[0] * dx[j][0], (float)(c[0] * 254 + c[1]), acc[0][0]);
              acc[1][0] = fmaf(wd[1] * dx[j][0], (float)(c[2] * 254 + c[3]), acc[1][0]);
            } else if (MODE == Q8M_MODE_B) {
              int cl[4];
              mma_s8(cl, afr[0][0], afr[1][0], afr[0][1], afr[1][1], bl[j][0], bl[j][1]);
#pragma unroll
              for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int cidx = 0; cidx < 2; ++cidx)
                  acc[r][cidx] = fmaf(wd[r] * dx[j][cidx],
                                      (float)(c[2 * r + cidx] * 254 + cl[2 * r + cidx]),
                                      acc[r][cidx]);
            } else {
#pragma unroll
              for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int cidx = 0; cidx < 2; ++cidx)
                  acc[r][cidx] = fmaf(wd[r] * dx[j][cidx], (float)c[2 * r + cidx], acc[r][cidx]);
            }
          }
        }
        // this slot's registers are free: request the group PD ahead
        if (grp + PD < g_end) load_group(grp + PD, raw[gi % PD]);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          if (MODE == Q8M_MODE_A) {
            s_part[gi][warp][g + 8 * r][t] = acc[r][0];
          } else {
            s_part[gi][warp][g + 8 * r][2 * t] = acc[r][0];
            s_part[gi][warp][g + 8 * r][2 * t + 1] = acc[r][NCOL - 1];
          }
        }
      }
    }
    __syncthreads();
    // thread = (group of the pair, row, activation row): sum over the warps' K slices
    const int gcount = min(BATCH, g_end - gb);
    for (int idx = tid; idx < gcount * 16 * MC; idx += Q8M_THREADS) {
      const int gi = idx / (16 * MC), row = (idx / MC) % 16, m = idx % MC;
      if (m < a.M) {
        const int grp = gb + gi;
        int s = 0;
#pragma unroll
        for (int i = 1; i < Q8M_MAX_SEGS; ++i)
          if (i < a.nseg && grp >= a.seg[i].group_begin) s = i;
        const int64_t n = (int64_t)(grp - a.seg[s].group_begin) * 16 + row;
        if (n < a.seg[s].rows) {
          float sum = 0.f;
#pragma unroll
          for (int w = 0; w < Q8M_WARPS; ++w) sum += s_part[gi][w][row][m];
          float* dst = a.seg[s].y + (int64_t)m * a.seg[s].ldy + n;
          if (a.accumulate) {
            atomicAdd(dst, sum);
          } else {
            if (a.resid) sum += a.resid[(int64_t)m * a.ldr + n];
            *dst = sum;
          }
        }
      }
    }
    __syncthreads();
  }
}

template <int MODE>
static int32_t q8m_launch(kanso_cuda_ctx* ctx, const Q8mArgs& a, dim3 grid) {
  // up to two activation rows: the lanes quantise each (row, block) pair together
  cudaError_t e = a.M <= 2 ? launch_dependent(ctx, gemv_q8_mma_kernel<MODE, true>, grid,
                                              dim3(Q8M_THREADS), 0, a)
                           : launch_dependent(ctx, gemv_q8_mma_kernel<MODE, false>, grid,
                                              dim3(Q8M_THREADS), 0, a);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "gemv_q8_mma launch");
  return after_launch(ctx, "gemv_q8_mma");
}

// Up to three Q8_0 matrices against the same 1..8 activation rows, with the decode step's
// optional fusions. Sets *handled = false (and launches nothing) for shapes outside this
// kernel's range: K a multiple of 64, the matrices word-aligned, and K at most 1024 when a
// norm is folded in or several matrices share the launch.
int32_t q8_mma_matmul(kanso_cuda_ctx* ctx, int nseg, const void* const* w, float* const* y,
                      const int64_t* rows, const float* x, const float* x2, const float* norm_w,
                      float eps, const float* resid, int64_t K, int M, int32_t act_mode,
                      bool decode_chain, bool* handled) {
  *handled = false;
  if (nseg < 1 || nseg > Q8M_MAX_SEGS || M < 1 || M > 8) return KANSO_OK;
  if (K < 64 || K % 64 != 0 || K > (1 << 20)) return KANSO_OK;
  if ((reinterpret_cast<uintptr_t>(x) & 7) != 0 || (x2 && (reinterpret_cast<uintptr_t>(x2) & 7)) ||
      (norm_w && (reinterpret_cast<uintptr_t>(norm_w) & 7)))
    return KANSO_OK;
  const int bpr = (int)(K / 32);
  const int ksplit = (bpr + Q8M_NB * Q8M_WARPS - 1) / (Q8M_NB * Q8M_WARPS);
  if (ksplit > 1 && (norm_w || nseg != 1)) return KANSO_OK;
  if (ksplit > 65535) return KANSO_OK;
  // One activation row, called on its own: the streaming kernel (bulk copies into shared
  // memory, dp4a) sustains more launches per second, except on tall matrices with short rows
  // (an LM head). Inside the decode step's chain of dependent launches this kernel is used for
  // every row count: what counts there is the time from the arrival of the activations to the
  // last store, and this kernel has no block-wide activation staging in that path.
  {
    int64_t total_rows = 0;
    for (int i = 0; i < nseg; ++i) total_rows += rows[i];
    if (M == 1 && !decode_chain && !(ksplit == 1 && total_rows >= 16384)) return KANSO_OK;
  }
  Q8mArgs a;
  a.nseg = nseg;
  int groups = 0;
  for (int i = 0; i < nseg; ++i) {
    if (!w[i] || !y[i] || rows[i] < 1 || (reinterpret_cast<uintptr_t>(w[i]) & 3) != 0)
      return KANSO_OK;
    if (rows[i] > (int64_t(1) << 30)) return KANSO_OK;
    a.seg[i].w = (const uint8_t*)w[i];
    a.seg[i].y = y[i];
    a.seg[i].rows = rows[i];
    a.seg[i].ldy = rows[i];
    a.seg[i].group_begin = groups;
    groups += (int)((rows[i] + 15) / 16);
  }
  for (int i = nseg; i < Q8M_MAX_SEGS; ++i) a.seg[i] = a.seg[0];
  a.total_groups = groups;
  a.x = x;
  a.x2 = x2;
  a.norm_w = norm_w;
  a.eps = eps;
  a.resid = resid;
  a.ldr = nseg == 1 ? rows[0] : 0;
  a.ldx = K;
  a.K = (int)K;
  a.bpr = bpr;
  a.M = M;
  a.accumulate = 0;
  *handled = true;
  if (ksplit > 1) {
    // the K slices add into y: y must hold the residual (in place) or zeros
    a.accumulate = 1;
    if (!(resid && resid == y[0])) {
      if (resid)
        KANSO_CUDA_TRY(ctx,
                       cudaMemcpyAsync(y[0], resid, sizeof(float) * (size_t)M * rows[0],
                                       cudaMemcpyDeviceToDevice, ctx->stream),
                       "gemv_q8_mma: residual copy");
      else
        KANSO_CUDA_TRY(ctx,
                       cudaMemsetAsync(y[0], 0, sizeof(float) * (size_t)M * rows[0], ctx->stream),
                       "gemv_q8_mma: clear y");
    }
  }
  // two CTAs per SM are resident; never more CTAs along x than row groups
  int gx = (2 * ctx->sm_count + ksplit - 1) / ksplit;
  if (gx > groups) gx = groups;
  if (gx < 1) gx = 1;
  const dim3 grid(gx, ksplit);
  if (act_mode == KANSO_ACT_Q8) return q8m_launch<Q8M_MODE_C>(ctx, a, grid);
  return M <= 4 ? q8m_launch<Q8M_MODE_A>(ctx, a, grid) : q8m_launch<Q8M_MODE_B>(ctx, a, grid);
}

}  // namespace kanso
