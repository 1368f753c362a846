// Q4_K decode GEMV (and few-row GEMM): scalar_gemv_q4_k (src/quant/q4_k.rs:69-93) with
// super-blocks streamed straight from HBM into registers.
//
// The work is HBM-bound byte work, but Q4_K carries a 6-bit scale and min per 32 weights,
// so the instruction count per byte decides whether the loads can run at memory speed.
// Design:
//   * one persistent CTA of 16 warps per SM owns a contiguous range of weight rows, cut
//     into groups of 8 rows; a work item is (row group, super-block) = 8 x 144 bytes. Items
//     are ordered super-block-major and each warp takes a contiguous share of them, so the
//     activation fragments of a super-block stay in registers over a run of items;
//   * every warp runs its own ring of three to five shared-memory slots filled with 16-byte
//     cp.async copies (8 rows x 9 pieces per item, whole sectors of each row), so
//     60-100 KB per SM are in flight without holding registers. Rows sit 160 bytes apart in a
//     slot, which keeps the 64-bit fragment loads of a warp free of bank conflicts;
//   * a lane (gid = lane / 4, t = lane % 4) works on row gid of the group: the 16-byte
//     header (shared by the four lanes of a row) and, for each of the four 64-weight
//     groups, 8 of its 32 nibble bytes;
//   * nibbles are never widened: low nibbles are masked in place, high nibbles are used
//     as 16*q (mask 0xF0, the factor is folded into the scale). The masked words are
//     exactly the A fragments of the int8 tensor-core instruction
//     mma.sync.m16n8k32.u8.s8: fragment rows 0-7 hold the eight rows for one sub-block,
//     rows 8-15 hold the SAME eight rows for the neighbouring sub-block, and the B
//     columns carry the matching activations, so one instruction yields 8 rows x 2
//     sub-blocks x 2 activation planes (x 2 activation rows). The instruction replaces
//     64 dp4a and the shuffle reduction; it is used as a wide dot-product unit, the
//     kernel stays a GEMV that reads every weight byte once;
//   * activations are staged once per CTA as two int8 planes, x ~= d*(hi + lo/254) with
//     one d per 256 values (max error d/508, ~3e-5 of the output scale), so the 6-bit
//     sub-block scales can be applied to the int32 sums with integer multiply-adds and
//     one float scale per super-block. The -dmin*m term uses exact f32 sums of x per
//     sub-block;
//   * per-row results of a CTA are accumulated in shared memory and written once.
#include "ctx.h"
#include "shard.cuh"

namespace kanso {

constexpr int Q4M_ROW_STRIDE = 160;    // bytes between the rows of an item in a slot
constexpr int Q4M_SLOT = 8 * Q4M_ROW_STRIDE;
constexpr int Q4M_PLANE_PAD = 32;  // plane stride K+32: the B loads of a warp hit distinct banks

constexpr int Q4M_MAX_OUT = 8;

struct Q4kArgs {
  const uint8_t* w;
  const float* x;
  float* y;
  // row-sharded use: the CTA's rows are also stored into these result buffers (this GPU's
  // and its peers'), at row y_row_offset + r of rows of length ldy
  float* y_out[Q4M_MAX_OUT];
  int n_out;
  int64_t y_row_offset;
  int64_t rows, ldx, ldy;
  int K, bpr, M;
  int max_rows_cta;
  // row groups per CTA: the first groups_rem CTAs take groups_quot + 1, the others groups_quot
  int groups_quot, groups_rem;
  // sharded layer (shard != 0): the rows go to the exchange buffer of the current step in every
  // rank's region, and the grid's last CTA signals the peers
  int shard;
  ShardSignal sig;
};

struct Q4kLayout {
  int off_dxs, off_sum, off_planes, off_yacc, off_ring, plane_stride, total;
};
__host__ __device__ inline Q4kLayout q4k_layout(int K, int M, int max_rows_cta, int nwarps,
                                                int depth) {
  Q4kLayout L;
  int off = 0;
  L.off_dxs = off;
  off += M * (K / 256) * 4;
  off = (off + 15) & ~15;
  L.off_sum = off;
  off += M * (K / 32) * 4;
  off = (off + 127) & ~127;
  L.off_planes = off;
  L.plane_stride = K + Q4M_PLANE_PAD;
  off += M * 2 * L.plane_stride;
  off = (off + 15) & ~15;
  L.off_yacc = off;  // per-(activation row, super-block, weight row) partial sums
  off += M * (K / 256) * max_rows_cta * 4;
  off = (off + 127) & ~127;
  L.off_ring = off;
  off += nwarps * depth * Q4M_SLOT;
  L.total = off;
  return L;
}

// Packed f32x2 arithmetic (two floats per 64-bit register, one instruction for both).
__device__ __forceinline__ uint64_t f2pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t f2fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f2add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// The lowest bytes of the four 32-bit halves of a and b, a's low half first.
__device__ __forceinline__ uint32_t low_bytes4(uint64_t a, uint64_t b) {
  const uint32_t p01 = __byte_perm((uint32_t)a, (uint32_t)(a >> 32), 0x0040);
  const uint32_t p23 = __byte_perm((uint32_t)b, (uint32_t)(b >> 32), 0x0040);
  return __byte_perm(p01, p23, 0x5410);
}

// The calling warp stages the activation planes of super-blocks [s_first, s_last] of every
// activation row: the ones its own work items use (a neighbouring warp may stage a shared
// boundary super-block too; both write the same bytes). Lane l owns values [8l, 8l+8) of a
// 256-value block. The loads of up to four blocks are issued before any is processed.
__device__ __forceinline__ void q4k_stage_activations(const Q4kArgs& a, const Q4kLayout& L,
                                                      uint8_t* smem, int s_first, int s_last) {
  const int lane = threadIdx.x & 31;
  const int nsb = a.K / 256;
  float* dxs = reinterpret_cast<float*>(smem + L.off_dxs);
  float* xsum = reinterpret_cast<float*>(smem + L.off_sum);
  const int ns = s_last - s_first + 1;
  const int total = ns * a.M;  // (activation row, super-block) pairs, row-major in m
  for (int base = 0; base < total; base += 4) {
    float4 v0[4], v1[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int b = min(base + j, total - 1);
      const int m = b / ns, sb = s_first + (b - m * ns);
      const float4* src =
          reinterpret_cast<const float4*>(a.x + (int64_t)m * a.ldx + (int64_t)sb * 256) + 2 * lane;
      v0[j] = __ldg(src);
      v1[j] = __ldg(src + 1);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (base + j >= total) break;
      const int b = base + j;
      const int m = b / ns, sb = s_first + (b - m * ns);
      const float4 u0 = v0[j], u1 = v1[j];
      float amax = fmaxf(fmaxf(fmaxf(fabsf(u0.x), fabsf(u0.y)), fmaxf(fabsf(u0.z), fabsf(u0.w))),
                         fmaxf(fmaxf(fabsf(u1.x), fabsf(u1.y)), fmaxf(fabsf(u1.z), fabsf(u1.w))));
      float sum = ((u0.x + u0.y) + (u0.z + u0.w)) + ((u1.x + u1.y) + (u1.z + u1.w));
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
#pragma unroll
      for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      const float d = amax * (1.0f / 127.0f);
      const float id = d != 0.0f ? 1.0f / d : 0.0f;
      const float il = 254.0f * id;
      // Rounding by the 1.5 * 2^23 trick: v + MAGIC has the integer nearest to v (ties to even)
      // in its low mantissa bits, two's complement, so the int8 byte is the lowest byte of the
      // float and no conversion instruction is needed. |x * id| <= 127 and
      // |residual * il| <= 127 by construction (up to an ulp that rounds away): no clamps.
      const float MAGIC = 12582912.0f;
      const uint64_t magic2 = f2pack(MAGIC, MAGIC), nmagic2 = f2pack(-MAGIC, -MAGIC);
      const uint64_t id2 = f2pack(id, id), il2 = f2pack(il, il), nd2 = f2pack(-d, -d);
      const uint64_t xv[4] = {f2pack(u0.x, u0.y), f2pack(u0.z, u0.w), f2pack(u1.x, u1.y),
                              f2pack(u1.z, u1.w)};
      uint64_t th[4], tl[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        th[k] = f2fma(xv[k], id2, magic2);                  // MAGIC + hi
        const uint64_t hf = f2add(th[k], nmagic2);          // hi as a float
        tl[k] = f2fma(f2fma(nd2, hf, xv[k]), il2, magic2);  // MAGIC + lo
      }
      uint8_t* p0 = smem + L.off_planes + (m * 2) * L.plane_stride + sb * 256 + 8 * lane;
      *reinterpret_cast<uint2*>(p0) =
          make_uint2(low_bytes4(th[0], th[1]), low_bytes4(th[2], th[3]));
      *reinterpret_cast<uint2*>(p0 + L.plane_stride) =
          make_uint2(low_bytes4(tl[0], tl[1]), low_bytes4(tl[2], tl[3]));
      if ((lane & 3) == 0) xsum[m * (a.K / 32) + sb * 8 + (lane >> 2)] = sum;
      // low-nibble sums enter with a factor 16 (see the kernel), hence 1/(254*16)
      if (lane == 0) dxs[m * nsb + sb] = d * (1.0f / (254.0f * 16.0f));
    }
  }
}

// c = A*B (the accumulator input is zero)
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  // the zero goes in as one constant operand: no accumulator registers to clear per call
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// MSETS = number of activation-row pairs (M <= 2*MSETS).
//
// Fragment roles. A rows 0-7: the eight weight rows for sub-block family 0 (the 64-weight
// groups 0 and 2), A rows 8-15: the same eight rows for family 1 (groups 1 and 3).
// B column n: activation row (n >> 2) of the pair, plane (n >> 1) & 1 (hi / lo), family n & 1.
// Lane (gid, t) therefore finds in c[0] (A row gid, column 2t) the family-0 sum and in c[3]
// (A row gid+8, column 2t+1) the family-1 sum of weight row gid, for activation row t >> 1 and
// plane t & 1; c[1] and c[2] pair a family with the other family's activations and are unused.
template <int MSETS, int Q4M_WARPS, int Q4M_DEPTH>
__global__ void __launch_bounds__(Q4M_WARPS * 32, 1024 / (Q4M_WARPS * 32)) gemv_q4k_mma_kernel(const Q4kArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  // the shuffle makes the warp index provably warp-uniform, so that the loop bounds derived
  // from it stay in uniform registers and branches on them need no reconvergence barrier
  const int warp = __shfl_sync(0xFFFFFFFFu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int gid = lane >> 2, t = lane & 3;
  const Q4kLayout L = q4k_layout(a.K, a.M, a.max_rows_cta, Q4M_WARPS, Q4M_DEPTH);
  const int M = a.M, bpr = a.bpr, max_rows = a.max_rows_cta;

  // rows are dealt out in groups of 8 (the host guarantees rows % 8 == 0)
  const int cta = (int)blockIdx.x;
  const int g_begin = a.groups_quot * cta + min(cta, a.groups_rem);
  const int ngroups = a.groups_quot + (cta < a.groups_rem ? 1 : 0);
  const int nrows = ngroups * 8;
  const int64_t rb = (int64_t)g_begin * 8;
  const uint32_t row_bytes = (uint32_t)bpr * Q4K_BYTES;
  const uint8_t* wbase = a.w + rb * (int64_t)row_bytes;

  // Items in super-block-major order, i = S * ngroups + g; each warp owns a contiguous range,
  // so its activation fragments change only when S does.
  const int n_items = ngroups * bpr;
  // (n_items < 2^24: at most 227 KB / 4 bytes of per-item partial sums fit in shared memory)
  const int i0 = (int)((uint32_t)n_items * (uint32_t)warp / (uint32_t)Q4M_WARPS);
  const int i1 = (int)((uint32_t)n_items * (uint32_t)(warp + 1) / (uint32_t)Q4M_WARPS);

  // copy roles: lane (gid, t) copies pieces t, t+4 and (t == 0) 8 of row gid: 64 contiguous
  // bytes per row and instruction, at constant offsets from one pointer per lane
  const uint32_t lane_g = (uint32_t)gid * row_bytes + 16u * t;
  const uint32_t lane_s = (uint32_t)gid * Q4M_ROW_STRIDE + 16u * t;
  const bool third = t == 0;
  const uint32_t ring0 = smem_u32(smem + L.off_ring + warp * (Q4M_DEPTH * Q4M_SLOT));
  const uint32_t ring_end = ring0 + Q4M_DEPTH * Q4M_SLOT;
  const uint32_t gstep = 8u * row_bytes;
  int lS = ngroups > 0 ? i0 / ngroups : 0, lg = i0 - lS * ngroups, li = i0;
  const uint8_t* lsrc = wbase + (uint32_t)lS * Q4K_BYTES + (uint32_t)lg * gstep + lane_g;
  uint32_t ldst = ring0;  // slot base (warp-uniform)
  auto issue = [&]() {
    if (li < i1) {
      asm volatile(
          "cp.async.cg.shared.global [%0], [%1], 16;\n"
          "cp.async.cg.shared.global [%0+64], [%1+64], 16;\n" ::"r"(ldst + lane_s),
          "l"(lsrc)
          : "memory");
      if (third)
        asm volatile("cp.async.cg.shared.global [%0+128], [%1+128], 16;\n" ::"r"(ldst + lane_s),
                     "l"(lsrc)
                     : "memory");
      ++li;
      if (++lg == ngroups) {
        lg = 0;
        ++lS;
        lsrc = wbase + (uint32_t)lS * Q4K_BYTES + lane_g;
      } else {
        lsrc += gstep;
      }
    }
    cp_async_commit();  // always, so that the group count per slot stays uniform
    ldst += Q4M_SLOT;
    if (ldst == ring_end) ldst = ring0;
  };
#pragma unroll
  for (int k = 0; k < Q4M_DEPTH; ++k) issue();

  // Programmatic dependent launch: the weight copies above do not depend on the kernel
  // before this one in the stream (weights are read-only), everything below may. When the
  // launch did not ask for overlap both instructions are no-ops.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  float* ypart = reinterpret_cast<float*>(smem + L.off_yacc);  // [M][bpr][max_rows]
  // each warp stages only the super-blocks of the activations that its own items read
  if (i0 < i1) q4k_stage_activations(a, L, smem, i0 / ngroups, (i1 - 1) / ngroups);
  __syncwarp();

  const float* dxs = reinterpret_cast<const float*>(smem + L.off_dxs);
  const float* xsum = reinterpret_cast<const float*>(smem + L.off_sum);
  const int nsb = a.K / 256, nblk = a.K / 32;
  const int bn_m = gid >> 2, bn_plane = (gid >> 1) & 1, bn_fam = gid & 1;  // B-fragment role
  const int out_m = t >> 1, plane = t & 1;                                  // result role
  const float plane_w = plane ? 1.0f : 254.0f;

  // per-super-block state, reloaded when S changes
  uint2 bf[MSETS][4];   // B fragments: [pair][low0, high0, low1, high1]
  float4 xs[MSETS];     // f32 sums of x over this lane's four sub-blocks
  float dx[MSETS];
  bool ok[MSETS];       // does this lane publish a result for activation-row pair ms?
#pragma unroll
  for (int ms = 0; ms < MSETS; ++ms) ok[ms] = plane == 0 && 2 * ms + out_m < M;
  auto load_x = [&](int S) {
#pragma unroll
    for (int ms = 0; ms < MSETS; ++ms) {
      const int m_b = min(2 * ms + bn_m, M - 1);  // unused columns repeat a valid row
      const uint8_t* xb = smem + L.off_planes + (m_b * 2 + bn_plane) * L.plane_stride + S * 256 +
                          64 * bn_fam + 8 * t;
      bf[ms][0] = *reinterpret_cast<const uint2*>(xb);
      bf[ms][1] = *reinterpret_cast<const uint2*>(xb + 32);
      bf[ms][2] = *reinterpret_cast<const uint2*>(xb + 128);
      bf[ms][3] = *reinterpret_cast<const uint2*>(xb + 160);
      const int m_o = min(2 * ms + out_m, M - 1);
      xs[ms] = *reinterpret_cast<const float4*>(xsum + m_o * nblk + S * 8 + 4 * plane);
      dx[ms] = dxs[m_o * nsb + S];
    }
  };

  // compute side
  int gS = ngroups > 0 ? i0 / ngroups : 0, gg = i0 - gS * ngroups;
  if (i0 < i1) load_x(gS);
  uint32_t csrc = ring0 + (uint32_t)gid * Q4M_ROW_STRIDE + 8u * t;  // this lane's row in the slot
  const uint32_t csrc_end = csrc + Q4M_DEPTH * Q4M_SLOT;
  // shared-memory address of ypart[out_m][S][row gid of group gg]; every (S, row) cell is
  // written by exactly one item, so plain stores suffice
  const uint32_t ypart_lane = smem_u32(ypart) + 4u * (uint32_t)(out_m * bpr * max_rows + gid);
  uint32_t yaddr = ypart_lane + 4u * (uint32_t)(gS * max_rows + gg * 8);
  const uint32_t LO = 0x0F0F0F0Fu, HI = 0xF0F0F0F0u;
  for (int i = i0; i < i1; ++i) {
    cp_async_wait<Q4M_DEPTH - 1>();  // the oldest copy group (this slot) has landed
    __syncwarp();
    uint4 hdr;
    uint2 q0, q1, q2, q3;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(hdr.x), "=r"(hdr.y), "=r"(hdr.z), "=r"(hdr.w)
                 : "r"(csrc - 8u * t));
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+16];" : "=r"(q0.x), "=r"(q0.y) : "r"(csrc));
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+48];" : "=r"(q1.x), "=r"(q1.y) : "r"(csrc));
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+80];" : "=r"(q2.x), "=r"(q2.y) : "r"(csrc));
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+112];" : "=r"(q3.x), "=r"(q3.y) : "r"(csrc));
    const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
    uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
    unpack_scales_k4(hdr.y, hdr.z, hdr.w, sc_lo, sc_hi, mn_lo, mn_hi);
    // sub-block s = 2*group + nibble; family 0 = groups 0,2, family 1 = groups 1,3
    const int s0 = (int)__byte_perm(sc_lo, 0, 0x4440), s1 = (int)__byte_perm(sc_lo, 0, 0x4441);
    const int s2 = (int)__byte_perm(sc_lo, 0, 0x4442), s3 = (int)__byte_perm(sc_lo, 0, 0x4443);
    const int s4 = (int)__byte_perm(sc_hi, 0, 0x4440), s5 = (int)__byte_perm(sc_hi, 0, 0x4441);
    const int s6 = (int)__byte_perm(sc_hi, 0, 0x4442), s7 = (int)__byte_perm(sc_hi, 0, 0x4443);
    const uint32_t mw = plane ? mn_hi : mn_lo;  // this lane sums the mins of sub-blocks 4*plane..
#pragma unroll
    for (int ms = 0; ms < MSETS; ++ms) {
      int c[4];
      // groups 0 (family 0) and 1 (family 1): sub-blocks 0,2 (low nibbles) and 1,3 (high)
      mma_u8s8(c, q0.x & LO, q1.x & LO, q0.y & LO, q1.y & LO, bf[ms][0].x, bf[ms][0].y);
      int accL = s0 * c[0] + s2 * c[3];
      mma_u8s8(c, q0.x & HI, q1.x & HI, q0.y & HI, q1.y & HI, bf[ms][1].x, bf[ms][1].y);
      int accH = s1 * c[0] + s3 * c[3];
      // groups 2 and 3: sub-blocks 4,6 and 5,7
      mma_u8s8(c, q2.x & LO, q3.x & LO, q2.y & LO, q3.y & LO, bf[ms][2].x, bf[ms][2].y);
      accL += s4 * c[0] + s6 * c[3];
      mma_u8s8(c, q2.x & HI, q3.x & HI, q2.y & HI, q3.y & HI, bf[ms][3].x, bf[ms][3].y);
      accH += s5 * c[0] + s7 * c[3];
      // low-nibble sums count 16x so that they add to the 16*q high-nibble sums
      const float f = plane_w * (float)(accL * 16 + accH);
      float mins = (float)(mw & 0xFF) * xs[ms].x;
      mins = fmaf((float)((mw >> 8) & 0xFF), xs[ms].y, mins);
      mins = fmaf((float)((mw >> 16) & 0xFF), xs[ms].z, mins);
      mins = fmaf((float)(mw >> 24), xs[ms].w, mins);
      float v = fmaf(d * dx[ms], f, -dmin * mins);
      v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);  // hi plane + lo plane (and both halves of mins)
      if (ok[ms])
        asm volatile("st.shared.f32 [%0], %1;" ::"r"(yaddr + 8u * (uint32_t)(ms * bpr * max_rows)),
                     "f"(v)
                     : "memory");
    }
    yaddr += 32u;
    if (++gg == ngroups) {
      gg = 0;
      ++gS;
      yaddr = ypart_lane + 4u * (uint32_t)(gS * max_rows);
      if (i + 1 < i1) load_x(gS);
    }
    csrc += Q4M_SLOT;
    if (csrc == csrc_end) csrc -= Q4M_DEPTH * Q4M_SLOT;
    __syncwarp();  // every lane is done reading the slot before it is refilled
    issue();
  }
  cp_async_wait<0>();
  __syncthreads();
  for (int i = threadIdx.x; i < M * nrows; i += blockDim.x) {
    const int m = i / nrows, r = i - m * nrows;
    const float* p = ypart + (size_t)m * bpr * max_rows + r;
    float acc = 0.f;
    for (int S = 0; S < bpr; ++S) acc += p[S * max_rows];
    if (a.n_out == 0) {
      a.y[(int64_t)m * a.ldy + rb + r] = acc;  // sharded layer: y is the local staging slice
    } else {
      for (int o = 0; o < a.n_out; ++o)  // plain stores, also into peers' memory over NVLink
        a.y_out[o][(int64_t)m * a.ldy + a.y_row_offset + rb + r] = acc;
    }
  }
  if (a.shard) {
    // Sharded layer: the CTA that draws the last ticket publishes the whole slice to the peers
    // and, for a K shard, waits for theirs and adds them up (shard_tail); all others are done.
    // (the flag lives in dynamic shared memory that the main loop no longer needs: a static
    // variable would come off the opt-in maximum the launch asks for)
    volatile unsigned int* s_last = reinterpret_cast<volatile unsigned int*>(smem + L.off_dxs);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int drawn = atomicAdd(a.sig.ticket, 1u);
      *s_last = drawn == gridDim.x - 1;
      if (*s_last) *a.sig.ticket = 0;  // every CTA has drawn: ready for the next launch
    }
    __syncthreads();
    if (!*s_last) return;
    __threadfence();
    shard_tail(a.sig);
  }
}

template <int MSETS, int NW, int DEPTH>
static int32_t launch_q4k_mma(kanso_cuda_ctx* ctx, const Q4kArgs& a, int grid, int smem) {
  auto kern = gemv_q4k_mma_kernel<MSETS, NW, DEPTH>;
  static int smem_set[16] = {0};
  if (smem > smem_set[ctx->device & 15]) {
    KANSO_CUDA_TRY(ctx,
                   cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        ctx->smem_optin),
                   "gemv_q4k: shared memory opt-in");
    smem_set[ctx->device & 15] = ctx->smem_optin;
  }
  prefer_max_shared(ctx, reinterpret_cast<const void*>(kern));
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(grid);
  lc.blockDim = dim3(NW * 32);
  lc.dynamicSmemBytes = smem;
  lc.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = ctx->overlap_weight_prefetch ? 1 : 0;
  lc.attrs = attr;
  lc.numAttrs = 1;
  KANSO_CUDA_TRY(ctx, cudaLaunchKernelEx(&lc, kern, a), "gemv_q4k launch");
  return after_launch(ctx, "gemv_q4k_mma");
}

template <int NW, int DEPTH>
static int32_t dispatch_q4k_msets(kanso_cuda_ctx* ctx, const Q4kArgs& a, int grid, int smem) {
  switch ((a.M + 1) / 2) {
    case 1: return launch_q4k_mma<1, NW, DEPTH>(ctx, a, grid, smem);
    case 2: return launch_q4k_mma<2, NW, DEPTH>(ctx, a, grid, smem);
    case 3: return launch_q4k_mma<3, NW, DEPTH>(ctx, a, grid, smem);
    default: return launch_q4k_mma<4, NW, DEPTH>(ctx, a, grid, smem);
  }
}

constexpr int Q4M_NW = 16;  // warps per CTA

// Sets *handled when this kernel took the call; leaves it false when the shape is outside
// its range (the caller then uses the general streaming kernel).
int32_t q4k_direct_matmul_out(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                              int64_t M, int64_t N, int64_t K, bool* handled, float* const* y_out,
                              int n_out, int64_t ld_out, int64_t row_offset);

int32_t q4k_direct_matmul(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y, int64_t M,
                          int64_t N, int64_t K, bool* handled) {
  return q4k_direct_matmul_out(ctx, w, x, y, M, N, K, handled, nullptr, 0, N, 0);
}

static int32_t q4k_direct_matmul_impl(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                                      int64_t M, int64_t N, int64_t K, bool* handled,
                                      float* const* y_out, int n_out, int64_t ld_out,
                                      int64_t row_offset, const ShardSignal* sig);

int32_t q4k_direct_matmul_out(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                              int64_t M, int64_t N, int64_t K, bool* handled, float* const* y_out,
                              int n_out, int64_t ld_out, int64_t row_offset) {
  return q4k_direct_matmul_impl(ctx, w, x, y, M, N, K, handled, y_out, n_out, ld_out, row_offset,
                                nullptr);
}

// The sharded form: this pass's rows go to `stage` (this rank's memory); the grid's last CTA runs
// shard_tail (publish to the peers, signal, and for a K shard wait and sum) when sig.signal is
// set, i.e. on the last pass.
int32_t q4k_direct_matmul_shard(kanso_cuda_ctx* ctx, const void* w, const float* x, float* stage,
                                int64_t M, int64_t N, int64_t K, bool* handled,
                                const ShardSignal& sig) {
  return q4k_direct_matmul_impl(ctx, w, x, stage, M, N, K, handled, nullptr, 0, N, 0, &sig);
}

static int32_t q4k_direct_matmul_impl(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                                      int64_t M, int64_t N, int64_t K, bool* handled,
                                      float* const* y_out, int n_out, int64_t ld_out,
                                      int64_t row_offset, const ShardSignal* sig) {
  *handled = false;
  if (n_out < 0 || n_out > Q4M_MAX_OUT) return KANSO_OK;
  if (K % 256 != 0 || M < 1 || M > 8 || N < 8 || N % 8 != 0) return KANSO_OK;
  int grid = ctx->sm_count;
  if (N / 8 < grid) grid = (int)(N / 8);  // every CTA gets at least one group of 8 rows
  const int max_rows_cta = (int)(((N / 8 + grid - 1) / grid) * 8);
  // The deepest ring (5..3 slots per warp) with which two CTAs fit on an SM: under
  // dependent-launch overlap the next GEMV's CTA then moves in beside this one and has its
  // ring filled when this kernel ends, which is worth more than the fifth slot. Shapes whose
  // activation planes leave no room for two CTAs take four slots, or three if four do not
  // fit at all.
  int depth = 0;
  auto total = [&](int d) { return q4k_layout((int)K, (int)M, max_rows_cta, Q4M_NW, d).total; };
  for (int d = 5; d >= 3 && !depth; --d)
    if (2 * (total(d) + 1024) <= ctx->smem_per_sm) depth = d;  // 1 KB per CTA is reserved
  if (!depth) depth = total(4) <= ctx->smem_optin ? 4 : 3;
  Q4kLayout L = q4k_layout((int)K, (int)M, max_rows_cta, Q4M_NW, depth);
  if (L.total > ctx->smem_optin) return KANSO_OK;
  Q4kArgs a;
  a.w = (const uint8_t*)w;
  a.x = x;
  a.y = y;
  a.rows = N;
  a.ldx = K;
  a.ldy = n_out ? ld_out : N;
  a.shard = sig ? 1 : 0;
  a.sig = sig ? *sig : ShardSignal{};
  a.n_out = n_out;
  a.y_row_offset = row_offset;
  for (int o = 0; o < Q4M_MAX_OUT; ++o) a.y_out[o] = o < n_out ? y_out[o] : nullptr;
  a.K = (int)K;
  a.bpr = (int)(K / 256);
  a.M = (int)M;
  a.max_rows_cta = max_rows_cta;
  a.groups_quot = (int)((N / 8) / grid);
  a.groups_rem = (int)((N / 8) % grid);
  *handled = true;
  switch (depth) {
    case 5: return dispatch_q4k_msets<Q4M_NW, 5>(ctx, a, grid, L.total);
    case 4: return dispatch_q4k_msets<Q4M_NW, 4>(ctx, a, grid, L.total);
    default: return dispatch_q4k_msets<Q4M_NW, 3>(ctx, a, grid, L.total);
  }
}

}  // namespace kanso
