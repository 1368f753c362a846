// Batched Q8_0 x Q8 GEMM on tcgen05 kind::i8: LinearWeight::forward for more than 8 activation
// rows in KANSO_ACT_Q8 mode, i.e. with the arithmetic the reference's production matmul uses on
// the CPU (tests/test_quantized_weights.rs:352-355): every activation row is quantised per 32
// values by quantize_row_q8_0 and each (weight block, activation block) pair contributes
// w.d * x.d * (f32)sum_i with an exact int32 sum_i (scalar_dot_q8_0_q8_0,
// src/quant/q8_0.rs:43-66), added over the blocks of a row in order
// (scalar_gemv_q8_0, src/quant/q8_0.rs:82-92).
//
// The int32 sums come from the tensor cores and are exact by construction; the scaling and the
// f32 additions are done with separately rounded multiplies and adds in block order, so with an
// unsplit K the result is bit-identical to the CPU statement, not merely close to it.
//
//   * weights: 2-D tensor-map boxes of 128 rows x 128 bytes of the block matrix land in a ring
//     of swizzled shared-memory slots (one elected thread; rows and bytes past the matrix are
//     zero-filled). The int8 values are NOT converted: 16 worker warps only move each block's 32
//     bytes (2-byte aligned in the stream) into the K-major core-matrix layout of the A operand
//     and note the block's f16 scale;
//   * activations: a pack kernel quantises them once (bit-exact quantize_row_q8_0) into the B
//     operand layout, one unit per block with its f32 scales behind it; a loader thread streams
//     the units of a stage with one bulk copy;
//   * one thread issues ONE tcgen05.mma.kind::i8 (M = 128 weight rows, N = 64 or 128 activation
//     rows, K = 32) per block, each into its own quarter of TMEM (four rotating accumulators,
//     never accumulated across blocks) and commits it to that accumulator's mbarrier;
//   * the worker warps drain an accumulator as soon as its block is done (tcgen05.ld), scale by
//     d_w * d_x and add into f32 registers (thread = weight row x a quarter of the activation
//     rows), while the next blocks' MMAs run.
// A stage is one box: the blocks whose last byte lies in it (3 or 4). Waits are bounded; a wait
// that runs out sets the status word, drains the CTA's copies, frees TMEM and returns.
#include <cuda.h>

#include "ctx.h"
#include "tc05.cuh"

namespace kanso {

int32_t tma_encode_weight_map(const void* w, int64_t row_bytes, int64_t N, CUtensorMap* map);

constexpr int I8_WORKERS = 512;            // 16 warps: realign + drain
constexpr int I8_THREADS = I8_WORKERS + 96;  // + MMA issuer, weight loader, activation loader
constexpr int I8_TILE_N = 128;
constexpr int I8_BOX = 128 * 128;
constexpr int I8_RAW_SLOTS = 5;
constexpr int I8_A_BLOCK = 128 * 32;                    // A tile of one block
constexpr int I8_A_STAGE = 4 * I8_A_BLOCK + 4 * 128 * 4;  // four blocks + their scales
constexpr int I8_B_SLOTS = 3;
constexpr int I8_NBUF = 4;  // TMEM accumulators in rotation

struct I8Args {
  float* y;
  const uint8_t* bp;  // per block: [2 k-chunks][Mt rows][16 int8] then Mt f32 scales
  int64_t N;
  int M, Mt;          // Mt = 64 or 128
  int nblocks;        // K / 32
  int boxes_total;
  int ksplit;
  int* status;
};

struct I8Zero {
  float* p;
  int64_t n;
};

// quantize_row_q8_0 (src/quant/q8_0.rs:13-32,43-48) of every activation row, written in the B
// operand layout. One warp per (row, block), lane = value.
__global__ void i8_pack_kernel(const float* __restrict__ x, uint8_t* __restrict__ bp, int M,
                               int Mt, int K, const I8Zero zero) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = gtid; j < zero.n; j += nthreads) zero.p[j] = 0.f;
  const int lane = threadIdx.x & 31;
  const int nb = K / 32;
  const int64_t total = (int64_t)nb * Mt;
  for (int64_t wi = gtid >> 5; wi < total; wi += nthreads >> 5) {
    const int m = (int)(wi % Mt), b = (int)(wi / Mt);
    uint8_t* unit = bp + (size_t)b * 36 * Mt;
    float d = 0.f;
    int8_t q = 0;
    if (m < M) {
      const float v = x[(int64_t)m * K + b * 32 + lane];
      float amax = fabsf(v);
#pragma unroll
      for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      d = __fdiv_rn(amax, 127.0f);
      const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
      float r = roundf(__fmul_rn(v, id));  // half away from zero, as f32::round
      r = fminf(fmaxf(r, -128.0f), 127.0f);
      q = (int8_t)r;
    }
    unit[(lane >> 4) * (Mt * 16) + m * 16 + (lane & 15)] = (uint8_t)q;
    if (lane == 0) reinterpret_cast<float*>(unit + 32 * Mt)[m] = d;
  }
}

__device__ __forceinline__ void i8_tma_load_2d(void* dst_smem, const CUtensorMap* map, int x, int y,
                                               uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%2, %3}], [%4];" ::"r"(smem_u32(dst_smem)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, 0, 0;\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc)
      : "memory");
}
// Instruction descriptor for kind::i8: s8 x s8 -> s32, both operands K-major.
__host__ __device__ inline uint32_t tc_idesc_i8(int m, int n) {
  uint32_t d = 0;
  d |= 2u << 4;                   // accumulator format s32
  d |= 1u << 7;                   // A format signed 8-bit
  d |= 1u << 10;                  // B format signed 8-bit
  d |= (uint32_t)(n >> 3) << 17;  // N / 8
  d |= (uint32_t)(m >> 4) << 24;  // M / 16
  return d;
}
__device__ __forceinline__ bool i8_wait_polite(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 21); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(20);
  }
  return false;
}
// Every lane polls, so that the warp stays converged through the wait (a poll loop entered by
// lane 0 alone made the compiler lay the code after it out twice: see gemm_tma.cu).
__device__ __forceinline__ bool i8_warp_wait(uint64_t* bar, uint32_t parity, int lane) {
  (void)lane;
  return __all_sync(0xFFFFFFFFu, i8_wait_polite(bar, parity)) != 0;
}
// First block whose last byte (stream offset 34 b + 33) lies in box s or later.
__device__ __forceinline__ int i8_first_block(int s) { return (128 * s) / 34; }

__global__ void __launch_bounds__(I8_THREADS, 1)
    gemm_i8_kernel(const __grid_constant__ CUtensorMap tmap, const I8Args a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t unit_bytes = 36u * (uint32_t)a.Mt;
  const uint32_t bslot_bytes = 4u * unit_bytes;
  uint8_t* Raw = smem;
  uint8_t* As = Raw + I8_RAW_SLOTS * I8_BOX;
  uint8_t* Bs = As + 2 * I8_A_STAGE;
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(Bs + I8_B_SLOTS * bslot_bytes);
  uint64_t* raw_empty = raw_full + I8_RAW_SLOTS;
  uint64_t* a_full = raw_empty + I8_RAW_SLOTS;
  uint64_t* a_empty = a_full + 2;
  uint64_t* b_full = a_empty + 2;
  uint64_t* b_empty = b_full + I8_B_SLOTS;
  uint64_t* d_full = b_empty + I8_B_SLOTS;
  uint64_t* d_empty = d_full + I8_NBUF;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_empty + I8_NBUF);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int n0 = (int)blockIdx.x * I8_TILE_N;
  const int b0 = (int)((int64_t)a.boxes_total * blockIdx.y / a.ksplit);
  const int b1 = (int)((int64_t)a.boxes_total * (blockIdx.y + 1) / a.ksplit);
  const int first = b0 > 0 ? b0 - 1 : 0;  // a block that ends in box b0 may start in the box before
  const uint32_t ncols = (uint32_t)(I8_NBUF * a.Mt);  // 256 or 512
  // blocks [blk_lo(s), blk_hi(s)) end in box s
  auto blk_lo = [&](int s) { return min(i8_first_block(s), a.nblocks); };

  if (warp == 0) tmem_alloc(tmem_slot, ncols);
  if (tid == 32) {
    for (int i = 0; i < I8_RAW_SLOTS; ++i) {
      mbar_init(&raw_full[i], 1);
      mbar_init(&raw_empty[i], I8_WORKERS / 32);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&a_full[i], I8_WORKERS / 32);
      mbar_init(&a_empty[i], 1 + I8_WORKERS / 32);  // the MMAs' commit + every worker warp
    }
    for (int i = 0; i < I8_B_SLOTS; ++i) {
      mbar_init(&b_full[i], 1);
      mbar_init(&b_empty[i], 1 + I8_WORKERS / 32);
    }
    for (int i = 0; i < I8_NBUF; ++i) {
      mbar_init(&d_full[i], 1);
      mbar_init(&d_empty[i], I8_WORKERS / 32);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  // accumulators of a worker thread: weight row 32 * (warp % 4) + lane, activation rows
  // [(warp / 4) * Mt / 4, +Mt / 4)
  float acc[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) acc[i] = 0.f;

  if (warp < I8_WORKERS / 32) {
    const int row = tid & 127, j = tid >> 7;  // realign task: block j of the stage, this row
    const int q = warp & 3, cg = warp >> 2;
    const int ncol = a.Mt >> 2;                // 16 or 32 activation rows per thread
    uint32_t g_drain = 0;                      // blocks drained so far (accumulator rotation)
    const int nst = b1 - b0;
    for (int it = 0, idx = (b0 > first ? 1 : 0); it <= nst; ++it, ++idx) {
      // ---- realign stage `it` (box b0 + it) ----
      if (it < nst) {
        const int box = b0 + it;
        if (it == 0 && b0 > first) {
          // the history box: wait for it once, nothing to process
          if (!i8_warp_wait(&raw_full[0], 0, lane)) *abort_flag = 1;
        }
        if (!i8_warp_wait(&raw_full[idx % I8_RAW_SLOTS], (uint32_t)(idx / I8_RAW_SLOTS) & 1u, lane))
          *abort_flag = 1;
        const int abuf = it & 1;
        if (!i8_warp_wait(&a_empty[abuf], (((uint32_t)it >> 1) & 1u) ^ 1u, lane)) *abort_flag = 1;
        if (*abort_flag) break;
        const int lo = blk_lo(box), hi = blk_lo(box + 1);
        if (lo + j < hi) {
          const uint32_t qo = 34u * (uint32_t)(lo + j) + 2u;  // stream offset of the 32 values
          const uint32_t c0 = qo >> 4, sh = qo & 15u;          // first chunk, offset in it (even)
          uint32_t w[12];
#pragma unroll
          for (int k = 0; k < 3; ++k) {
            // chunk c0 + k: in this box or the one before it (both in the ring)
            const uint32_t c = c0 + k, cbox = c >> 3;
            const int back = box - (int)cbox;  // 0 or 1 (a chunk past this box is never needed)
            uint4 v = make_uint4(0, 0, 0, 0);
            if (back >= 0 && back <= 1 && (k < 2 || sh != 0)) {
              const uint8_t* slot = Raw + ((idx - back) % I8_RAW_SLOTS) * I8_BOX;
              v = *reinterpret_cast<const uint4*>(slot + row * 128 + (((c & 7u) ^ (row & 7)) << 4));
            }
            w[4 * k] = v.x;
            w[4 * k + 1] = v.y;
            w[4 * k + 2] = v.z;
            w[4 * k + 3] = v.w;
          }
          // the block's scale: the two bytes before its values
          const uint32_t dofs = qo - 2u, dbox = dofs >> 7;
          const uint8_t* dslot = Raw + ((idx - (box - (int)dbox)) % I8_RAW_SLOTS) * I8_BOX;
          const __half dh = *reinterpret_cast<const __half*>(
              dslot + row * 128 + (((((dofs & 127u) >> 4)) ^ (row & 7)) << 4) + (dofs & 15u));
          uint32_t o[8];
          const uint32_t bits = (sh & 2u) * 8u;  // 0 or 16
          switch (sh >> 2) {
            case 0:
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] = __funnelshift_r(w[i], w[i + 1], bits);
              break;
            case 1:
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] = __funnelshift_r(w[i + 1], w[i + 2], bits);
              break;
            case 2:
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] = __funnelshift_r(w[i + 2], w[i + 3], bits);
              break;
            default:
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] = __funnelshift_r(w[i + 3], w[i + 4], bits);
              break;
          }
          uint8_t* Ab = As + abuf * I8_A_STAGE + j * I8_A_BLOCK + row * 16;
          *reinterpret_cast<uint4*>(Ab) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(Ab + 128 * 16) = make_uint4(o[4], o[5], o[6], o[7]);
          reinterpret_cast<float*>(As + abuf * I8_A_STAGE + 4 * I8_A_BLOCK)[j * 128 + row] =
              __half2float(dh);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&a_full[abuf]);
          if (idx >= 1) mbar_arrive(&raw_empty[(idx - 1) % I8_RAW_SLOTS]);
        }
      }
      // ---- drain stage `it - 1` ----
      if (it >= 1) {
        const int ds = it - 1, box = b0 + ds, abuf = ds & 1, bslot = ds % I8_B_SLOTS;
        const int lo = blk_lo(box), hi = blk_lo(box + 1);
        const float* dws = reinterpret_cast<const float*>(As + abuf * I8_A_STAGE + 4 * I8_A_BLOCK);
        for (int jb = 0; jb < hi - lo; ++jb, ++g_drain) {
          const uint32_t buf = g_drain & (I8_NBUF - 1);
          if (!i8_warp_wait(&d_full[buf], (g_drain / I8_NBUF) & 1u, lane)) *abort_flag = 1;
          if (*abort_flag) break;
          tc_fence_after();
          const float dw = dws[jb * 128 + q * 32 + lane];
          const float* dx = reinterpret_cast<const float*>(Bs + bslot * bslot_bytes +
                                                           jb * unit_bytes + 32 * a.Mt) +
                            cg * ncol;
          uint32_t r[16];
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * (uint32_t)a.Mt +
                                 (uint32_t)(cg * ncol);
          tmem_ld16(taddr, r);
#pragma unroll
          for (int i = 0; i < 16; ++i)
            acc[i] = __fadd_rn(acc[i], __fmul_rn(__fmul_rn(dw, dx[i]), (float)(int)r[i]));
          if (ncol == 32) {
            tmem_ld16(taddr + 16, r);
#pragma unroll
            for (int i = 0; i < 16; ++i)
              acc[16 + i] = __fadd_rn(acc[16 + i],
                                      __fmul_rn(__fmul_rn(dw, dx[16 + i]), (float)(int)r[i]));
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&d_empty[buf]);
        }
        if (*abort_flag) break;
        __syncwarp();
        if (lane == 0) {  // this warp is done with the stage's scales and activation scales
          mbar_arrive(&a_empty[abuf]);
          mbar_arrive(&b_empty[bslot]);
        }
      }
    }
  } else if (warp == I8_WORKERS / 32) {
    // ---- MMA issuer ----
    if (lane == 0) {
      const uint32_t idesc = tc_idesc_i8(I8_TILE_N, a.Mt);
      const uint64_t adesc0 = tc_smem_desc(smem_u32(As), 128 * 16, 128);
      const uint64_t bdesc0 = tc_smem_desc(smem_u32(Bs), (uint32_t)a.Mt * 16u, 128);
      uint32_t g = 0;
      bool ok = true;
      for (int s = 0; s < b1 - b0 && ok; ++s) {
        const int box = b0 + s, abuf = s & 1, bslot = s % I8_B_SLOTS;
        const int nblk = blk_lo(box + 1) - blk_lo(box);
        if (!mbar_wait_bounded(&a_full[abuf], ((uint32_t)s >> 1) & 1u) ||
            !mbar_wait_bounded(&b_full[bslot], ((uint32_t)s / I8_B_SLOTS) & 1u)) {
          ok = false;
          break;
        }
        tc_fence_after();
        for (int jb = 0; jb < nblk; ++jb, ++g) {
          const uint32_t buf = g & (I8_NBUF - 1);
          if (!mbar_wait_bounded(&d_empty[buf], ((g / I8_NBUF) & 1u) ^ 1u)) {
            ok = false;
            break;
          }
          tc_fence_after();
          tc_mma_i8(tmem_base + buf * (uint32_t)a.Mt,
                    adesc0 + (uint64_t)((uint32_t)(abuf * I8_A_STAGE + jb * I8_A_BLOCK) >> 4),
                    bdesc0 + (uint64_t)((bslot * bslot_bytes + jb * unit_bytes) >> 4), idesc);
          tc_commit(&d_full[buf]);
        }
        tc_commit(&a_empty[abuf]);
        tc_commit(&b_empty[bslot]);
      }
      if (!ok) *abort_flag = 1;
    }
    __syncwarp();
  } else if (warp == I8_WORKERS / 32 + 1) {
    // ---- weight loader ----
    if (lane == 0) {
      int issued = 0;
      for (int box = first, idx = 0; box < b1; ++box, ++idx) {
        const int slot = idx % I8_RAW_SLOTS;
        if (!i8_wait_polite(&raw_empty[slot], ((uint32_t)(idx / I8_RAW_SLOTS) & 1u) ^ 1u) ||
            *abort_flag) {
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&raw_full[slot], I8_BOX);
        i8_tma_load_2d(Raw + slot * I8_BOX, &tmap, box * 128, n0, &raw_full[slot]);
        issued = idx + 1;
      }
      for (int idx = max(0, issued - I8_RAW_SLOTS); idx < issued; ++idx)
        i8_wait_polite(&raw_full[idx % I8_RAW_SLOTS], (uint32_t)(idx / I8_RAW_SLOTS) & 1u);
    }
    __syncwarp();
  } else {
    // ---- activation loader: the units of a stage's blocks are contiguous ----
    if (lane == 0) {
      pdl_wait();
      int issued = 0;
      for (int s = 0; s < b1 - b0; ++s) {
        const int box = b0 + s, slot = s % I8_B_SLOTS;
        const int lo = blk_lo(box), nblk = blk_lo(box + 1) - lo;
        if (!i8_wait_polite(&b_empty[slot], (((uint32_t)s / I8_B_SLOTS) & 1u) ^ 1u) || *abort_flag) {
          *abort_flag = 1;
          break;
        }
        if (nblk > 0) {
          mbar_arrive_expect_tx(&b_full[slot], (uint32_t)nblk * unit_bytes);
          bulk_g2s(Bs + slot * bslot_bytes, a.bp + (size_t)lo * unit_bytes,
                   (uint32_t)nblk * unit_bytes, &b_full[slot]);
        } else {
          mbar_arrive(&b_full[slot]);
        }
        issued = s + 1;
      }
      for (int s = max(0, issued - I8_B_SLOTS); s < issued; ++s)
        i8_wait_polite(&b_full[s % I8_B_SLOTS], ((uint32_t)s / I8_B_SLOTS) & 1u);
    }
    __syncwarp();
  }

  __syncthreads();
  int failed = __syncthreads_or(*abort_flag != 0) ? 1 : 0;
  pdl_wait();
  if (!failed && warp < I8_WORKERS / 32) {
    const int q = warp & 3, cg = warp >> 2, ncol = a.Mt >> 2;
    const int64_t n = (int64_t)n0 + q * 32 + lane;
    if (n < a.N) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int m = cg * ncol + i;
        if (i < ncol && m < a.M) {
          float* dst = a.y + (int64_t)m * a.N + n;
          if (a.ksplit == 1)
            *dst = acc[i];
          else
            atomicAdd(dst, acc[i]);
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

// y[M,N] = x[M,K] @ W^T in KANSO_ACT_Q8 arithmetic for 9..128 activation rows per pass. Sets
// *handled = false (and launches nothing) when the shape is outside this kernel's range (rows of
// the block matrix must start on 16-byte boundaries: K % 256 == 0).
int32_t i8_matmul(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y, int64_t M,
                  int64_t N, int64_t K, bool* handled) {
  *handled = false;
  if (M < 9 || M > 128 || N < 1 || K < 256 || K % 256 != 0 || !w || !x || !y) return KANSO_OK;
  const int64_t row_bytes = K / 32 * Q8_BYTES;
  if (!aligned16(w) || row_bytes > (1 << 28) || N > (1 << 30)) return KANSO_OK;
  CUtensorMap tmap;
  const int32_t es = tma_encode_weight_map(w, row_bytes, N, &tmap);
  if (es == KANSO_ERR_UNSUPPORTED) return KANSO_OK;  // no encoder on this driver
  if (es) return fail(ctx, KANSO_ERR_DEVICE, "gemm_i8: cuTensorMapEncodeTiled failed");
  const int Mt = M <= 64 ? 64 : 128;
  const int nblocks = (int)(K / 32);
  const int boxes_total = (int)((row_bytes + 127) / 128);
  const int tiles_n = (int)((N + I8_TILE_N - 1) / I8_TILE_N);
  int ksplit = 1;
  while (tiles_n * ksplit * 2 <= ctx->sm_count + ctx->sm_count / 4 &&
         boxes_total / (ksplit * 2) >= 4)
    ksplit *= 2;
  const size_t bp_bytes = (size_t)nblocks * 36 * Mt;
  uint8_t* scratch = (uint8_t*)ctx_scratch(ctx, bp_bytes + 256);
  if (!scratch) return KANSO_ERR_DEVICE;
  *handled = true;
  I8Zero zero = {nullptr, 0};
  if (ksplit > 1) {
    zero.p = y;
    zero.n = M * N;
  }
  int64_t pack_blocks = ((int64_t)nblocks * Mt * 32 + 255) / 256;
  if (pack_blocks > 8 * ctx->sm_count) pack_blocks = 8 * ctx->sm_count;
  cudaError_t le = launch_dependent(ctx, i8_pack_kernel, dim3((unsigned)pack_blocks), dim3(256), 0,
                                    x, scratch, (int)M, Mt, (int)K, zero);
  if (le != cudaSuccess) return cuda_fail(ctx, le, "gemm_i8 pack launch");
  int32_t st = after_launch(ctx, "gemm_i8 pack activations");
  if (st) return st;
  I8Args a;
  a.y = y;
  a.bp = scratch;
  a.N = N;
  a.M = (int)M;
  a.Mt = Mt;
  a.nblocks = nblocks;
  a.boxes_total = boxes_total;
  a.ksplit = ksplit;
  a.status = ctx->dev_status;
  const size_t smem = (size_t)I8_RAW_SLOTS * I8_BOX + 2 * I8_A_STAGE +
                      (size_t)I8_B_SLOTS * 4 * 36 * Mt + 256;
  static bool attr_set[16] = {};
  if (!attr_set[ctx->device & 15]) {
    KANSO_CUDA_TRY(ctx,
                   cudaFuncSetAttribute(gemm_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        ctx->smem_optin),
                   "gemm_i8: shared memory opt-in");
    attr_set[ctx->device & 15] = true;
  }
  le = launch_dependent(ctx, gemm_i8_kernel, dim3(tiles_n, ksplit), dim3(I8_THREADS), smem, tmap, a);
  if (le != cudaSuccess) return cuda_fail(ctx, le, "gemm_i8 launch");
  return after_launch(ctx, "gemm_i8");
}

}  // namespace kanso
