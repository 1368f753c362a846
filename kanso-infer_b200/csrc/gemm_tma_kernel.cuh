// Device side of the TMA-staged batched GEMM: constants, the launch arguments, the stream-order
// index functions shared with the activation pack kernel, the dequantising producers and the
// kernel itself. The description of the design is at the top of gemm_tma.cu. The kernel is
// instantiated once per weight format in a translation unit of its own (gemm_tma_q8_0.cu,
// gemm_tma_q4_k.cu): its switch over dequantising bodies is the longest compile of the library,
// and the two formats then build side by side.
#pragma once
#include <cuda.h>  // CUtensorMap and its enums only; the encoder is looked up through the runtime

#include <mutex>
#include <type_traits>

#include "ctx.h"
#include "tc05.cuh"

namespace kanso {

constexpr int TM_PRODUCERS = 512;              // 16 warps: dequantise, then run the epilogue
constexpr int TM_THREADS = 768;  // 24 warps: scheduler 0 holds the MMA issuer and the two loaders
constexpr int TM_TILE_N = 128;                 // weight rows per CTA = MMA M
constexpr int TM_BOX_W = 128;                  // bytes of a weight row per box (the swizzle span)
constexpr int TM_BOX = TM_TILE_N * TM_BOX_W;   // 16 KB per ring slot
constexpr int TM_RAW_SLOTS = 5;  // measured: 4..7 slots and 2 or 3 A stages all within 3 %
constexpr int TM_A_STAGES = 2;
constexpr int TM_A_STAGE = 32768;  // 16 k-chunks of 8 positions x 128 rows x 16 bytes
constexpr int TM_B_SLOTS = 4;
constexpr int TM_FMT_Q8_0 = 0;
constexpr int TM_FMT_Q4_K = 1;
constexpr int TM_MAX_M = 512;
#ifndef TM_POLL_NS
#define TM_POLL_NS 20
#endif

struct TmArgs {
  float* y;            // [M, N]
  const uint8_t* bp;   // packed activations: units of [2 k-chunks][Mt rows][8 f16]
  int64_t N;
  int M, Mt;           // Mt = M rounded up to 16
  int row_bytes;       // bytes of one weight row
  int boxes_total;     // ceil(row_bytes / 128)
  int ksplit;          // CTAs along the stream; > 1: partial sums are added into y with atomics
  int ub;              // activation units per ring slot (1, 2, 4 or 8)
  int* status;
};

// Result buffer the pack kernel clears on the way (a split launch adds into it).
struct TmZero {
  float* p;
  int64_t n;
};

// The k index a stream position stands for, or -1 where the byte is not a weight.
// Q8_0: chunk `gc` of the row stream, byte j of it.
__device__ __forceinline__ int tm_k_of_q8_0(int gc, int j) {
  const int o = 16 * gc + j;
  const int blk = o / 34, within = o - 34 * blk;
  return within >= 2 ? 32 * blk + within - 2 : -1;
}
// Q4_K: nibble chunk; hs = 0 low nibbles, 1 high nibbles; q = position 0..15 inside the k-step.
// Inside a 32-bit word the positions run over bytes 0, 2, 1, 3: that is how the masked half2
// pairs fall out of the word in the producer.
__device__ __forceinline__ int tm_k_of_q4_k(int gc, int hs, int q) {
  const int o = 16 * gc;
  const int sb = o / 144, rem = o - 144 * sb;
  if (rem == 0) return -1;  // header chunk
  const int i = (rem >> 4) - 1;
  const int r = q & 3;
  const int byte = 4 * (q >> 2) + (r == 0 ? 0 : r == 1 ? 2 : r == 2 ? 1 : 3);
  const int nb = 16 * i + byte;
  return 256 * sb + 64 * (nb >> 5) + (nb & 31) + 32 * hs;
}

// x f32 [M,K] -> f16 in stream order. One thread per (unit, k-chunk of 8, row): 16 bytes.

__device__ __forceinline__ void tma_load_2d(void* dst_smem, const CUtensorMap* map, int x, int y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%2, %3}], [%4];" ::"r"(smem_u32(dst_smem)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Address of 16-byte chunk `chunk` of row `row` inside a swizzled box.
__device__ __forceinline__ const uint8_t* tm_chunk(const uint8_t* slot, int row, int chunk) {
  return slot + row * TM_BOX_W + ((chunk ^ (row & 7)) << 4);
}

// Broadcasts the low (HI = 0) or high (HI = 1) 16 bits of a word into both halves.
template <int HI>
__device__ __forceinline__ __half2 tm_bcast_half(uint32_t w) {
  return u32_as_h2(__byte_perm(w, w, HI ? 0x3232 : 0x1010));
}

// Q8_0: 32 consecutive stream bytes of this thread's row (chunks 2c and 2c+1 of the box) -> two
// k-steps of 16 f16 values d*q in the A tile. W0 = offset of the first of those bytes inside its
// 34-byte block: even, 0..32, and a compile-time constant, because the 17 possible phases are
// dispatched by a switch in the caller: which byte pair holds a scale and which scale every other
// pair takes is then known to the compiler and costs no instruction. A pair that holds a scale's
// own bytes is converted like any other: its activation is zero in the packed stream, and the
// product of two finite f16 numbers with zero is zero.
//   W0 == 0 : pair 0 is the scale of the block the 15 pairs after it belong to;
//   W0 == 2 : all 16 pairs belong to the block whose scale sits 2 bytes before them;
//   W0 >= 4 : pairs [0, SB) belong to the block whose scale sits W0 bytes back, pair
//             SB = 17 - W0/2 is the next block's scale, the pairs after it are that block's.
// A scale that precedes the 32 bytes lies at most 32 bytes back: in this box (`cur`) or, for the
// first two chunks of a box, in the one before it (`prev`), which is still in the ring.
template <int W0>
__device__ __forceinline__ void tm_dequant_q8_0(const uint8_t* cur, const uint8_t* prev, int c,
                                                uint32_t row_off, uint32_t rsw, uint8_t* dst) {
  constexpr int SB = W0 == 0 ? 0 : 17 - W0 / 2;
  const uint8_t* rb = cur + row_off;
  const uint4 v0 = *reinterpret_cast<const uint4*>(rb + ((((uint32_t)(2 * c)) ^ rsw) << 4));
  const uint4 v1 = *reinterpret_cast<const uint4*>(rb + ((((uint32_t)(2 * c + 1)) ^ rsw) << 4));
  const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
  __half2 da, db;
  if (W0 == 0) {
    da = tm_bcast_half<0>(w[0]);
    db = da;
  } else {
    const uint32_t bo = (uint32_t)(32 * c - W0) & 127u;  // warp-uniform
    const uint8_t* src = (32 * c < W0 ? prev : cur) + row_off;
    const unsigned short bits =
        *reinterpret_cast<const unsigned short*>(src + ((((bo >> 4) ^ rsw) << 4) | (bo & 15u)));
    da = __half2half2(__ushort_as_half(bits));
    db = SB <= 15 ? tm_bcast_half<SB & 1>(w[(SB <= 15 ? SB : 0) >> 1]) : da;
  }
  const __half2 bias = __floats2half2_rn(1152.f, 1152.f);  // 1024 + 128, exact in f16
  uint32_t out[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t q = w[i] ^ 0x80808080u;
    // 0x6400 | byte = 1024 + (q + 128) as f16, exactly
    const __half2 q01 = __hsub2(u32_as_h2(__byte_perm(q, 0x64646464u, 0x4140)), bias);
    const __half2 q23 = __hsub2(u32_as_h2(__byte_perm(q, 0x64646464u, 0x4342)), bias);
    out[2 * i] = h2_as_u32(__hmul2(q01, (2 * i < SB) ? da : db));
    out[2 * i + 1] = h2_as_u32(__hmul2(q23, (2 * i + 1 < SB) ? da : db));
  }
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(dst + j * (TM_TILE_N * 16)) =
        make_uint4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
}

// Scale or minimum `j` (0..7) of a Q4_K header from the three words of its 12 packed bytes
// (get_scale_min_k4, src/quant/q4_k.rs:13-28); j is a compile-time constant.
template <int J, bool MIN>
__device__ __forceinline__ uint32_t tm_k4_field(uint32_t y, uint32_t z, uint32_t w) {
  if constexpr (J < 4) {
    return ((MIN ? z : y) >> (8 * J)) & 63u;
  } else {
    const uint32_t lo = (w >> (8 * (J - 4) + (MIN ? 4 : 0))) & 0xFu;
    const uint32_t hi = ((MIN ? z : y) >> (8 * (J - 4) + 6)) & 3u;
    return lo | (hi << 4);
  }
}

// Q4_K: this thread's nibble chunk -> two k-steps of 16 f16 values (low nibbles = sub-block 2g,
// high nibbles = sub-block 2g+1 of the chunk's 64-weight group). w = d1*(q-8) - (m1 - 8*d1) with
// d1 = d*sc, m1 = dmin*m (src/quant/q4_k.rs:30-55): centred on 8 so that the two f16 factors
// carry a small constant instead of one the size of the weight range. CM = the chunk's index
// inside its 144-byte super-block (1..8; 0 is the header chunk, which produces nothing), a
// compile-time constant dispatched by a switch in the caller: the group, its two scale fields
// and the header's distance are then fixed. The header lies CM chunks back: in this box or in
// the one before it.
template <int CM>
__device__ __forceinline__ void tm_dequant_q4_k(const uint8_t* cur, const uint8_t* prev, int cib,
                                                uint32_t row_off, uint32_t rsw, uint8_t* dst) {
  constexpr int G = (CM - 1) >> 1;  // 64-weight group; sub-blocks 2G (low) and 2G+1 (high)
  const uint4 qv = *reinterpret_cast<const uint4*>(cur + row_off + ((((uint32_t)cib) ^ rsw) << 4));
  const uint32_t hc = (uint32_t)(cib - CM) & 7u;  // warp-uniform
  const uint4 hdr = *reinterpret_cast<const uint4*>((cib < CM ? prev : cur) + row_off +
                                                    ((hc ^ rsw) << 4));
  const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
  const float d1l = d * (float)tm_k4_field<2 * G, false>(hdr.y, hdr.z, hdr.w);
  const float d1h = d * (float)tm_k4_field<2 * G + 1, false>(hdr.y, hdr.z, hdr.w);
  const float m1l = dmin * (float)tm_k4_field<2 * G, true>(hdr.y, hdr.z, hdr.w);
  const float m1h = dmin * (float)tm_k4_field<2 * G + 1, true>(hdr.y, hdr.z, hdr.w);
  const __half2 dl2 = __float2half2_rn(d1l), dh2 = __float2half2_rn(d1h);
  const __half2 cl2 = __float2half2_rn(8.0f * d1l - m1l), ch2 = __float2half2_rn(8.0f * d1h - m1h);
  // low nibble: 0x6400 | q = 1024 + q; high nibble left in place: 0x6400 | 16q = 1024 + 16q, and
  // (1024 + 16q) / 16 - 72 = q - 8 in one exact fused multiply-add
  const __half2 bias = __floats2half2_rn(1032.f, 1032.f);
  const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
  const __half2 m72 = __floats2half2_rn(-72.f, -72.f);
  const uint32_t w[4] = {qv.x, qv.y, qv.z, qv.w};
  uint32_t lo[8], hi[8];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    // pairs (byte 0, byte 2) and (byte 1, byte 3) of the word
    const uint32_t w8 = w[k] >> 8;
    const __half2 l0 = __hsub2(u32_as_h2((w[k] & 0x000F000Fu) | 0x64006400u), bias);
    const __half2 h0 = __hfma2(u32_as_h2((w[k] & 0x00F000F0u) | 0x64006400u), sixteenth, m72);
    const __half2 l1 = __hsub2(u32_as_h2((w8 & 0x000F000Fu) | 0x64006400u), bias);
    const __half2 h1 = __hfma2(u32_as_h2((w8 & 0x00F000F0u) | 0x64006400u), sixteenth, m72);
    lo[2 * k] = h2_as_u32(__hfma2(l0, dl2, cl2));
    lo[2 * k + 1] = h2_as_u32(__hfma2(l1, dl2, cl2));
    hi[2 * k] = h2_as_u32(__hfma2(h0, dh2, ch2));
    hi[2 * k + 1] = h2_as_u32(__hfma2(h1, dh2, ch2));
  }
  // k-steps 2c (low) and 2c+1 (high) of the stage
  *reinterpret_cast<uint4*>(dst) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  *reinterpret_cast<uint4*>(dst + TM_TILE_N * 16) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
  *reinterpret_cast<uint4*>(dst + 2 * TM_TILE_N * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
  *reinterpret_cast<uint4*>(dst + 3 * TM_TILE_N * 16) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
}

// Bounded wait for the roles that are NOT the MMA issuer: between polls the thread sleeps, so
// that its polling does not crowd the issuer's own barrier and tensor-core instructions out of
// the SM's shared-memory instruction queue.
__device__ __forceinline__ bool tm_wait_polite(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 21); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(TM_POLL_NS);
  }
  return false;
}
// The producers' form: every lane of the warp polls (one warp-wide instruction on one
// shared-memory word, as cheap as a single lane's) and the warp stays converged through the
// wait. With lane 0 alone in the poll loop the code that follows a wait was laid out once for
// lane 0 and once for the other 31 lanes, and the whole dequantising body ran twice per stage
// (79 us against 38 us for a 14336 x 4096 Q8_0 matrix at 32 rows). The abort word is only
// looked at while the barrier is not ready, and it is set here when the wait runs out, so that
// the CTA's other roles give up at their next poll.
__device__ __forceinline__ bool tm_warp_wait(uint64_t* bar, uint32_t parity, int lane,
                                             volatile uint32_t* abort_flag,
                                             uint64_t* bar2 = nullptr, uint32_t parity2 = 0) {
  (void)lane;
  bool ok = false, ok1 = false, ok2 = bar2 == nullptr;
  for (uint32_t i = 0; i < (1u << 21); ++i) {
    if (!ok1) ok1 = mbar_try_wait(bar, parity);
    if (!ok2) ok2 = mbar_try_wait(bar2, parity2);
    if (ok1 && ok2) {
      ok = true;
      break;
    }
    if (*abort_flag) break;
    __nanosleep(TM_POLL_NS);
  }
  ok = __all_sync(0xFFFFFFFFu, ok) != 0;
  if (!ok) *abort_flag = 1;
  return ok;
}

template <int FMT>
__global__ void __launch_bounds__(TM_THREADS, 1)
    gemm_tma_kernel(const __grid_constant__ CUtensorMap tmap, const TmArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int UPC = FMT == TM_FMT_Q8_0 ? 1 : 2;  // activation units (k-steps) per chunk
  // Chunks per A stage: both formats fill a 32 KB stage (Q8_0: a whole box, Q4_K: half a box).
  // Every hand-off between the roles costs a few hundred cycles, so stages are as large as the
  // shared memory allows.
  constexpr int CH = FMT == TM_FMT_Q8_0 ? 8 : 4;
  constexpr int SPB = 8 / CH;  // stages per box
  // Warp w runs on warp scheduler w % 4. Every instruction of the MMA issuer is on the CTA's
  // critical path, so scheduler 0 carries only that warp and the two loaders (one thread each,
  // mostly asleep on a barrier); the 16 dequantising warps sit on schedulers 1..3.
  const int pw = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // role: 0..15 producer, 16 first MMA issuer, 17 weight loader, 18 activation loader, 19 none,
  // 20 second MMA issuer
  int warp;
  if ((pw & 3) == 0)
    warp = (pw >> 2) < 3 ? 16 + (pw >> 2) : (pw >> 2) == 3 ? 20 : 19;
  else
    warp = (pw & 3) - 1 + 3 * (pw >> 2);
  if (warp >= 16 && warp != 20 && (pw & 3) != 0) warp = 19;
  const int tid = warp * 32 + lane;
  const uint32_t unit_bytes = 32u * (uint32_t)a.Mt;
  const uint32_t bslot_bytes = (uint32_t)a.ub * unit_bytes;
  uint8_t* Raw = smem;
  uint8_t* As = Raw + TM_RAW_SLOTS * TM_BOX;
  uint8_t* Bs = As + TM_A_STAGES * TM_A_STAGE;
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(Bs + TM_B_SLOTS * bslot_bytes);
  uint64_t* raw_empty = raw_full + TM_RAW_SLOTS;
  uint64_t* a_full = raw_empty + TM_RAW_SLOTS;
  uint64_t* a_empty = a_full + TM_A_STAGES;
  uint64_t* b_full = a_empty + TM_A_STAGES;
  uint64_t* b_empty = b_full + TM_B_SLOTS;
  uint64_t* acc_full = b_empty + TM_B_SLOTS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* issued_any = abort_flag + 1;  // [2]: did issuer i accumulate anything

  const int n0 = (int)blockIdx.x * TM_TILE_N;
  const int b0 = (int)((int64_t)a.boxes_total * blockIdx.y / a.ksplit);
  const int b1 = (int)((int64_t)a.boxes_total * (blockIdx.y + 1) / a.ksplit);
  // a chunk at the start of this CTA's range may need a scale or header from the box before it
  const int first = b0 > 0 ? b0 - 1 : 0;
  // Up to 128 activation rows: two issuing threads, each with its own accumulator (even and
  // odd stages), because a tcgen05.mma of few columns is bound by the issuing thread, not by the
  // tensor core (measured: 8 MMAs + commit cost one thread 873 cycles at N = 32 whether or not a
  // second thread issues beside it). The epilogue adds the two accumulators. With more rows a
  // stage takes all four activation slots, so both threads would use every slot in turn and the
  // second would have to wait for a slot's second filling without having seen its first (a
  // parity wait cannot express that); those sizes are bound by the tensor core anyway.
  const int nissue = a.Mt <= 128 ? 2 : 1;
  uint32_t acc_cols = 32;
  while (acc_cols < (uint32_t)a.Mt) acc_cols <<= 1;
  const uint32_t ncols = acc_cols * (uint32_t)nissue;  // <= 512

  if (pw == 0) tmem_alloc(tmem_slot, ncols);
  if (threadIdx.x == 32) {
    for (int i = 0; i < TM_RAW_SLOTS; ++i) {
      mbar_init(&raw_full[i], 1);
      mbar_init(&raw_empty[i], TM_PRODUCERS / 32);
    }
    for (int i = 0; i < TM_A_STAGES; ++i) {
      mbar_init(&a_full[i], TM_PRODUCERS / 32);
      mbar_init(&a_empty[i], 1);
    }
    for (int i = 0; i < TM_B_SLOTS; ++i) {
      mbar_init(&b_full[i], 1);
      mbar_init(&b_empty[i], 1);
    }
    mbar_init(acc_full, nissue);
    *abort_flag = 0;
    issued_any[0] = issued_any[1] = 0;
    mbar_fence_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // The weights never depend on the kernel before this one (the activation pack): their boxes
  // are requested at once; the activation loader waits for the pack.
  pdl_launch_dependents();

  if (warp < TM_PRODUCERS / 32) {
    const int row = tid & 127, c = tid >> 7;  // c: quarter of the stage's chunks, warp-uniform
    const uint32_t row_off = (uint32_t)row * TM_BOX_W, rsw = (uint32_t)row & 7u;
    int abuf = 0;
    uint32_t a_par = 1;  // parity that an unused a_empty barrier already satisfies
    int slot = 0, prev_slot = 0;
    uint32_t raw_par = 0;
    // Q8_0: phase of this thread's 32 bytes inside the 34-byte blocks, (128*box + 32*c) % 34 / 2;
    // Q4_K: index of this thread's chunk inside the 9-chunk super-blocks, (8*box + c) % 9
    uint32_t ph = FMT == TM_FMT_Q8_0 ? (uint32_t)((64 * (int64_t)first + 16 * c) % 17)
                                     : (uint32_t)((8 * (int64_t)first + c) % 9);
    for (int box = first; box < b1; ++box) {
      // a box that will be dequantised: its arrival and the A buffer of its first stage are
      // waited for in one poll loop (each wait costs a round trip even when it is complete)
      if (!tm_warp_wait(&raw_full[slot], raw_par, lane, abort_flag,
                        box >= b0 ? &a_empty[abuf] : nullptr, a_par))
        break;
      const uint8_t* cur = Raw + slot * TM_BOX;
      const uint8_t* prev = Raw + prev_slot * TM_BOX;
      if (box >= b0) {
#pragma unroll 1
        for (int st = 0; st < SPB; ++st) {
          if (st > 0 && !tm_warp_wait(&a_empty[abuf], a_par, lane, abort_flag)) break;
          uint8_t* dst = As + abuf * TM_A_STAGE + c * (4 * TM_TILE_N * 16) + row * 16;
          if (FMT == TM_FMT_Q8_0) {
            switch (ph) {
#define TM_Q8_CASE(P) \
  case P:             \
    tm_dequant_q8_0<2 * P>(cur, prev, c, row_off, rsw, dst); \
    break;
              TM_Q8_CASE(0) TM_Q8_CASE(1) TM_Q8_CASE(2) TM_Q8_CASE(3) TM_Q8_CASE(4) TM_Q8_CASE(5)
              TM_Q8_CASE(6) TM_Q8_CASE(7) TM_Q8_CASE(8) TM_Q8_CASE(9) TM_Q8_CASE(10)
              TM_Q8_CASE(11) TM_Q8_CASE(12) TM_Q8_CASE(13) TM_Q8_CASE(14) TM_Q8_CASE(15)
              TM_Q8_CASE(16)
#undef TM_Q8_CASE
              default:
                break;
            }
          } else {
            const int cib = st * CH + c;
            switch (ph) {
#define TM_Q4_CASE(P) \
  case P:             \
    tm_dequant_q4_k<P>(cur, prev, cib, row_off, rsw, dst); \
    break;
              TM_Q4_CASE(1) TM_Q4_CASE(2) TM_Q4_CASE(3) TM_Q4_CASE(4) TM_Q4_CASE(5) TM_Q4_CASE(6)
              TM_Q4_CASE(7) TM_Q4_CASE(8)
#undef TM_Q4_CASE
              default:  // 0: the header chunk; the MMA issuer skips its two k-steps
                break;
            }
            ph = ph >= 5u ? ph - 5u : ph + 4u;  // four chunks on, modulo 9
          }
          fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
          __syncwarp();
          if (lane == 0) mbar_arrive(&a_full[abuf]);
          if (++abuf == TM_A_STAGES) {
            abuf = 0;
            a_par ^= 1u;
          }
        }
      } else if (FMT == TM_FMT_Q4_K) {
        ph = ph == 0u ? 8u : ph - 1u;  // a box that is only read for its headers: eight chunks on
      }
      if (FMT == TM_FMT_Q8_0) ph = ph >= 4u ? ph - 4u : ph + 13u;  // 128 bytes on, modulo 34
      // the box before this one is no longer needed (scales and headers reach one box back)
      __syncwarp();
      if (box > first && lane == 0) mbar_arrive(&raw_empty[prev_slot]);
      prev_slot = slot;
      if (++slot == TM_RAW_SLOTS) {
        slot = 0;
        raw_par ^= 1u;
      }
    }
  } else if (warp == TM_PRODUCERS / 32 || warp == 20) {
    // ---- MMA issuers: one thread each, and every instruction they execute sits on the critical
    // path of the stages they own, so a stage is straight-line code per slot size with every
    // descriptor a constant offset from the stage's first. Issuer i owns the stages j = i,
    // i + nissue, ...: A buffer j % 2 and the TMEM columns [i * acc_cols, i * acc_cols + Mt).
    const int me = warp == 20 ? 1 : 0;
    if (lane == 0 && me < nissue) {
      const bool two = a.Mt > 256;  // a second chunk of columns 256.. (single issuer only)
      const uint32_t idesc0 = tc_idesc_f16(TM_TILE_N, two ? 256 : a.Mt);
      const uint32_t idesc1 = tc_idesc_f16(TM_TILE_N, two ? a.Mt - 256 : 16);
      const uint64_t adesc_buf0 = tc_smem_desc(smem_u32(As), TM_TILE_N * 16, 128);
      const uint64_t bdesc_base = tc_smem_desc(smem_u32(Bs), (uint32_t)a.Mt * 16u, 128);
      const uint32_t a_kstep = (2u * (TM_TILE_N * 16)) >> 4;  // descriptor units per k-step of A
      const uint32_t b_unit = unit_bytes >> 4, b_slot = bslot_bytes >> 4;
      const uint32_t ub = (uint32_t)a.ub, row_bytes = (uint32_t)a.row_bytes;
      const uint32_t adesc_hi = (uint32_t)(adesc_buf0 >> 32), bdesc_hi = (uint32_t)(bdesc_base >> 32);
      const uint32_t adesc_lo0 = (uint32_t)adesc_buf0, bdesc_lo0 = (uint32_t)bdesc_base;
      const uint32_t acc_tmem = tmem_base + (uint32_t)me * acc_cols;
      const uint32_t sps = 8u / ub;  // activation slots per stage (a stage is 8 k-steps)
      const int nstages = SPB * (b1 - b0);
      uint32_t acc = 0;
      bool ok = true;
      for (int j = me; j < nstages && ok; j += nissue) {
        const uint32_t abuf = (uint32_t)j % TM_A_STAGES;
        const uint32_t a_par = ((uint32_t)j / TM_A_STAGES) & 1u;
        const uint32_t l0 = (uint32_t)j * sps;  // first activation slot group of the stage
        // the activations of a stage arrive long before its weights are dequantised: their
        // barrier is looked at first, so that one fence covers both waits
        if (!mbar_wait_bounded(&b_full[l0 % TM_B_SLOTS], (l0 / TM_B_SLOTS) & 1u)) ok = false;
        if (!mbar_wait_bounded(&a_full[abuf], a_par)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t chunk0 = (uint32_t)b0 * 8u + (uint32_t)j * CH;  // first chunk of the stage
        const uint32_t o0 = chunk0 * 16u;
        // chunks that are not weights: a Q4_K header (one in nine), bytes past the row's end
        const uint32_t cm = FMT == TM_FMT_Q4_K ? chunk0 % 9u : 1u;
        const uint32_t hdr = FMT == TM_FMT_Q4_K ? (cm == 0u ? 0u : 9u - cm) : 99u;
        const uint32_t nvalid = o0 >= row_bytes ? 0u : min((uint32_t)CH, (row_bytes - o0 + 15u) >> 4);
        const uint32_t alo = adesc_lo0 + abuf * (TM_A_STAGE >> 4);
        auto run = [&](auto ub_tag) {
          constexpr int UB = decltype(ub_tag)::value;
#pragma unroll
          for (int g = 0; g < CH * UPC / UB; ++g) {
            const uint32_t l = l0 + (uint32_t)g, bslot = l % TM_B_SLOTS;
            if (g > 0) {
              if (!mbar_wait_bounded(&b_full[bslot], (l / TM_B_SLOTS) & 1u)) ok = false;
              tc_fence_after();
            }
            uint32_t blo = bdesc_lo0 + bslot * b_slot;
#pragma unroll
            for (int u = 0; u < UB; ++u) {
              const int ks = g * UB + u;
              const uint32_t c = (uint32_t)(ks / UPC);
              const bool skip = c == hdr || c >= nvalid;
              if (!skip && ok) {
                const uint64_t ad = tc_desc_join(alo + (uint32_t)ks * a_kstep, adesc_hi);
                const uint64_t bd = tc_desc_join(blo, bdesc_hi);
                tc_mma_f16(acc_tmem, ad, bd, idesc0, acc);
                if (UB == 1 && two)
                  tc_mma_f16(acc_tmem + 256u, ad, tc_desc_join(blo + 256u, bdesc_hi), idesc1, acc);
                acc = 1;
              }
              blo += b_unit;
            }
            tc_commit(&b_empty[bslot]);
          }
        };
        if (ub == 8u)
          run(std::integral_constant<int, 8>{});
        else if (ub == 4u)
          run(std::integral_constant<int, 4>{});
        else if (ub == 2u)
          run(std::integral_constant<int, 2>{});
        else
          run(std::integral_constant<int, 1>{});
        tc_commit(&a_empty[abuf]);
      }
      issued_any[me] = acc;
      if (ok)
        tc_commit(acc_full);
      else
        *abort_flag = 1;
    }
    __syncwarp();
  } else if (warp == TM_PRODUCERS / 32 + 1) {
    // ---- weight loader: one box per ring slot, as far ahead as the ring allows ----
    if (lane == 0) {
      int issued = 0;
      for (int box = first, idx = 0; box < b1; ++box, ++idx) {
        const int slot = idx % TM_RAW_SLOTS;
        if (!tm_wait_polite(&raw_empty[slot], ((uint32_t)(idx / TM_RAW_SLOTS) & 1u) ^ 1u) ||
            *abort_flag) {
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&raw_full[slot], TM_BOX);
        tma_load_2d(Raw + slot * TM_BOX, &tmap, box * TM_BOX_W, n0, &raw_full[slot]);
        issued = idx + 1;
      }
      // leave only when every copy this thread started has landed (bounded)
      for (int idx = max(0, issued - TM_RAW_SLOTS); idx < issued; ++idx)
        tm_wait_polite(&raw_full[idx % TM_RAW_SLOTS], (uint32_t)(idx / TM_RAW_SLOTS) & 1u);
    }
    __syncwarp();
  } else if (warp == TM_PRODUCERS / 32 + 2) {
    // ---- activation loader: ring slots of `ub` units, contiguous in the packed buffer ----
    if (lane == 0) {
      pdl_wait();  // the pack kernel has written the activations
      const uint32_t g0 = (uint32_t)b0 * 8u * UPC / (uint32_t)a.ub;
      const uint32_t g1 = (uint32_t)b1 * 8u * UPC / (uint32_t)a.ub;
      uint32_t issued = 0;
      for (uint32_t g = g0; g < g1; ++g) {
        const uint32_t l = g - g0, slot = l % TM_B_SLOTS;
        if (!tm_wait_polite(&b_empty[slot], ((l / TM_B_SLOTS) & 1u) ^ 1u) || *abort_flag) {
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&b_full[slot], bslot_bytes);
        bulk_g2s(Bs + slot * bslot_bytes, a.bp + (size_t)g * bslot_bytes, bslot_bytes,
                 &b_full[slot]);
        issued = l + 1;
      }
      for (uint32_t l = issued > TM_B_SLOTS ? issued - TM_B_SLOTS : 0; l < issued; ++l)
        tm_wait_polite(&b_full[l % TM_B_SLOTS], (l / TM_B_SLOTS) & 1u);
    }
    __syncwarp();
  }

  __syncthreads();
  int failed = *abort_flag != 0;
  if (!failed) failed = !tm_warp_wait(acc_full, 0, lane, abort_flag);
  failed = __syncthreads_or(failed) ? 1 : 0;
  tc_fence_after();
  pdl_wait();  // y (cleared by the pack kernel of a split launch) belongs to the kernel before
  if (!failed) {
    // every warp helps: lane = weight row inside the tile (a warp reaches the TMEM lanes of its
    // own quarter, warp % 4), TMEM column = activation row
    const int q = pw & 3;
    const int64_t n = (int64_t)n0 + q * 32 + lane;
    const bool any0 = issued_any[0] != 0, any1 = nissue == 2 && issued_any[1] != 0;
    for (int c16 = pw >> 2; c16 < a.Mt / 16; c16 += TM_THREADS / 128) {
      uint32_t r[16];
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) r[jj] = 0u;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c16 * 16);
      if (any0) tmem_ld16(taddr, r);
      if (any1) {  // the second issuer's accumulator: the odd stages
        uint32_t r1[16];
        tmem_ld16(taddr + acc_cols, r1);
#pragma unroll
        for (int jj = 0; jj < 16; ++jj)
          r[jj] = __float_as_uint(__uint_as_float(r[jj]) + __uint_as_float(r1[jj]));
      }
      if (n < a.N) {
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
          const int m = c16 * 16 + jj;
          if (m < a.M) {
            float* dst = a.y + (int64_t)m * a.N + n;
            if (a.ksplit == 1)
              *dst = __uint_as_float(r[jj]);
            else
              atomicAdd(dst, __uint_as_float(r[jj]));  // y was cleared by the pack kernel
          }
        }
      }
    }
  } else if (failed == 1 && threadIdx.x == 0) {
    atomicOr(a.status, DEV_WAIT_TIMEOUT);
  }
  tc_fence_before();
  __syncthreads();
  if (pw == 0) tmem_dealloc(tmem_base, ncols);
}

// Sets the kernel's shared-memory limit once per device and launches it after the activation
// pack (programmatic dependent launch where the context allows it).
template <int FMT>
static int32_t tm_launch(kanso_cuda_ctx* ctx, dim3 grid, size_t smem, const CUtensorMap& tmap,
                         const TmArgs& a) {
  static bool attr_set[16] = {};
  bool& done = attr_set[ctx->device & 15];
  if (!done) {
    KANSO_CUDA_TRY(ctx,
                   cudaFuncSetAttribute(gemm_tma_kernel<FMT>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        ctx->smem_optin),
                   "gemm_tma: shared memory opt-in");
    done = true;
  }
  const cudaError_t le =
      launch_dependent(ctx, gemm_tma_kernel<FMT>, grid, dim3(TM_THREADS), smem, tmap, a);
  if (le != cudaSuccess) return cuda_fail(ctx, le, "gemm_tma launch");
  return after_launch(ctx, "gemm_tma");
}

// One per format, each defined in its own translation unit.
int32_t tm_launch_q8_0(kanso_cuda_ctx* ctx, dim3 grid, size_t smem, const CUtensorMap& tmap,
                       const TmArgs& a);
int32_t tm_launch_q4_k(kanso_cuda_ctx* ctx, dim3 grid, size_t smem, const CUtensorMap& tmap,
                       const TmArgs& a);

}  // namespace kanso
