// Shared device/host helpers for the kanso sm_100a kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/kanso_cuda.h"

namespace kanso {

// ---- status word the kernels write instead of trapping ----
// Device code ORs one of these into ctx->dev_status; the host reads it at sync.
enum DevStatus : int {
  DEV_OK = 0,
  DEV_WAIT_TIMEOUT = 1,  // a bounded mbarrier / flag wait ran out
  DEV_BAD_INDEX = 2,     // a block-table entry, slot or token id was out of range
};

struct Ctx;  // defined in ctx.cu / ctx.h

constexpr int Q8_BYTES = KANSO_Q8_0_BYTES;
constexpr int Q4K_BYTES = KANSO_Q4_K_BYTES;

__device__ __forceinline__ float f16_bits_to_f32(uint32_t h16) {
  return __half2float(__ushort_as_half((unsigned short)(h16 & 0xFFFFu)));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier + bulk-copy wrappers (sm_90+/sm_100a PTX) ----
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls and returns false. Every caller then
// records DEV_WAIT_TIMEOUT and leaves the kernel; nothing spins for ever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  uint32_t limit = (1u << 22)) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// Global -> shared bulk async copy (the TMA engine's untiled form). src, dst and
// bytes must be multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// Programmatic dependent launch: let the next kernel of the stream start launching, and wait
// until the kernel before this one has completed and its writes are visible. Both are no-ops
// for a launch without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ int dp4a_ss(int a, int b, int c) { return __dp4a(a, b, c); }
// unsigned bytes of a times signed bytes of b
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// get_scale_min_k4 for all eight sub-blocks at once (src/quant/q4_k.rs:16-26).
// q0,q1,q2 = the 12 packed bytes as three little-endian words. Outputs hold one
// 6-bit value per byte: sc_lo = scales 0..3, sc_hi = scales 4..7, likewise mins.
__device__ __forceinline__ void unpack_scales_k4(uint32_t q0, uint32_t q1, uint32_t q2,
                                                 uint32_t& sc_lo, uint32_t& sc_hi,
                                                 uint32_t& mn_lo, uint32_t& mn_hi) {
  sc_lo = q0 & 0x3F3F3F3Fu;
  mn_lo = q1 & 0x3F3F3F3Fu;
  sc_hi = (q2 & 0x0F0F0F0Fu) | ((q0 >> 2) & 0x30303030u);
  mn_hi = ((q2 >> 4) & 0x0F0F0F0Fu) | ((q1 >> 2) & 0x30303030u);
}

}  // namespace kanso
