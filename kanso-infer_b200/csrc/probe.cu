// Measurement aid: the time a launch needs just to READ a buffer with 128-bit loads, no
// arithmetic. bench.py times it in the same captured sequence as the Q4_K GEMV over the same
// weight buffers: it is the floor that launch latency, drain between dependent kernels and the
// memory system put under any GEMV of that size, and the gap between the two is what the
// kernel's own instructions cost. No counterpart in the reference.
#include "ctx.h"

namespace kanso {
__global__ void __launch_bounds__(512) probe_read_kernel(const uint4* __restrict__ p, int64_t n,
                                                         uint32_t* __restrict__ sink) {
  pdl_launch_dependents();
  uint32_t acc = 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n; i += 4 * stride) {
    const uint4 a = __ldg(p + i), b = __ldg(p + i + stride), c = __ldg(p + i + 2 * stride),
                d = __ldg(p + i + 3 * stride);
    acc += a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w ^ c.x ^ c.y ^ c.z ^ c.w ^ d.x ^ d.y ^
           d.z ^ d.w;
  }
  for (; i < n; i += stride) {
    const uint4 a = __ldg(p + i);
    acc += a.x ^ a.y ^ a.z ^ a.w;
  }
  pdl_wait();
  if (acc == 0x12345678u) sink[0] = acc;  // keeps the loads alive; practically never taken
}
}  // namespace kanso

using namespace kanso;

extern "C" int32_t kanso_cuda_probe_read(kanso_cuda_ctx* ctx, const void* buf, size_t nbytes) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "probe_read: ctx is NULL");
  if (!buf || !aligned16(buf)) return fail(ctx, KANSO_ERR_SHAPE, "probe_read: buffer not 16-byte aligned");
  uint32_t* sink = reinterpret_cast<uint32_t*>(ctx_scratch(ctx, 256));
  if (!sink) return KANSO_ERR_DEVICE;
  KANSO_CUDA_TRY(ctx,
                 launch_dependent(ctx, probe_read_kernel, dim3(2 * ctx->sm_count), dim3(512), 0,
                                  reinterpret_cast<const uint4*>(buf), (int64_t)(nbytes / 16), sink),
                 "probe_read launch");
  return after_launch(ctx, "probe_read");
}
