// Internal definition of the context and of the handles behind the C ABI.
#pragma once
#include <cstdarg>
#include <cstdio>
#include <utility>
#include <vector>

#include "common.cuh"

struct kanso_cuda_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  int sm_count = 0;
  int smem_optin = 0;      // max dynamic shared memory per block (opt-in), bytes
  int smem_per_sm = 0;     // shared memory of one SM, bytes
  int* dev_status = nullptr;  // one int on the device, OR of kanso::DevStatus
  int* host_status = nullptr;  // pinned: the status word lands here with the stream's other work
  // arrival counters of the split-context attention (one per sequence and KV head); all zero
  // between calls: the CTA that takes the last ticket of a counter resets it
  uint32_t* pa_tickets = nullptr;
  static constexpr uint32_t kPaTickets = 16384;
  uint64_t launches = 0;
  // weight buffers are never written by work enqueued before a matmul on this stream, so a
  // matmul may start fetching weights while the kernel before it is still running
  bool overlap_weight_prefetch = false;
  std::string last_error;
  // Scratch owned by the context (split-KV partials, staged activations). Grows on demand.
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  // Pinned host staging + device staging for the host-buffer entry points.
  void* pinned = nullptr;
  size_t pinned_bytes = 0;
  void* stage_dev = nullptr;
  size_t stage_dev_bytes = 0;
  // bumped whenever scratch, pinned or device staging is reallocated: captured graphs that
  // hold the old addresses are stale
  uint64_t buf_gen = 0;
};

// One captured host call of a weight (kanso_cuda_linear_host): copy in, matmul, copy out and
// status word as a single graph launch.
struct kanso_host_graph {
  int64_t M = 0;
  int32_t act_mode = 0;
  uint64_t buf_gen = 0;
  bool overlap = false;
  cudaGraphExec_t exec = nullptr;  // nullptr: capture was tried and is not possible
};

struct kanso_cuda_weight {
  kanso_cuda_ctx* ctx = nullptr;
  void* dev = nullptr;
  size_t nbytes = 0;
  int32_t dtype = 0;
  int64_t rows = 0, cols = 0;
  uint32_t host_calls = 0;
  std::vector<kanso_host_graph> host_graphs;
};

namespace kanso {

int32_t fail(kanso_cuda_ctx* ctx, int32_t code, const char* fmt, ...);
// Turns a CUDA runtime error into KANSO_ERR_DEVICE with its message.
int32_t cuda_fail(kanso_cuda_ctx* ctx, cudaError_t e, const char* what);
// Makes sure ctx->scratch holds at least `bytes`; nullptr + error on failure.
void* ctx_scratch(kanso_cuda_ctx* ctx, size_t bytes);
int32_t ctx_pinned(kanso_cuda_ctx* ctx, size_t bytes);
int32_t ctx_stage_dev(kanso_cuda_ctx* ctx, size_t bytes);
// Checks the launch, counts it.
int32_t after_launch(kanso_cuda_ctx* ctx, const char* what);
// Turns the status word that has landed in ctx->host_status into a return code (and clears it).
int32_t status_word_result(kanso_cuda_ctx* ctx);

// Asks, once per device, for the largest shared-memory carveout for `kern`. A launch that
// overlaps the kernel before it can only share an SM with it when both run under the same
// L1/shared split; with per-launch splits the SM drains and switches between launches of
// different shared-memory sizes. For kernels that stage through shared memory and do not
// depend on a large L1 (the Q4_K GEMV); the Q8_0 tensor-core GEMV reads its activations
// through L1 and keeps the default split (42.5 against 37 us at 8 rows with the large
// carveout).
void prefer_max_shared(kanso_cuda_ctx* ctx, const void* kern);

// Launches `kern` on the context's stream. When the context allows overlap
// (KANSO_OPT_OVERLAP_WEIGHT_PREFETCH) the launch carries the programmatic-stream-serialization
// attribute; such a kernel MUST execute griddepcontrol.wait before it touches anything an
// earlier kernel may have written.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(kanso_cuda_ctx* ctx, void (*kern)(KArgs...), dim3 grid,
                                    dim3 block, size_t smem, Args&&... args) {
  cudaLaunchConfig_t lc = {};
  lc.gridDim = grid;
  lc.blockDim = block;
  lc.dynamicSmemBytes = smem;
  lc.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = ctx->overlap_weight_prefetch ? 1 : 0;
  lc.attrs = attr;
  lc.numAttrs = 1;
  return cudaLaunchKernelEx(&lc, kern, std::forward<Args>(args)...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define KANSO_CUDA_TRY(ctx, expr, what)                          \
  do {                                                           \
    cudaError_t _e = (expr);                                     \
    if (_e != cudaSuccess) return kanso::cuda_fail(ctx, _e, what); \
  } while (0)

}  // namespace kanso
