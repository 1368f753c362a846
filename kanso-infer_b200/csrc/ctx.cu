// Context lifetime, error reporting, scratch management.
#include "ctx.h"

#include <mutex>
#include <unordered_set>

namespace {
thread_local std::string g_no_ctx_error = "";
}

namespace kanso {

int32_t fail(kanso_cuda_ctx* ctx, int32_t code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx)
    ctx->last_error = buf;
  else
    g_no_ctx_error = buf;
  return code;
}

int32_t cuda_fail(kanso_cuda_ctx* ctx, cudaError_t e, const char* what) {
  return fail(ctx, KANSO_ERR_DEVICE, "%s: %s (%s)", what, cudaGetErrorString(e),
              cudaGetErrorName(e));
}

void* ctx_scratch(kanso_cuda_ctx* ctx, size_t bytes) {
  if (bytes <= ctx->scratch_bytes) return ctx->scratch;
  // Growing reallocates: wait for work that may still read the old buffer.
  cudaStreamSynchronize(ctx->stream);
  if (ctx->scratch) cudaFree(ctx->scratch);
  ctx->scratch = nullptr;
  ctx->scratch_bytes = 0;
  size_t want = bytes + (bytes >> 2);
  cudaError_t e = cudaMalloc(&ctx->scratch, want);
  if (e != cudaSuccess) {
    cuda_fail(ctx, e, "scratch allocation");
    return nullptr;
  }
  ctx->scratch_bytes = want;
  ctx->buf_gen++;
  return ctx->scratch;
}

int32_t ctx_pinned(kanso_cuda_ctx* ctx, size_t bytes) {
  if (bytes <= ctx->pinned_bytes) return KANSO_OK;
  cudaStreamSynchronize(ctx->stream);
  if (ctx->pinned) cudaFreeHost(ctx->pinned);
  ctx->pinned = nullptr;
  ctx->pinned_bytes = 0;
  KANSO_CUDA_TRY(ctx, cudaMallocHost(&ctx->pinned, bytes), "pinned staging allocation");
  ctx->pinned_bytes = bytes;
  ctx->buf_gen++;
  return KANSO_OK;
}

int32_t ctx_stage_dev(kanso_cuda_ctx* ctx, size_t bytes) {
  if (bytes <= ctx->stage_dev_bytes) return KANSO_OK;
  cudaStreamSynchronize(ctx->stream);
  if (ctx->stage_dev) cudaFree(ctx->stage_dev);
  ctx->stage_dev = nullptr;
  ctx->stage_dev_bytes = 0;
  KANSO_CUDA_TRY(ctx, cudaMalloc(&ctx->stage_dev, bytes), "device staging allocation");
  ctx->stage_dev_bytes = bytes;
  ctx->buf_gen++;
  return KANSO_OK;
}

void prefer_max_shared(kanso_cuda_ctx* ctx, const void* kern) {
  static std::mutex mu;
  static std::unordered_set<uintptr_t> done;  // (kernel, device) pairs already set
  const uintptr_t key = reinterpret_cast<uintptr_t>(kern) * 16u + (uintptr_t)(ctx->device & 15);
  std::lock_guard<std::mutex> lock(mu);
  if (!done.insert(key).second) return;
  // a preference only: a refusal changes nothing about the result
  if (cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                           cudaSharedmemCarveoutMaxShared) != cudaSuccess)
    cudaGetLastError();
}

int32_t after_launch(kanso_cuda_ctx* ctx, const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(ctx, e, what);
  ctx->launches++;
  return KANSO_OK;
}

}  // namespace kanso

using namespace kanso;

extern "C" {

int32_t kanso_cuda_ctx_create(int32_t device, void* stream, kanso_cuda_ctx** out) {
  if (!out) return fail(nullptr, KANSO_ERR_CONFIG, "ctx_create: out is NULL");
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return fail(nullptr, KANSO_ERR_DEVICE,
                "backend 'cuda' is not available: no CUDA device (%s); there is no CPU fallback",
                e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  if (device < 0 || device >= n)
    return fail(nullptr, KANSO_ERR_CONFIG, "ctx_create: device %d out of range (%d devices)",
                device, n);
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaGetDeviceProperties");
  if (prop.major != 10)
    return fail(nullptr, KANSO_ERR_DEVICE,
                "backend 'cuda' needs a compute capability 10.x GPU (sm_100a kernels); device %d "
                "is %d.%d",
                device, prop.major, prop.minor);
  e = cudaSetDevice(device);
  if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaSetDevice");
  auto* ctx = new kanso_cuda_ctx;
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->smem_optin = (int)prop.sharedMemPerBlockOptin;
  ctx->smem_per_sm = (int)prop.sharedMemPerMultiprocessor;
  if (stream) {
    ctx->stream = (cudaStream_t)stream;
  } else {
    e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
      delete ctx;
      return cuda_fail(nullptr, e, "cudaStreamCreate");
    }
    ctx->own_stream = true;
  }
  e = cudaMalloc(&ctx->dev_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(ctx->dev_status, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaMallocHost(&ctx->host_status, sizeof(int));
  if (e == cudaSuccess)
    e = cudaMalloc(&ctx->pa_tickets, sizeof(uint32_t) * kanso_cuda_ctx::kPaTickets);
  if (e == cudaSuccess)
    e = cudaMemset(ctx->pa_tickets, 0, sizeof(uint32_t) * kanso_cuda_ctx::kPaTickets);
  if (e != cudaSuccess) {
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return cuda_fail(nullptr, e, "status word allocation");
  }
  *out = ctx;
  return KANSO_OK;
}

int32_t kanso_cuda_ctx_destroy(kanso_cuda_ctx* ctx) {
  if (!ctx) return KANSO_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->stage_dev) cudaFree(ctx->stage_dev);
  if (ctx->pinned) cudaFreeHost(ctx->pinned);
  if (ctx->dev_status) cudaFree(ctx->dev_status);
  if (ctx->host_status) cudaFreeHost(ctx->host_status);
  if (ctx->pa_tickets) cudaFree(ctx->pa_tickets);
  if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
  return KANSO_OK;
}

int32_t kanso_cuda_sync(kanso_cuda_ctx* ctx) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "sync: ctx is NULL");
  // the status word rides behind the stream's work into pinned memory: one wait for both
  KANSO_CUDA_TRY(ctx,
                 cudaMemcpyAsync(ctx->host_status, ctx->dev_status, sizeof(int),
                                 cudaMemcpyDeviceToHost, ctx->stream),
                 "status word read");
  KANSO_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream), "stream synchronize");
  return status_word_result(ctx);
}

}  // extern "C"

namespace kanso {
int32_t status_word_result(kanso_cuda_ctx* ctx) {
  const int st = *ctx->host_status;
  if (st != 0) {
    cudaMemset(ctx->dev_status, 0, sizeof(int));
    // a kernel that gave up may have left attention tickets taken
    cudaMemset(ctx->pa_tickets, 0, sizeof(uint32_t) * kanso_cuda_ctx::kPaTickets);
    if (st & DEV_WAIT_TIMEOUT)
      return fail(ctx, KANSO_ERR_TIMEOUT, "a kernel gave up a bounded wait (status word %d)", st);
    return fail(ctx, KANSO_ERR_SHAPE,
                "a kernel met an out-of-range block id, slot or token id (status word %d)", st);
  }
  return KANSO_OK;
}
}  // namespace kanso

extern "C" {

const char* kanso_cuda_last_error(const kanso_cuda_ctx* ctx) {
  return ctx ? ctx->last_error.c_str() : g_no_ctx_error.c_str();
}

int32_t kanso_cuda_ctx_set_option(kanso_cuda_ctx* ctx, int32_t option, int32_t value) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "ctx_set_option: ctx is NULL");
  switch (option) {
    case KANSO_OPT_OVERLAP_WEIGHT_PREFETCH:
      ctx->overlap_weight_prefetch = value != 0;
      return KANSO_OK;
    default:
      return fail(ctx, KANSO_ERR_CONFIG, "ctx_set_option: unknown option %d", option);
  }
}

uint64_t kanso_cuda_launch_count(const kanso_cuda_ctx* ctx) { return ctx ? ctx->launches : 0; }
int32_t kanso_cuda_sm_count(const kanso_cuda_ctx* ctx) { return ctx ? ctx->sm_count : 0; }

}  // extern "C"
