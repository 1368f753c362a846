// Device-resident weights and the Model::linear call on them.
#include <atomic>
#include <chrono>
#include <cstring>

#include "ctx.h"

namespace kanso {
int32_t stream_matmul(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x, float* y,
                      int64_t M, int64_t N, int64_t K, int32_t act_mode);
int32_t matmul_dispatch(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x,
                        float* y, int64_t M, int64_t N, int64_t K, int32_t act_mode);

// LinearWeight::embed (src/weights.rs:50-57): dequantise the selected Q8_0 rows.
__global__ void embed_q8_0_kernel(const uint8_t* __restrict__ w, const uint32_t* __restrict__ ids,
                                  float* __restrict__ out, int64_t rows, int cols, int* status) {
  int t = blockIdx.x;
  uint32_t id = ids[t];
  if (id >= rows) {
    if (threadIdx.x == 0) atomicOr(status, DEV_BAD_INDEX);
    return;
  }
  const uint8_t* row = w + (int64_t)id * (cols / 32) * Q8_BYTES;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    const uint8_t* blk = row + (i >> 5) * Q8_BYTES;
    float d = f16_bits_to_f32(blk[0] | (blk[1] << 8));
    out[(int64_t)t * cols + i] = __fmul_rn(d, (float)(int8_t)blk[2 + (i & 31)]);
  }
}
}  // namespace kanso

using namespace kanso;

extern "C" {

int32_t kanso_cuda_weight_upload(kanso_cuda_ctx* ctx, const void* host_bytes, size_t nbytes,
                                 int32_t dtype, int64_t rows, int64_t cols,
                                 kanso_cuda_weight** out) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "weight_upload: ctx is NULL");
  if (!out || !host_bytes) return fail(ctx, KANSO_ERR_SHAPE, "weight_upload: NULL pointer");
  *out = nullptr;
  int blk, bb;
  if (dtype == KANSO_DTYPE_Q8_0) {
    blk = 32;
    bb = Q8_BYTES;
  } else if (dtype == KANSO_DTYPE_Q4_K) {
    blk = 256;
    bb = Q4K_BYTES;
  } else {
    return fail(ctx, KANSO_ERR_UNSUPPORTED, "weight_upload: dtype %d is neither Q8_0 (8) nor Q4_K (12)",
                dtype);
  }
  if (rows <= 0 || cols <= 0 || cols % blk != 0)
    return fail(ctx, KANSO_ERR_SHAPE,
                "weight_upload: [%lld x %lld] needs cols %% %d == 0 (a block may not straddle a row)",
                (long long)rows, (long long)cols, blk);
  size_t expect = (size_t)rows * (size_t)(cols / blk) * bb;
  if (nbytes != expect)
    return fail(ctx, KANSO_ERR_SHAPE, "weight_upload: %zu bytes given, [%lld x %lld] needs %zu",
                nbytes, (long long)rows, (long long)cols, expect);
  auto* w = new kanso_cuda_weight;
  w->ctx = ctx;
  w->nbytes = nbytes;
  w->dtype = dtype;
  w->rows = rows;
  w->cols = cols;
  cudaError_t e = cudaMalloc(&w->dev, (nbytes + 255) & ~size_t(255));
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(w->dev, host_bytes, nbytes, cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  if (e != cudaSuccess) {
    if (w->dev) cudaFree(w->dev);
    delete w;
    return cuda_fail(ctx, e, "weight_upload");
  }
  *out = w;
  return KANSO_OK;
}

int32_t kanso_cuda_weight_free(kanso_cuda_weight* w) {
  if (!w) return KANSO_OK;
  cudaDeviceSynchronize();  // the context may already be destroyed
  for (auto& g : w->host_graphs)
    if (g.exec) cudaGraphExecDestroy(g.exec);
  cudaFree(w->dev);
  delete w;
  return KANSO_OK;
}

const void* kanso_cuda_weight_ptr(const kanso_cuda_weight* w) { return w ? w->dev : nullptr; }

int32_t kanso_cuda_linear(kanso_cuda_ctx* ctx, const kanso_cuda_weight* w, const float* x,
                          float* y, int64_t M, int32_t act_mode) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "linear: ctx is NULL");
  if (!w) return fail(ctx, KANSO_ERR_SHAPE, "linear: weight is NULL");
  return matmul_dispatch(ctx, w->dtype, w->dev, x, y, M, w->rows, w->cols, act_mode);
}

// Model::linear with host activations. The first call of a (weight, M, mode) runs the plain
// sequence: copy in, matmul, copy out, status word, wait. From the second call on the same
// sequence is replayed as ONE captured graph launch (the staging addresses are fixed, the
// matmul has already sized the context's scratch, so nothing allocates during the capture):
// four driver calls and their gaps on the stream become one, which is most of what a host
// call costs around a 10 us kernel. A capture that cannot be made (the caller is itself
// capturing this stream, or the driver refuses) leaves the plain sequence in place.
// The device status word -> the pinned host word the caller watches. It runs after the matmul
// on the same stream, so the result the matmul stored into host memory is complete before it.
static __global__ void host_status_kernel(const int* dev_status, int* host_status) {
  *host_status = *dev_status;
}

static int32_t linear_host_enqueue(kanso_cuda_ctx* ctx, const kanso_cuda_weight* w, char* ph,
                                   char* pd, size_t xb, size_t xb_al, size_t yb, int64_t M,
                                   int32_t act_mode) {
  KANSO_CUDA_TRY(ctx, cudaMemcpyAsync(pd, ph, xb, cudaMemcpyHostToDevice, ctx->stream),
                 "linear_host: activations to device");
  // The batch-1..6 Q4_K GEMV writes every result element exactly once with a plain store and
  // never reads y: it can store straight into the pinned host buffer (posted writes over PCIe,
  // 16-57 KB), and a one-thread kernel passes the status word on, which leaves the graph one
  // copy and two kernels instead of three copies and a kernel. Every other kernel (atomics onto
  // a cleared y, several passes) keeps the device result and the copy back.
  const bool direct_y = w->dtype == KANSO_DTYPE_Q4_K && act_mode == KANSO_ACT_F32 && M <= 6 &&
                        w->cols % 256 == 0 && w->rows % 8 == 0 && w->rows >= 8;
  float* yd = direct_y ? (float*)(ph + xb_al) : (float*)(pd + xb_al);
  int32_t st = matmul_dispatch(ctx, w->dtype, w->dev, (const float*)pd, yd, M, w->rows, w->cols,
                               act_mode);
  if (st) return st;
  if (direct_y) {
    host_status_kernel<<<1, 1, 0, ctx->stream>>>(ctx->dev_status, ctx->host_status);
    return after_launch(ctx, "linear_host: status word");
  }
  KANSO_CUDA_TRY(ctx,
                 cudaMemcpyAsync(ph + xb_al, pd + xb_al, yb, cudaMemcpyDeviceToHost, ctx->stream),
                 "linear_host: result to host");
  KANSO_CUDA_TRY(ctx,
                 cudaMemcpyAsync(ctx->host_status, ctx->dev_status, sizeof(int),
                                 cudaMemcpyDeviceToHost, ctx->stream),
                 "linear_host: status word");
  return KANSO_OK;
}

int32_t kanso_cuda_linear_host(kanso_cuda_ctx* ctx, const kanso_cuda_weight* w_in,
                               const float* x_host, float* y_host, int64_t M, int32_t act_mode) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "linear_host: ctx is NULL");
  if (!w_in || !x_host || !y_host) return fail(ctx, KANSO_ERR_SHAPE, "linear_host: NULL pointer");
  if (M <= 0) return M == 0 ? KANSO_OK : fail(ctx, KANSO_ERR_SHAPE, "linear_host: M < 0");
  // the handle caches its captured calls: the cache is bookkeeping, not part of the weight
  kanso_cuda_weight* w = const_cast<kanso_cuda_weight*>(w_in);
  size_t xb = sizeof(float) * (size_t)M * w->cols, yb = sizeof(float) * (size_t)M * w->rows;
  size_t xb_al = (xb + 255) & ~size_t(255);
  int32_t st = ctx_pinned(ctx, xb_al + yb);
  if (st) return st;
  st = ctx_stage_dev(ctx, xb_al + yb);
  if (st) return st;
  char* ph = (char*)ctx->pinned;
  char* pd = (char*)ctx->stage_dev;
  std::memcpy(ph, x_host, xb);

  kanso_host_graph* hg = nullptr;
  for (auto& g : w->host_graphs)
    if (g.M == M && g.act_mode == act_mode) hg = &g;
  if (hg && (hg->buf_gen != ctx->buf_gen || hg->overlap != ctx->overlap_weight_prefetch)) {
    if (hg->exec) cudaGraphExecDestroy(hg->exec);  // the staging buffers moved: capture again
    *hg = kanso_host_graph{};
    hg->M = -1;
    hg = nullptr;
  }
  if (!hg && w->host_calls >= 1) {
    // second call of this shape: the plain sequence has run once, capture it now
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(ctx->stream, &cs) == cudaSuccess &&
        cs == cudaStreamCaptureStatusNone) {
      kanso_host_graph g;
      g.M = M;
      g.act_mode = act_mode;
      g.buf_gen = ctx->buf_gen;
      g.overlap = ctx->overlap_weight_prefetch;
      const uint64_t launches0 = ctx->launches;
      if (cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
        const int32_t est = linear_host_enqueue(ctx, w, ph, pd, xb, xb_al, yb, M, act_mode);
        cudaGraph_t graph = nullptr;
        const cudaError_t ee = cudaStreamEndCapture(ctx->stream, &graph);
        if (est == KANSO_OK && ee == cudaSuccess && graph && g.buf_gen == ctx->buf_gen &&
            cudaGraphInstantiate(&g.exec, graph, 0) != cudaSuccess)
          g.exec = nullptr;
        if (est != KANSO_OK || ee != cudaSuccess || g.buf_gen != ctx->buf_gen) g.exec = nullptr;
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
      }
      ctx->launches = launches0;  // nothing has run yet
      // remember the kernels one replay stands for
      w->host_graphs.push_back(g);
      hg = &w->host_graphs.back();
    }
  }
  w->host_calls++;
  // The status word is the last thing the stream copies to the host. With a sentinel in its
  // place the host can watch that pinned word instead of asking the driver: when it changes,
  // the result (copied before it, on the same stream) has landed too.
  volatile int* hs = ctx->host_status;
  *hs = -1;
  if (hg && hg->exec) {
    KANSO_CUDA_TRY(ctx, cudaGraphLaunch(hg->exec, ctx->stream), "linear_host: graph launch");
    ctx->launches += 1;  // at least the matmul kernel (its activation pack, if any, not counted)
  } else {
    st = linear_host_enqueue(ctx, w, ph, pd, xb, xb_al, yb, M, act_mode);
    if (st) return st;
  }
  {
    const auto t0 = std::chrono::steady_clock::now();
    uint32_t spins = 0;
    while (*hs == -1) {
      if ((++spins & 0xFFFu) == 0 &&
          std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(200)) {
        // something is slow (or failed): let the driver wait and report
        KANSO_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream), "linear_host: wait");
        break;
      }
    }
    std::atomic_thread_fence(std::memory_order_acquire);
  }
  st = status_word_result(ctx);
  if (st) return st;
  std::memcpy(y_host, ph + xb_al, yb);
  return KANSO_OK;
}

int32_t kanso_cuda_embed(kanso_cuda_ctx* ctx, const kanso_cuda_weight* w, const uint32_t* ids,
                         float* out, int64_t T) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "embed: ctx is NULL");
  if (!w || !ids || !out) return fail(ctx, KANSO_ERR_SHAPE, "embed: NULL pointer");
  if (w->dtype != KANSO_DTYPE_Q8_0)
    return fail(ctx, KANSO_ERR_UNSUPPORTED, "embed: only Q8_0 embedding tables are supported");
  if (T <= 0) return T == 0 ? KANSO_OK : fail(ctx, KANSO_ERR_SHAPE, "embed: T < 0");
  embed_q8_0_kernel<<<(unsigned)T, 256, 0, ctx->stream>>>((const uint8_t*)w->dev, ids, out,
                                                          w->rows, (int)w->cols, ctx->dev_status);
  return after_launch(ctx, "embed");
}

}  // extern "C"
