// Device-resident weights and the Model::linear call on them.
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

int32_t kanso_cuda_linear_host(kanso_cuda_ctx* ctx, const kanso_cuda_weight* w,
                               const float* x_host, float* y_host, int64_t M, int32_t act_mode) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "linear_host: ctx is NULL");
  if (!w || !x_host || !y_host) return fail(ctx, KANSO_ERR_SHAPE, "linear_host: NULL pointer");
  if (M <= 0) return M == 0 ? KANSO_OK : fail(ctx, KANSO_ERR_SHAPE, "linear_host: M < 0");
  size_t xb = sizeof(float) * (size_t)M * w->cols, yb = sizeof(float) * (size_t)M * w->rows;
  size_t xb_al = (xb + 255) & ~size_t(255);
  int32_t st = ctx_pinned(ctx, xb_al + yb);
  if (st) return st;
  st = ctx_stage_dev(ctx, xb_al + yb);
  if (st) return st;
  char* ph = (char*)ctx->pinned;
  char* pd = (char*)ctx->stage_dev;
  std::memcpy(ph, x_host, xb);
  KANSO_CUDA_TRY(ctx, cudaMemcpyAsync(pd, ph, xb, cudaMemcpyHostToDevice, ctx->stream),
                 "linear_host: activations to device");
  st = matmul_dispatch(ctx, w->dtype, w->dev, (const float*)pd, (float*)(pd + xb_al), M, w->rows,
                       w->cols, act_mode);
  if (st) return st;
  KANSO_CUDA_TRY(ctx,
                 cudaMemcpyAsync(ph + xb_al, pd + xb_al, yb, cudaMemcpyDeviceToHost, ctx->stream),
                 "linear_host: result to host");
  st = kanso_cuda_sync(ctx);
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
