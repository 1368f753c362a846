// Sharded linear layers behind the C ABI: peer-visible buffers, the exchange protocol and the
// row-sharded / K-sharded forward. The reference has no multi-GPU code (docs/SPEC.md:125); this
// extends LinearWeight::to_device and Model::linear (src/weights.rs:140-158,
// src/model.rs:390-397) to one process per GPU on one node.
//
// Memory. Every rank allocates one region with cudaMalloc and exports it as a CUDA IPC handle;
// the caller exchanges the handles by its own means (the harness uses torch.distributed, a Rust
// caller its own channel) and every rank maps its peers' regions. Layers carve their exchange
// buffers out of the region in creation order, so the same offset names the same buffer on
// every rank (every rank must create the same layers in the same order).
//
// Protocol of one exchange (no host state, so a captured CUDA graph replays correctly):
//   * each layer owns, in every rank's region, a flag array (one u64 per peer), a step counter
//     and a ticket; its data lives in TWO exchange buffers used alternately, chosen on the
//     device by the parity of the step counter;
//   * the producing kernel (the matmul's own epilogue, or the scatter kernel after a matmul
//     that cannot store to peers itself) writes its slice into buffer (step & 1) of EVERY rank
//     with plain stores over NVLink, fences, and takes a ticket; the CTA that draws the last
//     ticket advances the step and release-stores the new step number into its slot of every
//     peer's flag array;
//   * the consuming kernel (copy-out for a gathered row shard, the rank-ordered sum for a K
//     shard) acquire-polls its own flag array until every peer's slot has reached the step, at
//     most 2 s, then reads buffer ((step - 1) & 1) from its OWN memory.
// Why two buffers suffice: a rank can start storing exchange k+2 into the buffer of exchange k
// only after its own consumer of exchange k+1 has run, and that consumer waited for every
// peer's flag k+1, which a peer raises only after its consumer of exchange k (stream order).
// No multicast loads, no multimem, no load from peer memory at all: peers are only stored to.
#include <cstring>

#include "ctx.h"
#include "shard.cuh"

struct kanso_cuda_shard_group {
  kanso_cuda_ctx* ctx = nullptr;
  int rank = 0, world = 1;
  uint8_t* local = nullptr;
  size_t bytes = 0;
  uint8_t* peer[KANSO_MAX_PEERS] = {nullptr};
  bool opened[KANSO_MAX_PEERS] = {false};
  bool connected = false;
  size_t used = 0;      // bump pointer over the data part (identical on every rank)
  int next_slot = 0;    // control slots handed out so far
};

struct kanso_cuda_sharded_linear {
  kanso_cuda_shard_group* g = nullptr;
  kanso_cuda_weight* w = nullptr;
  int mode = 0;
  int64_t rows_total = 0, cols_total = 0, begin = 0, count = 0, max_m = 0;
  size_t buf_off = 0, buf_stride = 0;  // first exchange buffer, bytes between the two
  int64_t ld = 0;                      // floats per row of an exchange buffer
  float* y = nullptr;                  // fixed result [max_m, rows_total]
  float* y_slice = nullptr;            // row shard: this rank's rows only [max_m, count]
  float* stage = nullptr;              // few-row Q4_K path: this rank's slice before it is published
  int slot = 0;
};

namespace kanso {

constexpr size_t SG_CTRL_SLOT = 128;  // flags[8] u64, step u64, ticket u32
constexpr int SG_MAX_LAYERS = 256;
constexpr size_t SG_CTRL_BYTES = SG_CTRL_SLOT * SG_MAX_LAYERS;

int32_t matmul_dispatch(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x,
                        float* y, int64_t M, int64_t N, int64_t K, int32_t act_mode);

// src f32 [M, n] (this rank's slice, local) -> rows [col0, col0 + n) of buffer (step & 1) of
// every rank, then ticket + signal.
__global__ void shard_scatter_signal_kernel(const float* __restrict__ src, ShardSignal s,
                                            int64_t M, int64_t n, int64_t ld, int64_t col0) {
  __shared__ unsigned int s_last;
  pdl_launch_dependents();
  pdl_wait();
  const int64_t par = (int64_t)(*s.step & 1ull);
  const int64_t total = M * n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / n, c = i - m * n;
    const float v = src[i];
    for (int r = 0; r < s.world; ++r) s.out[r][par * s.buf_stride + m * ld + col0 + c] = v;
  }
  shard_ticket(s, gridDim.x, &s_last);
}

// Row shard, gathered: copies buffer ((step - 1) & 1) [M, ld] to the fixed result.
__global__ void shard_wait_copy_kernel(const float* __restrict__ buf0, int64_t buf_stride,
                                       const unsigned long long* mine,
                                       const unsigned long long* step, int world, int64_t M,
                                       int64_t ld, float* __restrict__ y, int* status) {
  pdl_launch_dependents();
  pdl_wait();  // the producing kernel has advanced the step
  const unsigned long long e = *step;
  shard_wait_flags(mine, world, e, status);
  const float* src = buf0 + (int64_t)((e - 1) & 1ull) * buf_stride;
  const int64_t total = M * ld;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x)
    y[i] = src[i];
}

// K shard: y[m, n] = sum over ranks r of buffer[m, r * rows + n], added in rank order (every
// rank gets the same bits).
__global__ void shard_wait_sum_kernel(const float* __restrict__ buf0, int64_t buf_stride,
                                      const unsigned long long* mine,
                                      const unsigned long long* step, int world, int64_t M,
                                      int64_t rows, float* __restrict__ y, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const unsigned long long e = *step;
  shard_wait_flags(mine, world, e, status);
  const float* src = buf0 + (int64_t)((e - 1) & 1ull) * buf_stride;
  const int64_t total = M * rows;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / rows, n = i - m * rows;
    const float* p = src + m * rows * world + n;
    float acc = 0.f;
    for (int r = 0; r < world; ++r) acc += p[(int64_t)r * rows];
    y[i] = acc;
  }
}

}  // namespace kanso

using namespace kanso;

namespace kanso {
int32_t q4k_direct_matmul_shard(kanso_cuda_ctx* ctx, const void* w, const float* x, float* stage,
                                int64_t M, int64_t N, int64_t K, bool* handled,
                                const ShardSignal& sig);

static unsigned long long* sg_flags(const kanso_cuda_shard_group* g, int r, int slot) {
  return reinterpret_cast<unsigned long long*>(g->peer[r] + (size_t)slot * SG_CTRL_SLOT);
}
static unsigned long long* sg_step(const kanso_cuda_shard_group* g, int slot) {
  return sg_flags(g, g->rank, slot) + KANSO_MAX_PEERS;
}
static unsigned int* sg_ticket(const kanso_cuda_shard_group* g, int slot) {
  return reinterpret_cast<unsigned int*>(sg_step(g, slot) + 1);
}

static ShardSignal sg_signal(const kanso_cuda_sharded_linear* L, int signal) {
  const kanso_cuda_shard_group* g = L->g;
  ShardSignal s = {};
  for (int r = 0; r < g->world; ++r) {
    s.out[r] = reinterpret_cast<float*>(g->peer[r] + SG_CTRL_BYTES + L->buf_off);
    s.flags[r] = sg_flags(g, r, L->slot);
  }
  s.step = sg_step(g, L->slot);
  s.ticket = sg_ticket(g, L->slot);
  s.buf_stride = (int64_t)(L->buf_stride / sizeof(float));
  s.world = g->world;
  s.rank = g->rank;
  s.signal = signal;
  return s;
}

// This rank's slice [M, n] -> columns [col0, col0 + n) of the current exchange buffer of every
// rank, followed by the signal. Q4_K with up to 8 activation rows stores from the matmul's own
// epilogue; every other shape goes through a staging buffer and the scatter kernel.
static int32_t sg_produce(kanso_cuda_sharded_linear* L, const float* x, int64_t M, int64_t n,
                          int64_t K, int64_t col0, int32_t act_mode, bool* fused) {
  kanso_cuda_ctx* ctx = L->g->ctx;
  *fused = false;
  if (L->w->dtype == KANSO_DTYPE_Q4_K && act_mode == KANSO_ACT_F32 && M <= 8) {
    // Up to 6 rows in one pass; 7 and 8 rows in two passes of 4. Every pass stores its rows into
    // the layer's staging slice; the last CTA of the LAST pass publishes all rows, signals, and
    // for a K shard waits for the peers and sums: one kernel per forward, no separate consumer.
    const int64_t mp = M > 6 ? 4 : M;
    bool all = true;
    for (int64_t m0 = 0; m0 < M && all; m0 += mp) {
      const int64_t mc = M - m0 < mp ? M - m0 : mp;
      ShardSignal s = sg_signal(L, m0 + mc >= M ? 1 : 0);
      s.stage = L->stage;
      s.y = L->y;
      s.ld = L->ld;
      s.col0 = col0;
      s.n = n;
      s.m_total = (int)M;
      s.sum = L->mode == KANSO_SHARD_K ? 1 : 0;
      s.status = ctx->dev_status;
      bool handled = false;
      int32_t st = q4k_direct_matmul_shard(ctx, L->w->dev, x + m0 * K, L->stage + m0 * n, mc, n, K,
                                           &handled, s);
      if (st) return st;
      if (!handled) {
        if (m0 != 0) return fail(ctx, KANSO_ERR_DEVICE, "sharded matmul: inconsistent passes");
        all = false;
      }
    }
    if (all) {
      *fused = true;
      return KANSO_OK;
    }
  }
  int32_t st = ctx_stage_dev(ctx, sizeof(float) * (size_t)M * (size_t)n);
  if (st) return st;
  float* tmp = (float*)ctx->stage_dev;
  st = matmul_dispatch(ctx, L->w->dtype, L->w->dev, x, tmp, M, n, K, act_mode);
  if (st) return st;
  const ShardSignal s = sg_signal(L, 1);
  int64_t blocks = (M * n + 255) / 256;
  if (blocks > 4 * ctx->sm_count) blocks = 4 * ctx->sm_count;
  KANSO_CUDA_TRY(ctx,
                 launch_dependent(ctx, shard_scatter_signal_kernel, dim3((unsigned)blocks),
                                  dim3(256), 0, (const float*)tmp, s, M, n, L->ld, col0),
                 "shard scatter launch");
  return after_launch(ctx, "shard scatter");
}
}  // namespace kanso

extern "C" {

int32_t kanso_cuda_shard_group_create(kanso_cuda_ctx* ctx, int32_t rank, int32_t world,
                                      size_t region_bytes, kanso_cuda_shard_group** out,
                                      void* handle_out) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "shard_group_create: ctx is NULL");
  if (!out || !handle_out) return fail(ctx, KANSO_ERR_SHAPE, "shard_group_create: NULL pointer");
  *out = nullptr;
  if (world < 1 || world > KANSO_MAX_PEERS || rank < 0 || rank >= world)
    return fail(ctx, KANSO_ERR_UNSUPPORTED, "shard_group_create: rank %d of %d (1..%d ranks)",
                rank, world, KANSO_MAX_PEERS);
  static_assert(sizeof(cudaIpcMemHandle_t) == KANSO_SHARD_HANDLE_BYTES, "handle size");
  auto* g = new kanso_cuda_shard_group;
  g->ctx = ctx;
  g->rank = rank;
  g->world = world;
  g->bytes = SG_CTRL_BYTES + ((region_bytes + 255) & ~size_t(255));
  cudaError_t e = cudaMalloc(&g->local, g->bytes);
  if (e == cudaSuccess) e = cudaMemsetAsync(g->local, 0, g->bytes, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, g->local);
  if (e != cudaSuccess) {
    if (g->local) cudaFree(g->local);
    delete g;
    return cuda_fail(ctx, e, "shard_group_create");
  }
  std::memcpy(handle_out, &h, sizeof h);
  g->peer[rank] = g->local;
  if (world == 1) g->connected = true;
  *out = g;
  return KANSO_OK;
}

int32_t kanso_cuda_shard_group_connect(kanso_cuda_shard_group* g, const void* all_handles) {
  if (!g) return fail(nullptr, KANSO_ERR_CONFIG, "shard_group_connect: group is NULL");
  if (!all_handles) return fail(g->ctx, KANSO_ERR_SHAPE, "shard_group_connect: NULL pointer");
  if (g->connected) return KANSO_OK;
  for (int r = 0; r < g->world; ++r) {
    if (r == g->rank) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, (const uint8_t*)all_handles + (size_t)r * KANSO_SHARD_HANDLE_BYTES, sizeof h);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail(g->ctx, e, "shard_group_connect: cudaIpcOpenMemHandle");
    g->peer[r] = (uint8_t*)p;
    g->opened[r] = true;
  }
  g->connected = true;
  return KANSO_OK;
}

int32_t kanso_cuda_shard_group_destroy(kanso_cuda_shard_group* g) {
  if (!g) return KANSO_OK;
  cudaDeviceSynchronize();
  for (int r = 0; r < g->world; ++r)
    if (g->opened[r]) cudaIpcCloseMemHandle(g->peer[r]);
  if (g->local) cudaFree(g->local);
  delete g;
  return KANSO_OK;
}

}  // extern "C"

extern "C" {

int32_t kanso_cuda_sharded_linear_create(kanso_cuda_shard_group* g, const void* shard_bytes,
                                         size_t nbytes, int32_t dtype, int64_t rows_total,
                                         int64_t cols_total, int32_t mode, int64_t max_m,
                                         kanso_cuda_sharded_linear** out) {
  if (!g) return fail(nullptr, KANSO_ERR_CONFIG, "sharded_linear_create: group is NULL");
  kanso_cuda_ctx* ctx = g->ctx;
  if (!out || !shard_bytes) return fail(ctx, KANSO_ERR_SHAPE, "sharded_linear_create: NULL pointer");
  *out = nullptr;
  if (!g->connected)
    return fail(ctx, KANSO_ERR_CONFIG, "sharded_linear_create: the group is not connected yet");
  if (mode != KANSO_SHARD_ROWS && mode != KANSO_SHARD_K)
    return fail(ctx, KANSO_ERR_CONFIG, "sharded_linear_create: mode %d is neither rows nor K", mode);
  if (max_m < 1) return fail(ctx, KANSO_ERR_SHAPE, "sharded_linear_create: max_m %lld", (long long)max_m);
  if (g->next_slot >= SG_MAX_LAYERS)
    return fail(ctx, KANSO_ERR_UNSUPPORTED, "sharded_linear_create: more than %d layers", SG_MAX_LAYERS);
  const int blk = dtype == KANSO_DTYPE_Q4_K ? 256 : 32;
  int64_t begin = 0, count = 0;
  const int32_t rs = mode == KANSO_SHARD_ROWS
                         ? kanso_cuda_shard_range(rows_total, g->rank, g->world, 8, &begin, &count)
                         : kanso_cuda_shard_range(cols_total, g->rank, g->world, blk, &begin, &count);
  if (rs != KANSO_OK || count == 0)
    return fail(ctx, KANSO_ERR_SHAPE,
                "sharded_linear_create: [%lld x %lld] does not split over %d ranks in units of %d",
                (long long)rows_total, (long long)cols_total, g->world,
                mode == KANSO_SHARD_ROWS ? 8 : blk);
  auto* L = new kanso_cuda_sharded_linear;
  L->g = g;
  L->mode = mode;
  L->rows_total = rows_total;
  L->cols_total = cols_total;
  L->begin = begin;
  L->count = count;
  L->max_m = max_m;
  // the exchange buffers: [max_m, rows_total] gathered rows, or [max_m, world * rows_total]
  // partial sums, twice
  L->ld = mode == KANSO_SHARD_ROWS ? rows_total : rows_total * g->world;
  const size_t one = ((size_t)max_m * (size_t)L->ld * sizeof(float) + 255) & ~size_t(255);
  if (g->used + 2 * one > g->bytes - SG_CTRL_BYTES) {
    delete L;
    return fail(ctx, KANSO_ERR_CONFIG,
                "sharded_linear_create: the group's region holds %zu bytes, %zu used, this layer "
                "needs %zu", g->bytes - SG_CTRL_BYTES, g->used, 2 * one);
  }
  L->buf_off = g->used;
  L->buf_stride = one;
  g->used += 2 * one;
  L->slot = g->next_slot++;
  int32_t st = mode == KANSO_SHARD_ROWS
                   ? kanso_cuda_weight_upload(ctx, shard_bytes, nbytes, dtype, count, cols_total, &L->w)
                   : kanso_cuda_weight_upload(ctx, shard_bytes, nbytes, dtype, rows_total, count, &L->w);
  cudaError_t e = cudaSuccess;
  if (st == KANSO_OK) {
    e = cudaMalloc(&L->y, sizeof(float) * (size_t)max_m * (size_t)rows_total);
    if (e == cudaSuccess && mode == KANSO_SHARD_ROWS)
      e = cudaMalloc(&L->y_slice, sizeof(float) * (size_t)max_m * (size_t)count);
    if (e == cudaSuccess)
      e = cudaMalloc(&L->stage, sizeof(float) * 8 *
                                    (size_t)(mode == KANSO_SHARD_ROWS ? count : rows_total));
    if (e != cudaSuccess) st = cuda_fail(ctx, e, "sharded_linear_create");
  }
  if (st != KANSO_OK) {
    kanso_cuda_sharded_linear_destroy(L);
    return st;
  }
  *out = L;
  return KANSO_OK;
}

int32_t kanso_cuda_sharded_linear_destroy(kanso_cuda_sharded_linear* L) {
  if (!L) return KANSO_OK;
  cudaDeviceSynchronize();
  if (L->w) kanso_cuda_weight_free(L->w);
  if (L->y) cudaFree(L->y);
  if (L->y_slice) cudaFree(L->y_slice);
  if (L->stage) cudaFree(L->stage);
  delete L;
  return KANSO_OK;
}

int32_t kanso_cuda_sharded_linear_range(const kanso_cuda_sharded_linear* L, int64_t* begin,
                                        int64_t* count) {
  if (!L || !begin || !count) return KANSO_ERR_SHAPE;
  *begin = L->begin;
  *count = L->count;
  return KANSO_OK;
}

int32_t kanso_cuda_sharded_linear_forward(kanso_cuda_sharded_linear* L, const float* x, int64_t M,
                                          int32_t act_mode, int32_t flags, const float** y_out) {
  if (!L) return fail(nullptr, KANSO_ERR_CONFIG, "sharded_linear_forward: layer is NULL");
  kanso_cuda_shard_group* g = L->g;
  kanso_cuda_ctx* ctx = g->ctx;
  if (!x || !y_out) return fail(ctx, KANSO_ERR_SHAPE, "sharded_linear_forward: NULL pointer");
  if (M < 1 || M > L->max_m)
    return fail(ctx, KANSO_ERR_SHAPE, "sharded_linear_forward: M %lld outside 1..%lld",
                (long long)M, (long long)L->max_m);
  const unsigned long long* mine = (const unsigned long long*)(g->local + (size_t)L->slot * SG_CTRL_SLOT);
  const unsigned long long* step = mine + KANSO_MAX_PEERS;
  const float* buf0 = reinterpret_cast<const float*>(g->local + SG_CTRL_BYTES + L->buf_off);
  const int64_t stride = (int64_t)(L->buf_stride / sizeof(float));
  if (L->mode == KANSO_SHARD_ROWS) {
    if (flags & KANSO_SHARD_LOCAL_ONLY) {
      // the slice stays on this rank: it is the K slice of a K-sharded consumer
      int32_t st = matmul_dispatch(ctx, L->w->dtype, L->w->dev, x, L->y_slice, M, L->count,
                                   L->cols_total, act_mode);
      *y_out = L->y_slice;
      return st;
    }
    bool fused = false;
    int32_t st = sg_produce(L, x, M, L->count, L->cols_total, L->begin, act_mode, &fused);
    if (st) return st;
    int64_t blocks = (M * L->ld + 255) / 256;
    if (blocks > 2 * ctx->sm_count) blocks = 2 * ctx->sm_count;
    KANSO_CUDA_TRY(ctx,
                   launch_dependent(ctx, shard_wait_copy_kernel, dim3((unsigned)blocks), dim3(256),
                                    0, buf0, stride, mine, step, g->world, M, L->ld, L->y,
                                    ctx->dev_status),
                   "shard wait/copy launch");
    *y_out = L->y;
    return after_launch(ctx, "shard wait/copy");
  }
  // K shard: x is this rank's columns [begin, begin + count) of the activations
  bool fused = false;
  int32_t st = sg_produce(L, x, M, L->rows_total, L->count, (int64_t)g->rank * L->rows_total,
                          act_mode, &fused);
  if (st) return st;
  *y_out = L->y;
  if (fused) return KANSO_OK;  // the matmul's last CTA has waited for the peers and summed
  int64_t blocks = (M * L->rows_total + 255) / 256;
  if (blocks > 2 * ctx->sm_count) blocks = 2 * ctx->sm_count;
  KANSO_CUDA_TRY(ctx,
                 launch_dependent(ctx, shard_wait_sum_kernel, dim3((unsigned)blocks), dim3(256), 0,
                                  buf0, stride, mine, step, g->world, M, L->rows_total, L->y,
                                  ctx->dev_status),
                 "shard wait/sum launch");
  *y_out = L->y;
  return after_launch(ctx, "shard wait/sum");
}

}  // extern "C"
