// Sharding a quantized linear layer over the GPUs of one node. The reference has no
// multi-GPU code (docs/SPEC.md:125); the pieces here extend LinearWeight::to_device
// (src/weights.rs:140-158) and Model::linear (src/model.rs:390-397):
//   * output-row sharding: rank r holds a contiguous range of weight rows; every rank
//     produces its slice of y (an all-gather assembles the vector where it is needed);
//   * K sharding: rank r holds the blocks of a contiguous range of columns of every row,
//     re-packed into its own [rows x K/world] block matrix; partial results are summed.
// Blocks never straddle a shard: ranges are multiples of the block size (and of 8 rows).
#include <cstring>

#include "common.cuh"
#include "ctx.h"

#define KANSO_MAX_PEERS 8

namespace kanso {
int32_t matmul_dispatch(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x,
                        float* y, int64_t M, int64_t N, int64_t K, int32_t act_mode);
int32_t q4k_direct_matmul_out(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                              int64_t M, int64_t N, int64_t K, bool* handled, float* const* y_out,
                              int n_out, int64_t ld_out, int64_t row_offset);

struct ScatterArgs {
  float* out[8];
  int n_out;
};
// src f32 [M, rows] -> out[o][m * ld + row_offset + r] for every result buffer
__global__ void scatter_rows_kernel(const float* __restrict__ src, ScatterArgs a, int64_t M,
                                    int64_t rows, int64_t ld, int64_t row_offset) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * rows) return;
  int64_t m = i / rows, r = i - m * rows;
  float v = src[i];
  for (int o = 0; o < a.n_out; ++o) a.out[o][m * ld + row_offset + r] = v;
}
}  // namespace kanso

using namespace kanso;

// y[m, n] = sum over r of parts[m, r * rows + n], added in rank order (every rank gets the same
// bits).
__global__ void sum_shards_kernel(const float* __restrict__ parts, int64_t M, int64_t rows,
                                  int world, float* __restrict__ y) {
  // launched while the exchange before it still waits for the peers; nothing is read before
  // that kernel has ended
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * rows) return;
  const int64_t m = i / rows, n = i - m * rows;
  const float* p = parts + m * rows * world + n;
  float s = 0.f;
  for (int r = 0; r < world; ++r) s += p[(int64_t)r * rows];
  y[i] = s;
}

// One thread per rank. Thread r tells rank r that this rank's stores of the current step are
// done (release store of the step number into slot `rank` of rank r's flag array), then waits
// until rank r has said the same to this rank (slot r of the own array). The step number lives
// in device memory and advances by one per call, so a captured graph of calls stays valid
// across replays; every rank makes the same sequence of calls. The wait is bounded by wall
// time: a peer that never arrives ends it with DEV_WAIT_TIMEOUT in the status word.
struct ExchangeArgs {
  unsigned long long* flags[KANSO_MAX_PEERS];  // flags[r]: rank r's array of `world` slots
  unsigned long long* step;                   // this rank's step counter
  int world, rank;
  unsigned long long timeout_ns;
  int* status;
};
__device__ __forceinline__ void peer_exchange(const ExchangeArgs& a, unsigned long long* s_step) {
  // Programmatic dependent launch: the kernel after this one (a GEMV) may start at once and
  // fetch its first weight tiles while this one waits for the peers; it reads nothing an
  // earlier kernel wrote before its own griddepcontrol.wait, which this kernel's end releases.
  pdl_launch_dependents();
  pdl_wait();  // the kernels before this one are complete, their stores performed
  const int r = threadIdx.x;
  if (r == 0) *s_step = *a.step + 1;
  __syncthreads();
  const unsigned long long e = *s_step;
  if (r < a.world) {
    // make the stores of the earlier kernels to the peers visible before the flag is
    __threadfence_system();
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(a.flags[r] + a.rank), "l"(e)
                 : "memory");
    const unsigned long long* mine = a.flags[a.rank] + r;
    unsigned long long t0, t1, seen;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (;;) {
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(mine) : "memory");
      if (seen >= e) break;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
      if (t1 - t0 > a.timeout_ns) {
        atomicOr(a.status, (int)DEV_WAIT_TIMEOUT);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  if (r == 0) *a.step = e;
}

__global__ void peer_exchange_kernel(const ExchangeArgs a) {
  __shared__ unsigned long long s_step;
  peer_exchange(a, &s_step);
}

static int32_t exchange_args(kanso_cuda_ctx* ctx, void* const* flags, void* step, int32_t world,
                             int32_t rank, ExchangeArgs* a, const char* who) {
  if (!flags || !step || world < 1 || world > KANSO_MAX_PEERS || rank < 0 || rank >= world)
    return fail(ctx, KANSO_ERR_SHAPE, "%s: bad arguments (world %d, rank %d)", who, world, rank);
  *a = ExchangeArgs{};
  for (int r = 0; r < world; ++r) {
    if (!flags[r]) return fail(ctx, KANSO_ERR_SHAPE, "%s: flags[%d] is NULL", who, r);
    a->flags[r] = (unsigned long long*)flags[r];
  }
  a->step = (unsigned long long*)step;
  a->world = world;
  a->rank = rank;
  a->timeout_ns = 2000000000ull;  // 2 s
  a->status = ctx->dev_status;
  return KANSO_OK;
}

extern "C" {

int32_t kanso_cuda_peer_exchange(kanso_cuda_ctx* ctx, void* const* flags, void* step,
                                 int32_t world, int32_t rank) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "peer_exchange: ctx is NULL");
  ExchangeArgs a;
  int32_t st = exchange_args(ctx, flags, step, world, rank, &a, "peer_exchange");
  if (st) return st;
  KANSO_CUDA_TRY(ctx, launch_dependent(ctx, peer_exchange_kernel, dim3(1), dim3(32), 0, a),
                 "peer_exchange launch");
  return after_launch(ctx, "peer_exchange");
}

int32_t kanso_cuda_shard_range(int64_t n, int32_t rank, int32_t world, int64_t align,
                               int64_t* begin, int64_t* count) {
  if (!begin || !count || world < 1 || rank < 0 || rank >= world || align < 1 || n < 0 ||
      n % align != 0)
    return KANSO_ERR_SHAPE;
  const int64_t units = n / align;
  const int64_t b = units * rank / world, e = units * (rank + 1) / world;
  *begin = b * align;
  *count = (e - b) * align;
  return KANSO_OK;
}

int32_t kanso_cuda_shard_k_repack(const void* host_bytes, int32_t dtype, int64_t rows,
                                  int64_t cols, int64_t col_begin, int64_t col_count,
                                  void* out_bytes, size_t out_capacity) {
  int blk, bb;
  if (dtype == KANSO_DTYPE_Q8_0) {
    blk = 32;
    bb = Q8_BYTES;
  } else if (dtype == KANSO_DTYPE_Q4_K) {
    blk = 256;
    bb = Q4K_BYTES;
  } else {
    return KANSO_ERR_UNSUPPORTED;
  }
  if (!host_bytes || !out_bytes || rows < 0 || cols % blk || col_begin % blk || col_count % blk ||
      col_begin < 0 || col_count < 0 || col_begin + col_count > cols)
    return KANSO_ERR_SHAPE;
  const size_t row_in = (size_t)(cols / blk) * bb, row_out = (size_t)(col_count / blk) * bb;
  if (out_capacity < row_out * (size_t)rows) return KANSO_ERR_SHAPE;
  const uint8_t* src = (const uint8_t*)host_bytes + (size_t)(col_begin / blk) * bb;
  uint8_t* dst = (uint8_t*)out_bytes;
  for (int64_t r = 0; r < rows; ++r) std::memcpy(dst + r * row_out, src + r * row_in, row_out);
  return KANSO_OK;
}

int32_t kanso_cuda_linear_scatter_out(kanso_cuda_ctx* ctx, const kanso_cuda_weight* w,
                                      const float* x, int64_t M, float* const* y_out,
                                      int32_t n_out, int64_t n_total, int64_t row_offset,
                                      int32_t act_mode) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "linear_scatter_out: ctx is NULL");
  if (!w || !x || !y_out) return fail(ctx, KANSO_ERR_SHAPE, "linear_scatter_out: NULL pointer");
  if (n_out < 1 || n_out > 8)
    return fail(ctx, KANSO_ERR_UNSUPPORTED, "linear_scatter_out: %d result buffers (1..8)", n_out);
  if (row_offset < 0 || row_offset + w->rows > n_total)
    return fail(ctx, KANSO_ERR_SHAPE, "linear_scatter_out: rows [%lld, %lld) outside [0, %lld)",
                (long long)row_offset, (long long)(row_offset + w->rows), (long long)n_total);
  for (int o = 0; o < n_out; ++o)
    if (!y_out[o]) return fail(ctx, KANSO_ERR_SHAPE, "linear_scatter_out: y_out[%d] is NULL", o);
  if (M <= 0) return M == 0 ? KANSO_OK : fail(ctx, KANSO_ERR_SHAPE, "linear_scatter_out: M < 0");
  if (w->dtype == KANSO_DTYPE_Q4_K && act_mode == KANSO_ACT_F32 && M <= 8) {
    bool handled = false;
    int32_t st = q4k_direct_matmul_out(ctx, w->dev, x, nullptr, M, w->rows, w->cols, &handled,
                                       y_out, n_out, n_total, row_offset);
    if (st || handled) return st;
  }
  // other shapes: compute the slice into scratch, then one small scatter kernel
  float* tmp = nullptr;
  {
    // the matmul kernels may use the context scratch themselves: keep this slice in the
    // device staging buffer
    int32_t st = ctx_stage_dev(ctx, sizeof(float) * (size_t)M * w->rows);
    if (st) return st;
    tmp = (float*)ctx->stage_dev;
  }
  int32_t st = matmul_dispatch(ctx, w->dtype, w->dev, x, tmp, M, w->rows, w->cols, act_mode);
  if (st) return st;
  ScatterArgs sa;
  sa.n_out = n_out;
  for (int o = 0; o < 8; ++o) sa.out[o] = o < n_out ? y_out[o] : nullptr;
  const int64_t n = M * w->rows;
  scatter_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(tmp, sa, M, w->rows,
                                                                           n_total, row_offset);
  return after_launch(ctx, "linear_scatter_out");
}

int32_t kanso_cuda_sum_shards(kanso_cuda_ctx* ctx, const float* parts, int64_t M, int64_t rows,
                              int32_t world, float* y) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "sum_shards: ctx is NULL");
  if (!parts || !y) return fail(ctx, KANSO_ERR_SHAPE, "sum_shards: NULL pointer");
  if (M < 0 || rows < 0 || world < 1 || world > 64)
    return fail(ctx, KANSO_ERR_SHAPE, "sum_shards: bad shape (M %lld, rows %lld, world %d)",
                (long long)M, (long long)rows, world);
  const int64_t n = M * rows;
  if (n == 0) return KANSO_OK;
  KANSO_CUDA_TRY(ctx,
                 launch_dependent(ctx, sum_shards_kernel, dim3((unsigned)((n + 255) / 256)),
                                  dim3(256), 0, parts, M, rows, world, y),
                 "sum_shards launch");
  return after_launch(ctx, "sum_shards");
}

}  // extern "C"
