// The device side of a sharded layer's exchange, shared by the kernels that publish a slice
// (the Q4_K matmul's own epilogue, the scatter kernel). The protocol is described in
// shard_group.cu.
#pragma once
#include "common.cuh"

#define KANSO_MAX_PEERS 8

namespace kanso {

// What a producing kernel needs to publish its slice and signal the peers.
struct ShardSignal {
  float* out[KANSO_MAX_PEERS];                // buffer 0 of the layer in every rank's region
  unsigned long long* flags[KANSO_MAX_PEERS]; // the layer's flag array in every rank's region
  unsigned long long* step;                   // this rank's step counter of the layer
  unsigned int* ticket;                       // this rank's ticket of the layer
  int64_t buf_stride;                         // floats between the two exchange buffers
  int world, rank;
  int signal;                                 // 0: an earlier pass of a multi-pass matmul
  // The fused tail of the Q4_K matmul (shard_tail below): all rows of all passes, staged in
  // this rank's memory, and what to do with them.
  const float* stage;   // [m_total, n] this rank's slice
  float* y;             // K shard: the summed result [m_total, n]; row shard: unused
  int64_t ld, col0, n;  // row length of an exchange buffer, first column and width of the slice
  int m_total;
  int sum;              // 1: K shard (wait for the peers and add the partial results)
  int* status;          // the context's device status word
};

// The last CTA of the producing grid calls this after every CTA's stores are fenced.
__device__ __forceinline__ void shard_publish(const ShardSignal& s) {
  *s.ticket = 0;  // every CTA has drawn: ready for the next launch
  if (!s.signal) return;
  __threadfence_system();
  const unsigned long long e = *s.step + 1;
  *s.step = e;
  for (int r = 0; r < s.world; ++r)
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(s.flags[r] + s.rank), "l"(e)
                 : "memory");
}

// Called by every CTA of a producing grid after its stores; `s_last` is a shared-memory word.
__device__ __forceinline__ void shard_ticket(const ShardSignal& s, unsigned int total_ctas,
                                             unsigned int* s_last) {
  // One system-scope fence per CTA, not per thread (75 000 of them cost 20 us per launch): the
  // CTA barrier orders every thread's stores before thread 0, whose fence is cumulative over
  // what it has observed, so the stores are performed system-wide before the ticket is drawn.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int drawn = atomicAdd(s.ticket, 1u);
    *s_last = drawn == total_ctas - 1;
    if (*s_last) {
      __threadfence();
      shard_publish(s);
    }
  }
}

// Bounded wait until every peer's slot of this rank's flag array has reached `e` (threads
// 0..world-1 of the CTA poll, 2 s at most).
__device__ __forceinline__ void shard_wait_flags(const unsigned long long* mine, int world,
                                                 unsigned long long e, int* status) {
  if ((int)threadIdx.x < world) {
    unsigned long long t0 = 0, t1, seen;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];"
                   : "=l"(seen)
                   : "l"(mine + threadIdx.x)
                   : "memory");
      if (seen >= e) break;
      // the clock is only read once the flag was found unset (a read costs about 150 ns)
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
      if (t0 == 0) t0 = t1;
      if (t1 - t0 > 2000000000ull) {  // 2 s
        atomicOr(status, (int)DEV_WAIT_TIMEOUT);
        break;
      }
      __nanosleep(32);
    }
  }
  __syncthreads();
}

// The fused tail of a sharded Q4_K matmul with few activation rows, run by the ONE CTA that
// drew the grid's last ticket (every other CTA has stored its rows into `stage`, fenced and
// left, so the kernel after this one may already be fetching its weights): the slice goes into
// the current exchange buffer of every rank with plain stores, one system-scope fence, the
// step advances and the peers are signalled; a K shard then waits for the peers' signals and
// adds the partial results in rank order into y. Compute and collective are one kernel.
__device__ __forceinline__ void shard_tail(const ShardSignal& s) {
  if (!s.signal) return;  // an earlier pass: its rows are published by the last pass
  const unsigned long long e = *s.step + 1;
  const int64_t par = (int64_t)((e - 1) & 1ull) * s.buf_stride;
  const int n = (int)s.n, world = s.world, rank = s.rank;
  // 16-byte moves when every row of the slice starts on a 16-byte boundary in both places
  // (stage rows are n floats apart, buffer rows ld floats, the slice starts at col0)
  const bool vec = ((n | (int)s.col0 | (int)s.ld) & 3) == 0;
  // The slice goes to every PEER's buffer; this rank reads its own part from the stage.
  for (int m = 0; m < s.m_total; ++m) {
    const float* src = s.stage + (int64_t)m * n;
    const int64_t dst = par + (int64_t)m * s.ld + s.col0;
    if (vec) {
      for (int c = 4 * (int)threadIdx.x; c < n; c += 4 * (int)blockDim.x) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(src + c));
        for (int r = 0; r < world; ++r)
          if (r != rank || !s.sum) *reinterpret_cast<float4*>(s.out[r] + dst + c) = v;
      }
    } else {
      for (int c = (int)threadIdx.x; c < n; c += (int)blockDim.x) {
        const float v = __ldcg(src + c);
        for (int r = 0; r < world; ++r)
          if (r != rank || !s.sum) s.out[r][dst + c] = v;
      }
    }
  }
  // one system-scope fence per storing thread, then thread r tells rank r (one store each, in
  // parallel: a release store per peer from one thread would pay a fence per peer)
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < world)
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(s.flags[threadIdx.x] + rank),
                 "l"(e)
                 : "memory");
  if (threadIdx.x == 0) *s.step = e;
  if (!s.sum) return;
  shard_wait_flags(s.flags[rank], world, e, s.status);
  // K shard: the buffer holds `world` slices of n floats per row (slice r from rank r, col0 =
  // rank * n); add them in rank order, this rank's own from the stage
  const float* buf = s.out[rank] + par;
  for (int m = 0; m < s.m_total; ++m) {
    const float* mine = s.stage + (int64_t)m * n;
    const float* row = buf + (int64_t)m * s.ld;
    float* y = s.y + (int64_t)m * n;
    if (vec) {
      for (int c = 4 * (int)threadIdx.x; c < n; c += 4 * (int)blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < world; ++r) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(
              r == rank ? mine + c : row + (int64_t)r * n + c));
          acc.x += v.x;
          acc.y += v.y;
          acc.z += v.z;
          acc.w += v.w;
        }
        *reinterpret_cast<float4*>(y + c) = acc;
      }
    } else {
      for (int c = (int)threadIdx.x; c < n; c += (int)blockDim.x) {
        float acc = 0.f;
        for (int r = 0; r < world; ++r)
          acc += __ldcg(r == rank ? mine + c : row + (int64_t)r * n + c);
        y[c] = acc;
      }
    }
  }
}

}  // namespace kanso