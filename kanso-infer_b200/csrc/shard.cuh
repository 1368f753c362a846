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
  __threadfence_system();  // this thread's stores to the peers are performed system-wide
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int drawn = atomicAdd(s.ticket, 1u);
    *s_last = drawn == total_ctas - 1;
    if (*s_last) {
      __threadfence();
      shard_publish(s);
    }
  }
}

}  // namespace kanso
