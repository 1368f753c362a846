// Decode attention over the int8 KV pool, read through the block table.
//
// Math: cpu_paged_attention (src/metal/paged_attention.rs:84-178) on rows
// dequantised as (f32)q * scale (src/kv_cache/quantized_storage.rs:284-383).
// Nothing is materialised: no dequantised history, no score matrix.
//
// Stage 1, one CTA per (context partition, kv head, sequence): all query heads
// of the GQA group are served together so each K/V byte is read once.
//   * QK: one thread per token. The query rows are split into two int8 planes
//     (q ~= d*(hi + lo/254)), so the dot with the int8 K row is dp4a on the
//     packed bytes; the token's f32 K scale, the query scale and the softmax
//     scale multiply the int32 sum once.
//   * online softmax inside the partition (max, exp, sum) in shared memory.
//   * PV: threads tile (8-dim word, token slice); V bytes are widened with one
//     byte-permute each and accumulated in f32 with weight p * v_scale.
//   Emits the unnormalised accumulator and (max, sum) per partition.
// Stage 2 merges the partitions: out = sum acc_p e^{m_p-M} / sum l_p e^{m_p-M}. With a ticket
// array the merge runs inside stage 1, in the CTA that finishes last for its (sequence, kv head):
// every CTA publishes its partials, fences, and takes a ticket; the one that draws the last
// ticket reads all partials back. Nothing waits on anything, so there is no spin to bound.
#include <cuda_fp8.h>

#include <mutex>
#include <vector>

#include "glue.cuh"
#include "kv_pool.h"

namespace kanso {

constexpr int PA_THREADS = 128;
constexpr int PA_BIG_THREADS = 256;  // partitions of 256 tokens and more
__host__ inline uint32_t pa_threads(uint32_t pt) { return pt >= 256 ? PA_BIG_THREADS : PA_THREADS; }
constexpr int PA_MAX_GROUP = 8;      // MAX_KV_GROUP_SIZE, src/metal/paged_attention.rs:10
constexpr int PA_MAX_HEAD_DIM = 256; // MAX_HEAD_DIM, src/metal/paged_attention.rs:8

struct PaArgs {
  KvGeom g;
  uint32_t layer;
  const float* q;
  const uint32_t* tables;
  const uint32_t* lens;
  float* out;
  float* part_acc;  // [seq][head][part][hd]
  float* part_ml;   // [seq][head][part][2]
  uint32_t num_heads, max_blocks, part_tokens, num_parts;
  float scale;
  int* status;
  uint32_t* tickets;  // [seq][kv head], zero between calls; nullptr = separate stage-2 launch
  // Chunked prefill: grid row `seq` is one query token; row_seq[seq] names the sequence whose
  // block table it walks (nullptr: the row is the sequence, as in decode).
  const uint32_t* row_seq;
  // Decode-step fusion (src/model.rs:1141-1207), off when k_new is nullptr: q arrives
  // un-rotated and is rotated as it is staged; the CTA whose partition holds the newest token
  // (position context_len - 1) rotates that token's K, quantises K and V and stores them in
  // the pool slot slots[seq] before it reads the partition.
  const float* k_new;  // [seq][kv head][hd]
  const float* v_new;
  const uint32_t* positions;
  const uint32_t* slots;
  const float* cos_t;  // [table_len][hd / 2]
  const float* sin_t;
  int table_len;
  // Batched decode: the output is ALSO written as the f16 hi/lo activation tile that the
  // o-projection's tensor-core GEMM reads (stage of 64 k-values, plane, k-chunk of 8, row:
  // the layout of tc_pack_activations_kernel), which saves that GEMM its pack launch. xp_mt =
  // rows of the tile (the batch rounded up to 16; the rows past the batch are zeroed here).
  __half* xp;  // nullptr: off
  uint32_t xp_mt;
};

// One output element into the packed tile: row = sequence, kk = head * head_dim + d.
__device__ __forceinline__ void pa_store_packed(const PaArgs& a, uint32_t row, uint32_t kk,
                                                float v) {
  const __half hi = __float2half_rn(v);
  const __half lo = __float2half_rn(v - __half2float(hi));
  const uint32_t c = (kk >> 3) & 7u, e = kk & 7u;
  __half* base = a.xp + (size_t)(kk >> 6) * (128u * a.xp_mt);
  base[((size_t)c * a.xp_mt + row) * 8 + e] = hi;
  base[((size_t)(8 + c) * a.xp_mt + row) * 8 + e] = lo;
}
// The tile's rows past the batch, for the k range of one KV head's query heads.
__device__ __forceinline__ void pa_zero_packed_rows(const PaArgs& a, uint32_t rows, uint32_t k0,
                                                    uint32_t nk, uint32_t tid, uint32_t nt) {
  const uint32_t pad = a.xp_mt - rows;
  for (uint32_t i = tid; i < pad * nk; i += nt)
    pa_store_packed(a, rows + i / nk, k0 + i % nk, 0.f);
}

// (block, offset) of token i = i0, i0 + step, ... inside a partition, without a division per
// token (the block size is a run-time value).
struct PaTokenIter {
  uint32_t blk, off, adv_blk, adv_off, bs;
  __device__ __forceinline__ PaTokenIter(uint32_t i0, uint32_t step, uint32_t block_size)
      : blk(i0 / block_size), off(i0 % block_size), adv_blk(step / block_size),
        adv_off(step % block_size), bs(block_size) {}
  __device__ __forceinline__ void next() {
    blk += adv_blk;
    off += adv_off;
    if (off >= bs) {
      off -= bs;
      ++blk;
    }
  }
};

__device__ __forceinline__ float s8_to_f32(uint32_t biased_word, int k) {
  // biased_word = bytes ^ 0x80 (value + 128). Put byte k into the low mantissa bits of 2^23.
  uint32_t bits = __byte_perm(biased_word, 0x4B000000u, 0x7540 | k);
  return __uint_as_float(bits) - 8388736.0f;  // 2^23 + 128
}

// The context length a launch can serve: the table's capacity (max_blocks * block_size; the
// reference rejects a longer context on the host, src/metal/paged_attention.rs:343-355) and the
// window of partitions this grid was sized for. A device length beyond either is cut off there
// (the reference's kernel clamps its partition range the same way,
// src/metal/kernels/paged_attention_v2.metal:86-87) and reported through the status word, so no
// table entry, partial or scratch cell outside the launch's own range is ever addressed.
__device__ __forceinline__ uint32_t pa_clamp_ctx(const PaArgs& a, uint32_t ctx, bool report) {
  const uint64_t cap = (uint64_t)a.max_blocks * a.g.block_size;
  const uint64_t window = (uint64_t)a.num_parts * a.part_tokens;
  const uint64_t lim = cap < window ? cap : window;
  if ((uint64_t)ctx > lim) {
    if (report) atomicOr(a.status, DEV_BAD_INDEX);
    ctx = (uint32_t)lim;
  }
  return ctx;
}

// Eight E4M3 values (two words) -> f32, exactly (every E4M3 number is an f16 number).
__device__ __forceinline__ void e4m3x4_to_f32(uint32_t w, float* f) {
  const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xFFFFu), __NV_E4M3);
  const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3);
  const float2 a = __half22float2(__half2(lo)), b = __half22float2(__half2(hi));
  f[0] = a.x;
  f[1] = a.y;
  f[2] = b.x;
  f[3] = b.y;
}

// Bytes of the first shared-memory region of stage 1: the partition's records, or the PV
// reduction scratch [NT / (hd/8) slices][G][hd] f32 that later overlays them, whichever is larger.
__host__ __device__ inline uint32_t pa_region0_bytes(uint32_t record_bytes, uint32_t G, uint32_t hd,
                                                     uint32_t threads) {
  uint32_t red = (threads / (hd / 8)) * G * hd * 4;
  if (red < 128) red = 128;
  const uint32_t r = record_bytes > red ? record_bytes : red;
  return (r + 15u) & ~15u;
}

// NT = threads per CTA. FP8: the pool holds E4M3 bit patterns with power-of-two scales
// (src/kv_cache/quantized_storage.rs:470-484); the query then stays in f32 and the products are
// f32 multiply-adds on the exactly converted K and V values. Otherwise int8 with dp4a.
template <int G, int NT, bool FP8>
__global__ void __launch_bounds__(NT) paged_attn_stage1(const PaArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch_dependents();
  const uint32_t hd = a.g.head_dim, bs = a.g.block_size;
  const uint32_t part = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  // Inside the decode step (fused mode) the context lengths, positions, slots and the block
  // table are inputs of the whole step, written before its first kernel, and the cache rows of
  // earlier steps do not depend on the kernel before this one either: all of them are read
  // before the wait, and only q and the new K/V rows, which that kernel produces, after it.
  const bool fused = a.k_new != nullptr;
  uint32_t ctx = 0, pos = 0;
  if (fused) {
    ctx = a.lens[seq];
    pos = a.positions[seq];
  }
  if (!fused) {
    pdl_wait();  // q, the table and the lengths may come from earlier kernels
    ctx = a.lens[seq];
  }
  ctx = pa_clamp_ctx(a, ctx, part == 0 && kvh == 0 && threadIdx.x == 0);
  const uint32_t t0 = part * a.part_tokens;
  if (ctx == 0 && a.tickets && part == 0) {
    // the CPU statement leaves zeros (src/metal/paged_attention.rs:112-115)
    float* o = a.out + ((size_t)seq * a.num_heads + (size_t)kvh * G) * hd;
    for (uint32_t e = threadIdx.x; e < G * hd; e += NT) o[e] = 0.f;
    if (a.xp) {
      pdl_wait();  // the tile's last reader is an earlier kernel of the stream
      for (uint32_t e = threadIdx.x; e < G * hd; e += NT)
        pa_store_packed(a, seq, kvh * G * hd + e, 0.f);
      if (seq == 0) pa_zero_packed_rows(a, gridDim.z, kvh * G * hd, G * hd, threadIdx.x, NT);
    }
  }
  if (t0 >= ctx) return;
  const uint32_t n = min(a.part_tokens, ctx - t0);
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  // shared: the partition's block records (K, V and their scales, as they lie in the pool),
  // mbarrier, q planes, q scales, block ids, probabilities, reduction scratch
  const uint32_t max_blk = (a.part_tokens + bs - 1) / bs;
  uint8_t* tiles = smem;                                                    // 16-byte records
  // The PV reduction scratch lies over the records: it is written only after every thread has
  // finished reading them, and the region is sized for the larger of the two.
  uint64_t* bar = reinterpret_cast<uint64_t*>(
      tiles + pa_region0_bytes(max_blk * a.g.rec_bytes, G, hd, NT));
  int8_t* qhi = reinterpret_cast<int8_t*>(bar + 2);          // [G][hd]
  int8_t* qlo = qhi + G * hd;                                // [G][hd]
  float* qf = reinterpret_cast<float*>(qhi);                 // FP8: [G][hd] f32 instead of the planes
  float* qd = reinterpret_cast<float*>(qhi + (FP8 ? 4 : 2) * G * hd);  // [G] (d/254)
  uint32_t* blk = reinterpret_cast<uint32_t*>(qd + PA_MAX_GROUP);  // [part_tokens/bs + 1]
  const uint32_t nblk_part = (max_blk + 4) & ~3u;
  float* prob = reinterpret_cast<float*>(blk + nblk_part);   // [G][part_tokens]
  float* red = reinterpret_cast<float*>(tiles);              // PV scratch (see above)

  // physical blocks of this partition (bounds-checked once); partitions start on a block
  const uint32_t nb = (n + bs - 1) / bs;
  const uint32_t tseq = a.row_seq ? a.row_seq[seq] : seq;
  {
    const uint32_t first_blk = t0 / bs;
    for (uint32_t b = tid; b < nb; b += NT) {
      uint32_t phys = a.tables[(size_t)tseq * a.max_blocks + first_blk + b];
      if (phys >= a.g.num_blocks) {
        atomicOr(a.status, DEV_BAD_INDEX);
        phys = 0;
      }
      blk[b] = phys;
    }
  }
  // RoPE factors of this sequence's position, and the pool slot of its newest token
  __shared__ float s_cos[PA_MAX_HEAD_DIM / 2], s_sin[PA_MAX_HEAD_DIM / 2];
  uint32_t new_slot = 0;
  if (fused) {
    if (pos >= (uint32_t)a.table_len) {
      if (tid == 0) atomicOr(a.status, DEV_BAD_INDEX);
      pos = 0;
    }
    for (uint32_t j = tid; j < hd / 2; j += NT) {
      s_cos[j] = a.cos_t[(size_t)pos * (hd / 2) + j];
      s_sin[j] = a.sin_t[(size_t)pos * (hd / 2) + j];
    }
    new_slot = a.slots[seq];
  }
  if (tid == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  __syncthreads();  // block ids, RoPE factors and the barrier are in shared memory

  // One bulk copy per block record brings K, V and both scale rows of 16 tokens (2176 bytes at
  // head_dim 64) into shared memory; the whole partition is in flight at once.
  if (warp == 0) {
    if (lane == 0) mbar_arrive_expect_tx(bar, nb * a.g.rec_bytes);
    __syncwarp();
    for (uint32_t b = lane; b < nb; b += 32)
      bulk_g2s(tiles + (size_t)b * a.g.rec_bytes,
               a.g.pool + a.g.rec_offset(a.layer, blk[b], kvh), a.g.rec_bytes, bar);
  }
  // position of the newest token inside this partition (fused mode), else out of range
  const uint32_t i_new = (fused && ctx - 1 >= t0 && ctx - 1 < t0 + n) ? ctx - 1 - t0 : 0xFFFFFFFFu;
  if (fused) pdl_wait();  // q and the new K/V rows come from the kernel before this one
  if (a.xp && seq == 0 && part == 0)
    pa_zero_packed_rows(a, gridDim.z, kvh * G * hd, G * hd, threadIdx.x, NT);

  // --- stage the query heads of this group: warp w quantises heads w, w+4, ...
  constexpr int QE = PA_MAX_HEAD_DIM / 32;
  const uint32_t half = hd / 2;
  // element d of a head after rotate-half RoPE; multiplies and adds round separately, as
  // the reference's tensor ops do (the stored K bytes must equal the CPU path's)
  auto roped = [&](const float* row, uint32_t d) {
    if (!fused) return row[d];
    const uint32_t j = d < half ? d : d - half;
    const float x0 = row[j], x1 = row[j + half], c_ = s_cos[j], s_ = s_sin[j];
    return d < half ? __fsub_rn(__fmul_rn(x0, c_), __fmul_rn(x1, s_))
                    : __fadd_rn(__fmul_rn(x0, s_), __fmul_rn(x1, c_));
  };
  // the newest token's K (warp 0) and V (warp 1): rotated and quantised in registers first
  // (quantize_head_slice, src/kv_cache/quantized_storage.rs:452-469), stored once the copies
  // above have landed
  const bool writer = i_new != 0xFFFFFFFFu && warp < 2;
  float ne[QE];
  float new_scale = 1.0f, new_inv = 1.0f;
  if (writer) {
    const bool is_k = warp == 0;
    const float* src = (is_k ? a.k_new : a.v_new) + ((size_t)seq * a.g.kv_heads + kvh) * hd;
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < QE; ++i) {
      const uint32_t d = lane + 32 * i;
      ne[i] = 0.f;
      if (d < hd) {
        ne[i] = is_k ? roped(src, d) : src[d];
        amax = fmaxf(amax, fabsf(ne[i]));
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    new_scale = kv_scale_of(amax, FP8);
    new_inv = __fdiv_rn(1.0f, new_scale);
  }
  for (int gq = warp; gq < G; gq += NT / 32) {
    const float* qrow = a.q + ((size_t)seq * a.num_heads + (size_t)kvh * G + gq) * hd;
    float qe[QE];  // this lane's elements of the head, loaded (and rotated) once
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < QE; ++i) {
      const uint32_t d = lane + 32 * i;
      qe[i] = d < hd ? roped(qrow, d) : 0.f;
      amax = fmaxf(amax, fabsf(qe[i]));
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if (FP8) {
#pragma unroll
      for (int i = 0; i < QE; ++i) {
        const uint32_t d = lane + 32 * i;
        if (d < hd) qf[gq * hd + d] = qe[i];
      }
      continue;
    }
    float d_ = amax / 127.0f;
    float id = d_ != 0.f ? 1.0f / d_ : 0.f;
#pragma unroll
    for (int i = 0; i < QE; ++i) {
      const uint32_t d = lane + 32 * i;
      if (d < hd) {
        float x = qe[i];
        float h = fminf(fmaxf(rintf(x * id), -127.f), 127.f);
        float l = fminf(fmaxf(rintf(fmaf(-d_, h, x) * (254.0f * id)), -127.f), 127.f);
        qhi[gq * hd + d] = (int8_t)h;
        qlo[gq * hd + d] = (int8_t)l;
      }
    }
    if (lane == 0) qd[gq] = d_ * (1.0f / 254.0f);
  }
  // the partition's records are in shared memory from here on (bounded wait: a copy that
  // never lands is reported through the status word, the CTA carries on with what it has)
  if (!mbar_wait_bounded(bar, 0) && tid == 0) atomicOr(a.status, DEV_WAIT_TIMEOUT);
  if (writer) {
    const bool is_k = warp == 0;
    const uint32_t block = new_slot / bs, off = new_slot % bs;
    if (block >= a.g.num_blocks) {
      if (lane == 0) atomicOr(a.status, DEV_BAD_INDEX);
    } else {
      uint8_t* rec = a.g.pool + a.g.rec_offset(a.layer, block, kvh);
      uint8_t* tile = tiles + (size_t)(i_new / bs) * a.g.rec_bytes;  // this CTA's own copy
      const uint32_t row = (is_k ? a.g.k_off() : a.g.v_off());
      int8_t* dst = reinterpret_cast<int8_t*>(rec + row) + (size_t)off * hd;
      int8_t* mine = reinterpret_cast<int8_t*>(tile + row) + (size_t)(i_new % bs) * hd;
#pragma unroll
      for (int i = 0; i < QE; ++i) {
        const uint32_t d = lane + 32 * i;
        if (d < hd) {
          const float scaled = __fmul_rn(ne[i], new_inv);
          const int8_t qv =
              FP8 ? (int8_t)__nv_cvt_float_to_fp8(scaled, __NV_SATFINITE, __NV_E4M3)
                  : (int8_t)fminf(fmaxf(roundf(scaled), -127.f), 127.f);
          dst[d] = qv;
          mine[d] = qv;
        }
      }
      if (lane == 0) {
        const uint32_t so = is_k ? a.g.ks_off() : a.g.vs_off();
        reinterpret_cast<float*>(rec + so)[off] = new_scale;
        reinterpret_cast<float*>(tile + so)[i_new % bs] = new_scale;
      }
    }
  }
  __syncthreads();

  // --- QK: one thread per token, rows read from the staged records. Lanes start at different
  // 16-byte chunks of their rows (rows are 64 bytes apart at head_dim 64: without the rotation
  // eight lanes would share two banks).
  const uint32_t nchunk = hd / 16;
  float lmax[G];
#pragma unroll
  for (int gq = 0; gq < G; ++gq) lmax[gq] = -INFINITY;
  PaTokenIter qk_it(tid, NT, bs);
  for (uint32_t i = tid; i < n; i += NT, qk_it.next()) {
    const uint8_t* rec = tiles + (size_t)qk_it.blk * a.g.rec_bytes;
    const uint32_t off = qk_it.off;
    const uint4* krow = reinterpret_cast<const uint4*>(rec + a.g.k_off() + (size_t)off * hd);
    const float ksc = reinterpret_cast<const float*>(rec + a.g.ks_off())[off];
    if (FP8) {
      float dot[G];
#pragma unroll
      for (int gq = 0; gq < G; ++gq) dot[gq] = 0.f;
      for (uint32_t cc = 0; cc < nchunk; ++cc) {
        const uint32_t c = (cc + (i >> 1)) & (nchunk - 1);
        const uint4 kw = krow[c];
        float kf[16];
        e4m3x4_to_f32(kw.x, kf);
        e4m3x4_to_f32(kw.y, kf + 4);
        e4m3x4_to_f32(kw.z, kf + 8);
        e4m3x4_to_f32(kw.w, kf + 12);
#pragma unroll
        for (int gq = 0; gq < G; ++gq) {
          const float4* q4 = reinterpret_cast<const float4*>(qf + gq * hd + 16 * c);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 qq = q4[j];
            dot[gq] = fmaf(kf[4 * j], qq.x, dot[gq]);
            dot[gq] = fmaf(kf[4 * j + 1], qq.y, dot[gq]);
            dot[gq] = fmaf(kf[4 * j + 2], qq.z, dot[gq]);
            dot[gq] = fmaf(kf[4 * j + 3], qq.w, dot[gq]);
          }
        }
      }
#pragma unroll
      for (int gq = 0; gq < G; ++gq) {
        const float sc = dot[gq] * ksc * a.scale;
        prob[gq * a.part_tokens + i] = sc;
        lmax[gq] = fmaxf(lmax[gq], sc);
      }
      continue;
    }
    int ih[G], il[G];
#pragma unroll
    for (int gq = 0; gq < G; ++gq) ih[gq] = il[gq] = 0;
    for (uint32_t cc = 0; cc < nchunk; ++cc) {
      const uint32_t c = (cc + (i >> 1)) & (nchunk - 1);
      const uint4 kw = krow[c];
#pragma unroll
      for (int gq = 0; gq < G; ++gq) {
        const uint4 h4 = *reinterpret_cast<const uint4*>(qhi + gq * hd + 16 * c);
        const uint4 l4 = *reinterpret_cast<const uint4*>(qlo + gq * hd + 16 * c);
        ih[gq] = dp4a_ss((int)kw.x, (int)h4.x, ih[gq]);
        ih[gq] = dp4a_ss((int)kw.y, (int)h4.y, ih[gq]);
        ih[gq] = dp4a_ss((int)kw.z, (int)h4.z, ih[gq]);
        ih[gq] = dp4a_ss((int)kw.w, (int)h4.w, ih[gq]);
        il[gq] = dp4a_ss((int)kw.x, (int)l4.x, il[gq]);
        il[gq] = dp4a_ss((int)kw.y, (int)l4.y, il[gq]);
        il[gq] = dp4a_ss((int)kw.z, (int)l4.z, il[gq]);
        il[gq] = dp4a_ss((int)kw.w, (int)l4.w, il[gq]);
      }
    }
#pragma unroll
    for (int gq = 0; gq < G; ++gq) {
      float sc = (float)(ih[gq] * 254 + il[gq]) * (qd[gq] * ksc) * a.scale;
      prob[gq * a.part_tokens + i] = sc;
      lmax[gq] = fmaxf(lmax[gq], sc);
    }
  }
  // --- softmax inside the partition; the G heads share each block-wide reduction
  __shared__ float s_redm[PA_MAX_GROUP * (NT / 32)], s_reds[PA_MAX_GROUP * (NT / 32)];
  float pmax[G], psum[G];
#pragma unroll
  for (int gq = 0; gq < G; ++gq) {
    float m = lmax[gq];
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (lane == 0) s_redm[gq * (NT / 32) + warp] = m;
  }
  __syncthreads();
#pragma unroll
  for (int gq = 0; gq < G; ++gq) {
    float m = s_redm[gq * (NT / 32)];
#pragma unroll
    for (int w = 1; w < NT / 32; ++w) m = fmaxf(m, s_redm[gq * (NT / 32) + w]);
    pmax[gq] = m;
    psum[gq] = 0.f;
  }
  PaTokenIter sm_it(tid, NT, bs);
  for (uint32_t i = tid; i < n; i += NT, sm_it.next()) {
    const uint8_t* rec = tiles + (size_t)sm_it.blk * a.g.rec_bytes;
    const float vsc = reinterpret_cast<const float*>(rec + a.g.vs_off())[sm_it.off];
#pragma unroll
    for (int gq = 0; gq < G; ++gq) {
      float e = expf(prob[gq * a.part_tokens + i] - pmax[gq]);
      psum[gq] += e;
      prob[gq * a.part_tokens + i] = e * vsc;  // weight applied to the raw int8 V row
    }
  }
#pragma unroll
  for (int gq = 0; gq < G; ++gq) {
    float t = psum[gq];
#pragma unroll
    for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
    if (lane == 0) s_reds[gq * (NT / 32) + warp] = t;
  }
  __syncthreads();  // also: every probability is written before PV reads them
#pragma unroll
  for (int gq = 0; gq < G; ++gq) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < NT / 32; ++w) t += s_reds[gq * (NT / 32) + w];
    psum[gq] = t;
  }

  // --- PV: thread = (8 dims = one 64-bit word c of the V row, token slice)
  const uint32_t dwords = hd / 8;
  const uint32_t nslice = NT / dwords;  // hd in {16..256} -> dwords in {2..32}
  const uint32_t c = tid % dwords, slice = tid / dwords;
  float acc[G][8];
#pragma unroll
  for (int gq = 0; gq < G; ++gq)
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[gq][k] = 0.f;
  PaTokenIter pv_it(slice, nslice, bs);
  for (uint32_t i = slice; i < n; i += nslice, pv_it.next()) {
    const uint8_t* rec = tiles + (size_t)pv_it.blk * a.g.rec_bytes;
    const uint2 vw =
        reinterpret_cast<const uint2*>(rec + a.g.v_off() + (size_t)pv_it.off * hd)[c];
    float f[8];
    if (FP8) {
      e4m3x4_to_f32(vw.x, f);
      e4m3x4_to_f32(vw.y, f + 4);
    } else {
      const uint32_t lo = vw.x ^ 0x80808080u, hi = vw.y ^ 0x80808080u;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        f[k] = s8_to_f32(lo, k);
        f[4 + k] = s8_to_f32(hi, k);
      }
    }
#pragma unroll
    for (int gq = 0; gq < G; ++gq) {
      const float p = prob[gq * a.part_tokens + i];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[gq][k] = fmaf(p, f[k], acc[gq][k]);
    }
  }
  // reduce over token slices through shared memory: red[slice][G][hd]
  __syncthreads();  // every thread is done with the records the scratch overlays
  float4* red4 = reinterpret_cast<float4*>(red);
#pragma unroll
  for (int gq = 0; gq < G; ++gq) {
    red4[((slice * G + gq) * dwords + c) * 2] =
        make_float4(acc[gq][0], acc[gq][1], acc[gq][2], acc[gq][3]);
    red4[((slice * G + gq) * dwords + c) * 2 + 1] =
        make_float4(acc[gq][4], acc[gq][5], acc[gq][6], acc[gq][7]);
  }
  __syncthreads();
  // partitions that exist in this grid (a context longer than the host said is cut off there)
  const uint32_t np = min((ctx + a.part_tokens - 1) / a.part_tokens, a.num_parts);
  const bool single = a.tickets && np == 1;  // the only partition: normalise and finish here
  for (uint32_t e = tid; e < G * hd; e += NT) {
    float s = 0.f;
    for (uint32_t sl = 0; sl < nslice; ++sl) s += red[sl * G * hd + e];
    const uint32_t gq = e / hd, d = e % hd;
    const size_t head = (size_t)seq * a.num_heads + (size_t)kvh * G + gq;
    if (single) {
      float l = 0.f;
#pragma unroll
      for (int k = 0; k < G; ++k)
        if (k == (int)gq) l = psum[k];
      const float o = l > 0.f ? s / l : 0.f;
      a.out[head * hd + d] = o;
      if (a.xp) pa_store_packed(a, seq, (kvh * G + gq) * hd + d, o);
    } else {
      a.part_acc[(head * a.num_parts + part) * hd + d] = s;
    }
  }
  if (single) return;
  if (tid < G) {
    const size_t head = (size_t)seq * a.num_heads + (size_t)kvh * G + tid;
    float m = 0.f, l = 0.f;
#pragma unroll
    for (int gq = 0; gq < G; ++gq)
      if (gq == tid) {
        m = pmax[gq];
        l = psum[gq];
      }
    a.part_ml[(head * a.num_parts + part) * 2 + 0] = m;
    a.part_ml[(head * a.num_parts + part) * 2 + 1] = l;
  }
  if (!a.tickets) return;  // a separate stage-2 launch merges

  // --- merge, by the CTA that draws the last ticket of this (sequence, kv head)
  __shared__ uint32_t s_last;
  // This CTA's partials must be visible device-wide before its ticket is drawn. One fence by
  // the thread that draws it is enough: the block barrier orders every thread's stores before
  // that thread, and its fence is cumulative over what it has observed (256 fences per CTA
  // showed up as 0.47 membar stall cycles per issued instruction).
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    uint32_t* ticket = a.tickets + (size_t)seq * a.g.kv_heads + kvh;
    const uint32_t drawn = atomicAdd(ticket, 1u);
    s_last = drawn == np - 1;
    if (s_last) *ticket = 0;  // every CTA of the group has drawn: ready for the next call
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // Each thread merges its output elements on its own: the (max, sum) pairs and the
  // accumulators of up to 16 partitions are requested together (one trip to L2), then folded
  // in with the running-maximum form of the softmax merge.
  for (uint32_t e = tid; e < G * hd; e += NT) {
    const uint32_t gq = e / hd, d = e % hd;
    const size_t head = (size_t)seq * a.num_heads + (size_t)kvh * G + gq;
    const float* ml = a.part_ml + head * a.num_parts * 2;
    const float* pa = a.part_acc + head * a.num_parts * hd + d;
    float M = -INFINITY, s = 0.f, l = 0.f;
    for (uint32_t p0 = 0; p0 < np; p0 += 16) {
      float2 mlv[16];
      float av[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const uint32_t pp = min(p0 + k, np - 1);
        mlv[k] = __ldcg(reinterpret_cast<const float2*>(ml) + pp);
        av[k] = __ldcg(pa + (size_t)pp * hd);
      }
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        if (p0 + k < np) {
          const float Mn = fmaxf(M, mlv[k].x);
          const float so = expf(M - Mn), sn = expf(mlv[k].x - Mn);
          s = s * so + av[k] * sn;
          l = l * so + mlv[k].y * sn;
          M = Mn;
        }
      }
    }
    const float o = l > 0.f ? s / l : 0.f;
    a.out[head * hd + d] = o;
    if (a.xp) pa_store_packed(a, seq, (kvh * G + gq) * hd + d, o);
  }
}

// Stage 2: merge the partitions of one (sequence, head)
// (paged_attention_v2_reduce_kernel's role, src/metal/kernels/paged_attention_v2.metal:154-205).
__global__ void paged_attn_stage2(const PaArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t head = blockIdx.x, seq = blockIdx.y, hd = a.g.head_dim;
  // the same cut-off as stage 1: only partitions that stage 1 wrote are read
  const uint32_t ctx = pa_clamp_ctx(a, a.lens[seq], false);
  const size_t hidx = (size_t)seq * a.num_heads + head;
  float* o = a.out + hidx * hd;
  if (ctx == 0) {  // the CPU statement leaves zeros (src/metal/paged_attention.rs:112-115)
    for (uint32_t d = threadIdx.x; d < hd; d += blockDim.x) o[d] = 0.f;
    return;
  }
  const uint32_t np = min((ctx + a.part_tokens - 1) / a.part_tokens, a.num_parts);
  const float* ml = a.part_ml + hidx * a.num_parts * 2;
  float M = -INFINITY;
  for (uint32_t p = 0; p < np; ++p) M = fmaxf(M, ml[2 * p]);
  float denom = 0.f;
  for (uint32_t p = 0; p < np; ++p) denom += ml[2 * p + 1] * expf(ml[2 * p] - M);
  const float inv = denom > 0.f ? 1.0f / denom : 0.f;
  for (uint32_t d = threadIdx.x; d < hd; d += blockDim.x) {
    float s = 0.f;
    for (uint32_t p = 0; p < np; ++p)
      s += a.part_acc[(hidx * a.num_parts + p) * hd + d] * expf(ml[2 * p] - M);
    o[d] = s * inv;
  }
}

static int32_t validate_params(const kanso_paged_attention_params* p, char* msg, size_t n) {
  auto bad = [&](const char* fmt, unsigned a0 = 0, unsigned a1 = 0) {
    if (msg && n) snprintf(msg, n, fmt, a0, a1);
    return KANSO_ERR_UNSUPPORTED;
  };
  if (!p) return bad("paged attention: params is NULL");
  if (p->num_seqs == 0 || p->num_heads == 0 || p->num_kv_heads == 0)
    return bad("paged attention: empty shape");
  if (p->num_heads % p->num_kv_heads != 0)
    return bad("paged attention: num_heads %u not divisible by num_kv_heads %u", p->num_heads,
               p->num_kv_heads);
  unsigned group = p->num_heads / p->num_kv_heads;
  if (group > PA_MAX_GROUP)
    return bad("paged attention: GQA group size %u exceeds kernel limit %u", group, PA_MAX_GROUP);
  if (p->head_dim == 0 || p->head_dim > PA_MAX_HEAD_DIM)
    return bad("paged attention: head_dim %u outside kernel range 1..=%u", p->head_dim,
               PA_MAX_HEAD_DIM);
  if (p->block_size == 0 || p->max_num_blocks_per_seq == 0)
    return bad("paged attention: block_size %u / max_num_blocks_per_seq %u must be non-zero",
               p->block_size, p->max_num_blocks_per_seq);
  uint64_t cap = (uint64_t)p->max_num_blocks_per_seq * p->block_size;
  if (cap > 0xFFFFFFFFull) cap = 0xFFFFFFFFull;
  uint64_t parts = (cap + 255) / 256;
  if (parts < 1) parts = 1;
  if ((uint64_t)p->num_seqs * p->num_heads * parts * p->head_dim > (1ull << 31))
    return bad("paged attention: partial elements exceed 32-bit kernel indexing");
  return KANSO_OK;
}

// Dynamic shared memory of stage 1: the partition's block records, query planes and scales,
// block ids, probabilities, PV reduction scratch.
static size_t pa_stage1_smem(uint32_t G, uint32_t hd, uint32_t pt, uint32_t block_size,
                             uint32_t rec_bytes, uint32_t threads, bool fp8 = false) {
  const uint32_t max_blk = (pt + block_size - 1) / block_size;
  const uint32_t nblk_part = (max_blk + 4) & ~3u;
  return (size_t)pa_region0_bytes(max_blk * rec_bytes, G, hd, threads) + 16 +
         (fp8 ? 4 : 2) * G * hd + PA_MAX_GROUP * 4 + nblk_part * 4 +
         (size_t)((G * pt + 3) & ~3u) * 4 + 16;
}

// Tokens per context partition. Enough CTAs to cover the SMs, but no smaller than 64 tokens; the
// partition's records are staged in shared memory, so the size also decides how many CTAs share
// an SM: with plenty of CTAs (large batches) the largest whole-block size that lets THREE CTAs
// fit is taken (measured on 64 sequences of 256..4096 tokens, 5 kv heads x 3 query heads:
// 512 tokens = two CTAs per SM 61.0 us, 448 = three 54.6 us, 384 57.4 us, 256 67.1 us), else two.
static uint32_t pa_partition_tokens(const kanso_cuda_ctx* ctx, const kanso_paged_attention_params* p,
                                    const KvGeom& g, uint64_t cap) {
  const uint32_t G = p->num_heads / p->num_kv_heads, hd = p->head_dim, bs = p->block_size;
  auto smem_of = [&](uint32_t pt) {
    return pa_stage1_smem(G, hd, pt, bs, g.rec_bytes, pa_threads(pt), g.fp8 != 0);
  };
  uint32_t pt = 512;
  while (pt > 64 && (uint64_t)p->num_seqs * p->num_kv_heads * ((cap + pt - 1) / pt) <
                        (uint64_t)ctx->sm_count / 2)
    pt >>= 1;
  while (pt > 64 && smem_of(pt) > (size_t)ctx->smem_optin / 2) pt >>= 1;
  if (pt % bs) pt = ((pt + bs - 1) / bs) * bs;  // a partition starts on a block record
  if (pt == 512 && bs <= 64) {
    // 2.5 KB per CTA for the kernel's static arrays and the driver's reserve
    const size_t budget = (size_t)ctx->smem_per_sm / 3 - 2560;
    uint32_t pt3 = 512 / bs * bs;
    while (pt3 > 256 && smem_of(pt3) > budget) pt3 -= bs;
    const uint64_t ctas3 = (uint64_t)p->num_seqs * p->num_kv_heads * ((cap + pt3 - 1) / pt3);
    if (pt3 >= 384 && smem_of(pt3) <= budget && ctas3 >= 6ull * ctx->sm_count) pt = pt3;
  }
  return pt;
}

template <int G, int NT, bool FP8>
static void launch_stage1_nt(kanso_cuda_ctx* ctx, const PaArgs& a, dim3 grid, size_t smem) {
  static size_t smem_set[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > smem_set[dev & 15]) {
    cudaFuncSetAttribute(paged_attn_stage1<G, NT, FP8>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    smem_set[dev & 15] = smem;
  }
  launch_dependent(ctx, paged_attn_stage1<G, NT, FP8>, grid, dim3(NT), smem, a);
}
template <int G>
static void launch_stage1(kanso_cuda_ctx* ctx, const PaArgs& a, dim3 grid, size_t smem) {
  const bool big = pa_threads(a.part_tokens) == PA_BIG_THREADS;
  if (a.g.fp8) {
    if (big)
      launch_stage1_nt<G, PA_BIG_THREADS, true>(ctx, a, grid, smem);
    else
      launch_stage1_nt<G, PA_THREADS, true>(ctx, a, grid, smem);
  } else {
    if (big)
      launch_stage1_nt<G, PA_BIG_THREADS, false>(ctx, a, grid, smem);
    else
      launch_stage1_nt<G, PA_THREADS, false>(ctx, a, grid, smem);
  }
}

int32_t launch_paged_attention_rows(kanso_cuda_ctx* ctx, const kanso_cuda_kv* kv, uint32_t layer,
                                    const float* q, const uint32_t* tables, const uint32_t* lens,
                                    float* out, const kanso_paged_attention_params* p,
                                    uint32_t max_ctx_hint, const PaDecodeFusion* fusion,
                                    const uint32_t* row_seq);

int32_t launch_paged_attention(kanso_cuda_ctx* ctx, const kanso_cuda_kv* kv, uint32_t layer,
                               const float* q, const uint32_t* tables, const uint32_t* lens,
                               float* out, const kanso_paged_attention_params* p,
                               uint32_t max_ctx_hint, const PaDecodeFusion* fusion) {
  return launch_paged_attention_rows(ctx, kv, layer, q, tables, lens, out, p, max_ctx_hint,
                                     fusion, nullptr);
}

// p->num_seqs is the number of grid rows (query tokens); with row_seq the block tables hold
// one row per SEQUENCE and row_seq maps each grid row to its sequence.
int32_t launch_paged_attention_rows(kanso_cuda_ctx* ctx, const kanso_cuda_kv* kv, uint32_t layer,
                                    const float* q, const uint32_t* tables, const uint32_t* lens,
                                    float* out, const kanso_paged_attention_params* p,
                                    uint32_t max_ctx_hint, const PaDecodeFusion* fusion,
                                    const uint32_t* row_seq) {
  KvGeom g = kv_geom(kv);
  const uint32_t G = p->num_heads / p->num_kv_heads;
  const uint32_t hd = p->head_dim;
  uint64_t cap = (uint64_t)p->max_num_blocks_per_seq * p->block_size;
  if (max_ctx_hint && max_ctx_hint < cap) cap = max_ctx_hint;
  const uint32_t pt = pa_partition_tokens(ctx, p, g, cap);
  const uint32_t nparts = (uint32_t)((cap + pt - 1) / pt);
  const size_t nheads_total = (size_t)p->num_seqs * p->num_heads;
  const size_t acc_bytes = nheads_total * nparts * hd * sizeof(float);
  const size_t ml_bytes = nheads_total * nparts * 2 * sizeof(float);
  // merge inside stage 1 when the ticket array covers the batch and the partition weights fit
  // where the probabilities were
  const bool merge_in_stage1 =
      (uint64_t)p->num_seqs * p->num_kv_heads <= kanso_cuda_ctx::kPaTickets && nparts <= pt;
  // the packed copy of the output for the o-projection (decode fusion only; 64 | heads * head_dim)
  const uint32_t xp_mt = (p->num_seqs + 15u) / 16u * 16u;
  const bool want_packed = fusion && fusion->packed_out && !row_seq && merge_in_stage1 &&
                           (p->num_heads * hd) % 64 == 0;
  const size_t xp_off = (acc_bytes + ml_bytes + 511) & ~size_t(255);
  const size_t xp_bytes = want_packed ? 2 * (size_t)(p->num_heads * hd / 8) * xp_mt * 16 : 0;
  uint8_t* scratch = (uint8_t*)ctx_scratch(ctx, xp_off + xp_bytes + 256);
  if (!scratch) return KANSO_ERR_DEVICE;
  if (fusion && fusion->packed_out) *fusion->packed_out = want_packed ? scratch + xp_off : nullptr;

  PaArgs a;
  a.g = g;
  a.layer = layer;
  a.q = q;
  a.tables = tables;
  a.lens = lens;
  a.out = out;
  a.part_acc = reinterpret_cast<float*>(scratch);
  a.part_ml = reinterpret_cast<float*>(scratch + ((acc_bytes + 255) & ~size_t(255)));
  a.num_heads = p->num_heads;
  a.max_blocks = p->max_num_blocks_per_seq;
  a.part_tokens = pt;
  a.num_parts = nparts;
  a.scale = p->scale;
  a.status = ctx->dev_status;
  a.tickets = merge_in_stage1 ? ctx->pa_tickets : nullptr;
  a.xp = want_packed ? reinterpret_cast<__half*>(scratch + xp_off) : nullptr;
  a.xp_mt = xp_mt;
  a.row_seq = row_seq;
  a.k_new = a.v_new = a.cos_t = a.sin_t = nullptr;
  a.positions = a.slots = nullptr;
  a.table_len = 0;
  if (fusion) {
    a.k_new = fusion->k_new;
    a.v_new = fusion->v_new;
    a.positions = fusion->positions;
    a.slots = fusion->slots;
    a.cos_t = fusion->cos_t;
    a.sin_t = fusion->sin_t;
    a.table_len = fusion->table_len;
  }

  const size_t smem = pa_stage1_smem(G, hd, pt, p->block_size, g.rec_bytes, pa_threads(pt), g.fp8 != 0);
  if (smem > (size_t)ctx->smem_optin)
    return fail(ctx, KANSO_ERR_UNSUPPORTED, "paged attention: %zu bytes of shared memory needed",
                smem);
  dim3 grid(nparts, p->num_kv_heads, p->num_seqs);
  switch (G) {
    case 1: launch_stage1<1>(ctx, a, grid, smem); break;
    case 2: launch_stage1<2>(ctx, a, grid, smem); break;
    case 3: launch_stage1<3>(ctx, a, grid, smem); break;
    case 4: launch_stage1<4>(ctx, a, grid, smem); break;
    case 5: launch_stage1<5>(ctx, a, grid, smem); break;
    case 6: launch_stage1<6>(ctx, a, grid, smem); break;
    case 7: launch_stage1<7>(ctx, a, grid, smem); break;
    default: launch_stage1<8>(ctx, a, grid, smem); break;
  }
  int32_t st = after_launch(ctx, "paged_attention stage 1");
  if (st || merge_in_stage1) return st;
  launch_dependent(ctx, paged_attn_stage2, dim3(p->num_heads, p->num_seqs), dim3(64), 0, a);
  return after_launch(ctx, "paged_attention stage 2");
}

}  // namespace kanso

using namespace kanso;

extern "C" {

int32_t kanso_cuda_validate_paged_attention_params(const kanso_paged_attention_params* params,
                                                   char* msg, size_t msg_len) {
  return validate_params(params, msg, msg_len);
}

int32_t kanso_cuda_paged_attention(kanso_cuda_ctx* ctx, const kanso_cuda_kv* kv, uint32_t layer,
                                   const float* q, const uint32_t* block_tables,
                                   const uint32_t* context_lens, float* out,
                                   const kanso_paged_attention_params* params,
                                   const uint32_t* host_context_lens) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "paged_attention: ctx is NULL");
  char msg[256];
  int32_t st = validate_params(params, msg, sizeof msg);
  if (st) return fail(ctx, st, "%s", msg);
  if (!kv || !q || !block_tables || !context_lens || !out)
    return fail(ctx, KANSO_ERR_SHAPE, "paged_attention: NULL pointer");
  if (layer >= kv->layers)
    return fail(ctx, KANSO_ERR_SHAPE, "Layer index %u out of bounds (%u)", layer, kv->layers);
  if (params->num_kv_heads != kv->kv_heads || params->head_dim != kv->head_dim ||
      params->block_size != kv->block_size)
    return fail(ctx, KANSO_ERR_SHAPE,
                "paged attention: params (kv_heads %u, head_dim %u, block_size %u) do not match "
                "the pool (%u, %u, %u)",
                params->num_kv_heads, params->head_dim, params->block_size, kv->kv_heads,
                kv->head_dim, kv->block_size);
  const uint32_t hd = params->head_dim;
  if (hd < 16 || (hd & (hd - 1)) != 0)
    return fail(ctx, KANSO_ERR_UNSUPPORTED,
                "paged attention: head_dim %u is not one of 16, 32, 64, 128, 256", hd);
  uint32_t max_ctx = 0;
  if (host_context_lens) {
    // gpu_paged_attention_v2 rejects these on the host (src/metal/paged_attention.rs:343-355)
    uint64_t cap = (uint64_t)params->max_num_blocks_per_seq * params->block_size;
    for (uint32_t s = 0; s < params->num_seqs; ++s) {
      if (host_context_lens[s] == 0)
        return fail(ctx, KANSO_ERR_UNSUPPORTED, "paged attention: sequence %u has context 0", s);
      if (host_context_lens[s] > cap)
        return fail(ctx, KANSO_ERR_UNSUPPORTED,
                    "paged attention: sequence %u context %u exceeds table capacity %llu", s,
                    host_context_lens[s], (unsigned long long)cap);
      if (host_context_lens[s] > max_ctx) max_ctx = host_context_lens[s];
    }
  }
  return launch_paged_attention(ctx, kv, layer, q, block_tables, context_lens, out, params,
                                max_ctx, nullptr);
}

// Chunked-prefill attention: every query token of every sequence is one grid row whose context
// is the prefix up to and including itself; the rows of a sequence share its block-table row.
// The arithmetic per row is exactly the decode attention's (the reference adds -1e9 to the
// masked scores, src/model.rs:1027-1043, which leaves exp() == 0 for them).
int32_t kanso_cuda_paged_attention_prefill(kanso_cuda_ctx* ctx, const kanso_cuda_kv* kv,
                                           uint32_t layer, const float* q,
                                           const uint32_t* block_tables,
                                           const uint32_t* host_context_lens,
                                           const uint32_t* host_query_lens, float* out,
                                           const kanso_paged_attention_params* params) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "paged_attention_prefill: ctx is NULL");
  char msg[256];
  int32_t st = validate_params(params, msg, sizeof msg);
  if (st) return fail(ctx, st, "%s", msg);
  if (!kv || !q || !block_tables || !host_context_lens || !host_query_lens || !out)
    return fail(ctx, KANSO_ERR_SHAPE, "paged_attention_prefill: NULL pointer");
  if (layer >= kv->layers)
    return fail(ctx, KANSO_ERR_SHAPE, "Layer index %u out of bounds (%u)", layer, kv->layers);
  if (params->num_kv_heads != kv->kv_heads || params->head_dim != kv->head_dim ||
      params->block_size != kv->block_size)
    return fail(ctx, KANSO_ERR_SHAPE, "paged attention: params do not match the pool");
  const uint32_t hd = params->head_dim;
  if (hd < 16 || (hd & (hd - 1)) != 0)
    return fail(ctx, KANSO_ERR_UNSUPPORTED,
                "paged attention: head_dim %u is not one of 16, 32, 64, 128, 256", hd);
  // The per-row arrays are built here on the host for this call's lengths and copied from a
  // temporary: a captured graph would replay the copy from memory that no longer exists.
  cudaStreamCaptureStatus cap_st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(ctx->stream, &cap_st) == cudaSuccess &&
      cap_st != cudaStreamCaptureStatusNone)
    return fail(ctx, KANSO_ERR_UNSUPPORTED,
                "paged_attention_prefill cannot be captured in a CUDA graph (its row arrays are "
                "per-call host data)");
  const uint64_t cap = (uint64_t)params->max_num_blocks_per_seq * params->block_size;
  std::vector<uint32_t> rows;  // [row_seq | row_ctx]
  uint64_t T = 0;
  for (uint32_t s = 0; s < params->num_seqs; ++s) T += host_query_lens[s];
  if (T == 0) return fail(ctx, KANSO_ERR_SHAPE, "paged_attention_prefill: no query tokens");
  if (T > (1u << 20))
    return fail(ctx, KANSO_ERR_UNSUPPORTED, "paged_attention_prefill: %llu query tokens",
                (unsigned long long)T);
  rows.resize(2 * T);
  uint32_t max_ctx = 0;
  uint64_t t = 0;
  for (uint32_t s = 0; s < params->num_seqs; ++s) {
    const uint32_t ql = host_query_lens[s], cl = host_context_lens[s];
    // forward_batch_rows' checks (src/model.rs:1434-1455): the context includes the chunk
    if (cl < ql || cl > cap)
      return fail(ctx, KANSO_ERR_SHAPE,
                  "paged_attention_prefill: sequence %u: context %u, %u query tokens, table "
                  "capacity %llu", s, cl, ql, (unsigned long long)cap);
    for (uint32_t i = 0; i < ql; ++i, ++t) {
      rows[t] = s;
      rows[T + t] = cl - ql + i + 1;  // query i sits at position cl - ql + i
    }
    if (cl > max_ctx) max_ctx = cl;
  }
  // one grid row per query token; the row arrays are stream-ordered temporaries
  kanso_paged_attention_params pr = *params;
  pr.num_seqs = (uint32_t)T;
  if ((st = validate_params(&pr, msg, sizeof msg))) return fail(ctx, st, "%s", msg);
  uint32_t* drows = nullptr;
  KANSO_CUDA_TRY(ctx, cudaMallocAsync((void**)&drows, 2 * T * sizeof(uint32_t), ctx->stream),
                 "paged_attention_prefill: row arrays");
  cudaError_t ce = cudaMemcpyAsync(drows, rows.data(), 2 * T * sizeof(uint32_t),
                                   cudaMemcpyHostToDevice, ctx->stream);
  if (ce == cudaSuccess) {
    st = launch_paged_attention_rows(ctx, kv, layer, q, block_tables, drows + T, out, &pr, max_ctx,
                                     nullptr, drows);
  } else {
    st = cuda_fail(ctx, ce, "paged_attention_prefill: row arrays to device");
  }
  cudaFreeAsync(drows, ctx->stream);
  return st;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// An engine that plans all of its device memory up front (the KV pool is sized from a memory
// budget when the engine starts, and nothing may grow afterwards), or that calls from a place
// where cudaMalloc is off limits because it synchronises the whole device (a latency-critical
// serving loop, a thread that holds a lock other GPU work waits on), cannot use the entry
// point above: its split-context partials live in context scratch that grows on demand. This
// variant keeps the partials in a fixed array that is part of the loaded library image, so the
// call itself performs no allocation of any kind.
namespace kanso {

// Every GPU that loads the library carries this array until the process exits.
constexpr size_t PA_STATIC_SCRATCH_BYTES = size_t(8) << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_pa_static_scratch[PA_STATIC_SCRATCH_BYTES];

// Device address of the array, looked up once per device. In host code the symbol's name is
// only a handle for the runtime, not a device pointer, so it must never be handed to a kernel
// directly; cudaGetSymbolAddress translates it for the device that is current.
// Contexts are single-caller, but two contexts on different threads may make their first calls
// at the same time: the table is filled under a mutex. The caller's current device is put back
// before returning.
static unsigned char* pa_static_scratch_ptr(kanso_cuda_ctx* ctx, int32_t* status) {
  static unsigned char* per_device[64] = {nullptr};
  static std::mutex mu;
  *status = KANSO_OK;
  const int dev = ctx->device;
  if (dev < 0 || dev >= 64) {
    *status = fail(ctx, KANSO_ERR_UNSUPPORTED, "paged_attention_noalloc: device index %d", dev);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!per_device[dev]) {
    int cur = -1;
    cudaError_t e = cudaGetDevice(&cur);
    const bool switched = e == cudaSuccess && cur != dev;
    if (switched) e = cudaSetDevice(dev);
    unsigned char* p = nullptr;
    if (e == cudaSuccess) e = cudaGetSymbolAddress((void**)&p, g_pa_static_scratch);
    if (switched) {
      const cudaError_t back = cudaSetDevice(cur);
      if (e == cudaSuccess) e = back;
    }
    if (e != cudaSuccess || !p) {
      *status = cuda_fail(ctx, e, "paged_attention_noalloc: cudaGetSymbolAddress");
      return nullptr;
    }
    per_device[dev] = p;
  }
  return per_device[dev];
}

static int32_t launch_paged_attention_static(kanso_cuda_ctx* ctx, const kanso_cuda_kv* kv,
                                             uint32_t layer, const float* q,
                                             const uint32_t* tables, const uint32_t* lens,
                                             float* out, const kanso_paged_attention_params* p,
                                             uint32_t max_ctx_hint) {
  KvGeom g = kv_geom(kv);
  const uint32_t G = p->num_heads / p->num_kv_heads;
  const uint32_t hd = p->head_dim;
  uint64_t cap = (uint64_t)p->max_num_blocks_per_seq * p->block_size;
  if (max_ctx_hint && max_ctx_hint < cap) cap = max_ctx_hint;
  const uint32_t pt = pa_partition_tokens(ctx, p, g, cap);
  const uint32_t nparts = (uint32_t)((cap + pt - 1) / pt);

  const size_t nheads_total = (size_t)p->num_seqs * p->num_heads;
  const size_t acc_bytes = nheads_total * nparts * hd * sizeof(float);
  const size_t acc_al = (acc_bytes + 255) & ~size_t(255);
  const size_t ml_bytes = nheads_total * nparts * 2 * sizeof(float);
  if (acc_al + ml_bytes > PA_STATIC_SCRATCH_BYTES)
    return fail(ctx, KANSO_ERR_UNSUPPORTED,
                "paged_attention_noalloc: this batch needs %zu bytes of partials (%u sequences x "
                "%u heads x %u partitions x head_dim %u); the built-in scratch holds %zu. Split "
                "the batch or use kanso_cuda_paged_attention",
                acc_al + ml_bytes, p->num_seqs, p->num_heads, nparts, hd,
                (size_t)PA_STATIC_SCRATCH_BYTES);
  int32_t st;
  unsigned char* scratch = pa_static_scratch_ptr(ctx, &st);
  if (!scratch) return st;

  PaArgs a;
  a.g = g;
  a.layer = layer;
  a.q = q;
  a.tables = tables;
  a.lens = lens;
  a.out = out;
  // Nothing in the array has to start at zero: stage 1 writes every partition that stage 2
  // reads for a sequence (those below its context length), so stale contents are never used.
  a.part_acc = reinterpret_cast<float*>(scratch);
  a.part_ml = reinterpret_cast<float*>(scratch + acc_al);
  a.num_heads = p->num_heads;
  a.max_blocks = p->max_num_blocks_per_seq;
  a.part_tokens = pt;
  a.num_parts = nparts;
  a.scale = p->scale;
  a.status = ctx->dev_status;
  a.tickets = nullptr;  // two launches: stage 2 merges
  a.row_seq = nullptr;
  a.xp = nullptr;
  a.xp_mt = 0;
  a.k_new = a.v_new = a.cos_t = a.sin_t = nullptr;
  a.positions = a.slots = nullptr;
  a.table_len = 0;

  const size_t smem = pa_stage1_smem(G, hd, pt, p->block_size, g.rec_bytes, pa_threads(pt), g.fp8 != 0);
  if (smem > (size_t)ctx->smem_optin)
    return fail(ctx, KANSO_ERR_UNSUPPORTED,
                "paged_attention_noalloc: %zu bytes of shared memory needed", smem);
  dim3 grid(nparts, p->num_kv_heads, p->num_seqs);
  switch (G) {
    case 1: launch_stage1<1>(ctx, a, grid, smem); break;
    case 2: launch_stage1<2>(ctx, a, grid, smem); break;
    case 3: launch_stage1<3>(ctx, a, grid, smem); break;
    case 4: launch_stage1<4>(ctx, a, grid, smem); break;
    case 5: launch_stage1<5>(ctx, a, grid, smem); break;
    case 6: launch_stage1<6>(ctx, a, grid, smem); break;
    case 7: launch_stage1<7>(ctx, a, grid, smem); break;
    default: launch_stage1<8>(ctx, a, grid, smem); break;
  }
  st = after_launch(ctx, "paged_attention_noalloc stage 1");
  if (st) return st;
  launch_dependent(ctx, paged_attn_stage2, dim3(p->num_heads, p->num_seqs), dim3(64), 0, a);
  return after_launch(ctx, "paged_attention_noalloc stage 2");
}

}  // namespace kanso

extern "C" int32_t kanso_cuda_paged_attention_noalloc(
    kanso_cuda_ctx* ctx, const kanso_cuda_kv* kv, uint32_t layer, const float* q,
    const uint32_t* block_tables, const uint32_t* context_lens, float* out,
    const kanso_paged_attention_params* params, const uint32_t* host_context_lens) {
  if (!ctx) return kanso::fail(nullptr, KANSO_ERR_CONFIG, "paged_attention_noalloc: ctx is NULL");
  char msg[256];
  int32_t st = kanso::validate_params(params, msg, sizeof msg);
  if (st) return kanso::fail(ctx, st, "%s", msg);
  if (!kv || !q || !block_tables || !context_lens || !out)
    return kanso::fail(ctx, KANSO_ERR_SHAPE, "paged_attention_noalloc: NULL pointer");
  if (layer >= kv->layers)
    return kanso::fail(ctx, KANSO_ERR_SHAPE, "Layer index %u out of bounds (%u)", layer,
                       kv->layers);
  if (params->num_kv_heads != kv->kv_heads || params->head_dim != kv->head_dim ||
      params->block_size != kv->block_size)
    return kanso::fail(ctx, KANSO_ERR_SHAPE,
                       "paged attention: params (kv_heads %u, head_dim %u, block_size %u) do not "
                       "match the pool (%u, %u, %u)",
                       params->num_kv_heads, params->head_dim, params->block_size, kv->kv_heads,
                       kv->head_dim, kv->block_size);
  const uint32_t hd = params->head_dim;
  if (hd < 16 || (hd & (hd - 1)) != 0)
    return kanso::fail(ctx, KANSO_ERR_UNSUPPORTED,
                       "paged attention: head_dim %u is not one of 16, 32, 64, 128, 256", hd);
  uint32_t max_ctx = 0;
  if (host_context_lens) {
    const uint64_t cap = (uint64_t)params->max_num_blocks_per_seq * params->block_size;
    for (uint32_t s = 0; s < params->num_seqs; ++s) {
      if (host_context_lens[s] == 0)
        return kanso::fail(ctx, KANSO_ERR_UNSUPPORTED,
                           "paged attention: sequence %u has context 0", s);
      if (host_context_lens[s] > cap)
        return kanso::fail(ctx, KANSO_ERR_UNSUPPORTED,
                           "paged attention: sequence %u context %u exceeds table capacity %llu",
                           s, host_context_lens[s], (unsigned long long)cap);
      if (host_context_lens[s] > max_ctx) max_ctx = host_context_lens[s];
    }
  }
  return kanso::launch_paged_attention_static(ctx, kv, layer, q, block_tables, context_lens, out,
                                              params, max_ctx);
}
