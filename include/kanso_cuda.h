/*
 * kanso_cuda.h — C ABI of the B200 (sm_100a) `cuda` backend for kanso-infer's
 * quantized-weight matmul and int8 paged decode attention.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, and
 * returns an int32 status (0 = OK). Nothing here falls back to the CPU: an
 * unsupported shape is an error, a missing GPU is an error.
 *
 * Citations are file:line inside the kanso-infer source tree and name the
 * reference interface each entry point replaces.
 *
 * Threading: a context is single-caller (the reference drives its engine from
 * exactly one thread, src/server/engine_loop.rs:1-7). Calls are asynchronous on
 * the context's stream; kanso_cuda_sync() waits for them.
 */
#ifndef KANSO_CUDA_H
#define KANSO_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes: the reference's EngineError variants (src/error.rs:3-11) ---- */
#define KANSO_OK 0
#define KANSO_ERR_CONFIG 1      /* EngineError::Config  — startup misconfiguration      */
#define KANSO_ERR_SHAPE 2       /* EngineError::Model   — shape / bounds problems        */
#define KANSO_ERR_UNSUPPORTED 3 /* new EngineError::Cuda — geometry the kernels lack     */
#define KANSO_ERR_DEVICE 4      /* new EngineError::Cuda — CUDA runtime / NCCL failure    */
#define KANSO_ERR_TIMEOUT 5     /* new EngineError::Cuda — a bounded device wait ran out  */

/* ---- block formats (values are the GGML type ids of the GGUF file format) ---- */
#define KANSO_DTYPE_Q8_0 8  /* 34 B: f16 d, 32 x int8       (src/quant/q8_0.rs:1-9 with d as f16) */
#define KANSO_DTYPE_Q4_K 12 /* 144 B: f16 d, f16 dmin, 12 B scales, 128 B nibbles (src/quant/q4_k.rs:1-12) */

#define KANSO_QK8_0 32
#define KANSO_Q8_0_BYTES 34
#define KANSO_QK_K 256
#define KANSO_Q4_K_BYTES 144

/* ---- activation handling of the matmul ---- */
#define KANSO_ACT_F32 0 /* f32 activations, as scalar_dot_q8_0 / scalar_dot_q4_k (q8_0.rs:51-57, q4_k.rs:58-66) */
#define KANSO_ACT_Q8 1  /* activations quantized per 32 by quantize_row_q8_0, int32 block sums as scalar_dot_q8_0_q8_0 (q8_0.rs:43-66) */

/* ---- KV pool element type: the reference's KvCacheType flag (src/kv_cache/kind.rs:31-73) ---- */
#define KANSO_KV_F32 0
#define KANSO_KV_INT8 1
#define KANSO_KV_FP8 2 /* E4M3 bytes, power-of-two scale per (token, kv head) */

typedef struct kanso_cuda_ctx kanso_cuda_ctx;
typedef struct kanso_cuda_weight kanso_cuda_weight;
typedef struct kanso_cuda_kv kanso_cuda_kv;
typedef struct kanso_cuda_model kanso_cuda_model;

/* Same field order and types as the reference's #[repr(C)] PagedAttentionParams
 * (src/metal/paged_attention.rs:12-22). */
typedef struct kanso_paged_attention_params {
  uint32_t num_seqs;
  uint32_t num_heads;
  uint32_t num_kv_heads;
  uint32_t head_dim;
  uint32_t block_size;
  uint32_t max_num_blocks_per_seq;
  float scale;
} kanso_paged_attention_params;

/* The fields of the reference's ModelConfig that the decode step reads
 * (src/config.rs:8-40; preset src/config.rs:71-90). rope_theta is a parameter
 * because the GGUF loader overrides the preset (src/weights.rs:397-399). */
typedef struct kanso_model_config {
  uint32_t hidden_size;
  uint32_t num_attention_heads;
  uint32_t num_key_value_heads;
  uint32_t num_hidden_layers;
  uint32_t intermediate_size;
  uint32_t vocab_size;
  uint32_t block_size;
  uint32_t max_seq_len;
  float rms_norm_eps;
  float rope_theta;
} kanso_model_config;

/* Names of the per-layer tensors (src/weights.rs:429-447) for kanso_cuda_model_set_weight. */
#define KANSO_W_ATTN_Q 0
#define KANSO_W_ATTN_K 1
#define KANSO_W_ATTN_V 2
#define KANSO_W_ATTN_OUTPUT 3
#define KANSO_W_FFN_GATE 4
#define KANSO_W_FFN_UP 5
#define KANSO_W_FFN_DOWN 6
#define KANSO_W_TOKEN_EMBD 7 /* layer argument ignored; also the tied lm_head (src/weights.rs:418-422) */
#define KANSO_W_OUTPUT 8     /* layer argument ignored; optional untied lm_head */
#define KANSO_NORM_ATTN 0
#define KANSO_NORM_FFN 1
#define KANSO_NORM_FINAL 2 /* layer argument ignored */

/* ------------------------------------------------------------------------- */
/* Context. Replaces the per-backend seam state the reference keeps in
 * MetalContext (src/metal/context.rs:6-16): device, stream, scratch, counters. */

/* `stream` is a cudaStream_t the caller owns (work is enqueued there), or NULL
 * for a stream the context creates. Fails with KANSO_ERR_DEVICE when the device
 * is absent or is not compute capability 10.x. */
int32_t kanso_cuda_ctx_create(int32_t device, void* stream, kanso_cuda_ctx** out);
int32_t kanso_cuda_ctx_destroy(kanso_cuda_ctx* ctx);
int32_t kanso_cuda_sync(kanso_cuda_ctx* ctx);
/* Message of the last failing call on this context (or on no context when ctx
 * is NULL: creation failures). Never NULL. */
const char* kanso_cuda_last_error(const kanso_cuda_ctx* ctx);
/* Options of a context. KANSO_OPT_OVERLAP_WEIGHT_PREFETCH (default 0): the caller promises
 * that the weight blocks given to matmul calls are not written by work enqueued earlier on
 * the stream (they are model parameters, uploaded and left alone, as LinearWeight storage is
 * in the reference, src/weights.rs:22). A matmul kernel may then be launched with
 * programmatic dependent launch and fetch its first weight tiles while the kernel before it
 * drains; it still waits for that kernel before it reads activations or writes results. */
#define KANSO_OPT_OVERLAP_WEIGHT_PREFETCH 1
int32_t kanso_cuda_ctx_set_option(kanso_cuda_ctx* ctx, int32_t option, int32_t value);
/* Kernels launched by this context since creation (the reference counts seam
 * calls the same way, src/model.rs:246-301). */
uint64_t kanso_cuda_launch_count(const kanso_cuda_ctx* ctx);
/* Number of streaming multiprocessors of the context's device. */
int32_t kanso_cuda_sm_count(const kanso_cuda_ctx* ctx);
/* Measurement aid, no counterpart in the reference: one launch that only reads `nbytes` of a
 * device buffer with 128-bit loads. Timed beside a GEMV over the same buffer it gives the floor
 * that launch latency and the memory system put under that GEMV. */
int32_t kanso_cuda_probe_read(kanso_cuda_ctx* ctx, const void* buf, size_t nbytes);

/* ------------------------------------------------------------------------- */
/* Block kernels: src/quant. All pointers are device pointers, 16-byte aligned. */

/* scalar_gemv_q8_0(weights, x, out, rows, cols) — src/quant/q8_0.rs:69-93.
 * w: rows * cols/32 GGUF Q8_0 blocks, row-major. x f32[cols], y f32[rows].
 * cols % 32 != 0 -> KANSO_ERR_SHAPE. */
int32_t kanso_cuda_gemv_q8_0(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                             int64_t rows, int64_t cols);
/* scalar_gemv_q4_k(weights, x, out, rows, cols) — src/quant/q4_k.rs:69-93.
 * cols % 256 != 0 -> KANSO_ERR_SHAPE. */
int32_t kanso_cuda_gemv_q4_k(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                             int64_t rows, int64_t cols);

/* LinearWeight::forward, y[M,N] = x[M,K] @ W[N,K]^T — src/weights.rs:43-45,
 * callers src/model.rs:390-397. x f32[M,K] row-major, y f32[M,N] row-major.
 * act_mode is KANSO_ACT_F32 or KANSO_ACT_Q8 (Q4_K accepts KANSO_ACT_F32 only). */
int32_t kanso_cuda_gemm_q8_0(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                             int64_t M, int64_t N, int64_t K, int32_t act_mode);
int32_t kanso_cuda_gemm_q4_k(kanso_cuda_ctx* ctx, const void* w, const float* x, float* y,
                             int64_t M, int64_t N, int64_t K, int32_t act_mode);

/* quantize_row_q8_0(xs, blocks) — src/quant/q8_0.rs:13-32,43-48. The reference's
 * in-memory block keeps an f32 d, so the result is two planes:
 * d_out f32[cols/32], qs_out int8[cols]. */
int32_t kanso_cuda_quantize_row_q8_0(kanso_cuda_ctx* ctx, const float* x, float* d_out,
                                     int8_t* qs_out, int64_t cols);

/* BlockQ8_0::dequantize over nblocks GGUF blocks — src/quant/q8_0.rs:35-39. out f32[32*nblocks]. */
int32_t kanso_cuda_dequantize_q8_0(kanso_cuda_ctx* ctx, const void* w, float* out, int64_t nblocks);
/* BlockQ4_K::dequantize over nblocks GGUF super-blocks — src/quant/q4_k.rs:30-55. out f32[256*nblocks]. */
int32_t kanso_cuda_dequantize_q4_k(kanso_cuda_ctx* ctx, const void* w, float* out, int64_t nblocks);
/* get_scale_min_k4 for all 8 sub-blocks of nblocks super-blocks — src/quant/q4_k.rs:16-26.
 * out u8[nblocks*16]: 8 scales then 8 mins per super-block. */
int32_t kanso_cuda_unpack_scales_q4_k(kanso_cuda_ctx* ctx, const void* w, uint8_t* out,
                                      int64_t nblocks);
/* The int32 inner sums of scalar_dot_q8_0_q8_0 — src/quant/q8_0.rs:60-66 — for every
 * (row, block) against activations quantized by quantize_row_q8_0.
 * x_qs int8[cols]; isums int32[rows * cols/32]. */
int32_t kanso_cuda_block_isums_q8_0(kanso_cuda_ctx* ctx, const void* w, const int8_t* x_qs,
                                    int32_t* isums, int64_t rows, int64_t cols);

/* ------------------------------------------------------------------------- */
/* Weights resident on the device: LinearWeight::to_device rebuilding the block
 * storage from raw bytes — src/weights.rs:140-158. */

/* host_bytes: rows * cols/blk blocks in GGUF layout (host memory). */
int32_t kanso_cuda_weight_upload(kanso_cuda_ctx* ctx, const void* host_bytes, size_t nbytes,
                                 int32_t dtype, int64_t rows, int64_t cols,
                                 kanso_cuda_weight** out);
int32_t kanso_cuda_weight_free(kanso_cuda_weight* w);
/* Device address of the blocks (for the pointer-level entry points above). */
const void* kanso_cuda_weight_ptr(const kanso_cuda_weight* w);
/* Model::linear(w, x) with host activations — src/model.rs:390-397: copies
 * x_host f32[M,K] to the device, runs the matmul, copies y f32[M,N] back and
 * synchronises. This is the call whose timing is the end-to-end figure. */
int32_t kanso_cuda_linear_host(kanso_cuda_ctx* ctx, const kanso_cuda_weight* w,
                               const float* x_host, float* y_host, int64_t M, int32_t act_mode);
/* Same with device activations, asynchronous. */
int32_t kanso_cuda_linear(kanso_cuda_ctx* ctx, const kanso_cuda_weight* w, const float* x,
                          float* y, int64_t M, int32_t act_mode);
/* ---- sharding one linear layer over the GPUs of a node (one process per GPU). The reference
 * has no multi-GPU path (docs/SPEC.md:125); these extend LinearWeight::to_device and
 * Model::linear (src/weights.rs:140-158, src/model.rs:390-397). ---- */
/* The part of [0, n) that rank `rank` of `world` owns, in multiples of `align`
 * (8 rows for output-row sharding, the block size for K sharding). Host only. */
int32_t kanso_cuda_shard_range(int64_t n, int32_t rank, int32_t world, int64_t align,
                               int64_t* begin, int64_t* count);
/* K sharding: copies the blocks of columns [col_begin, col_begin + col_count) of every row
 * into a contiguous [rows x col_count] block matrix (host to host). */
int32_t kanso_cuda_shard_k_repack(const void* host_bytes, int32_t dtype, int64_t rows,
                                  int64_t cols, int64_t col_begin, int64_t col_count,
                                  void* out_bytes, size_t out_capacity);
/* Output-row sharding with the gather fused into the matmul's epilogue: w holds rows
 * [row_offset, row_offset + w.rows) of an [n_total x cols] weight; the slice
 * y[m, row_offset + r] is stored into every one of the n_out (<= 8) result buffers
 * y_out[i] (f32 [M, n_total]; this GPU's own and its peers' buffers mapped into this
 * process, e.g. symmetric memory). Stores to peers are plain stores over NVLink; the caller
 * orders them against the readers with a cross-GPU barrier (kanso_cuda_peer_exchange below is
 * one, as a kernel on the same stream). */
int32_t kanso_cuda_linear_scatter_out(kanso_cuda_ctx* ctx, const kanso_cuda_weight* w,
                                      const float* x, int64_t M, float* const* y_out,
                                      int32_t n_out, int64_t n_total, int64_t row_offset,
                                      int32_t act_mode);
/* K sharding with the reduction done through the same peer stores: every rank stores its
 * partial y into slice [rank * rows, (rank + 1) * rows) of every rank's parts buffer
 * (f32 [M, world * rows]) with kanso_cuda_linear_scatter_out(n_total = world * rows,
 * row_offset = rank * rows); after the cross-GPU barrier (kanso_cuda_peer_exchange) this
 * adds the slices in rank order: y[m, n] = sum_r parts[m, r * rows + n]. No counterpart in
 * the reference. */
int32_t kanso_cuda_sum_shards(kanso_cuda_ctx* ctx, const float* parts, int64_t M, int64_t rows,
                              int32_t world, float* y);
/* The cross-GPU barrier of the two sharded forms above, as one small kernel on the context's
 * stream: tells every peer that this rank's stores of the step are done and waits (at most
 * 2 s, then KANSO_ERR_TIMEOUT at the next kanso_cuda_sync) until every peer has said the same.
 * flags[r] (r < world <= 8): rank r's array of `world` u64 slots, zeroed once, mapped into this
 * process (symmetric memory); step: one u64 in this GPU's memory, zeroed once, advanced by
 * every call. Every rank makes the same sequence of calls; no host state, so the calls can be
 * captured in a CUDA graph. No counterpart in the reference. */
int32_t kanso_cuda_peer_exchange(kanso_cuda_ctx* ctx, void* const* flags, void* step,
                                 int32_t world, int32_t rank);
/* NOTE on the three pointer-level calls above (scatter_out / sum_shards / peer_exchange): one
 * exchange orders the stores of a call against its readers, but it does NOT protect the next
 * call's stores from a peer that is still reading: a rank one call ahead would overwrite the
 * buffer under a slower peer. Consecutive calls on the same layer must therefore alternate
 * between TWO result (or parts) buffers, or be separated by a second exchange placed after the
 * readers. The sharded-layer objects below do this themselves. */

/* ---- sharded layers as objects: peer-visible memory, the exchange and the forward call, so
 * that a caller without any Python (Model::linear, src/model.rs:390-397) can shard a layer.
 * No counterpart in the reference. ---- */
typedef struct kanso_cuda_shard_group kanso_cuda_shard_group;
typedef struct kanso_cuda_sharded_linear kanso_cuda_sharded_linear;
#define KANSO_SHARD_HANDLE_BYTES 64
#define KANSO_SHARD_ROWS 0 /* output rows split over the ranks; x replicated */
#define KANSO_SHARD_K 1    /* columns (K) split at block boundaries; partial results summed */
#define KANSO_SHARD_LOCAL_ONLY 1 /* forward flag, row shard: keep the slice on this rank */
/* Step 1, every rank: allocates this rank's region of `region_bytes` (the exchange buffers of
 * all layers created later: 2 * max_m * rows_total * 4 bytes per row-sharded layer,
 * 2 * max_m * world * rows_total * 4 per K-sharded layer) and writes its 64-byte inter-process
 * handle to handle_out. world <= 8, all ranks on one node. */
int32_t kanso_cuda_shard_group_create(kanso_cuda_ctx* ctx, int32_t rank, int32_t world,
                                      size_t region_bytes, kanso_cuda_shard_group** out,
                                      void* handle_out);
/* Step 2: the caller gathers the handles of all ranks (world * 64 bytes, in rank order) over its
 * own channel and hands them in; the peers' regions are mapped into this process. */
int32_t kanso_cuda_shard_group_connect(kanso_cuda_shard_group* g, const void* all_handles);
int32_t kanso_cuda_shard_group_destroy(kanso_cuda_shard_group* g);
/* LinearWeight::to_device for this rank's shard of an [rows_total x cols_total] weight
 * (src/weights.rs:140-158). shard_bytes: the blocks of this rank's rows
 * (kanso_cuda_shard_range(rows_total, rank, world, 8)) for KANSO_SHARD_ROWS, or this rank's
 * columns re-packed by kanso_cuda_shard_k_repack for KANSO_SHARD_K. Every rank creates the same
 * layers in the same order (their buffers are found by offset). */
int32_t kanso_cuda_sharded_linear_create(kanso_cuda_shard_group* g, const void* shard_bytes,
                                         size_t nbytes, int32_t dtype, int64_t rows_total,
                                         int64_t cols_total, int32_t mode, int64_t max_m,
                                         kanso_cuda_sharded_linear** out);
int32_t kanso_cuda_sharded_linear_destroy(kanso_cuda_sharded_linear* layer);
/* The rows (row shard) or columns (K shard) this rank holds. */
int32_t kanso_cuda_sharded_linear_range(const kanso_cuda_sharded_linear* layer, int64_t* begin,
                                        int64_t* count);
/* Model::linear on the sharded layer, asynchronous on the context's stream; *y_out is a device
 * buffer owned by the layer, valid until its next forward.
 *   row shard: x f32 [M, cols_total] (replicated). Default: y f32 [M, rows_total] gathered on
 *     every rank (each rank's matmul stores its rows into every rank's memory, a consumer
 *     kernel waits for the peers' signals). KANSO_SHARD_LOCAL_ONLY: y f32 [M, count], this
 *     rank's rows only and no exchange at all: exactly the K slice a K-sharded layer wants.
 *   K shard: x f32 [M, count] = this rank's columns of the activations; y f32 [M, rows_total],
 *     the partial results of all ranks added in rank order (same bits on every rank).
 * Every rank makes the same sequence of calls. A peer that never arrives ends the wait after
 * 2 s with KANSO_ERR_TIMEOUT at the next kanso_cuda_sync. No host state changes per call, so a
 * sequence of forwards may be captured in a CUDA graph and replayed. */
int32_t kanso_cuda_sharded_linear_forward(kanso_cuda_sharded_linear* layer, const float* x,
                                          int64_t M, int32_t act_mode, int32_t flags,
                                          const float** y_out);
/* LinearWeight::embed — src/weights.rs:50-57: dequantise the selected rows.
 * ids u32[T] (device), out f32[T, cols] (device). An id >= rows -> KANSO_ERR_SHAPE
 * is reported by the device status word at the next kanso_cuda_sync. */
int32_t kanso_cuda_embed(kanso_cuda_ctx* ctx, const kanso_cuda_weight* w, const uint32_t* ids,
                         float* out, int64_t T);

/* ------------------------------------------------------------------------- */
/* KV pool: KvStorageKind with the KvCacheType flag — src/kv_cache/kind.rs:176-494,
 * int8 / fp8 pool src/kv_cache/quantized_storage.rs. */

/* QuantizedKvStorage::new — quantized_storage.rs:56-105. New blocks hold quants 0
 * and scales 1.0 (quantized_storage.rs:24-33). kv_type KANSO_KV_INT8 (QuantMode::Int8) or
 * KANSO_KV_FP8 (QuantMode::Fp8, new_fp8 quantized_storage.rs:109-131: scale =
 * 2^ceil(log2(amax / 64)), values rounded to nearest-even E4M3, quantized_storage.rs:470-484);
 * every call that takes the pool (write, read, reset, decode / prefill attention, the decode
 * step) works on either. KANSO_KV_F32 -> KANSO_ERR_UNSUPPORTED. */
int32_t kanso_cuda_kv_create(kanso_cuda_ctx* ctx, uint32_t num_layers, uint32_t num_blocks,
                             uint32_t block_size, uint32_t num_kv_heads, uint32_t head_dim,
                             int32_t kv_type, kanso_cuda_kv** out);
int32_t kanso_cuda_kv_destroy(kanso_cuda_kv* kv);
/* KvStorageKind::write_kv_slots — kind.rs:348; per token quantize_head_slice +
 * write_quantized_kv_token — quantized_storage.rs:143-204,452-469.
 * slots u32[T] (slot = block*block_size + offset, kind.rs:111), k,v f32[T,kvh,hd], all device.
 * host_slots (optional, may be NULL) lets the call bounds-check on the host like
 * KvSlotPlan::new (kind.rs:123-147); device-side the check sets the status word. */
int32_t kanso_cuda_kv_write_slots(kanso_cuda_ctx* ctx, kanso_cuda_kv* kv, uint32_t layer,
                                  const uint32_t* slots, const float* k, const float* v,
                                  int64_t T, const uint32_t* host_slots);
/* QuantizedKvStorage::reset_block — quantized_storage.rs:134-140: all layers. */
int32_t kanso_cuda_kv_reset_block(kanso_cuda_ctx* ctx, kanso_cuda_kv* kv, uint32_t block);
/* read_quantized_kv_token — quantized_storage.rs:219-270. Copies one token's
 * stored form to host: k_q,v_q int8[kvh*hd] (may be NULL), k_scale,v_scale f32[kvh]
 * (may be NULL), k_deq,v_deq f32[kvh*hd] = (f32)q*scale (may be NULL). Synchronous. */
int32_t kanso_cuda_kv_read_token(kanso_cuda_ctx* ctx, const kanso_cuda_kv* kv, uint32_t layer,
                                 uint32_t block, uint32_t offset, int8_t* k_q, int8_t* v_q,
                                 float* k_scale, float* v_scale, float* k_deq, float* v_deq);
/* QuantizedKvStorage::memory_bytes_per_token — quantized_storage.rs:414-419. */
uint64_t kanso_cuda_kv_bytes_per_token(const kanso_cuda_kv* kv);

/* Decode attention over the pool through the block table: the call the reference
 * makes as metal_paged_attention / encode_paged_attention_v2
 * (src/model.rs:874-914, src/metal/paged_attention.rs:193-203), with the math of
 * cpu_paged_attention (paged_attention.rs:84-178) over the dequantised int8 pool
 * (quantized_storage.rs:284-383). q f32[num_seqs, num_heads, head_dim],
 * block_tables u32[num_seqs*max_blocks], context_lens u32[num_seqs],
 * out f32[num_seqs, num_heads*head_dim]; all device. host_context_lens (optional)
 * enables the reference's host checks: ctx 0 and ctx > capacity are rejected
 * (paged_attention.rs:343-355). head_dim must be a power of two from 16 to 256 (the reference's
 * validation only asks for 1..256 and a whole GQA ratio, paged_attention.rs:24-82; its presets use
 * 64 and 128): any other value returns KANSO_ERR_UNSUPPORTED. A device context length beyond
 * the table capacity or beyond the host's figure is cut off there and reported as
 * KANSO_ERR_SHAPE by the next kanso_cuda_sync. */
int32_t kanso_cuda_paged_attention(kanso_cuda_ctx* ctx, const kanso_cuda_kv* kv, uint32_t layer,
                                   const float* q, const uint32_t* block_tables,
                                   const uint32_t* context_lens, float* out,
                                   const kanso_paged_attention_params* params,
                                   const uint32_t* host_context_lens);
/* Chunked-prefill attention, query_len > 1: the attention of Model::forward_prefill and of the
 * mixed batches of forward_batch_rows (src/model.rs:1002-1099,1470-1529) over the int8 pool.
 * The chunk's K/V must already be in the pool (kanso_cuda_kv_write_slots). Sequence s has
 * host_query_lens[s] query tokens, the LAST tokens of its host_context_lens[s] (which counts the
 * chunk); query i attends keys 0 ..= context - query_len + i, which is what the reference's
 * offset causal mask of -1e9 leaves (src/model.rs:1027-1043). q and out f32
 * [sum of query_lens, num_heads*head_dim], rows in sequence order; block_tables device
 * u32[num_seqs*max_blocks]; the two length arrays are HOST arrays (they are host slices in the
 * reference's forward_batch, src/model.rs:1360-1369). Not capturable in a CUDA graph (the
 * per-row arrays are built on the host for each call): KANSO_ERR_UNSUPPORTED while the context's
 * stream is being captured. */
int32_t kanso_cuda_paged_attention_prefill(kanso_cuda_ctx* ctx, const kanso_cuda_kv* kv,
                                           uint32_t layer, const float* q,
                                           const uint32_t* block_tables,
                                           const uint32_t* host_context_lens,
                                           const uint32_t* host_query_lens, float* out,
                                           const kanso_paged_attention_params* params);
/* The same decode attention for callers that cannot allocate device memory. It has no
 * counterpart in the reference. kanso_cuda_paged_attention keeps its split-context partials
 * in context scratch that grows with cudaMalloc when a larger batch arrives; an engine whose
 * device memory is fully planned at start-up, or a caller for whom cudaMalloc's device-wide
 * synchronisation is unacceptable (a latency-critical loop, a thread holding a lock that other
 * GPU work waits on), uses this entry point instead: the partials live in an 8 MiB array built
 * into the library image (every GPU that loads the library holds it until the process exits)
 * and the call performs no cudaMalloc, cudaFree or other allocating call.
 *   - Arguments, checks and results are those of kanso_cuda_paged_attention.
 *   - A batch whose partials (num_seqs * num_heads * partitions * (head_dim + 2) floats) exceed
 *     8 MiB is refused with KANSO_ERR_UNSUPPORTED; the message gives the size needed.
 *   - The first call on a device looks up the array's device address; make that first call
 *     outside any stream capture.
 *   - All calls on a device share the one array, and it keeps the previous call's contents
 *     (nothing in it needs clearing: every cell read was written by the same call). Two calls
 *     whose kernels overlap on the GPU (different streams or contexts) would race on it:
 *     keep them on one stream or order them yourself. */
int32_t kanso_cuda_paged_attention_noalloc(kanso_cuda_ctx* ctx, const kanso_cuda_kv* kv,
                                           uint32_t layer, const float* q,
                                           const uint32_t* block_tables,
                                           const uint32_t* context_lens, float* out,
                                           const kanso_paged_attention_params* params,
                                           const uint32_t* host_context_lens);
/* validate_paged_attention_params — src/metal/paged_attention.rs:39-81 (no device work). */
int32_t kanso_cuda_validate_paged_attention_params(const kanso_paged_attention_params* params,
                                                   char* msg, size_t msg_len);

/* ------------------------------------------------------------------------- */
/* Glue ops of the decode step (src/model.rs:653-737,367-382; CPU statements in
 * src/metal/ops.rs:10-77). Device pointers, asynchronous. */
int32_t kanso_cuda_rmsnorm(kanso_cuda_ctx* ctx, const float* x, const float* weight, float* out,
                           int64_t rows, int64_t hidden, float eps);
/* Rotate-half RoPE in place on x f32[T, heads, head_dim] with positions u32[T]. */
int32_t kanso_cuda_rope(kanso_cuda_ctx* ctx, float* x, const uint32_t* positions, int64_t T,
                        int64_t heads, int64_t head_dim, float theta);
int32_t kanso_cuda_silu_mul(kanso_cuda_ctx* ctx, const float* gate, const float* up, float* out,
                            int64_t n);
int32_t kanso_cuda_residual_add(kanso_cuda_ctx* ctx, float* hidden, const float* proj, int64_t n);

/* ------------------------------------------------------------------------- */
/* Whole decode step: Model::forward_decode_step / forward_batch on a pure-decode
 * batch — src/model.rs:1101-1231,1360-1369,1418-1740. */
int32_t kanso_cuda_model_create(kanso_cuda_ctx* ctx, const kanso_model_config* cfg,
                                kanso_cuda_model** out);
int32_t kanso_cuda_model_destroy(kanso_cuda_model* m);
/* ModelWeights::load_from_gguf — src/weights.rs:332-493: reads a .gguf file (metadata keys
 * general.architecture, llama.block_count, llama.attention.head_count[_kv],
 * llama.embedding_length, llama.feed_forward_length, llama.attention.layer_norm_rms_epsilon
 * (default 1e-5), llama.rope.freq_base (default 10000); tensors token_embd.weight,
 * output_norm.weight, optional output.weight (absent = tied lm_head), blk.N.{attn_norm, attn_q,
 * attn_k, attn_v, attn_output, ffn_norm, ffn_gate, ffn_up, ffn_down}.weight), creates the model
 * and uploads every tensor. The Q and K projections' rows are permuted from llama.cpp's
 * interleaved head layout to rotate-half on the way (interleaved_permutation,
 * src/weights.rs:231-252; the reference permutes the projected activations instead,
 * src/model.rs:455-477). block_size / max_seq_len 0 = the loader's 16 / 2048. A missing key,
 * tensor or an unsupported architecture is KANSO_ERR_CONFIG with the reference's message;
 * 'granite' is recognised and refused (its multipliers are not wired). cfg_out may be NULL. */
int32_t kanso_cuda_model_load_gguf(kanso_cuda_ctx* ctx, const char* path, uint32_t block_size,
                                   uint32_t max_seq_len, kanso_cuda_model** out,
                                   kanso_model_config* cfg_out);
/* Projection weights: GGUF blocks in host memory (copied to the device). */
int32_t kanso_cuda_model_set_weight(kanso_cuda_model* m, uint32_t layer, int32_t which,
                                    const void* host_bytes, size_t nbytes, int32_t dtype,
                                    int64_t rows, int64_t cols);
/* Norm weights: f32[hidden] in host memory. */
int32_t kanso_cuda_model_set_norm(kanso_cuda_model* m, uint32_t layer, int32_t which,
                                  const float* host_weight, int64_t n);
/* One decode token per sequence. tokens, positions u32[B]; slots u32[B];
 * block_tables u32[B*max_blocks] padded as PaddedDecodeTables (src/model.rs:64-116);
 * context_lens u32[B] (= position + 1); all HOST arrays. logits_out f32[B, vocab] HOST.
 * Synchronous: copies the step's inputs in, runs, copies the logits back. */
int32_t kanso_cuda_decode_step(kanso_cuda_ctx* ctx, kanso_cuda_model* m, kanso_cuda_kv* kv,
                               const uint32_t* tokens, const uint32_t* positions,
                               const uint32_t* slots, const uint32_t* block_tables,
                               const uint32_t* context_lens, uint32_t B, uint32_t max_blocks,
                               int32_t act_mode, float* logits_out);
/* Same step, logits left on the device (f32[B,vocab]), asynchronous; inputs are device arrays.
 * max_ctx bounds the context lengths (sizes the split of the attention work). */
int32_t kanso_cuda_decode_step_device(kanso_cuda_ctx* ctx, kanso_cuda_model* m, kanso_cuda_kv* kv,
                                      const uint32_t* tokens, const uint32_t* positions,
                                      const uint32_t* slots, const uint32_t* block_tables,
                                      const uint32_t* context_lens, uint32_t B,
                                      uint32_t max_blocks, uint32_t max_ctx, int32_t act_mode,
                                      float* logits_dev);
/* sampler::greedy_token — src/sampler.rs:7-17 (first maximum wins). logits f32[B,vocab]
 * device, out u32[B] device. */
int32_t kanso_cuda_greedy_token(kanso_cuda_ctx* ctx, const float* logits, uint32_t* out,
                                int64_t B, int64_t vocab);

#ifdef __cplusplus
}
#endif
#endif /* KANSO_CUDA_H */
