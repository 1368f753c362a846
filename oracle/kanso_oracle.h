/*
 * kanso_oracle.h — CPU restatement of kanso-infer's quantized hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This library is the checker the CUDA kernels are
 * compared against; the product never links, loads or calls it. It is plain
 * single-threaded C++ compiled without FMA contraction so that every rounding
 * step is the one the reference's Rust source performs.
 *
 * Parity status: pinned on the reference's own test inputs where those carry
 * expected values (the hand-worked paged-attention example, the quantizer
 * round-trip bounds, the int8 KV round-trip bound, the Q8_0-vs-dense bound) and
 * on an independent numpy restatement plus the `gguf` Python package's block
 * decoders (tests/golden). The reference crate itself cannot be built where this
 * was written (no Rust toolchain), so no output of the reference binary backs it.
 *
 * Citations are file:line inside the kanso-infer source tree.
 *
 * Two scale layouts are offered: "gguf" = blocks as stored in a GGUF file (f16
 * scales: 34-byte Q8_0, 144-byte Q4_K), which is what the CUDA backend reads,
 * and "ref" = the reference's in-memory structs with f32 scales
 * (src/quant/q8_0.rs:4-9, src/quant/q4_k.rs:5-12), which is what the
 * reference's own tests construct. The arithmetic after the scale has been
 * widened to f32 is the same code.
 */
#ifndef KANSO_ORACLE_H
#define KANSO_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* IEEE binary16 <-> binary32, round to nearest even. */
uint16_t kanso_ref_f32_to_f16(float f);
float kanso_ref_f16_to_f32(uint16_t h);

/* ---- Q8_0: src/quant/q8_0.rs ---- */
/* quantize_row_q8_0 (q8_0.rs:13-32,43-48): d f32[cols/32], qs int8[cols]. */
void kanso_ref_quantize_row_q8_0(const float* x, int64_t cols, float* d_out, int8_t* qs_out);
/* Rule of from_f32_slice per 32 weights, then d rounded to f16; q stay as computed from the f32 d. */
void kanso_ref_quantize_weights_q8_0(const float* w, int64_t rows, int64_t cols, uint8_t* gguf_out);
/* BlockQ8_0::dequantize (q8_0.rs:35-39). */
void kanso_ref_dequantize_q8_0(const uint8_t* gguf, int64_t nblocks, float* out);
/* scalar_dot_q8_0 (q8_0.rs:51-57) on a ref-layout block. */
float kanso_ref_dot_q8_0_ref(float d, const int8_t* qs, const float* x);
/* scalar_dot_q8_0_q8_0 (q8_0.rs:60-66) on ref-layout blocks; *isum gets the int32 sum. */
float kanso_ref_dot_q8_0_q8_0_ref(float wd, const int8_t* wqs, float xd, const int8_t* xqs,
                                  int32_t* isum);
/* scalar_gemv_q8_0 (q8_0.rs:69-93). */
void kanso_ref_gemv_q8_0(const uint8_t* w, const float* x, float* out, int64_t rows, int64_t cols);
void kanso_ref_gemv_q8_0_ref(const float* d, const int8_t* qs, const float* x, float* out,
                             int64_t rows, int64_t cols);
/* quantize_row_q8_0 on x, then scalar_dot_q8_0_q8_0 per block, summed like scalar_gemv_q8_0. */
void kanso_ref_gemv_q8_0_q8(const uint8_t* w, const float* x, float* out, int64_t rows,
                            int64_t cols);
/* The int32 sums of scalar_dot_q8_0_q8_0 for every (row, block). */
void kanso_ref_block_isums_q8_0(const uint8_t* w, const int8_t* x_qs, int32_t* isums,
                                int64_t rows, int64_t cols);
/* LinearWeight::forward restated with the block kernels: y[M,N] = x[M,K] @ W[N,K]^T. */
void kanso_ref_gemm_q8_0(const uint8_t* w, const float* x, float* y, int64_t M, int64_t N,
                         int64_t K, int32_t act_mode);

/* ---- Q4_K: src/quant/q4_k.rs ---- */
/* get_scale_min_k4 (q4_k.rs:16-26). */
void kanso_ref_get_scale_min_k4(int32_t j, const uint8_t* scales12, uint8_t* sc, uint8_t* m);
/* 8 scales then 8 mins per super-block. */
void kanso_ref_unpack_scales_q4_k(const uint8_t* gguf, int64_t nblocks, uint8_t* out);
/* BlockQ4_K::dequantize (q4_k.rs:30-55). */
void kanso_ref_dequantize_q4_k(const uint8_t* gguf, int64_t nblocks, float* out);
void kanso_ref_dequantize_q4_k_ref(float d, float dmin, const uint8_t* scales12,
                                   const uint8_t* qs128, float* out256);
/* scalar_dot_q4_k (q4_k.rs:58-66). */
float kanso_ref_dot_q4_k_ref(float d, float dmin, const uint8_t* scales12, const uint8_t* qs128,
                             const float* x256);
/* scalar_gemv_q4_k (q4_k.rs:69-93). */
void kanso_ref_gemv_q4_k(const uint8_t* w, const float* x, float* out, int64_t rows, int64_t cols);
void kanso_ref_gemm_q4_k(const uint8_t* w, const float* x, float* y, int64_t M, int64_t N,
                         int64_t K);
/* Generator of VALID Q4_K super-blocks from f32 weights. The reference tree holds no
 * Q4_K quantizer (it calls candle's); parity is defined on the decoded blocks, so any
 * valid encoder serves. Not claimed to match candle/ggml byte for byte. */
void kanso_ref_quantize_weights_q4_k(const float* w, int64_t rows, int64_t cols,
                                     uint8_t* gguf_out);

/* ---- int8 / fp8 KV pool: src/kv_cache/quantized_storage.rs ---- */
typedef struct kanso_ref_kv kanso_ref_kv;
/* quantize_head_slice, Int8 arm (quantized_storage.rs:452-469). Returns the scale. */
float kanso_ref_kv_quantize_head(const float* x, int32_t n, int8_t* q);
kanso_ref_kv* kanso_ref_kv_create(uint32_t layers, uint32_t num_blocks, uint32_t block_size,
                                  uint32_t kv_heads, uint32_t head_dim);
/* The same pool in QuantMode::Fp8 when fp8 != 0 (QuantizedKvStorage::new_fp8,
 * quantized_storage.rs:109-131). */
kanso_ref_kv* kanso_ref_kv_create_typed(uint32_t layers, uint32_t num_blocks, uint32_t block_size,
                                        uint32_t kv_heads, uint32_t head_dim, int32_t fp8);
/* quantize_head_slice, Fp8 arm (quantized_storage.rs:470-484); E4M3 per the float8 crate. */
float kanso_ref_kv_quantize_head_fp8(const float* x, int32_t n, int8_t* q);
float kanso_ref_fp8_e4m3_to_f32(uint8_t bits);
uint8_t kanso_ref_fp8_e4m3_from_f32(float x);
void kanso_ref_kv_destroy(kanso_ref_kv* kv);
/* write_quantized_kv_token (quantized_storage.rs:143-204); status as the C ABI's. */
int32_t kanso_ref_kv_write_token(kanso_ref_kv* kv, uint32_t layer, uint32_t block,
                                 uint32_t offset, const float* k, const float* v);
/* KvStorageKind::write_kv_slots (src/kv_cache/kind.rs:348): T tokens, slot = block*block_size +
 * offset (kind.rs:111), k and v f32[T, kvh*hd]; each token through write_quantized_kv_token. */
int32_t kanso_ref_kv_write_slots(kanso_ref_kv* kv, uint32_t layer, const uint32_t* slots,
                                 const float* k, const float* v, int64_t T);
/* reset_block (quantized_storage.rs:134-140). */
void kanso_ref_kv_reset_block(kanso_ref_kv* kv, uint32_t block);
/* read_quantized_kv_token (quantized_storage.rs:219-270). Any output may be NULL. */
int32_t kanso_ref_kv_read_token(const kanso_ref_kv* kv, uint32_t layer, uint32_t block,
                                uint32_t offset, int8_t* k_q, int8_t* v_q, float* k_scale,
                                float* v_scale, float* k_deq, float* v_deq);
/* gather_dequantized_blocks (quantized_storage.rs:284-383): out f32[num_tokens,kvh,hd]. */
int32_t kanso_ref_kv_gather(const kanso_ref_kv* kv, uint32_t layer, const uint32_t* blocks,
                            uint32_t nblocks, uint32_t num_tokens, float* k_out, float* v_out);

/* ---- paged attention: src/metal/paged_attention.rs ---- */
typedef struct kanso_ref_pa_params {
  uint32_t num_seqs, num_heads, num_kv_heads, head_dim, block_size, max_num_blocks_per_seq;
  float scale;
} kanso_ref_pa_params;
/* validate_paged_attention_params (paged_attention.rs:39-81). 0 = ok. */
int32_t kanso_ref_validate_pa_params(const kanso_ref_pa_params* p);
/* paged_attention_num_partitions (paged_attention.rs:27-32). */
uint32_t kanso_ref_pa_num_partitions(const kanso_ref_pa_params* p);
/* cpu_paged_attention (paged_attention.rs:84-178) over f32 caches. */
void kanso_ref_paged_attention_f32(const float* q, const float* k_cache, const float* v_cache,
                                   const uint32_t* block_tables, const uint32_t* context_lens,
                                   const kanso_ref_pa_params* p, float* out);
/* The same attention over the int8 pool: per sequence gather_dequantized_blocks then
 * the math of cpu_paged_attention on the dequantised rows. */
int32_t kanso_ref_paged_attention_int8(const kanso_ref_kv* kv, uint32_t layer, const float* q,
                                       const uint32_t* block_tables,
                                       const uint32_t* context_lens,
                                       const kanso_ref_pa_params* p, float* out);

/* Chunked-prefill attention of one sequence as Model::forward_prefill computes it
 * (src/model.rs:1027-1085, gqa_attention src/model.rs:764-795): the prefix 0..start_pos+chunk_len
 * gathered from the int8 pool, an offset causal mask of -1e9 added to the scaled scores, softmax,
 * P.V. q and out f32 [chunk_len, num_heads, head_dim]. */
int32_t kanso_ref_prefill_attention_int8(const kanso_ref_kv* kv, uint32_t layer, const float* q,
                                         const uint32_t* blocks, uint32_t nblocks,
                                         uint32_t start_pos, uint32_t chunk_len,
                                         uint32_t num_heads, float scale, float* out);

/* ---- glue: src/model.rs:653-737,367-382; src/sampler.rs:7-17 ---- */
void kanso_ref_rmsnorm(const float* x, const float* w, float* out, int64_t rows, int64_t hidden,
                       float eps);
/* cos/sin rows of build_rope_table (model.rs:698-719): f32[len, head_dim/2] each. */
void kanso_ref_rope_table(float theta, int64_t len, int64_t head_dim, float* cos_out,
                          float* sin_out);
/* rope_apply (model.rs:721-737) in place on x f32[T, heads, head_dim]. */
void kanso_ref_rope(float* x, const uint32_t* positions, int64_t T, int64_t heads,
                    int64_t head_dim, float theta);
void kanso_ref_silu_mul(const float* gate, const float* up, float* out, int64_t n);
uint32_t kanso_ref_greedy_token(const float* logits, int64_t n);
/* PaddedDecodeTables::new (model.rs:64-116). tables: concatenated per-sequence tables with
 * table_lens[s] entries each. out u32[num_seqs*max_blocks]; returns max_blocks, or 0 with
 * *status set when a table is shorter than ceil(ctx/bs). */
uint32_t kanso_ref_padded_decode_tables(uint32_t block_size, const uint32_t* tables,
                                        const uint32_t* table_lens, const uint32_t* context_lens,
                                        uint32_t num_seqs, uint32_t* out, uint32_t out_capacity,
                                        int32_t* status);

/* ---- decode step: src/model.rs:1101-1231 per sequence ---- */
typedef struct kanso_ref_model kanso_ref_model;
typedef struct kanso_ref_model_config {
  uint32_t hidden_size, num_attention_heads, num_key_value_heads, num_hidden_layers,
      intermediate_size, vocab_size, block_size, max_seq_len;
  float rms_norm_eps, rope_theta;
} kanso_ref_model_config;
kanso_ref_model* kanso_ref_model_create(const kanso_ref_model_config* cfg);
void kanso_ref_model_destroy(kanso_ref_model* m);
/* Pointers are borrowed: the caller keeps the block bytes alive. Only Q8_0 (dtype 8). */
int32_t kanso_ref_model_set_weight(kanso_ref_model* m, uint32_t layer, int32_t which,
                                   const uint8_t* gguf, int64_t rows, int64_t cols);
int32_t kanso_ref_model_set_norm(kanso_ref_model* m, uint32_t layer, int32_t which,
                                 const float* w, int64_t n);
/* One decode token for each of B sequences, each through forward_decode_step's order of
 * operations. last_layers > 0 runs only that many layers (for bounded CPU timing). */
int32_t kanso_ref_decode_step(const kanso_ref_model* m, kanso_ref_kv* kv, const uint32_t* tokens,
                              const uint32_t* positions, const uint32_t* slots,
                              const uint32_t* block_tables, const uint32_t* context_lens,
                              uint32_t B, uint32_t max_blocks, int32_t act_mode,
                              uint32_t num_layers_to_run, float* logits_out);

#ifdef __cplusplus
}
#endif
#endif
