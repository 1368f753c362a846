// Decode step of a Llama-architecture model on the cuda backend:
// Model::forward_decode_step / forward_batch on a pure-decode batch
// (src/model.rs:1101-1231,1418-1740), one token per sequence.
#include <cmath>
#include <cstring>

#include "glue.cuh"
#include "kv_pool.h"

namespace kanso {
int32_t launch_paged_attention(kanso_cuda_ctx* ctx, const kanso_cuda_kv* kv, uint32_t layer,
                               const float* q, const uint32_t* tables, const uint32_t* lens,
                               float* out, const kanso_paged_attention_params* p,
                               uint32_t max_ctx_hint, const PaDecodeFusion* fusion);
int32_t tc_matmul_multi(kanso_cuda_ctx* ctx, int32_t dtype, int nseg, const void* const* w,
                        float* const* y, const int64_t* rows, const float* x, const float* x2,
                        const float* norm_w, float eps, const float* resid, int64_t M, int64_t K,
                        bool* handled, const void* prepacked);

// Embedding rows of a Q8_0 table (src/weights.rs:50-57), bit-exact d * (f32)q.
__global__ void model_embed_kernel(const uint8_t* __restrict__ w, const uint32_t* __restrict__ ids,
                                   float* __restrict__ out, int64_t rows, int cols, int* status) {
  int t = blockIdx.x;
  uint32_t id = ids[t];
  if (id >= rows) {
    if (threadIdx.x == 0) atomicOr(status, DEV_BAD_INDEX);
    id = 0;
  }
  const uint8_t* row = w + (int64_t)id * (cols / 32) * Q8_BYTES;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    const uint8_t* blk = row + (i >> 5) * Q8_BYTES;
    float d = f16_bits_to_f32(blk[0] | (blk[1] << 8));
    out[(int64_t)t * cols + i] = __fmul_rn(d, (float)(int8_t)blk[2 + (i & 31)]);
  }
}
}  // namespace kanso

struct ModelLin {
  void* dev = nullptr;
  int32_t dtype = 0;
  int64_t rows = 0, cols = 0;
};

struct kanso_cuda_model {
  kanso_cuda_ctx* ctx = nullptr;
  kanso_model_config cfg{};
  struct Layer {
    ModelLin w[7];
    float* attn_norm = nullptr;
    float* ffn_norm = nullptr;
  };
  std::vector<Layer> layers;
  ModelLin token_embd, output;
  float* final_norm = nullptr;
  // RoPE table rows [max_seq_len][head_dim/2], built on the host like build_rope_table
  float* rope_cos = nullptr;
  float* rope_sin = nullptr;
  int rope_len = 0;
  // workspace for B sequences
  uint32_t ws_B = 0, ws_max_blocks = 0;
  float *hidden = nullptr, *normed = nullptr, *qkv = nullptr, *attn = nullptr, *proj = nullptr,
        *gate = nullptr, *up = nullptr, *act = nullptr, *logits = nullptr;
  uint32_t *d_tokens = nullptr, *d_positions = nullptr, *d_slots = nullptr, *d_tables = nullptr,
           *d_lens = nullptr;
};

using namespace kanso;

static void free_ws(kanso_cuda_model* m) {
  for (float** p : {&m->hidden, &m->normed, &m->qkv, &m->attn, &m->proj, &m->gate, &m->up, &m->act,
                    &m->logits}) {
    if (*p) cudaFree(*p);
    *p = nullptr;
  }
  for (uint32_t** p : {&m->d_tokens, &m->d_positions, &m->d_slots, &m->d_tables, &m->d_lens}) {
    if (*p) cudaFree(*p);
    *p = nullptr;
  }
  m->ws_B = m->ws_max_blocks = 0;
}

static int32_t ensure_ws(kanso_cuda_model* m, uint32_t B, uint32_t max_blocks) {
  kanso_cuda_ctx* ctx = m->ctx;
  if (B <= m->ws_B && max_blocks <= m->ws_max_blocks) return KANSO_OK;
  cudaStreamSynchronize(ctx->stream);
  if (B < m->ws_B) B = m->ws_B;
  if (max_blocks < m->ws_max_blocks) max_blocks = m->ws_max_blocks;
  free_ws(m);
  const auto& c = m->cfg;
  const uint32_t hd = c.hidden_size / c.num_attention_heads;
  const size_t qkv_w = (size_t)(c.num_attention_heads + 2 * c.num_key_value_heads) * hd;
  struct {
    float** p;
    size_t n;
  } fb[] = {{&m->hidden, (size_t)B * c.hidden_size},
            {&m->normed, (size_t)B * c.hidden_size},
            {&m->qkv, (size_t)B * qkv_w},
            {&m->attn, (size_t)B * c.num_attention_heads * hd},
            {&m->proj, (size_t)B * c.hidden_size},
            {&m->gate, (size_t)B * c.intermediate_size},
            {&m->up, (size_t)B * c.intermediate_size},
            {&m->act, (size_t)B * c.intermediate_size},
            {&m->logits, (size_t)B * c.vocab_size}};
  for (auto& b : fb) KANSO_CUDA_TRY(ctx, cudaMalloc((void**)b.p, b.n * sizeof(float)), "workspace");
  struct {
    uint32_t** p;
    size_t n;
  } ib[] = {{&m->d_tokens, B}, {&m->d_positions, B}, {&m->d_slots, B},
            {&m->d_tables, (size_t)B * max_blocks}, {&m->d_lens, B}};
  for (auto& b : ib)
    KANSO_CUDA_TRY(ctx, cudaMalloc((void**)b.p, b.n * sizeof(uint32_t)), "workspace");
  m->ws_B = B;
  m->ws_max_blocks = max_blocks;
  return KANSO_OK;
}

// Up to three projections of the same activations in one tensor-core GEMM launch (9..128
// activation rows), with rmsnorm (norm_w) or the SwiGLU product (x2) folded into the activation
// pack and the residual add into the epilogue (resid). *handled = false, nothing launched, when the
// weights or shapes are outside that kernel's range: the caller then runs the pieces singly.
static int32_t lin_multi(kanso_cuda_ctx* ctx, int n, const ModelLin* const* l, float* const* y,
                         const float* x, const float* x2, const float* norm_w, float eps,
                         const float* resid, int64_t M, int32_t act_mode, bool* handled,
                         const void* prepacked = nullptr) {
  *handled = false;
  if (act_mode != KANSO_ACT_F32 || M <= 8 || M > 128) return KANSO_OK;
  const void* w[3];
  int64_t rows[3];
  for (int i = 0; i < n; ++i) {
    if (!l[i]->dev || l[i]->dtype != l[0]->dtype || l[i]->cols != l[0]->cols) return KANSO_OK;
    w[i] = l[i]->dev;
    rows[i] = l[i]->rows;
  }
  if (l[0]->dtype != KANSO_DTYPE_Q8_0 && l[0]->dtype != KANSO_DTYPE_Q4_K) return KANSO_OK;
  return tc_matmul_multi(ctx, l[0]->dtype, n, w, y, rows, x, x2, norm_w, eps, resid, M,
                         l[0]->cols, handled, prepacked);
}

static int32_t lin(kanso_cuda_ctx* ctx, const ModelLin& l, const float* x, float* y, int64_t M,
                   int32_t act_mode) {
  if (!l.dev) return fail(ctx, KANSO_ERR_CONFIG, "decode_step: a projection weight is not set");
  return matmul_dispatch(ctx, l.dtype, l.dev, x, y, M, l.rows, l.cols, act_mode);
}

extern "C" {

int32_t kanso_cuda_model_create(kanso_cuda_ctx* ctx, const kanso_model_config* cfg,
                                kanso_cuda_model** out) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "model_create: ctx is NULL");
  if (!cfg || !out) return fail(ctx, KANSO_ERR_CONFIG, "model_create: NULL argument");
  *out = nullptr;
  if (!cfg->hidden_size || !cfg->num_attention_heads || !cfg->num_key_value_heads ||
      !cfg->num_hidden_layers || !cfg->intermediate_size || !cfg->vocab_size || !cfg->max_seq_len)
    return fail(ctx, KANSO_ERR_CONFIG, "model_create: every dimension must be non-zero");
  if (cfg->hidden_size % cfg->num_attention_heads ||
      cfg->num_attention_heads % cfg->num_key_value_heads)
    return fail(ctx, KANSO_ERR_CONFIG,
                "model_create: hidden %u / heads %u / kv heads %u do not divide", cfg->hidden_size,
                cfg->num_attention_heads, cfg->num_key_value_heads);
  const uint32_t hd = cfg->hidden_size / cfg->num_attention_heads;
  if (hd % 2) return fail(ctx, KANSO_ERR_CONFIG, "model_create: head_dim %u is odd", hd);
  auto* m = new kanso_cuda_model;
  m->ctx = ctx;
  m->cfg = *cfg;
  m->layers.resize(cfg->num_hidden_layers);
  // build_rope_table (src/model.rs:698-719), on the host with the same libm calls
  const uint32_t half = hd / 2;
  m->rope_len = (int)cfg->max_seq_len;
  std::vector<float> c((size_t)m->rope_len * half), s((size_t)m->rope_len * half), freq(half);
  for (uint32_t j = 0; j < half; ++j)
    freq[j] = std::pow(cfg->rope_theta, -2.0f * (float)j / (float)hd);
  for (int p = 0; p < m->rope_len; ++p)
    for (uint32_t j = 0; j < half; ++j) {
      float a = (float)p * freq[j];
      c[(size_t)p * half + j] = std::cos(a);
      s[(size_t)p * half + j] = std::sin(a);
    }
  cudaError_t e = cudaMalloc((void**)&m->rope_cos, c.size() * 4);
  if (e == cudaSuccess) e = cudaMalloc((void**)&m->rope_sin, s.size() * 4);
  if (e == cudaSuccess) e = cudaMemcpy(m->rope_cos, c.data(), c.size() * 4, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(m->rope_sin, s.data(), s.size() * 4, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    kanso_cuda_model_destroy(m);
    return cuda_fail(ctx, e, "model_create: rope table");
  }
  *out = m;
  return KANSO_OK;
}

int32_t kanso_cuda_model_destroy(kanso_cuda_model* m) {
  if (!m) return KANSO_OK;
  cudaDeviceSynchronize();  // the context may already be destroyed
  free_ws(m);
  for (auto& l : m->layers) {
    for (auto& w : l.w)
      if (w.dev) cudaFree(w.dev);
    if (l.attn_norm) cudaFree(l.attn_norm);
    if (l.ffn_norm) cudaFree(l.ffn_norm);
  }
  if (m->token_embd.dev) cudaFree(m->token_embd.dev);
  if (m->output.dev) cudaFree(m->output.dev);
  if (m->final_norm) cudaFree(m->final_norm);
  if (m->rope_cos) cudaFree(m->rope_cos);
  if (m->rope_sin) cudaFree(m->rope_sin);
  delete m;
  return KANSO_OK;
}

int32_t kanso_cuda_model_set_weight(kanso_cuda_model* m, uint32_t layer, int32_t which,
                                    const void* host_bytes, size_t nbytes, int32_t dtype,
                                    int64_t rows, int64_t cols) {
  if (!m) return fail(nullptr, KANSO_ERR_CONFIG, "model_set_weight: model is NULL");
  kanso_cuda_ctx* ctx = m->ctx;
  const auto& c = m->cfg;
  const uint32_t hd = c.hidden_size / c.num_attention_heads;
  int64_t er, ec;
  switch (which) {
    case KANSO_W_ATTN_Q: er = (int64_t)c.num_attention_heads * hd; ec = c.hidden_size; break;
    case KANSO_W_ATTN_K:
    case KANSO_W_ATTN_V: er = (int64_t)c.num_key_value_heads * hd; ec = c.hidden_size; break;
    case KANSO_W_ATTN_OUTPUT: er = c.hidden_size; ec = (int64_t)c.num_attention_heads * hd; break;
    case KANSO_W_FFN_GATE:
    case KANSO_W_FFN_UP: er = c.intermediate_size; ec = c.hidden_size; break;
    case KANSO_W_FFN_DOWN: er = c.hidden_size; ec = c.intermediate_size; break;
    case KANSO_W_TOKEN_EMBD:
    case KANSO_W_OUTPUT: er = c.vocab_size; ec = c.hidden_size; break;
    default: return fail(ctx, KANSO_ERR_CONFIG, "model_set_weight: unknown tensor %d", which);
  }
  if (rows != er || cols != ec)
    return fail(ctx, KANSO_ERR_SHAPE, "model_set_weight: tensor %d is [%lld x %lld], config needs [%lld x %lld]",
                which, (long long)rows, (long long)cols, (long long)er, (long long)ec);
  if (which < KANSO_W_TOKEN_EMBD && layer >= m->layers.size())
    return fail(ctx, KANSO_ERR_SHAPE, "Layer index %u out of bounds (%zu)", layer,
                m->layers.size());
  if (which == KANSO_W_TOKEN_EMBD && dtype != KANSO_DTYPE_Q8_0)
    return fail(ctx, KANSO_ERR_UNSUPPORTED, "model_set_weight: token_embd must be Q8_0");
  kanso_cuda_weight* tmp = nullptr;
  int32_t st = kanso_cuda_weight_upload(ctx, host_bytes, nbytes, dtype, rows, cols, &tmp);
  if (st) return st;
  ModelLin& dst = which == KANSO_W_TOKEN_EMBD ? m->token_embd
                  : which == KANSO_W_OUTPUT   ? m->output
                                              : m->layers[layer].w[which];
  if (dst.dev) cudaFree(dst.dev);
  dst.dev = tmp->dev;
  dst.dtype = dtype;
  dst.rows = rows;
  dst.cols = cols;
  delete tmp;  // the device buffer now belongs to the model
  return KANSO_OK;
}

int32_t kanso_cuda_model_set_norm(kanso_cuda_model* m, uint32_t layer, int32_t which,
                                  const float* host_weight, int64_t n) {
  if (!m) return fail(nullptr, KANSO_ERR_CONFIG, "model_set_norm: model is NULL");
  kanso_cuda_ctx* ctx = m->ctx;
  if (n != (int64_t)m->cfg.hidden_size)
    return fail(ctx, KANSO_ERR_SHAPE, "model_set_norm: %lld weights, hidden size is %u",
                (long long)n, m->cfg.hidden_size);
  float** dst;
  if (which == KANSO_NORM_FINAL) {
    dst = &m->final_norm;
  } else if (which == KANSO_NORM_ATTN || which == KANSO_NORM_FFN) {
    if (layer >= m->layers.size())
      return fail(ctx, KANSO_ERR_SHAPE, "Layer index %u out of bounds (%zu)", layer,
                  m->layers.size());
    dst = which == KANSO_NORM_ATTN ? &m->layers[layer].attn_norm : &m->layers[layer].ffn_norm;
  } else {
    return fail(ctx, KANSO_ERR_CONFIG, "model_set_norm: unknown norm %d", which);
  }
  if (!*dst) KANSO_CUDA_TRY(ctx, cudaMalloc((void**)dst, n * 4), "model_set_norm");
  KANSO_CUDA_TRY(ctx, cudaMemcpy(*dst, host_weight, n * 4, cudaMemcpyHostToDevice),
                 "model_set_norm");
  return KANSO_OK;
}

int32_t kanso_cuda_decode_step_device(kanso_cuda_ctx* ctx, kanso_cuda_model* m, kanso_cuda_kv* kv,
                                      const uint32_t* tokens, const uint32_t* positions,
                                      const uint32_t* slots, const uint32_t* block_tables,
                                      const uint32_t* context_lens, uint32_t B,
                                      uint32_t max_blocks, uint32_t max_ctx, int32_t act_mode,
                                      float* logits_dev) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "decode_step: ctx is NULL");
  if (!m || !kv) return fail(ctx, KANSO_ERR_SHAPE, "decode_step: model or pool is NULL");
  if (B == 0) return KANSO_OK;
  const auto& c = m->cfg;
  const uint32_t H = c.num_attention_heads, KH = c.num_key_value_heads;
  const uint32_t hd = c.hidden_size / H, hidden = c.hidden_size, inter = c.intermediate_size;
  if (kv->layers < c.num_hidden_layers || kv->kv_heads != KH || kv->head_dim != hd)
    return fail(ctx, KANSO_ERR_SHAPE,
                "decode_step: pool geometry (layers %u, kv_heads %u, head_dim %u) does not match "
                "the model (%u, %u, %u)",
                kv->layers, kv->kv_heads, kv->head_dim, c.num_hidden_layers, KH, hd);
  if (!m->token_embd.dev || !m->final_norm)
    return fail(ctx, KANSO_ERR_CONFIG, "decode_step: token_embd / final norm not set");
  int32_t st = ensure_ws(m, B, max_blocks);
  if (st) return st;
  const size_t qw = (size_t)H * hd, kw = (size_t)KH * hd;
  float* q = m->qkv;
  float* k = m->qkv + (size_t)B * qw;
  float* v = k + (size_t)B * kw;
  kanso_paged_attention_params pa{B, H, KH, hd, kv->block_size, max_blocks,
                                  1.0f / std::sqrt((float)hd)};

  model_embed_kernel<<<B, 256, 0, ctx->stream>>>((const uint8_t*)m->token_embd.dev, tokens,
                                                 m->hidden, m->token_embd.rows, (int)hidden,
                                                 ctx->dev_status);
  if ((st = after_launch(ctx, "embed"))) return st;
  const ModelLin& head = m->output.dev ? m->output : m->token_embd;  // tied lm_head

  // RoPE of q and of the new k, and the int8 store of the new K/V rows, run inside the
  // attention kernel. context_lens counts the new token, whose row is slots[seq] and must be
  // where block_tables places position context_len - 1.
  const PaDecodeFusion fusion = {k, v, positions, slots, m->rope_cos, m->rope_sin, m->rope_len};

  // Up to 8 sequences on Q8_0 weights: 5 launches per layer. The norms are folded into the
  // activation staging of the projections that follow them, SiLU*up into ffn_down's, the
  // residual adds into the epilogues, the split-context merge into the attention kernel.
  bool fused = B <= 8 && head.dtype == KANSO_DTYPE_Q8_0;
  for (uint32_t l = 0; l < c.num_hidden_layers && fused; ++l)
    for (const auto& w : m->layers[l].w) fused = fused && w.dev && w.dtype == KANSO_DTYPE_Q8_0;
  if (fused) {
    for (uint32_t l = 0; l < c.num_hidden_layers; ++l) {
      auto& ly = m->layers[l];
      if (!ly.attn_norm || !ly.ffn_norm)
        return fail(ctx, KANSO_ERR_CONFIG, "decode_step: norm weights of layer %u not set", l);
      {
        const void* w3[3] = {ly.w[KANSO_W_ATTN_Q].dev, ly.w[KANSO_W_ATTN_K].dev,
                             ly.w[KANSO_W_ATTN_V].dev};
        float* y3[3] = {q, k, v};
        const int64_t r3[3] = {(int64_t)qw, (int64_t)kw, (int64_t)kw};
        if ((st = stream_fused_q8_0(ctx, 3, w3, y3, r3, m->hidden, nullptr, ly.attn_norm,
                                    c.rms_norm_eps, nullptr, hidden, (int)B, act_mode)))
          return st;
      }
      // RoPE of q and k and the int8 store of the new K/V rows happen inside the attention
      if ((st = launch_paged_attention(ctx, kv, l, q, block_tables, context_lens, m->attn, &pa,
                                       max_ctx, &fusion)))
        return st;
      {
        const void* w1[1] = {ly.w[KANSO_W_ATTN_OUTPUT].dev};
        float* y1[1] = {m->hidden};
        const int64_t r1[1] = {(int64_t)hidden};
        if ((st = stream_fused_q8_0(ctx, 1, w1, y1, r1, m->attn, nullptr, nullptr, 0.f, m->hidden,
                                    qw, (int)B, act_mode)))
          return st;
      }
      {
        const void* w2[2] = {ly.w[KANSO_W_FFN_GATE].dev, ly.w[KANSO_W_FFN_UP].dev};
        float* y2[2] = {m->gate, m->up};
        const int64_t r2[2] = {(int64_t)inter, (int64_t)inter};
        if ((st = stream_fused_q8_0(ctx, 2, w2, y2, r2, m->hidden, nullptr, ly.ffn_norm,
                                    c.rms_norm_eps, nullptr, hidden, (int)B, act_mode)))
          return st;
      }
      {
        const void* w1[1] = {ly.w[KANSO_W_FFN_DOWN].dev};
        float* y1[1] = {m->hidden};
        const int64_t r1[1] = {(int64_t)hidden};
        if ((st = stream_fused_q8_0(ctx, 1, w1, y1, r1, m->gate, m->up, nullptr, 0.f, m->hidden,
                                    inter, (int)B, act_mode)))
          return st;
      }
    }
    const void* w1[1] = {head.dev};
    float* y1[1] = {logits_dev};
    const int64_t r1[1] = {head.rows};
    return stream_fused_q8_0(ctx, 1, w1, y1, r1, m->hidden, nullptr, m->final_norm,
                             c.rms_norm_eps, nullptr, hidden, (int)B, act_mode);
  }

  for (uint32_t l = 0; l < c.num_hidden_layers; ++l) {
    auto& ly = m->layers[l];
    if (!ly.attn_norm || !ly.ffn_norm)
      return fail(ctx, KANSO_ERR_CONFIG, "decode_step: norm weights of layer %u not set", l);
    bool one = false;  // the launch below covered the whole group
    {
      const ModelLin* l3[3] = {&ly.w[KANSO_W_ATTN_Q], &ly.w[KANSO_W_ATTN_K], &ly.w[KANSO_W_ATTN_V]};
      float* y3[3] = {q, k, v};
      if ((st = lin_multi(ctx, 3, l3, y3, m->hidden, nullptr, ly.attn_norm, c.rms_norm_eps,
                          nullptr, B, act_mode, &one)))
        return st;
    }
    if (!one) {
      if ((st = launch_rmsnorm(ctx, m->hidden, ly.attn_norm, m->normed, B, hidden,
                               c.rms_norm_eps)))
        return st;
      if ((st = lin(ctx, ly.w[KANSO_W_ATTN_Q], m->normed, q, B, act_mode))) return st;
      if ((st = lin(ctx, ly.w[KANSO_W_ATTN_K], m->normed, k, B, act_mode))) return st;
      if ((st = lin(ctx, ly.w[KANSO_W_ATTN_V], m->normed, v, B, act_mode))) return st;
    }
    // The attention's merge also leaves its output as the packed f16 tile of the o-projection's
    // GEMM (when it can), which then starts without a pack launch of its own.
    const void* packed = nullptr;
    PaDecodeFusion fusion_l = fusion;
    if (act_mode == KANSO_ACT_F32) fusion_l.packed_out = &packed;
    if ((st = launch_paged_attention(ctx, kv, l, q, block_tables, context_lens, m->attn, &pa,
                                     max_ctx, &fusion_l)))
      return st;
    {
      const ModelLin* l1[1] = {&ly.w[KANSO_W_ATTN_OUTPUT]};
      float* y1[1] = {m->hidden};
      one = false;
      if (packed &&
          (st = lin_multi(ctx, 1, l1, y1, m->attn, nullptr, nullptr, 0.f, m->hidden, B, act_mode,
                          &one, packed)))
        return st;
      if (!one && (st = lin_multi(ctx, 1, l1, y1, m->attn, nullptr, nullptr, 0.f, m->hidden, B,
                                  act_mode, &one)))
        return st;
    }
    if (!one) {
      if ((st = lin(ctx, ly.w[KANSO_W_ATTN_OUTPUT], m->attn, m->proj, B, act_mode))) return st;
      if ((st = launch_residual_add(ctx, m->hidden, m->proj, (int64_t)B * hidden))) return st;
    }
    {
      const ModelLin* l2[2] = {&ly.w[KANSO_W_FFN_GATE], &ly.w[KANSO_W_FFN_UP]};
      float* y2[2] = {m->gate, m->up};
      if ((st = lin_multi(ctx, 2, l2, y2, m->hidden, nullptr, ly.ffn_norm, c.rms_norm_eps, nullptr,
                          B, act_mode, &one)))
        return st;
    }
    if (!one) {
      if ((st = launch_rmsnorm(ctx, m->hidden, ly.ffn_norm, m->normed, B, hidden, c.rms_norm_eps)))
        return st;
      if ((st = lin(ctx, ly.w[KANSO_W_FFN_GATE], m->normed, m->gate, B, act_mode))) return st;
      if ((st = lin(ctx, ly.w[KANSO_W_FFN_UP], m->normed, m->up, B, act_mode))) return st;
    }
    {
      const ModelLin* l1[1] = {&ly.w[KANSO_W_FFN_DOWN]};
      float* y1[1] = {m->hidden};
      if ((st = lin_multi(ctx, 1, l1, y1, m->gate, m->up, nullptr, 0.f, m->hidden, B, act_mode,
                          &one)))
        return st;
    }
    if (!one) {
      if ((st = launch_silu_mul(ctx, m->gate, m->up, m->act, (int64_t)B * inter))) return st;
      if ((st = lin(ctx, ly.w[KANSO_W_FFN_DOWN], m->act, m->proj, B, act_mode))) return st;
      if ((st = launch_residual_add(ctx, m->hidden, m->proj, (int64_t)B * hidden))) return st;
    }
  }
  {
    bool one = false;
    const ModelLin* l1[1] = {&head};
    float* y1[1] = {logits_dev};
    if ((st = lin_multi(ctx, 1, l1, y1, m->hidden, nullptr, m->final_norm, c.rms_norm_eps, nullptr,
                        B, act_mode, &one)) ||
        one)
      return st;
  }
  if ((st = launch_rmsnorm(ctx, m->hidden, m->final_norm, m->normed, B, hidden, c.rms_norm_eps)))
    return st;
  return lin(ctx, head, m->normed, logits_dev, B, act_mode);
}

int32_t kanso_cuda_decode_step(kanso_cuda_ctx* ctx, kanso_cuda_model* m, kanso_cuda_kv* kv,
                               const uint32_t* tokens, const uint32_t* positions,
                               const uint32_t* slots, const uint32_t* block_tables,
                               const uint32_t* context_lens, uint32_t B, uint32_t max_blocks,
                               int32_t act_mode, float* logits_out) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "decode_step: ctx is NULL");
  if (!m || !kv) return fail(ctx, KANSO_ERR_SHAPE, "decode_step: model or pool is NULL");
  if (B == 0) return KANSO_OK;
  if (!tokens || !positions || !slots || !block_tables || !context_lens || !logits_out)
    return fail(ctx, KANSO_ERR_SHAPE, "decode_step: NULL argument");
  if (max_blocks == 0) return fail(ctx, KANSO_ERR_SHAPE, "decode_step: max_blocks is 0");
  // host-side checks the reference makes before touching the pool
  const uint32_t bs = kv->block_size;
  uint32_t max_ctx = 0;
  for (uint32_t s = 0; s < B; ++s) {
    if (tokens[s] >= m->cfg.vocab_size)
      return fail(ctx, KANSO_ERR_SHAPE, "decode_step: token id %u out of range (vocab %u)",
                  tokens[s], m->cfg.vocab_size);
    if (positions[s] >= m->cfg.max_seq_len)
      return fail(ctx, KANSO_ERR_SHAPE, "decode_step: position %u beyond max_seq_len %u",
                  positions[s], m->cfg.max_seq_len);
    if ((uint64_t)slots[s] >= (uint64_t)kv->num_blocks * bs)
      return fail(ctx, KANSO_ERR_SHAPE, "Slot %u out of bounds for %u blocks of size %u", slots[s],
                  kv->num_blocks, bs);
    uint32_t ctxlen = context_lens[s];
    if (ctxlen == 0 || (ctxlen + bs - 1) / bs > max_blocks)
      // src/model.rs:92-101: a table shorter than ceil(ctx/bs) is an error, never a clamp
      return fail(ctx, KANSO_ERR_SHAPE,
                  "forward_batch: sequence %u attends %u tokens but its block table has %u of the "
                  "%u blocks needed",
                  s, ctxlen, max_blocks, (ctxlen + bs - 1) / bs);
    for (uint32_t b = 0; b < (ctxlen + bs - 1) / bs; ++b)
      if (block_tables[(size_t)s * max_blocks + b] >= kv->num_blocks)
        return fail(ctx, KANSO_ERR_SHAPE, "Physical block index %u out of bounds (%u)",
                    block_tables[(size_t)s * max_blocks + b], kv->num_blocks);
    if (ctxlen > max_ctx) max_ctx = ctxlen;
  }
  int32_t st = ensure_ws(m, B, max_blocks);
  if (st) return st;
  const size_t nb = (size_t)B * 4, tb = (size_t)B * max_blocks * 4;
  const size_t lb = (size_t)B * m->cfg.vocab_size * 4;
  if ((st = ctx_pinned(ctx, 4 * nb + tb + lb))) return st;
  char* ph = (char*)ctx->pinned;
  std::memcpy(ph, tokens, nb);
  std::memcpy(ph + nb, positions, nb);
  std::memcpy(ph + 2 * nb, slots, nb);
  std::memcpy(ph + 3 * nb, context_lens, nb);
  std::memcpy(ph + 4 * nb, block_tables, tb);
  cudaStream_t s = ctx->stream;
  KANSO_CUDA_TRY(ctx, cudaMemcpyAsync(m->d_tokens, ph, nb, cudaMemcpyHostToDevice, s), "h2d");
  KANSO_CUDA_TRY(ctx, cudaMemcpyAsync(m->d_positions, ph + nb, nb, cudaMemcpyHostToDevice, s),
                 "h2d");
  KANSO_CUDA_TRY(ctx, cudaMemcpyAsync(m->d_slots, ph + 2 * nb, nb, cudaMemcpyHostToDevice, s),
                 "h2d");
  KANSO_CUDA_TRY(ctx, cudaMemcpyAsync(m->d_lens, ph + 3 * nb, nb, cudaMemcpyHostToDevice, s),
                 "h2d");
  KANSO_CUDA_TRY(ctx, cudaMemcpyAsync(m->d_tables, ph + 4 * nb, tb, cudaMemcpyHostToDevice, s),
                 "h2d");
  st = kanso_cuda_decode_step_device(ctx, m, kv, m->d_tokens, m->d_positions, m->d_slots,
                                     m->d_tables, m->d_lens, B, max_blocks, max_ctx, act_mode,
                                     m->logits);
  if (st) return st;
  char* pl = ph + 4 * nb + tb;
  KANSO_CUDA_TRY(ctx, cudaMemcpyAsync(pl, m->logits, lb, cudaMemcpyDeviceToHost, s), "d2h");
  if ((st = kanso_cuda_sync(ctx))) return st;
  std::memcpy(logits_out, pl, lb);
  return KANSO_OK;
}

}  // extern "C"
