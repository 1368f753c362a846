// GGUF file -> model on the device: ModelWeights::load_from_gguf (src/weights.rs:332-493).
// Same metadata keys, tensor names, defaults and refusals as the reference's loader; projection
// weights keep the file's blocks (only Q8_0 is wired for the decode step, as the reference's
// Q8_0-resident path), the 1-D norms are widened to f32, a missing output.weight means a tied
// lm_head (src/weights.rs:418-422). llama.cpp stores Q and K projections with the two halves of
// every head interleaved; the reference undoes that with an index_select on the projected
// activations (interleaved_permutation, src/weights.rs:231-252, applied at
// src/model.rs:455-477). Selecting output j = old output perm[j] is the same as putting weight
// row perm[j] in row j, and a quantized row is a run of whole blocks, so here the permutation is
// folded into the upload as a row permutation and costs nothing per token.
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "ctx.h"

namespace kanso {
namespace {

struct GgufValue {
  uint32_t type = 0;
  uint64_t u = 0;
  double f = 0.0;
  std::string s;
};
struct GgufTensor {
  std::vector<uint64_t> dims;  // dims[0] is the innermost (columns)
  uint32_t type = 0;
  uint64_t offset = 0;
};

struct Reader {
  const uint8_t* p;
  size_t n, pos = 0;
  bool ok = true;
  template <typename T>
  T get() {
    T v{};
    if (pos + sizeof(T) > n) {
      ok = false;
      return v;
    }
    std::memcpy(&v, p + pos, sizeof(T));
    pos += sizeof(T);
    return v;
  }
  std::string str() {
    const uint64_t len = get<uint64_t>();
    if (!ok || len > n - pos) {
      ok = false;
      return {};
    }
    std::string s(reinterpret_cast<const char*>(p + pos), (size_t)len);
    pos += (size_t)len;
    return s;
  }
};

// Scalar sizes of the GGUF metadata value types 0..12 (8 = string, 9 = array).
size_t scalar_size(uint32_t t) {
  switch (t) {
    case 0: case 1: case 7: return 1;
    case 2: case 3: return 2;
    case 4: case 5: case 6: return 4;
    case 10: case 11: case 12: return 8;
    default: return 0;
  }
}

bool read_value(Reader& r, uint32_t type, GgufValue* out) {
  out->type = type;
  switch (type) {
    case 0: out->u = r.get<uint8_t>(); break;
    case 1: out->u = (uint64_t)(int64_t)r.get<int8_t>(); break;
    case 2: out->u = r.get<uint16_t>(); break;
    case 3: out->u = (uint64_t)(int64_t)r.get<int16_t>(); break;
    case 4: out->u = r.get<uint32_t>(); break;
    case 5: out->u = (uint64_t)(int64_t)r.get<int32_t>(); break;
    case 6: out->f = r.get<float>(); break;
    case 7: out->u = r.get<uint8_t>(); break;
    case 8: out->s = r.str(); break;
    case 10: out->u = r.get<uint64_t>(); break;
    case 11: out->u = (uint64_t)r.get<int64_t>(); break;
    case 12: out->f = r.get<double>(); break;
    case 9: {  // array: skipped (the loader reads no array-valued key)
      const uint32_t et = r.get<uint32_t>();
      const uint64_t cnt = r.get<uint64_t>();
      if (!r.ok) return false;
      if (et == 8) {
        for (uint64_t i = 0; i < cnt && r.ok; ++i) r.str();
      } else if (et == 9 || scalar_size(et) == 0) {
        return false;
      } else {
        const size_t bytes = scalar_size(et);
        if (cnt > (r.n - r.pos) / bytes) return false;
        r.pos += (size_t)cnt * bytes;
      }
      break;
    }
    default: return false;
  }
  return r.ok;
}

float f16_to_f32_host(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FF;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while (!(man & 0x400));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

}  // namespace
}  // namespace kanso

using namespace kanso;

extern "C" int32_t kanso_cuda_model_load_gguf(kanso_cuda_ctx* ctx, const char* path,
                                              uint32_t block_size, uint32_t max_seq_len,
                                              kanso_cuda_model** out, kanso_model_config* cfg_out) {
  if (!ctx) return fail(nullptr, KANSO_ERR_CONFIG, "model_load_gguf: ctx is NULL");
  if (!path || !out) return fail(ctx, KANSO_ERR_SHAPE, "model_load_gguf: NULL pointer");
  *out = nullptr;
  std::vector<uint8_t> file;
  {
    FILE* f = std::fopen(path, "rb");
    if (!f) return fail(ctx, KANSO_ERR_CONFIG, "Failed to open GGUF file %s", path);
    std::fseek(f, 0, SEEK_END);
    const long sz = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    if (sz > 0) {
      file.resize((size_t)sz);
      if (std::fread(file.data(), 1, file.size(), f) != file.size()) file.clear();
    }
    std::fclose(f);
  }
  Reader r{file.data(), file.size()};
  auto parse_fail = [&](const char* why) {
    return fail(ctx, KANSO_ERR_CONFIG, "Failed to parse GGUF file %s: %s", path, why);
  };
  if (r.get<uint32_t>() != 0x46554747u) return parse_fail("bad magic");
  const uint32_t version = r.get<uint32_t>();
  if (version < 2 || version > 3) return parse_fail("unsupported version");
  const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
  if (!r.ok || n_tensors > (1u << 20) || n_kv > (1u << 20)) return parse_fail("bad header");
  std::map<std::string, GgufValue> meta;
  for (uint64_t i = 0; i < n_kv; ++i) {
    std::string key = r.str();
    const uint32_t type = r.get<uint32_t>();
    GgufValue v;
    if (!r.ok || !read_value(r, type, &v)) return parse_fail("bad metadata");
    meta[key] = std::move(v);
  }
  std::map<std::string, GgufTensor> tensors;
  for (uint64_t i = 0; i < n_tensors; ++i) {
    std::string name = r.str();
    GgufTensor t;
    const uint32_t nd = r.get<uint32_t>();
    if (!r.ok || nd > 4) return parse_fail("bad tensor info");
    for (uint32_t d = 0; d < nd; ++d) t.dims.push_back(r.get<uint64_t>());
    t.type = r.get<uint32_t>();
    t.offset = r.get<uint64_t>();
    if (!r.ok) return parse_fail("bad tensor info");
    tensors[name] = std::move(t);
  }
  uint64_t align = 32;
  if (meta.count("general.alignment")) align = meta["general.alignment"].u;
  if (align == 0 || (align & (align - 1))) return parse_fail("bad alignment");
  const size_t data0 = (r.pos + align - 1) & ~(size_t)(align - 1);

  auto need = [&](const std::string& key, GgufValue* v) -> int32_t {
    auto it = meta.find(key);
    if (it == meta.end())
      return fail(ctx, KANSO_ERR_CONFIG, "Missing GGUF metadata key '%s'", key.c_str());
    *v = it->second;
    return KANSO_OK;
  };
  GgufValue v;
  if (!meta.count("general.architecture") || meta["general.architecture"].type != 8)
    return fail(ctx, KANSO_ERR_CONFIG,
                "Missing GGUF metadata key 'general.architecture': architecture must be "
                "explicitly specified (supported: 'llama', 'granite')");
  const std::string arch = meta["general.architecture"].s;
  if (arch == "granite")
    return fail(ctx, KANSO_ERR_UNSUPPORTED,
                "GGUF architecture 'granite': its embedding/attention/residual/logit multipliers "
                "are not wired in the cuda backend's decode step");
  if (arch != "llama")
    return fail(ctx, KANSO_ERR_CONFIG,
                "unsupported GGUF architecture '%s': only 'llama' and 'granite' (dense) load; "
                "hybrid SSM/conv models are roadmap, not wired", arch.c_str());
  const std::string px = arch + ".";
  kanso_model_config c = {};
  int32_t st;
  if ((st = need(px + "block_count", &v))) return st;
  c.num_hidden_layers = (uint32_t)v.u;
  if ((st = need(px + "attention.head_count", &v))) return st;
  c.num_attention_heads = (uint32_t)v.u;
  if ((st = need(px + "attention.head_count_kv", &v))) return st;
  c.num_key_value_heads = (uint32_t)v.u;
  if ((st = need(px + "embedding_length", &v))) return st;
  c.hidden_size = (uint32_t)v.u;
  if (c.num_attention_heads == 0 || c.num_key_value_heads == 0 ||
      c.hidden_size < c.num_attention_heads)
    return fail(ctx, KANSO_ERR_CONFIG,
                "cannot build KV storage: model declares %u attention heads, %u KV heads and "
                "hidden size %u", c.num_attention_heads, c.num_key_value_heads, c.hidden_size);
  if ((st = need(px + "feed_forward_length", &v))) return st;
  c.intermediate_size = (uint32_t)v.u;
  c.rms_norm_eps = 1e-5f;
  if (meta.count(px + "attention.layer_norm_rms_epsilon")) {
    const GgufValue& e = meta[px + "attention.layer_norm_rms_epsilon"];
    if (e.type == 6 || e.type == 12) c.rms_norm_eps = (float)e.f;
  }
  c.rope_theta = 10000.0f;
  if (meta.count(px + "rope.freq_base")) {
    const GgufValue& e = meta[px + "rope.freq_base"];
    if (e.type == 6 || e.type == 12) c.rope_theta = (float)e.f;
  }
  c.block_size = block_size ? block_size : 16;       // the reference's loader: 16
  c.max_seq_len = max_seq_len ? max_seq_len : 2048;  // and 2048 (src/weights.rs:462-463)

  auto find = [&](const std::string& name, const GgufTensor** t) -> int32_t {
    auto it = tensors.find(name);
    if (it == tensors.end())
      return fail(ctx, KANSO_ERR_CONFIG, "GGUF tensor '%s' is missing", name.c_str());
    *t = &it->second;
    return KANSO_OK;
  };
  auto block_of = [](uint32_t type, int* blk, int* bb) {
    if (type == KANSO_DTYPE_Q8_0) {
      *blk = 32;
      *bb = Q8_BYTES;
      return true;
    }
    if (type == KANSO_DTYPE_Q4_K) {
      *blk = 256;
      *bb = Q4K_BYTES;
      return true;
    }
    return false;
  };
  const GgufTensor* te = nullptr;
  if ((st = find("token_embd.weight", &te))) return st;
  if (te->dims.size() != 2 || te->dims[0] != c.hidden_size)
    return fail(ctx, KANSO_ERR_SHAPE, "GGUF tensor 'token_embd.weight' is not [vocab x %u]",
                c.hidden_size);
  c.vocab_size = (uint32_t)te->dims[1];

  kanso_cuda_model* m = nullptr;
  if ((st = kanso_cuda_model_create(ctx, &c, &m))) return st;
  const uint32_t hd = c.hidden_size / c.num_attention_heads;
  std::vector<uint8_t> permuted;
  auto put_weight = [&](const std::string& name, uint32_t layer, int32_t which,
                        uint32_t perm_heads) -> int32_t {
    const GgufTensor* t = nullptr;
    int32_t s2 = find(name, &t);
    if (s2) return s2;
    int blk, bb;
    if (t->dims.size() != 2 || !block_of(t->type, &blk, &bb))
      return fail(ctx, KANSO_ERR_UNSUPPORTED,
                  "GGUF tensor '%s': type %u is neither Q8_0 (8) nor Q4_K (12)", name.c_str(),
                  t->type);
    const uint64_t cols = t->dims[0], rows = t->dims[1];
    if (cols % blk) return fail(ctx, KANSO_ERR_SHAPE, "GGUF tensor '%s': %llu columns", name.c_str(),
                                (unsigned long long)cols);
    const size_t row_bytes = (size_t)(cols / blk) * bb, nbytes = row_bytes * (size_t)rows;
    if (data0 + t->offset > file.size() || nbytes > file.size() - data0 - t->offset)
      return fail(ctx, KANSO_ERR_CONFIG, "GGUF tensor '%s' runs past the end of the file",
                  name.c_str());
    const uint8_t* src = file.data() + data0 + t->offset;
    if (perm_heads) {
      // row j of the stored matrix = row perm[j] of the file's: evens of each head first, then
      // odds (interleaved_permutation, src/weights.rs:231-252)
      if (rows != (uint64_t)perm_heads * hd)
        return fail(ctx, KANSO_ERR_SHAPE, "GGUF tensor '%s' has %llu rows, %u heads x %u expected",
                    name.c_str(), (unsigned long long)rows, perm_heads, hd);
      permuted.resize(nbytes);
      const uint32_t half = hd / 2;
      for (uint32_t h = 0; h < perm_heads; ++h)
        for (uint32_t i = 0; i < hd; ++i) {
          const uint32_t from = h * hd + (i < half ? 2 * i : 2 * (i - half) + 1);
          std::memcpy(permuted.data() + (size_t)(h * hd + i) * row_bytes,
                      src + (size_t)from * row_bytes, row_bytes);
        }
      src = permuted.data();
    }
    return kanso_cuda_model_set_weight(m, layer, which, src, nbytes, (int32_t)t->type,
                                       (int64_t)rows, (int64_t)cols);
  };
  std::vector<float> normbuf;
  auto put_norm = [&](const std::string& name, uint32_t layer, int32_t which) -> int32_t {
    const GgufTensor* t = nullptr;
    int32_t s2 = find(name, &t);
    if (s2) return s2;
    if (t->dims.size() != 1 || t->dims[0] != c.hidden_size || (t->type != 0 && t->type != 1))
      return fail(ctx, KANSO_ERR_UNSUPPORTED, "GGUF tensor '%s' is not an F32/F16 vector of %u",
                  name.c_str(), c.hidden_size);
    const size_t nbytes = (size_t)c.hidden_size * (t->type == 0 ? 4 : 2);
    if (data0 + t->offset > file.size() || nbytes > file.size() - data0 - t->offset)
      return fail(ctx, KANSO_ERR_CONFIG, "GGUF tensor '%s' runs past the end of the file",
                  name.c_str());
    normbuf.resize(c.hidden_size);
    const uint8_t* src = file.data() + data0 + t->offset;
    if (t->type == 0) {
      std::memcpy(normbuf.data(), src, nbytes);
    } else {
      for (uint32_t i = 0; i < c.hidden_size; ++i) {
        uint16_t h;
        std::memcpy(&h, src + 2 * i, 2);
        normbuf[i] = f16_to_f32_host(h);
      }
    }
    return kanso_cuda_model_set_norm(m, layer, which, normbuf.data(), c.hidden_size);
  };
  st = put_weight("token_embd.weight", 0, KANSO_W_TOKEN_EMBD, 0);
  if (!st) st = put_norm("output_norm.weight", 0, KANSO_NORM_FINAL);
  if (!st && tensors.count("output.weight")) st = put_weight("output.weight", 0, KANSO_W_OUTPUT, 0);
  for (uint32_t l = 0; l < c.num_hidden_layers && !st; ++l) {
    const std::string b = "blk." + std::to_string(l) + ".";
    st = put_norm(b + "attn_norm.weight", l, KANSO_NORM_ATTN);
    if (!st) st = put_weight(b + "attn_q.weight", l, KANSO_W_ATTN_Q, c.num_attention_heads);
    if (!st) st = put_weight(b + "attn_k.weight", l, KANSO_W_ATTN_K, c.num_key_value_heads);
    if (!st) st = put_weight(b + "attn_v.weight", l, KANSO_W_ATTN_V, 0);
    if (!st) st = put_weight(b + "attn_output.weight", l, KANSO_W_ATTN_OUTPUT, 0);
    if (!st) st = put_norm(b + "ffn_norm.weight", l, KANSO_NORM_FFN);
    if (!st) st = put_weight(b + "ffn_gate.weight", l, KANSO_W_FFN_GATE, 0);
    if (!st) st = put_weight(b + "ffn_up.weight", l, KANSO_W_FFN_UP, 0);
    if (!st) st = put_weight(b + "ffn_down.weight", l, KANSO_W_FFN_DOWN, 0);
  }
  if (st) {
    const std::string keep = ctx->last_error;
    kanso_cuda_model_destroy(m);
    ctx->last_error = keep;
    return st;
  }
  if (cfg_out) *cfg_out = c;
  *out = m;
  return KANSO_OK;
}
