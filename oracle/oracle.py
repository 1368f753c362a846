"""ctypes binding of the CPU oracle (libkanso_oracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU
baseline leg of bench.py, as the checker. The product package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libkanso_oracle.so")

Q8_BYTES, QK8_0 = 34, 32
Q4K_BYTES, QK_K = 144, 256
ACT_F32, ACT_Q8 = 0, 1


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file (g++ only)."""
    src = os.path.join(_HERE, "kanso_oracle.cpp")
    stale = (not os.path.exists(_LIB_PATH)) or (
        os.path.exists(src) and os.path.getmtime(src) > os.path.getmtime(_LIB_PATH))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "libkanso_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


class PaParams(C.Structure):
    _fields_ = [("num_seqs", C.c_uint32), ("num_heads", C.c_uint32),
                ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("block_size", C.c_uint32), ("max_num_blocks_per_seq", C.c_uint32),
                ("scale", C.c_float)]


class ModelConfig(C.Structure):
    _fields_ = [("hidden_size", C.c_uint32), ("num_attention_heads", C.c_uint32),
                ("num_key_value_heads", C.c_uint32), ("num_hidden_layers", C.c_uint32),
                ("intermediate_size", C.c_uint32), ("vocab_size", C.c_uint32),
                ("block_size", C.c_uint32), ("max_seq_len", C.c_uint32),
                ("rms_norm_eps", C.c_float), ("rope_theta", C.c_float)]


def _p(a, t=C.c_void_p):
    if a is None:
        return None
    return a.ctypes.data_as(t)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.kanso_ref_f32_to_f16.restype = C.c_uint16
        L.kanso_ref_f32_to_f16.argtypes = [C.c_float]
        L.kanso_ref_f16_to_f32.restype = C.c_float
        L.kanso_ref_f16_to_f32.argtypes = [C.c_uint16]
        L.kanso_ref_dot_q8_0_ref.restype = C.c_float
        L.kanso_ref_dot_q8_0_ref.argtypes = [C.c_float, C.c_void_p, C.c_void_p]
        L.kanso_ref_dot_q8_0_q8_0_ref.restype = C.c_float
        L.kanso_ref_dot_q8_0_q8_0_ref.argtypes = [C.c_float, C.c_void_p, C.c_float, C.c_void_p,
                                                  C.c_void_p]
        L.kanso_ref_dot_q4_k_ref.restype = C.c_float
        L.kanso_ref_dot_q4_k_ref.argtypes = [C.c_float, C.c_float, C.c_void_p, C.c_void_p,
                                             C.c_void_p]
        L.kanso_ref_dequantize_q4_k_ref.argtypes = [C.c_float, C.c_float, C.c_void_p, C.c_void_p,
                                                    C.c_void_p]
        L.kanso_ref_kv_quantize_head.restype = C.c_float
        L.kanso_ref_kv_create.restype = C.c_void_p
        L.kanso_ref_kv_create.argtypes = [C.c_uint32] * 5
        L.kanso_ref_kv_create_typed.restype = C.c_void_p
        L.kanso_ref_kv_create_typed.argtypes = [C.c_uint32] * 5 + [C.c_int32]
        L.kanso_ref_kv_quantize_head_fp8.restype = C.c_float
        L.kanso_ref_fp8_e4m3_to_f32.restype = C.c_float
        L.kanso_ref_fp8_e4m3_to_f32.argtypes = [C.c_uint8]
        L.kanso_ref_fp8_e4m3_from_f32.restype = C.c_uint8
        L.kanso_ref_fp8_e4m3_from_f32.argtypes = [C.c_float]
        L.kanso_ref_kv_destroy.argtypes = [C.c_void_p]
        L.kanso_ref_model_create.restype = C.c_void_p
        L.kanso_ref_model_destroy.argtypes = [C.c_void_p]
        L.kanso_ref_pa_num_partitions.restype = C.c_uint32
        L.kanso_ref_greedy_token.restype = C.c_uint32
        L.kanso_ref_padded_decode_tables.restype = C.c_uint32
        _lib = L
    return _lib


# ----------------------------- Q8_0 -----------------------------
def f32_to_f16_bits(x: float) -> int:
    return lib().kanso_ref_f32_to_f16(C.c_float(x))


def f16_bits_to_f32(h: int) -> float:
    return lib().kanso_ref_f16_to_f32(C.c_uint16(h))


def quantize_row_q8_0(x):
    x = _f32(x)
    cols = x.size
    d = np.empty(cols // QK8_0, np.float32)
    qs = np.empty(cols, np.int8)
    lib().kanso_ref_quantize_row_q8_0(_p(x), C.c_int64(cols), _p(d), _p(qs))
    return d, qs


def quantize_weights_q8_0(w):
    w = _f32(w)
    rows, cols = w.shape
    out = np.empty(rows * (cols // QK8_0) * Q8_BYTES, np.uint8)
    lib().kanso_ref_quantize_weights_q8_0(_p(w), C.c_int64(rows), C.c_int64(cols), _p(out))
    return out


def dequantize_q8_0(blocks):
    blocks = _u8(blocks)
    nb = blocks.size // Q8_BYTES
    out = np.empty(nb * QK8_0, np.float32)
    lib().kanso_ref_dequantize_q8_0(_p(blocks), C.c_int64(nb), _p(out))
    return out


def dot_q8_0_ref(d, qs, x):
    qs = np.ascontiguousarray(qs, np.int8)
    x = _f32(x)
    return lib().kanso_ref_dot_q8_0_ref(C.c_float(d), _p(qs), _p(x))


def dot_q8_0_q8_0_ref(wd, wqs, xd, xqs):
    wqs = np.ascontiguousarray(wqs, np.int8)
    xqs = np.ascontiguousarray(xqs, np.int8)
    isum = C.c_int32(0)
    r = lib().kanso_ref_dot_q8_0_q8_0_ref(C.c_float(wd), _p(wqs), C.c_float(xd), _p(xqs),
                                          C.byref(isum))
    return r, isum.value


def gemv_q8_0(w, x, rows, cols):
    w, x = _u8(w), _f32(x)
    out = np.empty(rows, np.float32)
    lib().kanso_ref_gemv_q8_0(_p(w), _p(x), _p(out), C.c_int64(rows), C.c_int64(cols))
    return out


def gemv_q8_0_ref(d, qs, x, rows, cols):
    d, x = _f32(d), _f32(x)
    qs = np.ascontiguousarray(qs, np.int8)
    out = np.empty(rows, np.float32)
    lib().kanso_ref_gemv_q8_0_ref(_p(d), _p(qs), _p(x), _p(out), C.c_int64(rows), C.c_int64(cols))
    return out


def gemv_q8_0_q8(w, x, rows, cols):
    w, x = _u8(w), _f32(x)
    out = np.empty(rows, np.float32)
    lib().kanso_ref_gemv_q8_0_q8(_p(w), _p(x), _p(out), C.c_int64(rows), C.c_int64(cols))
    return out


def block_isums_q8_0(w, x_qs, rows, cols):
    w = _u8(w)
    x_qs = np.ascontiguousarray(x_qs, np.int8)
    out = np.empty(rows * (cols // QK8_0), np.int32)
    lib().kanso_ref_block_isums_q8_0(_p(w), _p(x_qs), _p(out), C.c_int64(rows), C.c_int64(cols))
    return out.reshape(rows, cols // QK8_0)


def gemm_q8_0(w, x, M, N, K, act_mode=ACT_F32):
    w, x = _u8(w), _f32(x)
    y = np.empty((M, N), np.float32)
    lib().kanso_ref_gemm_q8_0(_p(w), _p(x), _p(y), C.c_int64(M), C.c_int64(N), C.c_int64(K),
                              C.c_int32(act_mode))
    return y


# ----------------------------- Q4_K -----------------------------
def get_scale_min_k4(j, scales12):
    s = _u8(scales12)
    sc, m = C.c_uint8(0), C.c_uint8(0)
    lib().kanso_ref_get_scale_min_k4(C.c_int32(j), _p(s), C.byref(sc), C.byref(m))
    return sc.value, m.value


def unpack_scales_q4_k(blocks):
    blocks = _u8(blocks)
    nb = blocks.size // Q4K_BYTES
    out = np.empty(nb * 16, np.uint8)
    lib().kanso_ref_unpack_scales_q4_k(_p(blocks), C.c_int64(nb), _p(out))
    return out.reshape(nb, 16)


def dequantize_q4_k(blocks):
    blocks = _u8(blocks)
    nb = blocks.size // Q4K_BYTES
    out = np.empty(nb * QK_K, np.float32)
    lib().kanso_ref_dequantize_q4_k(_p(blocks), C.c_int64(nb), _p(out))
    return out


def dequantize_q4_k_ref(d, dmin, scales12, qs128):
    s, q = _u8(scales12), _u8(qs128)
    out = np.empty(QK_K, np.float32)
    lib().kanso_ref_dequantize_q4_k_ref(C.c_float(d), C.c_float(dmin), _p(s), _p(q), _p(out))
    return out


def dot_q4_k_ref(d, dmin, scales12, qs128, x):
    s, q, x = _u8(scales12), _u8(qs128), _f32(x)
    return lib().kanso_ref_dot_q4_k_ref(C.c_float(d), C.c_float(dmin), _p(s), _p(q), _p(x))


def gemv_q4_k(w, x, rows, cols):
    w, x = _u8(w), _f32(x)
    out = np.empty(rows, np.float32)
    lib().kanso_ref_gemv_q4_k(_p(w), _p(x), _p(out), C.c_int64(rows), C.c_int64(cols))
    return out


def gemm_q4_k(w, x, M, N, K):
    w, x = _u8(w), _f32(x)
    y = np.empty((M, N), np.float32)
    lib().kanso_ref_gemm_q4_k(_p(w), _p(x), _p(y), C.c_int64(M), C.c_int64(N), C.c_int64(K))
    return y


def quantize_weights_q4_k(w):
    w = _f32(w)
    rows, cols = w.shape
    out = np.empty(rows * (cols // QK_K) * Q4K_BYTES, np.uint8)
    lib().kanso_ref_quantize_weights_q4_k(_p(w), C.c_int64(rows), C.c_int64(cols), _p(out))
    return out


# ----------------------------- KV pool -----------------------------
def kv_quantize_head(x):
    x = _f32(x)
    q = np.empty(x.size, np.int8)
    s = lib().kanso_ref_kv_quantize_head(_p(x), C.c_int32(x.size), _p(q))
    return np.float32(s), q


def kv_quantize_head_fp8(x):
    x = _f32(x)
    q = np.empty(x.size, np.int8)
    s = lib().kanso_ref_kv_quantize_head_fp8(_p(x), C.c_int32(x.size), _p(q))
    return np.float32(s), q


def fp8_e4m3_to_f32(bits):
    return np.float32(lib().kanso_ref_fp8_e4m3_to_f32(C.c_uint8(int(bits) & 0xFF)))


def fp8_e4m3_from_f32(x):
    return int(lib().kanso_ref_fp8_e4m3_from_f32(C.c_float(float(x))))


class KvPool:
    def __init__(self, layers, num_blocks, block_size, kv_heads, head_dim, fp8=False):
        self.geom = (layers, num_blocks, block_size, kv_heads, head_dim)
        self.fp8 = bool(fp8)
        self.h = C.c_void_p(lib().kanso_ref_kv_create_typed(layers, num_blocks, block_size,
                                                            kv_heads, head_dim, int(self.fp8)))

    def __del__(self):
        if getattr(self, "h", None):
            lib().kanso_ref_kv_destroy(self.h)
            self.h = None

    def write_token(self, layer, block, offset, k, v):
        k, v = _f32(k), _f32(v)
        return lib().kanso_ref_kv_write_token(self.h, C.c_uint32(layer), C.c_uint32(block),
                                              C.c_uint32(offset), _p(k), _p(v))

    def write_slots(self, layer, slots, k, v):
        slots, k, v = _u32(slots), _f32(k), _f32(v)
        return lib().kanso_ref_kv_write_slots(self.h, C.c_uint32(layer), _p(slots), _p(k), _p(v),
                                              C.c_int64(slots.size))

    def reset_block(self, block):
        lib().kanso_ref_kv_reset_block(self.h, C.c_uint32(block))

    def read_token(self, layer, block, offset):
        _, _, _, H, hd = self.geom
        kq, vq = np.empty(H * hd, np.int8), np.empty(H * hd, np.int8)
        ks, vs = np.empty(H, np.float32), np.empty(H, np.float32)
        kd, vd = np.empty(H * hd, np.float32), np.empty(H * hd, np.float32)
        st = lib().kanso_ref_kv_read_token(self.h, C.c_uint32(layer), C.c_uint32(block),
                                           C.c_uint32(offset), _p(kq), _p(vq), _p(ks), _p(vs),
                                           _p(kd), _p(vd))
        return st, dict(k_q=kq, v_q=vq, k_scale=ks, v_scale=vs, k_deq=kd, v_deq=vd)

    def gather(self, layer, blocks, num_tokens):
        _, _, _, H, hd = self.geom
        blocks = _u32(blocks)
        k = np.empty((num_tokens, H, hd), np.float32)
        v = np.empty((num_tokens, H, hd), np.float32)
        st = lib().kanso_ref_kv_gather(self.h, C.c_uint32(layer), _p(blocks),
                                       C.c_uint32(blocks.size), C.c_uint32(num_tokens), _p(k),
                                       _p(v))
        return st, k, v


# ----------------------------- attention -----------------------------
def validate_pa_params(p: PaParams) -> int:
    return lib().kanso_ref_validate_pa_params(C.byref(p))


def pa_num_partitions(p: PaParams) -> int:
    return lib().kanso_ref_pa_num_partitions(C.byref(p))


def paged_attention_f32(q, k_cache, v_cache, block_tables, context_lens, p: PaParams):
    q, k_cache, v_cache = _f32(q), _f32(k_cache), _f32(v_cache)
    bt, cl = _u32(block_tables), _u32(context_lens)
    out = np.empty(p.num_seqs * p.num_heads * p.head_dim, np.float32)
    lib().kanso_ref_paged_attention_f32(_p(q), _p(k_cache), _p(v_cache), _p(bt), _p(cl),
                                        C.byref(p), _p(out))
    return out


def paged_attention_int8(pool: KvPool, layer, q, block_tables, context_lens, p: PaParams):
    q = _f32(q)
    bt, cl = _u32(block_tables), _u32(context_lens)
    out = np.empty((p.num_seqs, p.num_heads * p.head_dim), np.float32)
    st = lib().kanso_ref_paged_attention_int8(pool.h, C.c_uint32(layer), _p(q), _p(bt), _p(cl),
                                              C.byref(p), _p(out))
    return st, out


def prefill_attention_int8(pool: KvPool, layer, q, blocks, start_pos, num_heads, scale):
    """q f32 [chunk_len, num_heads*head_dim]; returns (status, out of the same shape)."""
    q = _f32(q)
    blocks = _u32(blocks)
    chunk = q.shape[0]
    out = np.empty_like(q)
    st = lib().kanso_ref_prefill_attention_int8(pool.h, C.c_uint32(layer), _p(q), _p(blocks),
                                                C.c_uint32(blocks.size), C.c_uint32(start_pos),
                                                C.c_uint32(chunk), C.c_uint32(num_heads),
                                                C.c_float(scale), _p(out))
    return st, out


# ----------------------------- glue -----------------------------
def rmsnorm(x, w, eps):
    x, w = _f32(x), _f32(w)
    rows, hidden = x.shape
    out = np.empty_like(x)
    lib().kanso_ref_rmsnorm(_p(x), _p(w), _p(out), C.c_int64(rows), C.c_int64(hidden),
                            C.c_float(eps))
    return out


def rope_table(theta, length, head_dim):
    c = np.empty((length, head_dim // 2), np.float32)
    s = np.empty((length, head_dim // 2), np.float32)
    lib().kanso_ref_rope_table(C.c_float(theta), C.c_int64(length), C.c_int64(head_dim), _p(c),
                               _p(s))
    return c, s


def rope(x, positions, theta):
    x = _f32(x).copy()
    T, heads, hd = x.shape
    pos = _u32(positions)
    lib().kanso_ref_rope(_p(x), _p(pos), C.c_int64(T), C.c_int64(heads), C.c_int64(hd),
                         C.c_float(theta))
    return x


def silu_mul(g, u):
    g, u = _f32(g), _f32(u)
    out = np.empty_like(g)
    lib().kanso_ref_silu_mul(_p(g), _p(u), _p(out), C.c_int64(g.size))
    return out


def greedy_token(logits):
    logits = _f32(logits)
    return lib().kanso_ref_greedy_token(_p(logits), C.c_int64(logits.size))


def padded_decode_tables(block_size, tables, context_lens):
    """tables: list of per-sequence lists. Returns (status, max_blocks, padded u32 array)."""
    lens = _u32([len(t) for t in tables])
    flat = _u32([b for t in tables for b in t] or [0])
    cl = _u32(context_lens)
    n = len(tables)
    cap = n * max(1, max((int(c) + block_size - 1) // block_size for c in cl))
    out = np.zeros(cap, np.uint32)
    st = C.c_int32(0)
    mb = lib().kanso_ref_padded_decode_tables(C.c_uint32(block_size), _p(flat), _p(lens), _p(cl),
                                              C.c_uint32(n), _p(out), C.c_uint32(cap),
                                              C.byref(st))
    return st.value, mb, out[: n * mb] if mb else out[:0]


# ----------------------------- decode step -----------------------------
class Model:
    """Holds references to the numpy block arrays it is given (the C side borrows them)."""

    def __init__(self, cfg: ModelConfig):
        self.cfg = cfg
        self.h = C.c_void_p(lib().kanso_ref_model_create(C.byref(cfg)))
        self._keep = []

    def __del__(self):
        if getattr(self, "h", None):
            lib().kanso_ref_model_destroy(self.h)
            self.h = None

    def set_weight(self, layer, which, blocks, rows, cols):
        blocks = _u8(blocks)
        self._keep.append(blocks)
        return lib().kanso_ref_model_set_weight(self.h, C.c_uint32(layer), C.c_int32(which),
                                                _p(blocks), C.c_int64(rows), C.c_int64(cols))

    def set_norm(self, layer, which, w):
        w = _f32(w)
        return lib().kanso_ref_model_set_norm(self.h, C.c_uint32(layer), C.c_int32(which), _p(w),
                                              C.c_int64(w.size))

    def decode_step(self, pool: KvPool, tokens, positions, slots, block_tables, context_lens,
                    max_blocks, act_mode=ACT_F32, num_layers_to_run=0):
        tokens, positions, slots = _u32(tokens), _u32(positions), _u32(slots)
        bt, cl = _u32(block_tables), _u32(context_lens)
        B = tokens.size
        logits = np.empty((B, self.cfg.vocab_size), np.float32)
        st = lib().kanso_ref_decode_step(self.h, pool.h, _p(tokens), _p(positions), _p(slots),
                                         _p(bt), _p(cl), C.c_uint32(B), C.c_uint32(max_blocks),
                                         C.c_int32(act_mode), C.c_uint32(num_layers_to_run),
                                         _p(logits))
        return st, logits
