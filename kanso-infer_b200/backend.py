"""ctypes binding of libkanso_cuda.so and a thin tensor-facing wrapper.

This is plumbing for tests and measurement: it passes device pointers of torch
tensors to the C ABI declared in include/kanso_cuda.h. It contains no arithmetic
and no fallback: if the shared library is missing or a call fails, it raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libkanso_cuda.so")

OK, ERR_CONFIG, ERR_SHAPE, ERR_UNSUPPORTED, ERR_DEVICE, ERR_TIMEOUT = range(6)
DTYPE_Q8_0, DTYPE_Q4_K = 8, 12
ACT_F32, ACT_Q8 = 0, 1
KV_F32, KV_INT8, KV_FP8 = 0, 1, 2
OPT_OVERLAP_WEIGHT_PREFETCH = 1
SHARD_ROWS, SHARD_K, SHARD_LOCAL_ONLY, SHARD_HANDLE_BYTES = 0, 1, 1, 64
Q8_BYTES, Q4K_BYTES = 34, 144
(W_ATTN_Q, W_ATTN_K, W_ATTN_V, W_ATTN_OUTPUT, W_FFN_GATE, W_FFN_UP, W_FFN_DOWN, W_TOKEN_EMBD,
 W_OUTPUT) = range(9)
NORM_ATTN, NORM_FFN, NORM_FINAL = range(3)

_STATUS_NAMES = {1: "Config", 2: "Model", 3: "Cuda(unsupported)", 4: "Cuda(device)",
                 5: "Cuda(timeout)"}


class KansoError(RuntimeError):
    """Mirror of the reference's EngineError (src/error.rs:3-11) for the cuda backend."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{_STATUS_NAMES.get(code, code)} error: {message}")
        self.code = code
        self.message = message


class PagedAttentionParams(C.Structure):
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


_P, _I32, _I64, _U32, _U64, _SZ, _F = (C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_uint64,
                                       C.c_size_t, C.c_float)

# name -> (restype, argtypes); one entry per declaration in include/kanso_cuda.h
PROTOTYPES = {
    "kanso_cuda_ctx_create": (_I32, [_I32, _P, C.POINTER(_P)]),
    "kanso_cuda_ctx_destroy": (_I32, [_P]),
    "kanso_cuda_sync": (_I32, [_P]),
    "kanso_cuda_last_error": (C.c_char_p, [_P]),
    "kanso_cuda_ctx_set_option": (_I32, [_P, _I32, _I32]),
    "kanso_cuda_launch_count": (_U64, [_P]),
    "kanso_cuda_sm_count": (_I32, [_P]),
    "kanso_cuda_probe_read": (_I32, [_P, _P, _SZ]),
    "kanso_cuda_gemv_q8_0": (_I32, [_P, _P, _P, _P, _I64, _I64]),
    "kanso_cuda_gemv_q4_k": (_I32, [_P, _P, _P, _P, _I64, _I64]),
    "kanso_cuda_gemm_q8_0": (_I32, [_P, _P, _P, _P, _I64, _I64, _I64, _I32]),
    "kanso_cuda_gemm_q4_k": (_I32, [_P, _P, _P, _P, _I64, _I64, _I64, _I32]),
    "kanso_cuda_quantize_row_q8_0": (_I32, [_P, _P, _P, _P, _I64]),
    "kanso_cuda_dequantize_q8_0": (_I32, [_P, _P, _P, _I64]),
    "kanso_cuda_dequantize_q4_k": (_I32, [_P, _P, _P, _I64]),
    "kanso_cuda_unpack_scales_q4_k": (_I32, [_P, _P, _P, _I64]),
    "kanso_cuda_block_isums_q8_0": (_I32, [_P, _P, _P, _P, _I64, _I64]),
    "kanso_cuda_weight_upload": (_I32, [_P, _P, _SZ, _I32, _I64, _I64, C.POINTER(_P)]),
    "kanso_cuda_weight_free": (_I32, [_P]),
    "kanso_cuda_weight_ptr": (_P, [_P]),
    "kanso_cuda_linear_host": (_I32, [_P, _P, _P, _P, _I64, _I32]),
    "kanso_cuda_linear": (_I32, [_P, _P, _P, _P, _I64, _I32]),
    "kanso_cuda_embed": (_I32, [_P, _P, _P, _P, _I64]),
    "kanso_cuda_shard_range": (_I32, [_I64, _I32, _I32, _I64, C.POINTER(_I64), C.POINTER(_I64)]),
    "kanso_cuda_shard_k_repack": (_I32, [_P, _I32, _I64, _I64, _I64, _I64, _P, _SZ]),
    "kanso_cuda_linear_scatter_out": (_I32, [_P, _P, _P, _I64, _P, _I32, _I64, _I64, _I32]),
    "kanso_cuda_sum_shards": (_I32, [_P, _P, _I64, _I64, _I32, _P]),
    "kanso_cuda_peer_exchange": (_I32, [_P, _P, _P, _I32, _I32]),
    "kanso_cuda_shard_group_create": (_I32, [_P, _I32, _I32, _SZ, C.POINTER(_P), _P]),
    "kanso_cuda_shard_group_connect": (_I32, [_P, _P]),
    "kanso_cuda_shard_group_destroy": (_I32, [_P]),
    "kanso_cuda_sharded_linear_create": (_I32, [_P, _P, _SZ, _I32, _I64, _I64, _I32, _I64,
                                                C.POINTER(_P)]),
    "kanso_cuda_sharded_linear_destroy": (_I32, [_P]),
    "kanso_cuda_sharded_linear_range": (_I32, [_P, C.POINTER(_I64), C.POINTER(_I64)]),
    "kanso_cuda_sharded_linear_forward": (_I32, [_P, _P, _I64, _I32, _I32, C.POINTER(_P)]),
    "kanso_cuda_kv_create": (_I32, [_P, _U32, _U32, _U32, _U32, _U32, _I32, C.POINTER(_P)]),
    "kanso_cuda_kv_destroy": (_I32, [_P]),
    "kanso_cuda_kv_write_slots": (_I32, [_P, _P, _U32, _P, _P, _P, _I64, _P]),
    "kanso_cuda_kv_reset_block": (_I32, [_P, _P, _U32]),
    "kanso_cuda_kv_read_token": (_I32, [_P, _P, _U32, _U32, _U32, _P, _P, _P, _P, _P, _P]),
    "kanso_cuda_kv_bytes_per_token": (_U64, [_P]),
    "kanso_cuda_paged_attention": (_I32, [_P, _P, _U32, _P, _P, _P, _P,
                                          C.POINTER(PagedAttentionParams), _P]),
    "kanso_cuda_paged_attention_prefill": (_I32, [_P, _P, _U32, _P, _P, _P, _P, _P,
                                                  C.POINTER(PagedAttentionParams)]),
    "kanso_cuda_paged_attention_noalloc": (_I32, [_P, _P, _U32, _P, _P, _P, _P,
                                                  C.POINTER(PagedAttentionParams), _P]),
    "kanso_cuda_validate_paged_attention_params": (_I32, [C.POINTER(PagedAttentionParams),
                                                          C.c_char_p, _SZ]),
    "kanso_cuda_rmsnorm": (_I32, [_P, _P, _P, _P, _I64, _I64, _F]),
    "kanso_cuda_rope": (_I32, [_P, _P, _P, _I64, _I64, _I64, _F]),
    "kanso_cuda_silu_mul": (_I32, [_P, _P, _P, _P, _I64]),
    "kanso_cuda_residual_add": (_I32, [_P, _P, _P, _I64]),
    "kanso_cuda_model_create": (_I32, [_P, C.POINTER(ModelConfig), C.POINTER(_P)]),
    "kanso_cuda_model_destroy": (_I32, [_P]),
    "kanso_cuda_model_load_gguf": (_I32, [_P, C.c_char_p, _U32, _U32, C.POINTER(_P),
                                          C.POINTER(ModelConfig)]),
    "kanso_cuda_model_set_weight": (_I32, [_P, _U32, _I32, _P, _SZ, _I32, _I64, _I64]),
    "kanso_cuda_model_set_norm": (_I32, [_P, _U32, _I32, _P, _I64]),
    "kanso_cuda_decode_step": (_I32, [_P, _P, _P, _P, _P, _P, _P, _P, _U32, _U32, _I32, _P]),
    "kanso_cuda_decode_step_device": (_I32, [_P, _P, _P, _P, _P, _P, _P, _P, _U32, _U32, _U32,
                                             _I32, _P]),
    "kanso_cuda_greedy_token": (_I32, [_P, _P, _P, _I64, _I64]),
}

_lib = None


def load():
    """Loads the shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise KansoError(ERR_CONFIG, f"backend 'cuda' is not built: {LIB_PATH} is missing "
                                         "(run kanso-infer_b200/build.py); there is no CPU fallback")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)  # AttributeError here = the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def _ptr(t):
    """Device (or host) address of a torch tensor / numpy array / int / None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data


class Context:
    """One context per GPU; single caller, asynchronous on its stream."""

    def __init__(self, device: int = 0, stream=None):
        self.lib = load()
        h = _P()
        sp = None
        if stream is not None:
            sp = stream if isinstance(stream, int) else stream.cuda_stream
        st = self.lib.kanso_cuda_ctx_create(device, sp, C.byref(h))
        if st != OK:
            raise KansoError(st, self.lib.kanso_cuda_last_error(None).decode())
        self.h = h
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            self.lib.kanso_cuda_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, st: int):
        if st != OK:
            raise KansoError(st, self.lib.kanso_cuda_last_error(self.h).decode())

    def call(self, name: str, *args):
        self.check(getattr(self.lib, name)(self.h, *args))

    def sync(self):
        self.check(self.lib.kanso_cuda_sync(self.h))

    def set_option(self, option: int, value: int):
        self.call("kanso_cuda_ctx_set_option", option, value)

    @property
    def launches(self) -> int:
        return self.lib.kanso_cuda_launch_count(self.h)

    @property
    def sm_count(self) -> int:
        return self.lib.kanso_cuda_sm_count(self.h)

    # ---- src/quant entry points (device tensors) ----
    def gemv_q8_0(self, w, x, y, rows, cols):
        self.call("kanso_cuda_gemv_q8_0", _ptr(w), _ptr(x), _ptr(y), rows, cols)

    def gemv_q4_k(self, w, x, y, rows, cols):
        self.call("kanso_cuda_gemv_q4_k", _ptr(w), _ptr(x), _ptr(y), rows, cols)

    def gemm_q8_0(self, w, x, y, M, N, K, act_mode=ACT_F32):
        self.call("kanso_cuda_gemm_q8_0", _ptr(w), _ptr(x), _ptr(y), M, N, K, act_mode)

    def gemm_q4_k(self, w, x, y, M, N, K, act_mode=ACT_F32):
        self.call("kanso_cuda_gemm_q4_k", _ptr(w), _ptr(x), _ptr(y), M, N, K, act_mode)

    def quantize_row_q8_0(self, x, d_out, qs_out, cols):
        self.call("kanso_cuda_quantize_row_q8_0", _ptr(x), _ptr(d_out), _ptr(qs_out), cols)

    def dequantize_q8_0(self, w, out, nblocks):
        self.call("kanso_cuda_dequantize_q8_0", _ptr(w), _ptr(out), nblocks)

    def dequantize_q4_k(self, w, out, nblocks):
        self.call("kanso_cuda_dequantize_q4_k", _ptr(w), _ptr(out), nblocks)

    def unpack_scales_q4_k(self, w, out, nblocks):
        self.call("kanso_cuda_unpack_scales_q4_k", _ptr(w), _ptr(out), nblocks)

    def block_isums_q8_0(self, w, x_qs, isums, rows, cols):
        self.call("kanso_cuda_block_isums_q8_0", _ptr(w), _ptr(x_qs), _ptr(isums), rows, cols)

    # ---- glue ----
    def rmsnorm(self, x, weight, out, rows, hidden, eps):
        self.call("kanso_cuda_rmsnorm", _ptr(x), _ptr(weight), _ptr(out), rows, hidden, eps)

    def rope(self, x, positions, T, heads, head_dim, theta):
        self.call("kanso_cuda_rope", _ptr(x), _ptr(positions), T, heads, head_dim, theta)

    def silu_mul(self, gate, up, out, n):
        self.call("kanso_cuda_silu_mul", _ptr(gate), _ptr(up), _ptr(out), n)

    def residual_add(self, hidden, proj, n):
        self.call("kanso_cuda_residual_add", _ptr(hidden), _ptr(proj), n)

    def greedy_token(self, logits, out, B, vocab):
        self.call("kanso_cuda_greedy_token", _ptr(logits), _ptr(out), B, vocab)


class Weight:
    """LinearWeight resident on the device (src/weights.rs:22,140-158)."""

    def __init__(self, ctx: Context, host_bytes, dtype: int, rows: int, cols: int):
        self.ctx = ctx
        h = _P()
        nbytes = host_bytes.nbytes if hasattr(host_bytes, "nbytes") else len(host_bytes)
        ctx.call("kanso_cuda_weight_upload", _ptr(host_bytes), nbytes, dtype, rows, cols,
                 C.byref(h))
        self.h, self.dtype, self.rows, self.cols, self.nbytes = h, dtype, rows, cols, nbytes

    @property
    def ptr(self) -> int:
        return self.ctx.lib.kanso_cuda_weight_ptr(self.h)

    def free(self):
        if getattr(self, "h", None):
            self.ctx.lib.kanso_cuda_weight_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def forward(self, x, y, M, act_mode=ACT_F32):
        """x, y device tensors; asynchronous."""
        self.ctx.call("kanso_cuda_linear", self.h, _ptr(x), _ptr(y), M, act_mode)

    def forward_host(self, x_host, y_host, M, act_mode=ACT_F32):
        """x, y host arrays; synchronous (copies in, runs, copies out)."""
        self.ctx.call("kanso_cuda_linear_host", self.h, _ptr(x_host), _ptr(y_host), M, act_mode)

    def embed(self, ids, out, T):
        self.ctx.call("kanso_cuda_embed", self.h, _ptr(ids), _ptr(out), T)


class KvPool:
    """KvStorageKind for the cuda backend (src/kv_cache/kind.rs:176)."""

    def __init__(self, ctx: Context, layers, num_blocks, block_size, kv_heads, head_dim,
                 kv_type=KV_INT8):
        self.ctx = ctx
        self.geom = (layers, num_blocks, block_size, kv_heads, head_dim)
        h = _P()
        ctx.call("kanso_cuda_kv_create", layers, num_blocks, block_size, kv_heads, head_dim,
                 kv_type, C.byref(h))
        self.h = h

    def destroy(self):
        if getattr(self, "h", None):
            self.ctx.lib.kanso_cuda_kv_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    def write_slots(self, layer, slots, k, v, T, host_slots=None):
        self.ctx.call("kanso_cuda_kv_write_slots", self.h, layer, _ptr(slots), _ptr(k), _ptr(v),
                      T, _ptr(host_slots))

    def reset_block(self, block):
        self.ctx.call("kanso_cuda_kv_reset_block", self.h, block)

    def read_token(self, layer, block, offset):
        import numpy as np
        _, _, _, H, hd = self.geom
        out = dict(k_q=np.empty(H * hd, np.int8), v_q=np.empty(H * hd, np.int8),
                   k_scale=np.empty(H, np.float32), v_scale=np.empty(H, np.float32),
                   k_deq=np.empty(H * hd, np.float32), v_deq=np.empty(H * hd, np.float32))
        self.ctx.call("kanso_cuda_kv_read_token", self.h, layer, block, offset, _ptr(out["k_q"]),
                      _ptr(out["v_q"]), _ptr(out["k_scale"]), _ptr(out["v_scale"]),
                      _ptr(out["k_deq"]), _ptr(out["v_deq"]))
        return out

    @property
    def bytes_per_token(self) -> int:
        return self.ctx.lib.kanso_cuda_kv_bytes_per_token(self.h)

    def paged_attention(self, layer, q, block_tables, context_lens, out,
                        params: PagedAttentionParams, host_context_lens=None):
        self.ctx.call("kanso_cuda_paged_attention", self.h, layer, _ptr(q), _ptr(block_tables),
                      _ptr(context_lens), _ptr(out), C.byref(params), _ptr(host_context_lens))


    def paged_attention_prefill(self, layer, q, block_tables, host_context_lens,
                                host_query_lens, out, params: PagedAttentionParams):
        """Chunked-prefill attention; the two length arrays are host uint32 arrays."""
        self.ctx.call("kanso_cuda_paged_attention_prefill", self.h, layer, _ptr(q),
                      _ptr(block_tables), _ptr(host_context_lens), _ptr(host_query_lens),
                      _ptr(out), C.byref(params))

    def paged_attention_noalloc(self, layer, q, block_tables, context_lens, out,
                                params: PagedAttentionParams, host_context_lens=None):
        """Same call with the partials in the library's built-in array (no allocation)."""
        self.ctx.call("kanso_cuda_paged_attention_noalloc", self.h, layer, _ptr(q),
                      _ptr(block_tables), _ptr(context_lens), _ptr(out), C.byref(params),
                      _ptr(host_context_lens))


def validate_paged_attention_params(params: PagedAttentionParams):
    buf = C.create_string_buffer(256)
    st = load().kanso_cuda_validate_paged_attention_params(C.byref(params), buf, 256)
    if st != OK:
        raise KansoError(st, buf.value.decode())


class Model:
    """Model::forward_decode_step / forward_batch on the cuda backend (src/model.rs:1101,1360)."""

    def __init__(self, ctx: Context, cfg: ModelConfig):
        self.ctx, self.cfg = ctx, cfg
        h = _P()
        ctx.call("kanso_cuda_model_create", C.byref(cfg), C.byref(h))
        self.h = h

    @classmethod
    def from_gguf(cls, ctx: Context, path: str, block_size: int = 0, max_seq_len: int = 0):
        """ModelWeights::load_from_gguf (src/weights.rs:332-493)."""
        self = cls.__new__(cls)
        self.ctx, self.cfg = ctx, ModelConfig()
        h = _P()
        ctx.call("kanso_cuda_model_load_gguf", path.encode(), block_size, max_seq_len, C.byref(h),
                 C.byref(self.cfg))
        self.h = h
        return self

    def destroy(self):
        if getattr(self, "h", None):
            self.ctx.lib.kanso_cuda_model_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    def set_weight(self, layer, which, host_bytes, dtype, rows, cols):
        self.ctx.check(self.ctx.lib.kanso_cuda_model_set_weight(
            self.h, layer, which, _ptr(host_bytes), host_bytes.nbytes, dtype, rows, cols))

    def set_norm(self, layer, which, w):
        self.ctx.check(self.ctx.lib.kanso_cuda_model_set_norm(self.h, layer, which, _ptr(w),
                                                              w.size))

    def decode_step(self, kv: KvPool, tokens, positions, slots, block_tables, context_lens,
                    max_blocks, logits_out, act_mode=ACT_F32):
        """All arguments are HOST numpy arrays (uint32 / float32); synchronous."""
        self.ctx.call("kanso_cuda_decode_step", self.h, kv.h, _ptr(tokens), _ptr(positions),
                      _ptr(slots), _ptr(block_tables), _ptr(context_lens), len(tokens),
                      max_blocks, act_mode, _ptr(logits_out))

    def decode_step_device(self, kv: KvPool, tokens, positions, slots, block_tables,
                           context_lens, B, max_blocks, max_ctx, logits, act_mode=ACT_F32):
        self.ctx.call("kanso_cuda_decode_step_device", self.h, kv.h, _ptr(tokens),
                      _ptr(positions), _ptr(slots), _ptr(block_tables), _ptr(context_lens), B,
                      max_blocks, max_ctx, act_mode, _ptr(logits))
