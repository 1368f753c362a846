"""GPU: a model loaded from a .gguf file through the C ABI equals the model built tensor by
tensor, and decodes like the oracle engine. The file is written here with the `gguf` Python
package (metadata keys and tensor names of src/weights.rs:332-493) with the Q and K projections
in llama.cpp's interleaved head layout, so the load has to undo it
(interleaved_permutation, src/weights.rs:231-252)."""
import numpy as np
import pytest

from conftest import golden
from test_decode_gpu import build_gpu_model, load_make_golden

pytestmark = pytest.mark.gpu
gguf = pytest.importorskip("gguf")

NAMES = {0: "attn_q", 1: "attn_k", 2: "attn_v", 3: "attn_output", 4: "ffn_gate", 5: "ffn_up",
         6: "ffn_down"}


def interleaved_permutation(heads, hd):
    half = hd // 2
    return np.array([h * hd + (2 * i if i < half else 2 * (i - half) + 1)
                     for h in range(heads) for i in range(hd)])


def write_gguf(path, cfg, shapes, blocks, norms, tied=True, arch="llama"):
    w = gguf.GGUFWriter(str(path), arch)
    w.add_uint32(f"{arch}.block_count", cfg.num_hidden_layers)
    w.add_uint32(f"{arch}.attention.head_count", cfg.num_attention_heads)
    w.add_uint32(f"{arch}.attention.head_count_kv", cfg.num_key_value_heads)
    w.add_uint32(f"{arch}.embedding_length", cfg.hidden_size)
    w.add_uint32(f"{arch}.feed_forward_length", cfg.intermediate_size)
    w.add_float32(f"{arch}.attention.layer_norm_rms_epsilon", cfg.rms_norm_eps)
    w.add_float32(f"{arch}.rope.freq_base", cfg.rope_theta)
    w.add_array("tokenizer.ggml.tokens", ["a", "b", "c"])  # an array-valued key to skip over
    hd = cfg.hidden_size // cfg.num_attention_heads
    q8 = gguf.GGMLQuantizationType.Q8_0

    def add_q8(name, b, rows, cols):
        w.add_tensor(name, np.ascontiguousarray(b).reshape(rows, cols // 32 * 34), raw_dtype=q8)

    add_q8("token_embd.weight", blocks[(0, 7)], cfg.vocab_size, cfg.hidden_size)
    w.add_tensor("output_norm.weight", norms[(0, 2)])
    if not tied:
        add_q8("output.weight", blocks[(0, 7)], cfg.vocab_size, cfg.hidden_size)
    for l in range(cfg.num_hidden_layers):
        w.add_tensor(f"blk.{l}.attn_norm.weight", norms[(l, 0)])
        w.add_tensor(f"blk.{l}.ffn_norm.weight", norms[(l, 1)].astype(np.float16))
        for which, nm in NAMES.items():
            rows, cols = shapes[which]
            b = np.ascontiguousarray(blocks[(l, which)]).reshape(rows, -1)
            if which in (0, 1):
                # the file holds the interleaved layout: file row perm[j] = engine row j
                heads = cfg.num_attention_heads if which == 0 else cfg.num_key_value_heads
                f = np.empty_like(b)
                f[interleaved_permutation(heads, hd)] = b
                b = f
            add_q8(f"blk.{l}.{nm}.weight", b, rows, cols)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def test_gguf_load_equals_tensor_by_tensor_model(ctx, kb, oracle, torch_cuda, tmp_path):
    mg = load_make_golden()
    g = golden("decode_tiny.npz")
    cfg, shapes, dense, blocks, norms = mg.tiny_model(int(g["seed"]))
    # the f16 norm in the file: both models use the rounded values
    for l in range(cfg.num_hidden_layers):
        norms[(l, 1)] = norms[(l, 1)].astype(np.float16).astype(np.float32)
    path = tmp_path / "tiny.gguf"
    write_gguf(path, cfg, shapes, blocks, norms)
    gm = kb.Model.from_gguf(ctx, str(path), cfg.block_size, cfg.max_seq_len)
    c = gm.cfg
    assert (c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.num_hidden_layers,
            c.intermediate_size, c.vocab_size) == (cfg.hidden_size, cfg.num_attention_heads,
                                                   cfg.num_key_value_heads,
                                                   cfg.num_hidden_layers, cfg.intermediate_size,
                                                   cfg.vocab_size)
    assert abs(c.rope_theta - cfg.rope_theta) < 1e-3 and abs(c.rms_norm_eps - 1e-5) < 1e-9
    ref_m = build_gpu_model(kb, ctx, cfg, shapes, blocks, norms)
    om = mg.build_oracle_model(cfg, shapes, blocks, norms)
    bs, hd = cfg.block_size, cfg.hidden_size // cfg.num_attention_heads
    pools = [kb.KvPool(ctx, cfg.num_hidden_layers, 8, bs, cfg.num_key_value_heads, hd)
             for _ in range(2)]
    opool = oracle.KvPool(cfg.num_hidden_layers, 8, bs, cfg.num_key_value_heads, hd)
    table = [int(b) for b in g["table"]]
    u = lambda a: np.array(a, np.uint32)
    for pos, tok in enumerate(g["tokens"][:6]):
        nb = pos // bs + 1
        slot = table[pos // bs] * bs + pos % bs
        outs = []
        for m, pool in zip((gm, ref_m), pools):
            got = np.empty((1, cfg.vocab_size), np.float32)
            m.decode_step(pool, u([tok]), u([pos]), u([slot]), u(table[:nb]), u([pos + 1]), nb, got)
            outs.append(got)
        assert np.array_equal(outs[0], outs[1])  # same weights on the device, same kernels
        st, ref = om.decode_step(opool, [tok], [pos], [slot], table[:nb], [pos + 1], nb)
        # (this toy model's logits reach +-6: the comparison is relative to their scale; the
        # 1e-2 absolute bound belongs to the benchmark model and is tested there)
        assert st == 0 and np.max(np.abs(outs[0] - ref)) <= 5e-3 * np.max(np.abs(ref))
    for p in pools:
        p.destroy()
    gm.destroy()
    ref_m.destroy()


def test_gguf_refusals(ctx, kb, tmp_path):
    mg = load_make_golden()
    cfg, shapes, dense, blocks, norms = mg.tiny_model(5)
    with pytest.raises(kb.KansoError) as e:
        kb.Model.from_gguf(ctx, str(tmp_path / "missing.gguf"))
    assert e.value.code == kb.ERR_CONFIG
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGUFxxxxxxxxxxxxxxxxxxxxxxxx")
    with pytest.raises(kb.KansoError) as e:
        kb.Model.from_gguf(ctx, str(bad))
    assert e.value.code == kb.ERR_CONFIG and "Failed to parse GGUF file" in e.value.message
    other = tmp_path / "mamba.gguf"
    write_gguf(other, cfg, shapes, blocks, norms, arch="mamba")
    with pytest.raises(kb.KansoError) as e:
        kb.Model.from_gguf(ctx, str(other))
    assert e.value.code == kb.ERR_CONFIG and "unsupported GGUF architecture 'mamba'" in e.value.message
    # untied output.weight is accepted
    untied = tmp_path / "untied.gguf"
    write_gguf(untied, cfg, shapes, blocks, norms, tied=False)
    kb.Model.from_gguf(ctx, str(untied)).destroy()
