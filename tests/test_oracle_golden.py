"""CPU: the oracle against the committed golden fixtures and the reference's own test bounds."""
import numpy as np
import pytest

from conftest import golden, rel_err


def test_q8_0_kat(oracle):
    g = golden("q8_0_kat.npz")
    assert oracle.dot_q8_0_ref(float(g["dot_d"]), g["dot_qs"], g["dot_x"]) == g["dot_expected"]
    xd, xq = oracle.quantize_row_q8_0(g["dot_x"])
    r, isum = oracle.dot_q8_0_q8_0_ref(float(g["dot_d"]), g["dot_qs"], float(xd[0]), xq)
    assert r == g["dot_q8_expected"] and isum == g["dot_q8_isum"]
    d, qs = oracle.quantize_row_q8_0(g["quant_x"])
    assert np.array_equal(d, g["quant_d"]) and np.array_equal(qs, g["quant_qs"])
    # tests/test_neon_simd_gemv.rs:63-68: round-trip error below one step
    assert np.all(np.abs(d[0] * qs[:32].astype(np.float32) - g["quant_x"][:32]) < d[0])
    out = oracle.gemv_q8_0_ref(g["gemv_d"], g["gemv_qs"], g["gemv_x"], 64, 128)
    assert np.array_equal(out, g["gemv_expected"])


def test_q4_k_kat(oracle):
    g = golden("q4_k_kat.npz")
    deq = oracle.dequantize_q4_k_ref(float(g["dot_d"]), float(g["dot_dmin"]), g["dot_scales"],
                                     g["dot_qs"])
    assert np.array_equal(deq, g["dot_dequant"])
    assert oracle.dot_q4_k_ref(float(g["dot_d"]), float(g["dot_dmin"]), g["dot_scales"],
                               g["dot_qs"], g["dot_x"]) == g["dot_expected"]
    for j in range(8):
        assert tuple(g["dot_unpacked"][j]) == oracle.get_scale_min_k4(j, g["dot_scales"])
    for r in range(32):
        got = oracle.dot_q4_k_ref(float(g["gemv_d"][r]), float(g["gemv_dmin"]), g["gemv_scales"],
                                  g["gemv_qs"][r], g["gemv_x"])
        assert got == g["gemv_expected"][r]


def test_gguf_blocks(oracle):
    g = golden("gguf_blocks.npz")
    assert np.array_equal(oracle.quantize_weights_q8_0(g["w"]), g["q8_0"])
    assert np.array_equal(oracle.dequantize_q8_0(g["q8_0"]), g["q8_0_dequant"])
    assert np.array_equal(oracle.quantize_weights_q4_k(g["w"]), g["q4_k"])
    assert np.array_equal(oracle.dequantize_q4_k(g["q4_k"]), g["q4_k_dequant"])
    assert np.array_equal(oracle.unpack_scales_q4_k(g["q4_k"]), g["q4_k_scales"])
    assert np.array_equal(oracle.gemv_q8_0(g["q8_0"], g["x"], 12, 512), g["gemv_q8_0"])
    assert np.array_equal(oracle.gemv_q8_0_q8(g["q8_0"], g["x"], 12, 512), g["gemv_q8_0_q8"])
    assert np.array_equal(oracle.gemv_q4_k(g["q4_k"], g["x"], 12, 512), g["gemv_q4_k"])
    assert np.array_equal(oracle.block_isums_q8_0(g["q8_0"], g["x_q8_qs"], 12, 512), g["isums"])
    # GEMM = the GEMV per activation row
    x2 = np.stack([g["x"], g["x"][::-1]])
    y = oracle.gemm_q8_0(g["q8_0"], x2, 2, 12, 512)
    assert np.array_equal(y[0], g["gemv_q8_0"])
    assert np.array_equal(y[1], oracle.gemv_q8_0(g["q8_0"], x2[1], 12, 512))
    y4 = oracle.gemm_q4_k(g["q4_k"], x2, 2, 12, 512)
    assert np.array_equal(y4[0], g["gemv_q4_k"])


def test_f16_roundtrip(oracle):
    # every f16 bit pattern widens and narrows back to itself (NaNs keep being NaN)
    for h in range(0, 1 << 16, 7):
        f = oracle.f16_bits_to_f32(h)
        if f != f:
            continue
        assert oracle.f32_to_f16_bits(f) == h
    assert np.array_equal(
        np.array([oracle.f16_bits_to_f32(h) for h in range(0, 0x7C00, 97)], np.float32),
        np.arange(0, 0x7C00, 97, dtype=np.uint16).view(np.float16).astype(np.float32))


def test_kv_int8(oracle):
    g = golden("kv_int8.npz")
    layers, nblocks, bs, H, hd = (int(v) for v in g["geom"])
    pool = oracle.KvPool(layers, nblocks, bs, H, hd)
    for t in range(6):
        block, off = [2, 0][t // bs], t % bs
        assert pool.write_token(1, block, off, g["k"][t], g["v"][t]) == 0
        st, got = pool.read_token(1, block, off)
        assert st == 0
        assert np.array_equal(got["k_q"], g["k_q"][t]) and np.array_equal(got["v_q"], g["v_q"][t])
        assert np.array_equal(got["k_scale"], g["k_scale"][t])
        # tests/test_quantized_kv_cache.rs:6-86: rel-L2 <= 1 %
        assert np.linalg.norm(got["k_deq"] - g["k"][t]) / np.linalg.norm(g["k"][t]) <= 0.01
        assert np.linalg.norm(got["v_deq"] - g["v"][t]) / np.linalg.norm(g["v"][t]) <= 0.01
    st, k, v = pool.gather(1, [2, 0], 6)
    assert st == 0 and np.array_equal(k, g["gather_k"]) and np.array_equal(v, g["gather_v"])
    # short table and out-of-range block are errors (quantized_storage.rs:319-333)
    assert pool.gather(1, [2], 6)[0] == 2
    assert pool.gather(1, [2, 9], 6)[0] == 2
    # reset: quants 0, scales 1.0 (quantized_storage.rs:35-40)
    pool.reset_block(2)
    st, got = pool.read_token(1, 2, 0)
    assert not got["k_q"].any() and np.all(got["k_scale"] == 1.0)
    # a recycled block in another layer is erased too
    st, got0 = pool.read_token(0, 2, 0)
    assert np.all(got0["v_scale"] == 1.0)


def test_kv_fp8(oracle):
    """QuantMode::Fp8 (src/kv_cache/quantized_storage.rs:109-131,440-449,470-484). E4M3 itself
    comes from the float8 crate, which the reference tree does not vendor: the restatement is
    pinned on the format's fixed points, on the reference's own test vector
    (tests/test_quantized_kv_cache.rs:88-166) and on an independent implementation (torch's
    float8_e4m3fn conversion) over seeded values of every binade, subnormals included."""
    torch = pytest.importorskip("torch")
    val = [oracle.fp8_e4m3_to_f32(b) for b in range(256)]
    assert val[0x7E] == 448.0 and val[0x08] == 2.0 ** -6 and val[0x01] == 2.0 ** -9
    assert val[0x38] == 1.0 and val[0xB8] == -1.0 and val[0x7F] != val[0x7F]
    for b in range(256):
        if val[b] == val[b] and val[b] != 0:
            assert oracle.fp8_e4m3_from_f32(val[b]) == b
    assert oracle.fp8_e4m3_from_f32(1.0625) == 0x38 and oracle.fp8_e4m3_from_f32(1.1875) == 0x3A
    rng = np.random.Generator(np.random.PCG64(0xB200F8))
    x = (rng.standard_normal(20000) * 10.0 ** rng.uniform(-4, 2, 20000)).astype(np.float32)
    x = x[np.abs(x) <= 448]
    ref = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = np.array([oracle.fp8_e4m3_from_f32(v) for v in x], np.uint8)
    assert np.array_equal(got, ref)
    back = torch.from_numpy(np.arange(256, dtype=np.uint8)).view(torch.float8_e4m3fn).float().numpy()
    assert all(back[b] == val[b] for b in range(256) if val[b] == val[b])
    # the reference's own case: values E4M3 holds exactly, bound 1 %, here zero
    n = 4 * 64
    k = np.array([((i % 16) * 0.5 - 3.5) or 1.0 for i in range(n)], np.float32)
    v = np.array([(i % 8) + 0.5 for i in range(n)], np.float32)
    pool = oracle.KvPool(2, 4, 4, 4, 64, fp8=True)
    assert pool.write_token(0, 0, 0, k, v) == 0
    st, got = pool.read_token(0, 0, 0)
    assert st == 0 and np.array_equal(got["k_deq"], k) and np.array_equal(got["v_deq"], v)
    assert np.all(got["k_scale"] == np.float32(2.0 ** -4)) and np.all(got["v_scale"] == 0.125)
    # seeded rows: scale is the smallest power of two >= amax / 64, error within half an E4M3 step
    xs = rng.standard_normal((16, 64)).astype(np.float32) * 3
    for row in xs:
        sc, q = oracle.kv_quantize_head_fp8(row)
        amax = float(np.max(np.abs(row)))
        assert sc >= amax / 64 > sc / 2 and np.log2(sc) == round(np.log2(sc))
        deq = np.array([oracle.fp8_e4m3_to_f32(int(b) & 0xFF) for b in q], np.float32) * sc
        assert np.all(np.abs(deq - row) <= np.maximum(np.abs(row) / 16, sc * 2.0 ** -10))
    # same byte count per token as int8 (quantized_storage.rs:414-419); fresh blocks: 0 / 1.0
    st, fresh = pool.read_token(1, 3, 1)
    assert not fresh["k_q"].any() and np.all(fresh["v_scale"] == 1.0)


def test_paged_attention_kat(oracle):
    g = golden("paged_attention_kat.npz")
    names = sorted({k.split("__")[0] for k in g.files})
    assert "basic" in names and "merge600" in names
    for n in names:
        S, H, KH, hd, bs, maxb = (int(v) for v in g[f"{n}__params"])
        p = oracle.PaParams(S, H, KH, hd, bs, maxb, 1.0 / np.sqrt(np.float32(hd)))
        out = oracle.paged_attention_f32(g[f"{n}__q"], g[f"{n}__k"], g[f"{n}__v"],
                                         g[f"{n}__tables"], g[f"{n}__lens"], p)
        assert np.array_equal(out, g[f"{n}__out"]), n
    b = g["basic__out"]  # tests/test_paged_attention_v2.rs:83-86
    assert abs(b[0] - 2.7407) < 1e-3 and abs(b[1] - 5.4814) < 1e-3
    assert abs(b[2] - 13.5558) < 1e-3 and b[3] == 0.0


def test_pa_params_validation(oracle):
    ok = oracle.PaParams(1, 8, 2, 64, 16, 4, 0.125)
    assert oracle.validate_pa_params(ok) == 0
    assert oracle.pa_num_partitions(ok) == 1
    assert oracle.pa_num_partitions(oracle.PaParams(1, 8, 2, 64, 16, 38, 0.125)) == 3
    for bad in [oracle.PaParams(0, 8, 2, 64, 16, 4, 1), oracle.PaParams(1, 7, 2, 64, 16, 4, 1),
                oracle.PaParams(1, 18, 2, 64, 16, 4, 1),  # group 9 > 8
                oracle.PaParams(1, 8, 2, 384, 16, 4, 1),  # tests/test_paged_attention_v2.rs:405-447
                oracle.PaParams(1, 8, 2, 64, 0, 4, 1), oracle.PaParams(1, 8, 2, 64, 16, 0, 1)]:
        assert oracle.validate_pa_params(bad) != 0


def test_int8_attention_matches_f32_attention_on_dequantised_pool(oracle):
    rng = np.random.Generator(np.random.PCG64(11))
    L, NB, bs, KH, hd, H = 1, 6, 4, 2, 16, 4
    pool = oracle.KvPool(L, NB, bs, KH, hd)
    table = [4, 1, 5]
    ctx = 10
    for t in range(ctx):
        pool.write_token(0, table[t // bs], t % bs, rng.standard_normal(KH * hd),
                         rng.standard_normal(KH * hd))
    q = rng.standard_normal(H * hd).astype(np.float32)
    p = oracle.PaParams(1, H, KH, hd, bs, 3, 0.25)
    st, out = oracle.paged_attention_int8(pool, 0, q, table, [ctx], p)
    assert st == 0
    # same numbers through the f32 statement on an explicitly dequantised pool
    kc = np.zeros((NB, bs, KH, hd), np.float32)
    vc = np.zeros_like(kc)
    for b in range(NB):
        for o in range(bs):
            _, r = pool.read_token(0, b, o)
            kc[b, o] = r["k_deq"].reshape(KH, hd)
            vc[b, o] = r["v_deq"].reshape(KH, hd)
    ref = oracle.paged_attention_f32(q, kc, vc, table, [ctx], p)
    assert np.array_equal(out.reshape(-1), ref)


def test_glue(oracle):
    rng = np.random.Generator(np.random.PCG64(5))
    x = rng.standard_normal((3, 64)).astype(np.float32)
    w = rng.standard_normal(64).astype(np.float32)
    ref = x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-5) * w
    assert rel_err(oracle.rmsnorm(x, w, 1e-5), ref) < 1e-6
    g, u = rng.standard_normal(100), rng.standard_normal(100)
    assert rel_err(oracle.silu_mul(g, u), g / (1 + np.exp(-g)) * u) < 1e-6
    c, s = oracle.rope_table(100000.0, 40, 16)
    j = np.arange(8)
    ang = np.arange(40)[:, None] * (100000.0 ** (-2.0 * j / 16))[None, :]
    assert np.max(np.abs(c - np.cos(ang))) < 1e-4 and np.max(np.abs(s - np.sin(ang))) < 1e-4
    v = rng.standard_normal((2, 3, 16)).astype(np.float32)
    r = oracle.rope(v, [5, 39], 100000.0)
    for t, pos in enumerate([5, 39]):
        a, b = v[t, :, :8], v[t, :, 8:]
        assert rel_err(r[t, :, :8], a * c[pos] - b * s[pos]) < 1e-6
        assert rel_err(r[t, :, 8:], a * s[pos] + b * c[pos]) < 1e-6
    assert oracle.greedy_token(np.array([1, 5, 5, 2], np.float32)) == 1  # first max wins


def test_padded_decode_tables(oracle):
    st, mb, out = oracle.padded_decode_tables(4, [[7, 3, 9], [5]], [9, 2])
    assert st == 0 and mb == 3
    assert list(out) == [7, 3, 9, 5, 5, 5]  # padding repeats the last needed block
    st, mb, _ = oracle.padded_decode_tables(4, [[7, 3], [5]], [9, 2])
    assert st == 2 and mb == 0  # a short table is an error, never a clamp


def test_decode_tiny_golden(oracle):
    import importlib.util, os
    spec = importlib.util.spec_from_file_location(
        "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    g = golden("decode_tiny.npz")
    cfg, shapes, dense, blocks, norms = mg.tiny_model(int(g["seed"]))
    m = mg.build_oracle_model(cfg, shapes, blocks, norms)
    bs = cfg.block_size
    pool = oracle.KvPool(cfg.num_hidden_layers, 8, bs, cfg.num_key_value_heads,
                         cfg.hidden_size // cfg.num_attention_heads)
    table = [int(b) for b in g["table"]]
    for pos, tok in enumerate(g["tokens"]):
        nb = pos // bs + 1
        st, logits = m.decode_step(pool, [tok], [pos], [table[pos // bs] * bs + pos % bs],
                                   table[:nb], [pos + 1], nb)
        assert st == 0 and np.array_equal(logits[0], g["logits"][pos])
