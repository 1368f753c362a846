"""Generates the golden fixtures in this directory.

Run from the repository root:  python tests/golden/make_golden.py

Each fixture stores inputs and expected outputs. The expected outputs come from
the CPU oracle (oracle/kanso_oracle.cpp); before anything is written they are
cross-checked against an INDEPENDENT restatement written here in numpy (and, for
the GGUF block decoders, against the `gguf` Python package), so that a mistake
in the oracle's reading of the reference shows up as a disagreement between two
separately written programs. Inputs are either the closed-form patterns of the
reference's own tests (tests/test_neon_simd_gemv.rs, tests/test_paged_attention_v2.rs,
tests/test_quantized_kv_cache.rs) or seeded numpy draws.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
f32 = np.float32


# ---------------------------------------------------------------- numpy restatement
def seq_sum(v):
    """Left-to-right f32 sum, as a scalar Rust loop performs it."""
    v = np.asarray(v, f32)
    return np.cumsum(v, dtype=f32)[-1] if v.size else f32(0)


def round_half_away(v):
    v = np.asarray(v, f32)
    return (np.sign(v) * np.floor(np.abs(v) + f32(0.5))).astype(f32)


def np_quantize_block_q8_0(x):
    x = np.asarray(x, f32)
    amax = np.max(np.abs(x)).astype(f32)
    d = f32(amax / f32(127.0))
    idv = f32(1.0) / d if d != 0 else f32(0)
    q = np.clip(round_half_away(x * idv), -128, 127).astype(np.int8)
    return d, q


def np_dot_q8_0(d, qs, x):
    return f32(d) * seq_sum(qs.astype(f32) * np.asarray(x, f32))


def np_scale_min(j, q):
    if j < 4:
        return q[j] & 63, q[j + 4] & 63
    return (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4), (q[j + 4] >> 4) | ((q[j] >> 6) << 4)


def np_dequant_q4_k(d, dmin, scales, qs):
    out = np.empty(256, f32)
    d, dmin = f32(d), f32(dmin)
    for g in range(4):
        q = qs[32 * g:32 * g + 32]
        sc1, m1 = np_scale_min(2 * g, scales)
        sc2, m2 = np_scale_min(2 * g + 1, scales)
        d1, min1 = f32(d * f32(sc1)), f32(dmin * f32(m1))
        d2, min2 = f32(d * f32(sc2)), f32(dmin * f32(m2))
        out[64 * g:64 * g + 32] = (d1 * (q & 0xF).astype(f32)).astype(f32) - min1
        out[64 * g + 32:64 * g + 64] = (d2 * (q >> 4).astype(f32)).astype(f32) - min2
    return out


def np_kv_quantize_head(x):
    x = np.asarray(x, f32)
    amax = np.max(np.abs(x)).astype(f32)
    scale = f32(amax / f32(127.0)) if amax > 0 else f32(1.0)
    inv = f32(1.0) / scale
    return scale, np.clip(round_half_away(x * inv), -127, 127).astype(np.int8)


def np_paged_attention(q, kc, vc, tables, lens, S, H, KH, hd, bs, maxb, scale):
    q = q.reshape(S, H, hd)
    kc = kc.reshape(-1, bs, KH, hd)
    vc = vc.reshape(-1, bs, KH, hd)
    out = np.zeros((S, H, hd), f32)
    g = H // KH
    for s in range(S):
        ctx = int(lens[s])
        if ctx == 0:
            continue
        t = np.arange(ctx)
        phys = np.asarray(tables, np.int64).reshape(S, maxb)[s, t // bs]
        for h in range(H):
            k = kc[phys, t % bs, h // g]
            v = vc[phys, t % bs, h // g]
            sc = (k.astype(np.float64) @ q[s, h].astype(np.float64)).astype(f32) * f32(scale)
            e = np.exp((sc - sc.max()).astype(f32)).astype(f32)
            w = e / e.sum(dtype=f32)
            out[s, h] = (w.astype(np.float64) @ v.astype(np.float64)).astype(f32)
    return out.reshape(-1)


def assert_close(a, b, tol, what):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    err = np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30)
    assert err <= tol, f"{what}: oracle vs numpy restatement differ by {err:.3e} (> {tol})"
    return err


# ---------------------------------------------------------------- fixtures
def fixture_q8_0():
    # tests/test_neon_simd_gemv.rs:9-44 — block dot pattern
    i = np.arange(32)
    qs = ((i * 7) % 255 - 128).astype(np.int8)
    x = (np.sin(i.astype(f32) * f32(0.13)).astype(f32) * f32(2.0)).astype(f32)
    dot = O.dot_q8_0_ref(0.025, qs, x)
    assert dot == np_dot_q8_0(f32(0.025), qs, x), "q8_0 block dot"
    xd, xq = np_quantize_block_q8_0(x)
    od, oq = O.quantize_row_q8_0(x)
    assert od[0] == xd and np.array_equal(oq, xq), "quantize_row_q8_0 on the dot pattern"
    dotq, isum = O.dot_q8_0_q8_0_ref(0.025, qs, xd, xq)
    assert isum == int(np.sum(qs.astype(np.int64) * xq.astype(np.int64)))
    assert dotq == f32(f32(f32(0.025) * xd) * f32(isum))

    # tests/test_neon_simd_gemv.rs:47-69 — quantize_row pattern and its round-trip bound
    xs = (np.arange(64).astype(f32) * f32(0.1) - f32(3.2)).astype(f32)
    qd, qq = O.quantize_row_q8_0(xs)
    for b in range(2):
        d_np, q_np = np_quantize_block_q8_0(xs[32 * b:32 * b + 32])
        assert qd[b] == d_np and np.array_equal(qq[32 * b:32 * b + 32], q_np)
    assert qd[0] > 0 and qd[1] > 0
    assert np.all(np.abs(qd[0] * qq[:32].astype(f32) - xs[:32]) < qd[0])

    # tests/test_neon_simd_gemv.rs:104-143 — GEMV 64x128 pattern (ref layout, f32 d)
    rows, cols, bpr = 64, 128, 4
    r = np.arange(rows)[:, None, None]
    b = np.arange(bpr)[None, :, None]
    k = np.arange(32)[None, None, :]
    gq = (((r * 31 + b * 17 + k * 5) % 255) - 128).astype(np.int8)
    gd = np.broadcast_to((f32(0.01) + (np.arange(rows).astype(f32) * f32(0.001)))[:, None],
                         (rows, bpr)).astype(f32).copy()
    gx = (np.sin(np.arange(cols).astype(f32) * f32(0.1)).astype(f32) * f32(1.2)).astype(f32)
    gout = O.gemv_q8_0_ref(gd, gq, gx, rows, cols)
    np_out = np.array([seq_sum([np_dot_q8_0(gd[rr, bb], gq[rr, bb], gx[32 * bb:32 * bb + 32])
                                for bb in range(bpr)]) for rr in range(rows)], f32)
    assert np.array_equal(gout, np_out), "q8_0 gemv pattern"

    # tests/test_neon_simd_gemv.rs:191-274 — Q8_0 GEMV vs dense f32 within 1e-2 (256x256 here)
    rows2 = cols2 = 256
    rr, cc = np.meshgrid(np.arange(rows2), np.arange(cols2), indexing="ij")
    wdense = (np.sin((rr * cols2 + cc).astype(f32) * f32(0.01)).astype(f32) * f32(0.5)).astype(f32)
    x2 = (np.cos(np.arange(cols2).astype(f32) * f32(0.05)).astype(f32)).astype(f32)
    wq = O.quantize_weights_q8_0(wdense)
    y_q = O.gemv_q8_0(wq, x2, rows2, cols2)
    y_dense = (wdense.astype(np.float64) @ x2.astype(np.float64))
    assert np.max(np.abs(y_q - y_dense)) < 5e-2, "q8_0 gemv vs dense"

    np.savez(os.path.join(HERE, "q8_0_kat.npz"), dot_qs=qs, dot_x=x, dot_d=f32(0.025),
             dot_expected=f32(dot), dot_q8_expected=f32(dotq), dot_q8_isum=np.int32(isum),
             quant_x=xs, quant_d=qd, quant_qs=qq, gemv_d=gd, gemv_qs=gq.reshape(-1), gemv_x=gx,
             gemv_expected=gout)


def fixture_q4_k():
    # tests/test_neon_simd_gemv.rs:72-101 — block dot pattern
    i = np.arange(128)
    qs = ((i * 17 + 5) & 0xFF).astype(np.uint8)
    scales = np.array([12, 24, 35, 48, 15, 20, 25, 30, 40, 50, 10, 5], np.uint8)
    x = (np.cos(np.arange(256).astype(f32) * f32(0.07)).astype(f32) * f32(1.5)).astype(f32)
    deq = O.dequantize_q4_k_ref(0.05, 0.02, scales, qs)
    assert np.array_equal(deq, np_dequant_q4_k(0.05, 0.02, scales, qs)), "q4_k dequant pattern"
    dot = O.dot_q4_k_ref(0.05, 0.02, scales, qs, x)
    assert dot == seq_sum(deq * x), "q4_k dot pattern"
    unp = [O.get_scale_min_k4(j, scales) for j in range(8)]
    assert unp == [tuple(int(v) for v in np_scale_min(j, scales)) for j in range(8)]

    # tests/test_neon_simd_gemv.rs:146-188 — GEMV 32x256 pattern (ref layout)
    rows = 32
    scales2 = np.array([10, 20, 30, 40, 15, 25, 35, 45, 5, 12, 18, 22], np.uint8)
    gout = np.empty(rows, f32)
    gx = (np.cos(np.arange(256).astype(f32) * f32(0.05)).astype(f32) * f32(2.0)).astype(f32)
    gqs = np.empty((rows, 128), np.uint8)
    gd = np.empty(rows, f32)
    for r in range(rows):
        gqs[r] = ((r * 13 + i * 7) & 0xFF).astype(np.uint8)
        gd[r] = f32(0.02) + f32(f32(r) * f32(0.001))
        gout[r] = O.dot_q4_k_ref(gd[r], 0.01, scales2, gqs[r], gx)
        assert gout[r] == seq_sum(np_dequant_q4_k(gd[r], 0.01, scales2, gqs[r]) * gx)

    np.savez(os.path.join(HERE, "q4_k_kat.npz"), dot_qs=qs, dot_scales=scales, dot_x=x,
             dot_d=f32(0.05), dot_dmin=f32(0.02), dot_dequant=deq, dot_expected=f32(dot),
             dot_unpacked=np.array(unp, np.uint8), gemv_qs=gqs, gemv_scales=scales2, gemv_d=gd,
             gemv_dmin=f32(0.01), gemv_x=gx, gemv_expected=gout)


def fixture_gguf_blocks():
    """Seeded N(0, 0.02) weights through the GGUF (f16-scale) layouts."""
    import gguf
    from gguf import quants as GQ

    rng = np.random.Generator(np.random.PCG64(0xB2000001))
    w = (rng.standard_normal((12, 512)) * 0.02).astype(f32)
    x = rng.standard_normal(512).astype(f32)

    q8 = O.quantize_weights_q8_0(w)
    d8 = O.dequantize_q8_0(q8)
    g8 = GQ.dequantize(q8.reshape(-1, 34), gguf.GGMLQuantizationType.Q8_0).reshape(-1)
    assert np.array_equal(d8, g8.astype(f32)), "Q8_0 dequant vs gguf package"
    # second opinion on the encoder: the gguf package rounds half-to-even and recomputes q
    # from the f16 d in places, so only near-equality is expected, not identity
    gq8 = GQ.quantize(w, gguf.GGMLQuantizationType.Q8_0).reshape(-1)
    mism = np.count_nonzero(gq8 != q8)
    assert mism <= q8.size // 50, f"Q8_0 encoder far from gguf package ({mism} bytes differ)"

    q4 = O.quantize_weights_q4_k(w)
    d4 = O.dequantize_q4_k(q4)
    g4 = GQ.dequantize(q4.reshape(-1, 144), gguf.GGMLQuantizationType.Q4_K).reshape(-1)
    assert np.array_equal(d4, g4.astype(f32)), "Q4_K dequant vs gguf package"
    # the generator must be a usable encoder: reconstruction within one grid step
    assert np.max(np.abs(d4 - w.reshape(-1))) < 0.02 * 8 / 15, "Q4_K encoder too coarse"
    sc = O.unpack_scales_q4_k(q4)
    blk = q4.reshape(-1, 144)
    for b in range(blk.shape[0]):
        for j in range(8):
            s_, m_ = np_scale_min(j, blk[b, 4:16])
            assert sc[b, j] == s_ and sc[b, 8 + j] == m_

    y8 = O.gemv_q8_0(q8, x, 12, 512)
    y8q = O.gemv_q8_0_q8(q8, x, 12, 512)
    y4 = O.gemv_q4_k(q4, x, 12, 512)
    assert_close(y8, d8.reshape(12, 512).astype(np.float64) @ x, 1e-5, "Q8_0 gemv")
    assert_close(y4, d4.reshape(12, 512).astype(np.float64) @ x, 1e-5, "Q4_K gemv")
    xd, xq = O.quantize_row_q8_0(x)
    isums = O.block_isums_q8_0(q8, xq, 12, 512)
    wq = q8.reshape(12, 16, 34)[:, :, 2:].view(np.int8).astype(np.int64)
    assert np.array_equal(isums, np.einsum("rbk,bk->rb", wq, xq.reshape(16, 32).astype(np.int64)))

    np.savez(os.path.join(HERE, "gguf_blocks.npz"), w=w, x=x, q8_0=q8, q8_0_dequant=d8, q4_k=q4,
             q4_k_dequant=d4, q4_k_scales=sc, gemv_q8_0=y8, gemv_q8_0_q8=y8q, gemv_q4_k=y4,
             x_q8_d=xd, x_q8_qs=xq, isums=isums)


def fixture_kv():
    # tests/test_quantized_kv_cache.rs:6-86 — int8 round trip on sin/cos patterns
    layers, nblocks, bs, H, hd = 2, 4, 4, 2, 8
    pool = O.KvPool(layers, nblocks, bs, H, hd)
    n = H * hd
    recs = []
    for t in range(6):
        k = (np.sin((np.arange(n) + t * n).astype(f32) * f32(0.1)) * f32(2.5)).astype(f32)
        v = (np.cos((np.arange(n) + t * n).astype(f32) * f32(0.15)) * f32(1.8)).astype(f32)
        block, off = [2, 0][t // bs], t % bs
        assert pool.write_token(1, block, off, k, v) == 0
        st, got = pool.read_token(1, block, off)
        assert st == 0
        for h in range(H):
            s_np, q_np = np_kv_quantize_head(k[h * hd:(h + 1) * hd])
            assert got["k_scale"][h] == s_np and np.array_equal(got["k_q"][h * hd:(h + 1) * hd],
                                                                q_np)
        rel = np.linalg.norm(got["k_deq"] - k) / np.linalg.norm(k)
        assert rel <= 0.01, "int8 KV round trip"
        recs.append((k, v, got))
    zero_scale, zero_q = O.kv_quantize_head(np.zeros(8, f32))
    assert zero_scale == 1.0 and not zero_q.any()
    assert pool.write_token(2, 0, 0, recs[0][0], recs[0][1]) == 2  # layer out of bounds
    assert pool.write_token(0, 4, 0, recs[0][0], recs[0][1]) == 2  # block out of bounds
    assert pool.write_token(0, 0, 4, recs[0][0], recs[0][1]) == 2  # offset out of bounds
    st, gk, gv = pool.gather(1, [2, 0], 6)
    assert st == 0
    np.savez(os.path.join(HERE, "kv_int8.npz"), geom=np.array([layers, nblocks, bs, H, hd]),
             k=np.stack([r[0] for r in recs]), v=np.stack([r[1] for r in recs]),
             k_q=np.stack([r[2]["k_q"] for r in recs]), v_q=np.stack([r[2]["v_q"] for r in recs]),
             k_scale=np.stack([r[2]["k_scale"] for r in recs]),
             v_scale=np.stack([r[2]["v_scale"] for r in recs]), gather_k=gk, gather_v=gv)


def pa_pattern_case(S, H, KH, hd, bs, maxb, lens, tables, nblocks):
    """Inputs in the style of tests/test_paged_attention_v2.rs:326-401."""
    nq, nkv = S * H * hd, nblocks * bs * KH * hd
    q = (((np.arange(nq) % 17) - 8).astype(f32) * f32(0.125)).astype(f32)
    kc = (((np.arange(nkv) % 19) - 9).astype(f32) * f32(0.1)).astype(f32)
    vc = (((np.arange(nkv) % 23) - 11).astype(f32) * f32(0.15)).astype(f32)
    p = O.PaParams(S, H, KH, hd, bs, maxb, 1.0 / np.sqrt(f32(hd)))
    out = O.paged_attention_f32(q, kc, vc, tables, lens, p)
    ref = np_paged_attention(q, kc, vc, tables, lens, S, H, KH, hd, bs, maxb, p.scale)
    assert_close(out, ref, 2e-5, f"paged attention {S}x{H}x{KH}x{hd}")
    return dict(q=q, k=kc, v=vc, tables=np.asarray(tables, np.uint32),
                lens=np.asarray(lens, np.uint32), out=out,
                params=np.array([S, H, KH, hd, bs, maxb], np.uint32))


def fixture_paged_attention():
    # tests/test_paged_attention_v2.rs:10-87 — the hand-worked example with expected outputs
    p = O.PaParams(1, 1, 1, 4, 2, 2, 0.5)
    q = np.array([1, 0, 1, 0], f32)
    kc = np.zeros(4 * 2 * 4, f32)
    vc = np.zeros(4 * 2 * 4, f32)
    o0, o1, o2 = (2 * 2) * 4, (2 * 2 + 1) * 4, 2 * 4
    kc[o0] = 1
    vc[o0] = 10
    kc[o1 + 2] = 1
    vc[o1 + 1] = 20
    kc[o2] = 1
    kc[o2 + 2] = 1
    vc[o2 + 2] = 30
    out = O.paged_attention_f32(q, kc, vc, [2, 1], [3], p)
    assert abs(out[0] - 2.7407) < 1e-3 and abs(out[1] - 5.4814) < 1e-3
    assert abs(out[2] - 13.5558) < 1e-3 and out[3] == 0.0
    # ctx 0 leaves zeros on the CPU path (paged_attention.rs:112-115)
    assert not O.paged_attention_f32(q, kc, vc, [2, 1], [0], p).any()

    cases = {"basic": dict(q=q, k=kc, v=vc, tables=np.array([2, 1], np.uint32),
                           lens=np.array([3], np.uint32), out=out,
                           params=np.array([1, 1, 1, 4, 2, 2], np.uint32))}
    # non-contiguous table, GQA 8:2, ragged 3-sequence batch, 3-partition merge at ctx 600
    cases["noncontig"] = pa_pattern_case(1, 4, 4, 64, 16, 4, [35], [7, 2, 5, 0], 8)
    cases["gqa"] = pa_pattern_case(1, 8, 2, 64, 16, 4, [50], [3, 1, 6, 4], 8)
    cases["ragged"] = pa_pattern_case(3, 4, 2, 32, 8, 4, [5, 17, 32],
                                      [1, 1, 1, 1, 4, 2, 9, 9, 8, 0, 3, 6], 10)
    cases["merge600"] = pa_pattern_case(1, 15, 5, 64, 16, 38, [600],
                                        list(np.random.Generator(np.random.PCG64(7))
                                             .permutation(40)[:38]), 40)
    flat = {f"{n}__{k}": v for n, c in cases.items() for k, v in c.items()}
    np.savez(os.path.join(HERE, "paged_attention_kat.npz"), **flat)


def tiny_model(seed=0xB2000004):
    """A seeded Q8_0 model small enough for a numpy restatement of the decode step."""
    cfg = O.ModelConfig(64, 4, 2, 2, 128, 96, 4, 64, 1e-5, 100000.0)
    rng = np.random.Generator(np.random.PCG64(seed))
    hd = cfg.hidden_size // cfg.num_attention_heads
    shapes = {0: (cfg.num_attention_heads * hd, 64), 1: (cfg.num_key_value_heads * hd, 64),
              2: (cfg.num_key_value_heads * hd, 64), 3: (64, cfg.num_attention_heads * hd),
              4: (128, 64), 5: (128, 64), 6: (64, 128)}
    dense, blocks, norms = {}, {}, {}
    for l in range(cfg.num_hidden_layers):
        for which, shp in shapes.items():
            w = (rng.standard_normal(shp) * 0.08).astype(f32)
            blocks[(l, which)] = O.quantize_weights_q8_0(w)
            dense[(l, which)] = O.dequantize_q8_0(blocks[(l, which)]).reshape(shp)
        norms[(l, 0)] = (1 + 0.1 * rng.standard_normal(64)).astype(f32)
        norms[(l, 1)] = (1 + 0.1 * rng.standard_normal(64)).astype(f32)
    emb = (rng.standard_normal((cfg.vocab_size, 64)) * 0.5).astype(f32)
    blocks[(0, 7)] = O.quantize_weights_q8_0(emb)
    dense[(0, 7)] = O.dequantize_q8_0(blocks[(0, 7)]).reshape(cfg.vocab_size, 64)
    norms[(0, 2)] = (1 + 0.1 * rng.standard_normal(64)).astype(f32)
    return cfg, shapes, dense, blocks, norms


def build_oracle_model(cfg, shapes, blocks, norms):
    m = O.Model(cfg)
    for (l, which), b in blocks.items():
        rows, cols = (cfg.vocab_size, cfg.hidden_size) if which == 7 else shapes[which]
        assert m.set_weight(l, which, b, rows, cols) == 0
    for (l, which), w in norms.items():
        assert m.set_norm(l, which, w) == 0
    return m


def np_decode_token(cfg, dense, norms, kcache, vcache, token, pos):
    """float64 restatement of src/model.rs:1101-1231 with an int8-quantised KV history kept
    as plain per-layer lists (no paging: the oracle's paging is checked separately)."""
    H, KH = cfg.num_attention_heads, cfg.num_key_value_heads
    hd = cfg.hidden_size // H
    half = hd // 2

    def rms(x, w):
        return x / np.sqrt(np.mean(x * x) + cfg.rms_norm_eps) * w

    def rope(v, nheads):
        v = v.reshape(nheads, hd).copy()
        j = np.arange(half)
        ang = pos * np.power(np.float64(cfg.rope_theta), -2.0 * j / hd)
        c, s = np.cos(ang), np.sin(ang)
        a, b = v[:, :half].copy(), v[:, half:].copy()
        v[:, :half], v[:, half:] = a * c - b * s, a * s + b * c
        return v

    h = dense[(0, 7)][token].astype(np.float64)
    for l in range(cfg.num_hidden_layers):
        n = rms(h, norms[(l, 0)])
        q = rope(dense[(l, 0)] @ n, H)
        k = rope(dense[(l, 1)] @ n, KH)
        v = (dense[(l, 2)] @ n).reshape(KH, hd)
        kq = np.stack([(lambda sq: sq[1].astype(np.float64) * np.float64(sq[0]))(
            np_kv_quantize_head(k[i].astype(f32))) for i in range(KH)])
        vq = np.stack([(lambda sq: sq[1].astype(np.float64) * np.float64(sq[0]))(
            np_kv_quantize_head(v[i].astype(f32))) for i in range(KH)])
        kcache[l].append(kq)
        vcache[l].append(vq)
        K, V = np.stack(kcache[l]), np.stack(vcache[l])  # [ctx, KH, hd]
        out = np.empty((H, hd))
        for hh in range(H):
            sc = K[:, hh // (H // KH)] @ q[hh] / np.sqrt(hd)
            e = np.exp(sc - sc.max())
            out[hh] = (e / e.sum()) @ V[:, hh // (H // KH)]
        h = h + dense[(l, 3)] @ out.reshape(-1)
        n = rms(h, norms[(l, 1)])
        g, u = dense[(l, 4)] @ n, dense[(l, 5)] @ n
        h = h + dense[(l, 6)] @ (g / (1 + np.exp(-g)) * u)
    return dense[(0, 7)] @ rms(h, norms[(0, 2)])


def fixture_decode():
    cfg, shapes, dense, blocks, norms = tiny_model()
    m = build_oracle_model(cfg, shapes, blocks, norms)
    bs, nblocks = cfg.block_size, 8
    pool = O.KvPool(cfg.num_hidden_layers, nblocks, bs, cfg.num_key_value_heads,
                    cfg.hidden_size // cfg.num_attention_heads)
    table = [5, 2, 7]  # permuted physical blocks
    tokens = [3, 17, 42, 8, 91, 60, 11, 29, 77]
    kc = [[] for _ in range(cfg.num_hidden_layers)]
    vc = [[] for _ in range(cfg.num_hidden_layers)]
    all_logits = []
    for pos, tok in enumerate(tokens):
        nb = pos // bs + 1
        slot = table[pos // bs] * bs + pos % bs
        st, logits = m.decode_step(pool, [tok], [pos], [slot], table[:nb], [pos + 1], nb)
        assert st == 0
        ref = np_decode_token(cfg, dense, norms, kc, vc, tok, pos)
        err = np.max(np.abs(logits[0] - ref))
        assert err < 2e-3, f"decode step pos {pos}: oracle vs numpy restatement differ by {err}"
        assert int(np.argmax(ref)) == O.greedy_token(logits[0])
        all_logits.append(logits[0])
    np.savez(os.path.join(HERE, "decode_tiny.npz"), tokens=np.array(tokens, np.uint32),
             table=np.array(table, np.uint32), logits=np.stack(all_logits),
             seed=np.uint64(0xB2000004))


def main():
    fixture_q8_0()
    fixture_q4_k()
    fixture_gguf_blocks()
    fixture_kv()
    fixture_paged_attention()
    fixture_decode()
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
