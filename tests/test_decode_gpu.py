"""GPU: the decode step against the oracle engine (logits within 1e-2 abs, same greedy token)."""
import importlib.util
import os

import numpy as np
import pytest

from conftest import golden, rel_err

pytestmark = pytest.mark.gpu


def load_make_golden():
    spec = importlib.util.spec_from_file_location(
        "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    return mg


def build_gpu_model(kb, ctx, cfg, shapes, blocks, norms):
    c = kb.ModelConfig(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                       cfg.num_hidden_layers, cfg.intermediate_size, cfg.vocab_size,
                       cfg.block_size, cfg.max_seq_len, cfg.rms_norm_eps, cfg.rope_theta)
    m = kb.Model(ctx, c)
    for (l, which), b in blocks.items():
        rows, cols = (cfg.vocab_size, cfg.hidden_size) if which == 7 else shapes[which]
        m.set_weight(l, which, b, kb.DTYPE_Q8_0, rows, cols)
    for (l, which), w in norms.items():
        m.set_norm(l, which, w)
    return m


def test_glue_ops(ctx, oracle, torch_cuda):
    torch = torch_cuda
    rng = np.random.Generator(np.random.PCG64(21))
    x = rng.standard_normal((5, 960)).astype(np.float32)
    w = rng.standard_normal(960).astype(np.float32)
    out = torch.empty((5, 960), device="cuda")
    ctx.rmsnorm(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), out, 5, 960, 1e-5)
    ctx.sync()
    assert rel_err(out.cpu().numpy(), oracle.rmsnorm(x, w, 1e-5)) <= 1e-5
    v = rng.standard_normal((3, 15, 64)).astype(np.float32)
    pos = np.array([0, 77, 4095], np.uint32)
    vd = torch.from_numpy(v).cuda()
    ctx.rope(vd, torch.from_numpy(pos.astype(np.int32)).cuda(), 3, 15, 64, 100000.0)
    ctx.sync()
    assert rel_err(vd.cpu().numpy(), oracle.rope(v, pos, 100000.0)) <= 1e-4
    g, u = rng.standard_normal(2560).astype(np.float32), rng.standard_normal(2560).astype(np.float32)
    o = torch.empty(2560, device="cuda")
    ctx.silu_mul(torch.from_numpy(g).cuda(), torch.from_numpy(u).cuda(), o, 2560)
    h = torch.from_numpy(g).cuda()
    ctx.residual_add(h, torch.from_numpy(u).cuda(), 2560)
    ctx.sync()
    assert rel_err(o.cpu().numpy(), oracle.silu_mul(g, u)) <= 1e-6
    assert np.array_equal(h.cpu().numpy(), g + u)
    logits = rng.standard_normal((4, 49152)).astype(np.float32)
    logits[1, 100] = logits[1, 7] = 50.0  # tie: the first maximum wins
    tok = torch.empty(4, dtype=torch.int32, device="cuda")
    ctx.greedy_token(torch.from_numpy(logits).cuda(), tok, 4, 49152)
    ctx.sync()
    assert [int(t) for t in tok.cpu()] == [oracle.greedy_token(r) for r in logits]
    assert int(tok[1]) == 7


@pytest.mark.parametrize("act", [0, 1])
def test_decode_tiny_model(ctx, kb, oracle, torch_cuda, act):
    mg = load_make_golden()
    g = golden("decode_tiny.npz")
    cfg, shapes, dense, blocks, norms = mg.tiny_model(int(g["seed"]))
    om = mg.build_oracle_model(cfg, shapes, blocks, norms)
    gm = build_gpu_model(kb, ctx, cfg, shapes, blocks, norms)
    bs, hd = cfg.block_size, cfg.hidden_size // cfg.num_attention_heads
    opool = oracle.KvPool(cfg.num_hidden_layers, 8, bs, cfg.num_key_value_heads, hd)
    gpool = kb.KvPool(ctx, cfg.num_hidden_layers, 8, bs, cfg.num_key_value_heads, hd)
    table = [int(b) for b in g["table"]]
    for pos, tok in enumerate(g["tokens"]):
        nb = pos // bs + 1
        slot = table[pos // bs] * bs + pos % bs
        u = lambda a: np.array(a, np.uint32)
        st, ref = om.decode_step(opool, [tok], [pos], [slot], table[:nb], [pos + 1], nb, act)
        assert st == 0
        got = np.empty((1, cfg.vocab_size), np.float32)
        gm.decode_step(gpool, u([tok]), u([pos]), u([slot]), u(table[:nb]), u([pos + 1]), nb, got,
                       act)
        assert np.max(np.abs(got - ref)) <= 1e-2
        assert int(np.argmax(got[0])) == oracle.greedy_token(ref[0])
        if act == 0:
            assert np.max(np.abs(got[0] - g["logits"][pos])) <= 1e-2


def test_decode_batch_of_ragged_sequences(ctx, kb, oracle, torch_cuda):
    """A pure-decode batch equals the per-sequence reference (tests/test_batched_forward.rs:52-201)."""
    mg = load_make_golden()
    cfg, shapes, dense, blocks, norms = mg.tiny_model(0xB2000009)
    om = mg.build_oracle_model(cfg, shapes, blocks, norms)
    gm = build_gpu_model(kb, ctx, cfg, shapes, blocks, norms)
    bs, hd, KH, L = cfg.block_size, 16, cfg.num_key_value_heads, cfg.num_hidden_layers
    rng = np.random.Generator(np.random.PCG64(77))
    B, NB = 5, 64
    lens = [1, 4, 9, 30, 17]  # context lengths including the token being decoded
    opool, gpool = oracle.KvPool(L, NB, bs, KH, hd), kb.KvPool(ctx, L, NB, bs, KH, hd)
    perm = [int(b) for b in rng.permutation(NB)]
    tables, used = [], 0
    for c in lens:
        need = (c + bs - 1) // bs
        tables.append(perm[used:used + need])
        used += need
    # history: random K/V written into both pools for every layer
    for s, c in enumerate(lens):
        for t in range(c - 1):
            slot = tables[s][t // bs] * bs + t % bs
            for l in range(L):
                k, v = rng.standard_normal(KH * hd), rng.standard_normal(KH * hd)
                opool.write_token(l, slot // bs, slot % bs, k, v)
                gpool.write_slots(l, torch_cuda.tensor([slot], dtype=torch_cuda.int32).cuda(),
                                  torch_cuda.from_numpy(k.astype(np.float32)).cuda(),
                                  torch_cuda.from_numpy(v.astype(np.float32)).cuda(), 1)
    st, maxb, padded = oracle.padded_decode_tables(bs, tables, lens)
    assert st == 0
    tokens = rng.integers(0, cfg.vocab_size, B).astype(np.uint32)
    positions = np.array([c - 1 for c in lens], np.uint32)
    slots = np.array([tables[s][(c - 1) // bs] * bs + (c - 1) % bs for s, c in enumerate(lens)],
                     np.uint32)
    st, ref = om.decode_step(opool, tokens, positions, slots, padded, lens, maxb)
    assert st == 0
    got = np.empty((B, cfg.vocab_size), np.float32)
    gm.decode_step(gpool, tokens, positions, slots, padded, np.array(lens, np.uint32), maxb, got)
    assert np.max(np.abs(got - ref)) <= 1e-2
    assert [int(np.argmax(r)) for r in got] == [oracle.greedy_token(r) for r in ref]
    # host-side rejections: short table, bad slot, bad token
    with pytest.raises(kb.KansoError) as e:
        gm.decode_step(gpool, tokens, positions, slots, padded, np.array([c + 64 for c in lens],
                                                                         np.uint32), maxb, got)
    assert e.value.code == kb.ERR_SHAPE
    bad = slots.copy()
    bad[0] = NB * bs
    with pytest.raises(kb.KansoError) as e:
        gm.decode_step(gpool, tokens, positions, bad, padded, np.array(lens, np.uint32), maxb, got)
    assert e.value.code == kb.ERR_SHAPE


@pytest.mark.parametrize("B,overlap", [(1, 1), (2, 1), (3, 1), (3, 0), (12, 1)])
def test_decode_smollm2_shapes(kb, oracle, torch_cuda, B, overlap):
    """SmolLM2-360M layer geometry (hidden 960, 15 query / 5 KV heads, head_dim 64, SwiGLU 2560,
    vocab 49152, RoPE theta 100000, 16-token blocks, permuted block tables), two layers, ragged
    contexts; B <= 8 takes the fused kernels, B = 12 the tensor-core GEMM. Logits within 1e-2 and
    the same greedy token as the oracle engine."""
    torch = torch_cuda
    ctx = kb.Context(0, torch.cuda.current_stream())
    ctx.set_option(kb.OPT_OVERLAP_WEIGHT_PREFETCH, overlap)
    L, hidden, H, KH, inter, vocab, bs = 2, 960, 15, 5, 2560, 49152, 16
    hd = hidden // H
    rng = np.random.Generator(np.random.PCG64(0xB2000D00 + B))
    ocfg = oracle.ModelConfig(hidden, H, KH, L, inter, vocab, bs, 1024, 1e-5, 100000.0)
    gcfg = kb.ModelConfig(hidden, H, KH, L, inter, vocab, bs, 1024, 1e-5, 100000.0)
    om, gm = oracle.Model(ocfg), kb.Model(ctx, gcfg)
    shapes = {0: (H * hd, hidden), 1: (KH * hd, hidden), 2: (KH * hd, hidden),
              3: (hidden, H * hd), 4: (inter, hidden), 5: (inter, hidden), 6: (hidden, inter)}
    for l in range(L):
        for which, (r, c) in shapes.items():
            blocks = oracle.quantize_weights_q8_0((rng.standard_normal((r, c)) * 0.02)
                                                 .astype(np.float32))
            assert om.set_weight(l, which, blocks, r, c) == 0
            gm.set_weight(l, which, blocks, kb.DTYPE_Q8_0, r, c)
        for which in (0, 1):
            nw = (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
            om.set_norm(l, which, nw)
            gm.set_norm(l, which, nw)
    emb = oracle.quantize_weights_q8_0((rng.standard_normal((vocab, hidden)) * 0.02)
                                       .astype(np.float32))
    om.set_weight(0, 7, emb, vocab, hidden)
    gm.set_weight(0, 7, emb, kb.DTYPE_Q8_0, vocab, hidden)
    fn = (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
    om.set_norm(0, 2, fn)
    gm.set_norm(0, 2, fn)

    lens = [int(x) for x in rng.integers(1, 400, size=B)]
    lens[0] = 1
    NB = sum((c + bs - 1) // bs for c in lens) + 4
    opool, gpool = oracle.KvPool(L, NB, bs, KH, hd), kb.KvPool(ctx, L, NB, bs, KH, hd)
    perm = [int(b) for b in rng.permutation(NB)]
    tables, used = [], 0
    for c in lens:
        need = (c + bs - 1) // bs
        tables.append(perm[used:used + need])
        used += need
    for l in range(L):
        hs, hk, hv = [], [], []
        for s, c in enumerate(lens):
            for t in range(c - 1):
                slot = tables[s][t // bs] * bs + t % bs
                k = rng.standard_normal(KH * hd).astype(np.float32)
                v = rng.standard_normal(KH * hd).astype(np.float32)
                opool.write_token(l, slot // bs, slot % bs, k, v)
                hs.append(slot)
                hk.append(k)
                hv.append(v)
        if hs:
            gpool.write_slots(l, torch.from_numpy(np.array(hs, np.int32)).cuda(),
                              torch.from_numpy(np.stack(hk)).cuda(),
                              torch.from_numpy(np.stack(hv)).cuda(), len(hs))
    st, maxb, padded = oracle.padded_decode_tables(bs, tables, lens)
    assert st == 0
    tokens = rng.integers(0, vocab, B).astype(np.uint32)
    positions = np.array([c - 1 for c in lens], np.uint32)
    slots = np.array([tables[s][(c - 1) // bs] * bs + (c - 1) % bs for s, c in enumerate(lens)],
                     np.uint32)
    st, ref = om.decode_step(opool, tokens, positions, slots, padded, lens, maxb)
    assert st == 0
    got = np.empty((B, vocab), np.float32)
    gm.decode_step(gpool, tokens, positions, slots, padded, np.array(lens, np.uint32), maxb, got)
    assert np.max(np.abs(got - ref)) <= 1e-2
    assert [int(np.argmax(r)) for r in got] == [oracle.greedy_token(r) for r in ref]
    # the K/V rows the step wrote are the bytes the CPU path stores
    for s in range(B):
        blk, off = int(slots[s]) // bs, int(slots[s]) % bs
        _, o = opool.read_token(L - 1, blk, off)
        gtok = gpool.read_token(L - 1, blk, off)
        # The layer's input differs from the CPU path's by the matmul tolerance (~1e-4 of the
        # scale), so a value that lies within that of a rounding boundary may land on the
        # other side: never by more than one step, and only for a small share of the bytes.
        dq = gtok["k_q"].astype(np.int32) - o["k_q"].astype(np.int32)
        assert np.max(np.abs(dq)) <= 1
        assert np.mean(dq != 0) <= 0.10
        assert np.allclose(gtok["k_scale"], o["k_scale"], rtol=1e-3)  # the matmul tolerance
    gm.destroy()
    gpool.destroy()
    ctx.close()
