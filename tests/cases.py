"""Seeded case builders shared by the GPU parity tests (and by nothing in the product)."""
import numpy as np

SMOLLM2 = dict(hidden=960, H=15, KH=5, inter=2560, vocab=49152, bs=16, eps=1e-5, theta=100000.0)


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def permuted_tables(rng, lens, bs, spare=4):
    """Per-sequence block tables drawn from one random permutation of the physical blocks."""
    NB = sum((c + bs - 1) // bs for c in lens) + spare
    perm = [int(b) for b in rng.permutation(NB)]
    tables, used = [], 0
    for c in lens:
        need = (c + bs - 1) // bs
        tables.append(perm[used:used + need])
        used += need
    return NB, tables


def history_slots(tables, lens, bs, upto_last=True):
    """Pool slots of every stored token: all but the newest token of each sequence when
    upto_last (the decode step writes that one itself), else all of them."""
    out = []
    for s, c in enumerate(lens):
        n = c - 1 if upto_last else c
        t = np.arange(n)
        out.append(np.asarray(tables[s], np.int64)[t // bs] * bs + t % bs)
    return np.concatenate(out).astype(np.uint32) if out else np.zeros(0, np.uint32)


def fill_history(torch, rng, gpool, opool, layers, slots, width):
    """Writes seeded N(0,1) K/V rows into both pools, layer by layer, in bulk."""
    if slots.size == 0:
        return
    sd = dev(torch, slots)
    for l in range(layers):
        k = rng.standard_normal((slots.size, width), dtype=np.float32)
        v = rng.standard_normal((slots.size, width), dtype=np.float32)
        assert opool.write_slots(l, slots, k, v) == 0
        gpool.write_slots(l, sd, dev(torch, k), dev(torch, v), slots.size)


def smollm2_models(kb, oracle, ctx, rng, layers, max_seq_len=4096):
    """The SmolLM2-360M layer geometry with `layers` layers: Q8_0 projections from N(0, 0.02),
    norm weights 1 + 0.1 N(0,1), tied lm_head. Returns (oracle model, gpu model)."""
    g = SMOLLM2
    hidden, H, KH, inter, vocab, bs = g["hidden"], g["H"], g["KH"], g["inter"], g["vocab"], g["bs"]
    hd = hidden // H
    ocfg = oracle.ModelConfig(hidden, H, KH, layers, inter, vocab, bs, max_seq_len, g["eps"],
                              g["theta"])
    gcfg = kb.ModelConfig(hidden, H, KH, layers, inter, vocab, bs, max_seq_len, g["eps"],
                          g["theta"])
    om, gm = oracle.Model(ocfg), kb.Model(ctx, gcfg)
    shapes = {0: (H * hd, hidden), 1: (KH * hd, hidden), 2: (KH * hd, hidden),
              3: (hidden, H * hd), 4: (inter, hidden), 5: (inter, hidden), 6: (hidden, inter)}
    for l in range(layers):
        for which, (r, c) in shapes.items():
            blocks = oracle.quantize_weights_q8_0(
                (rng.standard_normal((r, c), dtype=np.float32) * np.float32(0.02)))
            assert om.set_weight(l, which, blocks, r, c) == 0
            gm.set_weight(l, which, blocks, kb.DTYPE_Q8_0, r, c)
        for which in (0, 1):
            nw = (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
            om.set_norm(l, which, nw)
            gm.set_norm(l, which, nw)
    emb = oracle.quantize_weights_q8_0(
        (rng.standard_normal((vocab, hidden), dtype=np.float32) * np.float32(0.02)))
    om.set_weight(0, 7, emb, vocab, hidden)
    gm.set_weight(0, 7, emb, kb.DTYPE_Q8_0, vocab, hidden)
    fn = (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
    om.set_norm(0, 2, fn)
    gm.set_norm(0, 2, fn)
    return om, gm
