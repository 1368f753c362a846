"""GPU: the fp8 (E4M3, power-of-two scale) KV pool against the oracle's QuantMode::Fp8
(src/kv_cache/quantized_storage.rs:109-131,440-449,470-484): quantiser and read-back bit for
bit, decode / prefill / allocation-free attention within 1e-3, one decode step of a small model."""
import numpy as np
import pytest

from cases import dev, permuted_tables, history_slots
from conftest import rel_err

pytestmark = pytest.mark.gpu


def pools(kb, oracle, ctx, L, NB, bs, KH, hd):
    return kb.KvPool(ctx, L, NB, bs, KH, hd, kb.KV_FP8), oracle.KvPool(L, NB, bs, KH, hd, fp8=True)


def test_fp8_reference_vector_and_bit_exact_quantiser(ctx, kb, oracle, torch_cuda):
    """The reference's own fp8 case (tests/test_quantized_kv_cache.rs:88-166): values that E4M3
    holds exactly come back with zero error (its bound is 1 %); then seeded normal rows over six
    decades of magnitude, bytes, scales and dequantised values equal to the oracle's bit for bit."""
    torch = torch_cuda
    L, NB, bs, KH, hd = 2, 4, 4, 4, 64
    gp, op = pools(kb, oracle, ctx, L, NB, bs, KH, hd)
    n = KH * hd
    k = np.array([((i % 16) * 0.5 - 3.5) or 1.0 for i in range(n)], np.float32)
    v = np.array([(i % 8) + 0.5 for i in range(n)], np.float32)
    slot = np.array([0], np.uint32)
    gp.write_slots(0, dev(torch, slot), dev(torch, k[None]), dev(torch, v[None]), 1, slot)
    ctx.sync()
    got = gp.read_token(0, 0, 0)
    assert np.array_equal(got["k_deq"], k) and np.array_equal(got["v_deq"], v)
    assert np.all(got["k_scale"] == np.float32(2.0 ** -4)) and np.all(got["v_scale"] == 0.125)

    rng = np.random.Generator(np.random.PCG64(0xB200F8))
    T = NB * bs
    mags = (10.0 ** rng.uniform(-3, 3, size=(T, KH, 1))).astype(np.float32)
    kk = (rng.standard_normal((T, KH, hd), dtype=np.float32) * mags).reshape(T, n)
    vv = (rng.standard_normal((T, KH, hd), dtype=np.float32) * mags[::-1]).reshape(T, n)
    kk[3] = 0.0  # an all-zero slice keeps scale 1.0
    slots = rng.permutation(T).astype(np.uint32)
    gp.write_slots(1, dev(torch, slots), dev(torch, kk), dev(torch, vv), T, slots)
    assert op.write_slots(1, slots, kk, vv) == 0
    ctx.sync()
    for t in range(T):
        b, o = int(slots[t]) // bs, int(slots[t]) % bs
        got = gp.read_token(1, b, o)
        st, ref = op.read_token(1, b, o)
        assert st == 0
        for key in ("k_q", "v_q", "k_scale", "v_scale", "k_deq", "v_deq"):
            assert got[key].tobytes() == ref[key].tobytes(), (t, key)
    assert gp.bytes_per_token == 2 * KH * hd + 8 * KH
    gp.reset_block(int(slots[0]) // bs)
    ctx.sync()
    erased = gp.read_token(1, int(slots[0]) // bs, 0)
    assert not erased["k_q"].any() and np.all(erased["k_scale"] == 1.0)
    gp.destroy()


def fill(torch, rng, gp, op, layer, tables, lens, bs, width):
    slots = history_slots(tables, lens, bs, upto_last=False)
    k = rng.standard_normal((slots.size, width), dtype=np.float32)
    v = rng.standard_normal((slots.size, width), dtype=np.float32)
    gp.write_slots(layer, dev(torch, slots), dev(torch, k), dev(torch, v), slots.size)
    assert op.write_slots(layer, slots, k, v) == 0


def padded(tables, maxb):
    return np.array([t + [t[-1]] * (maxb - len(t)) for t in tables], np.uint32).reshape(-1)


@pytest.mark.parametrize("H,KH,hd,bs,lens", [
    (4, 4, 64, 16, [35]),
    (15, 5, 64, 16, [600, 17]),        # SmolLM2 heads, several partitions merged
    (8, 1, 128, 16, [100]),            # group 8, head_dim 128
    (5, 1, 256, 16, [70]),
    (2, 2, 16, 4, [1, 2, 3, 9]),
    (15, 5, 64, 16, [4096, 3000]),
])
def test_fp8_paged_attention_matches_oracle(ctx, kb, oracle, torch_cuda, H, KH, hd, bs, lens):
    torch = torch_cuda
    S = len(lens)
    rng = np.random.Generator(np.random.PCG64(0xB200F801 + H * 7 + hd + sum(lens)))
    NB, tables = permuted_tables(rng, lens, bs)
    gp, op = pools(kb, oracle, ctx, 2, NB, bs, KH, hd)
    fill(torch, rng, gp, op, 1, tables, lens, bs, KH * hd)
    maxb = max(len(t) for t in tables)
    tab = padded(tables, maxb)
    q = rng.standard_normal((S, H * hd), dtype=np.float32)
    lens_np = np.array(lens, np.uint32)
    p = kb.PagedAttentionParams(S, H, KH, hd, bs, maxb, 1.0 / np.sqrt(np.float32(hd)))
    st, ref = oracle.paged_attention_int8(op, 1, q, tab, lens_np,
                                          oracle.PaParams(S, H, KH, hd, bs, maxb, p.scale))
    assert st == 0
    out = torch.full((S, H * hd), float("nan"), dtype=torch.float32, device="cuda")
    gp.paged_attention(1, dev(torch, q), dev(torch, tab), dev(torch, lens_np), out, p, lens_np)
    ctx.sync()
    assert rel_err(out.cpu().numpy(), ref) <= 1e-3
    # the allocation-free entry point takes the same pool
    out2 = torch.full((S, H * hd), float("nan"), dtype=torch.float32, device="cuda")
    gp.paged_attention_noalloc(1, dev(torch, q), dev(torch, tab), dev(torch, lens_np), out2, p,
                               lens_np)
    ctx.sync()
    assert rel_err(out2.cpu().numpy(), ref) <= 1e-3
    gp.destroy()


def test_fp8_prefill_attention_matches_oracle(ctx, kb, oracle, torch_cuda):
    torch = torch_cuda
    H, KH, hd, bs = 6, 2, 64, 16
    ctx_lens, q_lens = [70, 33], [5, 33]  # a chunk on top of 65 cached tokens, and a whole prompt
    rng = np.random.Generator(np.random.PCG64(0xB200F802))
    NB, tables = permuted_tables(rng, ctx_lens, bs)
    gp, op = pools(kb, oracle, ctx, 1, NB, bs, KH, hd)
    fill(torch, rng, gp, op, 0, tables, ctx_lens, bs, KH * hd)
    maxb = max(len(t) for t in tables)
    T = sum(q_lens)
    q = rng.standard_normal((T, H * hd), dtype=np.float32)
    scale = 1.0 / np.sqrt(np.float32(hd))
    refs, r0 = [], 0
    for s in range(2):
        st, r = oracle.prefill_attention_int8(op, 0, q[r0:r0 + q_lens[s]], tables[s],
                                              ctx_lens[s] - q_lens[s], H, scale)
        assert st == 0
        refs.append(r)
        r0 += q_lens[s]
    ref = np.concatenate(refs)
    p = kb.PagedAttentionParams(2, H, KH, hd, bs, maxb, scale)
    out = torch.full((T, H * hd), float("nan"), dtype=torch.float32, device="cuda")
    gp.paged_attention_prefill(0, dev(torch, q), dev(torch, padded(tables, maxb)),
                               np.array(ctx_lens, np.uint32), np.array(q_lens, np.uint32), out, p)
    ctx.sync()
    assert rel_err(out.cpu().numpy(), ref.reshape(T, H * hd)) <= 1e-3
    gp.destroy()


@pytest.mark.parametrize("B", [3, 12])
def test_fp8_decode_step_matches_oracle(kb, oracle, torch_cuda, B):
    """One decode step of the SmolLM2-360M layer geometry (two layers) over an fp8 pool: the
    step's own K/V rows are rotated, quantised to E4M3 and stored inside the attention kernel;
    logits within 1e-2 of the oracle engine on its fp8 pool, same greedy token, and the new
    token's pool bytes equal to the oracle's."""
    from cases import fill_history, smollm2_models
    torch = torch_cuda
    ctx = kb.Context(0, torch.cuda.current_stream())
    ctx.set_option(kb.OPT_OVERLAP_WEIGHT_PREFETCH, 1)
    L, bs, KH, hd, vocab = 2, 16, 5, 64, 49152
    rng = np.random.Generator(np.random.PCG64(0xB200F810 + B))
    om, gm = smollm2_models(kb, oracle, ctx, rng, L, max_seq_len=1024)
    lens = [int(c) for c in rng.integers(20, 700, size=B)]
    NB, tables = permuted_tables(rng, lens, bs)
    gpool, opool = pools(kb, oracle, ctx, L, NB, bs, KH, hd)
    fill_history(torch, rng, gpool, opool, L, history_slots(tables, lens, bs), KH * hd)
    st, maxb, padded_t = oracle.padded_decode_tables(bs, tables, lens)
    assert st == 0
    tokens = rng.integers(0, vocab, B).astype(np.uint32)
    positions = np.array([c - 1 for c in lens], np.uint32)
    slots = np.array([tables[s][(c - 1) // bs] * bs + (c - 1) % bs for s, c in enumerate(lens)],
                     np.uint32)
    st, ref = om.decode_step(opool, tokens, positions, slots, padded_t, lens, maxb)
    assert st == 0
    got = np.empty((B, vocab), np.float32)
    gm.decode_step(gpool, tokens, positions, slots, padded_t, np.array(lens, np.uint32), maxb, got)
    assert np.isfinite(got).all()
    assert float(np.max(np.abs(got - ref))) <= 1e-2
    assert [int(np.argmax(r)) for r in got] == [oracle.greedy_token(r) for r in ref]
    # layer 0's new rows depend only on the embedding and the first projections: same bytes
    for s in range(B):
        b, o = int(slots[s]) // bs, int(slots[s]) % bs
        g0 = gpool.read_token(0, b, o)
        _, r0 = opool.read_token(0, b, o)
        same = np.mean(g0["k_q"] == r0["k_q"])
        assert same >= 0.99 and np.array_equal(g0["k_scale"], r0["k_scale"]), (s, same)
    gm.destroy()
    gpool.destroy()
    ctx.close()
