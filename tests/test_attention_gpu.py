"""GPU: int8 KV pool and paged decode attention against the oracle."""
import numpy as np
import pytest

from conftest import golden, rel_err

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def fill_pools(kb, ctx, oracle, torch, L, NB, bs, KH, hd, writes, layer=0):
    """writes: list of (slot, k[KH*hd], v[KH*hd]). Returns (gpu pool, oracle pool)."""
    gp = kb.KvPool(ctx, L, NB, bs, KH, hd)
    op = oracle.KvPool(L, NB, bs, KH, hd)
    slots = np.array([w[0] for w in writes], np.uint32)
    k = np.stack([w[1] for w in writes]).astype(np.float32)
    v = np.stack([w[2] for w in writes]).astype(np.float32)
    gp.write_slots(layer, dev(torch, slots), dev(torch, k), dev(torch, v), len(writes), slots)
    for s, kk, vv in writes:
        assert op.write_token(layer, int(s) // bs, int(s) % bs, kk, vv) == 0
    ctx.sync()
    return gp, op


def test_kv_write_read_bit_exact(ctx, kb, oracle, torch_cuda):
    g = golden("kv_int8.npz")
    L, NB, bs, H, hd = (int(v) for v in g["geom"])
    writes = [([2, 0][t // bs] * bs + t % bs, g["k"][t], g["v"][t]) for t in range(6)]
    gp, op = fill_pools(kb, ctx, oracle, torch_cuda, L, NB, bs, H, hd, writes, layer=1)
    for t in range(6):
        got = gp.read_token(1, [2, 0][t // bs], t % bs)
        assert np.array_equal(got["k_q"], g["k_q"][t]) and np.array_equal(got["v_q"], g["v_q"][t])
        assert got["k_scale"].tobytes() == g["k_scale"][t].tobytes()
        assert got["v_scale"].tobytes() == g["v_scale"][t].tobytes()
        _, ref = op.read_token(1, [2, 0][t // bs], t % bs)
        assert got["k_deq"].tobytes() == ref["k_deq"].tobytes()
    # untouched rows: quants 0, scales 1.0; reset erases every layer
    fresh = gp.read_token(0, 3, 1)
    assert not fresh["k_q"].any() and np.all(fresh["v_scale"] == 1.0)
    gp.reset_block(2)
    ctx.sync()
    erased = gp.read_token(1, 2, 0)
    assert not erased["k_q"].any() and np.all(erased["k_scale"] == 1.0)
    assert gp.bytes_per_token == 2 * H * hd + 8 * H
    # bounds errors (quantized_storage.rs:151-181)
    for args in [(L, 0, 0), (0, NB, 0), (0, 0, bs)]:
        with pytest.raises(kb.KansoError) as e:
            gp.read_token(*args)
        assert e.value.code == kb.ERR_SHAPE
    with pytest.raises(kb.KansoError) as e:
        bad = np.array([NB * bs], np.uint32)
        z = torch_cuda.zeros(H * hd, device="cuda")
        gp.write_slots(0, dev(torch_cuda, bad), z, z, 1, bad)
    assert e.value.code == kb.ERR_SHAPE


def test_kv_type_flag(ctx, kb):
    with pytest.raises(kb.KansoError) as e:
        kb.KvPool(ctx, 1, 4, 16, 5, 64, kb.KV_F32)
    assert e.value.code == kb.ERR_UNSUPPORTED
    kb.KvPool(ctx, 1, 4, 16, 5, 64, kb.KV_FP8).destroy()
    with pytest.raises(kb.KansoError) as e:
        kb.KvPool(ctx, 1, 4, 16, 5, 64, 9)
    assert e.value.code == kb.ERR_CONFIG


def random_case(rng, S, H, KH, hd, bs, lens, NB):
    maxb = max((c + bs - 1) // bs for c in lens)
    perm = rng.permutation(NB)
    tables, writes, used = [], [], 0
    for s in range(S):
        need = (lens[s] + bs - 1) // bs
        blocks = [int(b) for b in perm[used:used + need]]
        used += need
        tables.append(blocks + [blocks[-1]] * (maxb - need))  # PaddedDecodeTables rule
        for t in range(lens[s]):
            writes.append((blocks[t // bs] * bs + t % bs, rng.standard_normal(KH * hd),
                           rng.standard_normal(KH * hd)))
    q = rng.standard_normal((S, H * hd)).astype(np.float32)
    return maxb, np.array(tables, np.uint32).reshape(-1), writes, q


@pytest.mark.parametrize("S,H,KH,hd,bs,lens", [
    (1, 4, 4, 64, 16, [35]),              # non-contiguous table, 3 blocks
    (1, 8, 2, 64, 16, [50]),              # GQA 8:2
    (3, 4, 2, 32, 8, [5, 17, 32]),        # ragged batch
    (1, 15, 5, 64, 16, [600]),            # several partitions merged
    (2, 15, 5, 64, 16, [2048, 257]),      # long context
    (1, 8, 1, 128, 16, [100]),            # group 8, head_dim 128
    (1, 5, 1, 256, 16, [70]),             # group 5, head_dim 256
    (4, 2, 2, 16, 4, [1, 2, 3, 9]),       # tiny heads, context 1
    (2, 15, 5, 64, 16, [4096, 3000]),     # the longest context of the decode benchmark
])
def test_paged_attention_matches_oracle(ctx, kb, oracle, torch_cuda, S, H, KH, hd, bs, lens):
    torch = torch_cuda
    rng = np.random.Generator(np.random.PCG64(hash((S, H, KH, hd, bs, tuple(lens))) & 0xFFFFFFFF))
    NB = sum((c + bs - 1) // bs for c in lens) + 3
    maxb, tables, writes, q = random_case(rng, S, H, KH, hd, bs, lens, NB)
    gp, op = fill_pools(kb, ctx, oracle, torch, 2, NB, bs, KH, hd, writes, layer=1)
    p = kb.PagedAttentionParams(S, H, KH, hd, bs, maxb, 1.0 / np.sqrt(np.float32(hd)))
    out = torch.full((S, H * hd), float("nan"), dtype=torch.float32, device="cuda")
    lens_np = np.array(lens, np.uint32)
    gp.paged_attention(1, dev(torch, q), dev(torch, tables), dev(torch, lens_np), out, p, lens_np)
    ctx.sync()
    st, ref = oracle.paged_attention_int8(op, 1, q, tables, lens_np,
                                          oracle.PaParams(S, H, KH, hd, bs, maxb, p.scale))
    assert st == 0
    assert rel_err(out.cpu().numpy(), ref) <= 1e-3


def test_paged_attention_errors(ctx, kb, torch_cuda):
    torch = torch_cuda
    gp = kb.KvPool(ctx, 1, 8, 16, 2, 64)
    q = torch.zeros((1, 4 * 64), device="cuda")
    out = torch.zeros_like(q)
    tab = torch.zeros(4, dtype=torch.int32, device="cuda")
    lens = torch.ones(1, dtype=torch.int32, device="cuda")
    ok = kb.PagedAttentionParams(1, 4, 2, 64, 16, 4, 0.125)
    # ctx 0 and ctx > capacity are rejected on the host (src/metal/paged_attention.rs:343-355)
    for bad_len in (0, 65):
        with pytest.raises(kb.KansoError) as e:
            gp.paged_attention(0, q, tab, lens, out, ok, np.array([bad_len], np.uint32))
        assert e.value.code == kb.ERR_UNSUPPORTED
    with pytest.raises(kb.KansoError) as e:  # group 9
        gp.paged_attention(0, q, tab, lens, out, kb.PagedAttentionParams(1, 18, 2, 64, 16, 4, 1.0))
    assert e.value.code == kb.ERR_UNSUPPORTED
    with pytest.raises(kb.KansoError) as e:  # pool mismatch
        gp.paged_attention(0, q, tab, lens, out, kb.PagedAttentionParams(1, 4, 2, 128, 16, 4, 1.0))
    assert e.value.code == kb.ERR_SHAPE
    # an out-of-range block id is caught on the device and reported at sync, without a fault
    bad_tab = torch.full((4,), 99, dtype=torch.int32, device="cuda")
    gp.paged_attention(0, q, bad_tab, lens, out, ok)
    with pytest.raises(kb.KansoError) as e:
        ctx.sync()
    assert e.value.code == kb.ERR_SHAPE
    ctx.sync()  # the status word is cleared once reported


@pytest.mark.parametrize("hd", [64, 128, 256])
@pytest.mark.parametrize("group", [1, 4, 5, 8])
def test_paged_attention_reference_parity_matrix(ctx, kb, oracle, torch_cuda, hd, group):
    """The reference's parity matrix, head_dim {64, 128, 256} x GQA group {1, 4, 5, 8}, with its
    closed-form inputs and its non-contiguous table (tests/test_paged_attention_v2.rs:326-401).
    The reference runs it over an f32 cache; here every cache row goes through the int8 pool's
    quantiser on both sides, and the oracle's attention over that pool is the expected value."""
    torch = torch_cuda
    S, KH, bs, maxb, NB = 2, 2, 16, 4, 10
    H = KH * group
    lens = np.array([37, 16], np.uint32)
    q = ((np.arange(S * H * hd) % 17).astype(np.float32) - 8.0) * np.float32(0.125)
    n = NB * bs * KH * hd
    kc = ((np.arange(n) % 19).astype(np.float32) - 9.0) * np.float32(0.1)
    vc = ((np.arange(n) % 23).astype(np.float32) - 11.0) * np.float32(0.15)
    tables = np.array([5, 2, 7, 0, 3, 9, 1, 6], np.uint32)
    slots = np.arange(NB * bs, dtype=np.uint32)
    gp, op = kb.KvPool(ctx, 1, NB, bs, KH, hd), oracle.KvPool(1, NB, bs, KH, hd)
    k2, v2 = kc.reshape(NB * bs, KH * hd), vc.reshape(NB * bs, KH * hd)
    gp.write_slots(0, dev(torch, slots), dev(torch, k2), dev(torch, v2), slots.size, slots)
    assert op.write_slots(0, slots, k2, v2) == 0
    scale = np.float32(1.0) / np.sqrt(np.float32(hd))
    p = kb.PagedAttentionParams(S, H, KH, hd, bs, maxb, scale)
    out = torch.full((S, H * hd), float("nan"), dtype=torch.float32, device="cuda")
    gp.paged_attention(0, dev(torch, q.reshape(S, H * hd)), dev(torch, tables), dev(torch, lens),
                       out, p, lens)
    ctx.sync()
    st, ref = oracle.paged_attention_int8(op, 0, q, tables, lens,
                                          oracle.PaParams(S, H, KH, hd, bs, maxb, scale))
    assert st == 0
    assert rel_err(out.cpu().numpy(), ref) <= 1e-3
    # against the reference's own f32-cache expectation the int8 pool costs about a percent
    f32 = oracle.paged_attention_f32(q, kc, vc, tables, lens,
                                     oracle.PaParams(S, H, KH, hd, bs, maxb, scale))
    assert rel_err(out.cpu().numpy().reshape(-1), f32) <= 3e-2
    gp.destroy()


def test_paged_attention_flat_context_2048(ctx, kb, oracle, torch_cuda):
    """The reference's 2048-token case (tests/test_paged_attention_v2.rs:559-633): constant q,
    K and V, identity table; the output is finite, positive and equals V's constant."""
    torch = torch_cuda
    S, H, KH, hd, bs, ctx_len = 1, 4, 4, 64, 16, 2048
    maxb = ctx_len // bs
    NB = maxb + 4
    slots = np.arange(ctx_len, dtype=np.uint32)
    k = np.full((ctx_len, KH * hd), 0.05, np.float32)
    v = np.full((ctx_len, KH * hd), 0.02, np.float32)
    gp = kb.KvPool(ctx, 1, NB, bs, KH, hd)
    gp.write_slots(0, dev(torch, slots), dev(torch, k), dev(torch, v), ctx_len, slots)
    q = np.full((S, H * hd), 0.1, np.float32)
    lens = np.array([ctx_len], np.uint32)
    p = kb.PagedAttentionParams(S, H, KH, hd, bs, maxb, 0.125)
    out = torch.full((S, H * hd), float("nan"), dtype=torch.float32, device="cuda")
    gp.paged_attention(0, dev(torch, q), dev(torch, np.arange(maxb, dtype=np.uint32)),
                       dev(torch, lens), out, p, lens)
    ctx.sync()
    got = out.cpu().numpy()
    assert np.isfinite(got).all() and (got > 0).all()
    assert np.max(np.abs(got - 0.02)) <= 2e-5
    gp.destroy()


@pytest.mark.parametrize("entry", ["paged_attention", "paged_attention_noalloc"])
def test_device_length_beyond_the_launch_is_cut_off_and_reported(ctx, kb, oracle, torch_cuda,
                                                                 entry):
    """A device-side context length larger than what the launch was sized for (the host's hint,
    or the table's capacity when no hint is given) never reaches memory outside the launch's
    own partials or table rows: both kernels cut it off at the same place, the result is the
    attention over the tokens that remain, and the status word turns the next sync into a shape
    error. The reference rejects such a length on the host (src/metal/paged_attention.rs:343-355)
    and its kernel clamps the partition range (paged_attention_v2.metal:86-87)."""
    torch = torch_cuda
    S, H, KH, hd, bs = 1, 15, 5, 64, 16
    rng = np.random.Generator(np.random.PCG64(0xB2000500))
    stored = 704
    NB = stored // bs + 3
    maxb, tables, writes, q = random_case(rng, S, H, KH, hd, bs, [stored], NB)
    gp, op = fill_pools(kb, ctx, oracle, torch, 1, NB, bs, KH, hd, writes)
    p = kb.PagedAttentionParams(S, H, KH, hd, bs, maxb, 0.125)
    call = getattr(gp, entry)
    # (a) the host says 100 tokens, the device array says 700: the grid covers 128
    out = torch.full((S, H * hd), float("nan"), dtype=torch.float32, device="cuda")
    call(0, dev(torch, q), dev(torch, tables), dev(torch, np.array([700], np.uint32)), out, p,
         np.array([100], np.uint32))
    with pytest.raises(kb.KansoError) as e:
        ctx.sync()
    assert e.value.code == kb.ERR_SHAPE
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    cut = [c for c in (64, 128, 192, 256, 512) if c >= 100]
    refs = [oracle.paged_attention_int8(op, 0, q, tables, np.array([c], np.uint32),
                                        oracle.PaParams(S, H, KH, hd, bs, maxb, 0.125))[1]
            for c in cut]
    assert min(rel_err(got, r) for r in refs) <= 1e-3  # cut off at a whole partition
    # (b) no host lengths, device length beyond the table's capacity: cut off at the capacity
    out = torch.full((S, H * hd), float("nan"), dtype=torch.float32, device="cuda")
    call(0, dev(torch, q), dev(torch, tables), dev(torch, np.array([maxb * bs + 40], np.uint32)),
         out, p)
    with pytest.raises(kb.KansoError) as e:
        ctx.sync()
    assert e.value.code == kb.ERR_SHAPE
    _, ref = oracle.paged_attention_int8(op, 0, q, tables, np.array([maxb * bs], np.uint32),
                                         oracle.PaParams(S, H, KH, hd, bs, maxb, 0.125))
    assert rel_err(out.cpu().numpy(), ref) <= 1e-3
    ctx.sync()  # reported once, then clear
    gp.destroy()
