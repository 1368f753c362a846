"""GPU: the allocation-free decode-attention entry point against the regular one.

kanso_cuda_paged_attention_noalloc is for callers that may not allocate device memory when
they call (an engine with a fixed, pre-planned memory budget; a loop that cannot afford the
device-wide synchronisation of cudaMalloc). It keeps the split-context partials in an array
built into the library instead of context scratch. Its results must equal those of
kanso_cuda_paged_attention, call after call, because the array is reused and keeps the
previous call's contents. This file sorts last on purpose: it runs after every other test,
and it must also pass alone in a fresh process.
"""
import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-3  # the tolerance of the paged-attention parity tests


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_case(rng, torch, kb, ctx, S, H, KH, hd, bs, lens):
    NB = sum((c + bs - 1) // bs for c in lens) + 2
    maxb = max((c + bs - 1) // bs for c in lens)
    perm = rng.permutation(NB)
    pool = kb.KvPool(ctx, 1, NB, bs, KH, hd)
    tables, slots, used = [], [], 0
    for s in range(S):
        need = (lens[s] + bs - 1) // bs
        blocks = [int(b) for b in perm[used:used + need]]
        used += need
        tables.append(blocks + [blocks[-1]] * (maxb - need))
        slots += [blocks[t // bs] * bs + t % bs for t in range(lens[s])]
    T = len(slots)
    k = rng.standard_normal((T, KH * hd)).astype(np.float32)
    v = rng.standard_normal((T, KH * hd)).astype(np.float32)
    slots = np.array(slots, np.uint32)
    pool.write_slots(0, dev(torch, slots), dev(torch, k), dev(torch, v), T, slots)
    q = rng.standard_normal((S, H * hd)).astype(np.float32)
    p = kb.PagedAttentionParams(S, H, KH, hd, bs, maxb, 1.0 / np.sqrt(np.float32(hd)))
    return pool, dev(torch, q), dev(torch, np.array(tables, np.uint32).reshape(-1)), p


def test_noalloc_matches_regular_entry_point_twice(ctx, kb, torch_cuda):
    torch = torch_cuda
    rng = np.random.Generator(np.random.PCG64(0xB2000700))
    # two different shapes back to back: the second call finds the first call's partials in
    # the shared array and must not be disturbed by them
    for S, H, KH, hd, bs, lens in [(2, 15, 5, 64, 16, [700, 93]), (3, 8, 2, 128, 16, [40, 300, 1])]:
        pool, q, tables, p = make_case(rng, torch, kb, ctx, S, H, KH, hd, bs, lens)
        lens_np = np.array(lens, np.uint32)
        lens_d = dev(torch, lens_np)
        ref = torch.full((S, H * hd), float("nan"), dtype=torch.float32, device="cuda")
        pool.paged_attention(0, q, tables, lens_d, ref, p, lens_np)
        ctx.sync()
        for _ in range(2):
            out = torch.full((S, H * hd), float("nan"), dtype=torch.float32, device="cuda")
            pool.paged_attention_noalloc(0, q, tables, lens_d, out, p, lens_np)
            ctx.sync()
            assert rel_err(out.cpu().numpy(), ref.cpu().numpy()) <= TOL
        pool.destroy()


def test_noalloc_rejects_what_does_not_fit(ctx, kb, torch_cuda):
    torch = torch_cuda
    # 64 sequences x 32 heads x 128 partitions x head_dim 256 of partials is far beyond 8 MiB
    pool = kb.KvPool(ctx, 1, 4, 16, 4, 256)
    S, H, maxb = 64, 32, 512
    p = kb.PagedAttentionParams(S, H, 4, 256, 16, maxb, 0.0625)
    q = torch.zeros((S, H * 256), device="cuda")
    out = torch.zeros_like(q)
    tables = torch.zeros(S * maxb, dtype=torch.int32, device="cuda")
    lens = torch.ones(S, dtype=torch.int32, device="cuda")
    with pytest.raises(kb.KansoError) as e:
        pool.paged_attention_noalloc(0, q, tables, lens, out, p)
    assert e.value.code == kb.ERR_UNSUPPORTED and "8388608" in e.value.message
    # the same argument checks as the regular entry point
    with pytest.raises(kb.KansoError) as e:
        pool.paged_attention_noalloc(0, q, tables, lens, out,
                                     kb.PagedAttentionParams(1, 4, 4, 256, 16, 4, 1.0),
                                     np.array([0], np.uint32))
    assert e.value.code == kb.ERR_UNSUPPORTED
    ctx.sync()
    pool.destroy()
