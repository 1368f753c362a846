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


def make_case(rng, torch, kb, oracle, ctx, S, H, KH, hd, bs, lens):
    NB = sum((c + bs - 1) // bs for c in lens) + 2
    maxb = max((c + bs - 1) // bs for c in lens)
    perm = rng.permutation(NB)
    pool, opool = kb.KvPool(ctx, 1, NB, bs, KH, hd), oracle.KvPool(1, NB, bs, KH, hd)
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
    assert opool.write_slots(0, slots, k, v) == 0
    q = rng.standard_normal((S, H * hd)).astype(np.float32)
    scale = 1.0 / np.sqrt(np.float32(hd))
    p = kb.PagedAttentionParams(S, H, KH, hd, bs, maxb, scale)
    tables = np.array(tables, np.uint32).reshape(-1)
    _, expect = oracle.paged_attention_int8(opool, 0, q, tables, np.array(lens, np.uint32),
                                            oracle.PaParams(S, H, KH, hd, bs, maxb, scale))
    return pool, dev(torch, q), dev(torch, tables), p, expect


def test_noalloc_matches_regular_entry_point_twice(ctx, kb, oracle, torch_cuda):
    torch = torch_cuda
    rng = np.random.Generator(np.random.PCG64(0xB2000700))
    # two different shapes back to back: the second call finds the first call's partials in
    # the shared array and must not be disturbed by them
    for S, H, KH, hd, bs, lens in [(2, 15, 5, 64, 16, [700, 93]), (3, 8, 2, 128, 16, [40, 300, 1])]:
        pool, q, tables, p, expect = make_case(rng, torch, kb, oracle, ctx, S, H, KH, hd, bs, lens)
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
            # and against the CPU oracle directly: the two-launch merge this entry point uses
            # is not the one the regular entry point takes for batches of this size
            assert rel_err(out.cpu().numpy(), expect) <= TOL
        pool.destroy()


def test_noalloc_allocates_nothing(kb, oracle, torch_cuda):
    """What the entry point is for: on a context that has never run attention (so its own scratch
    is still empty) a call on a larger batch than anything before it leaves the device's free
    memory where it was. The first call on a device looks up the array's address and may load
    the kernels, so one small call comes first."""
    torch = torch_cuda
    fresh = kb.Context(0, torch.cuda.current_stream())
    rng = np.random.Generator(np.random.PCG64(0xB2000701))
    small = make_case(rng, torch, kb, oracle, fresh, 1, 15, 5, 64, 16, [40])
    big = make_case(rng, torch, kb, oracle, fresh, 6, 15, 5, 64, 16, [900, 511, 64, 1300, 7, 350])
    outs = [torch.full((c[3].num_seqs, 15 * 64), float("nan"), dtype=torch.float32, device="cuda")
            for c in (small, big)]
    lens = [dev(torch, np.array(l, np.uint32)) for l in ([40], [900, 511, 64, 1300, 7, 350])]
    small[0].paged_attention_noalloc(0, small[1], small[2], lens[0], outs[0], small[3])
    fresh.sync()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(2):
        big[0].paged_attention_noalloc(0, big[1], big[2], lens[1], outs[1], big[3])
        fresh.sync()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert rel_err(outs[1].cpu().numpy(), big[4]) <= TOL
    assert torch.cuda.current_device() == 0  # the caller's current device is left alone
    small[0].destroy()
    big[0].destroy()
    fresh.close()


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
