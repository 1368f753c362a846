"""GPU: chunked-prefill attention (query_len > 1) over the int8 pool against the oracle's
restatement of Model::forward_prefill's attention (src/model.rs:1027-1085): the whole prefix
gathered from the pool, an offset causal mask of -1e9, softmax, P.V."""
import numpy as np
import pytest

from cases import dev, permuted_tables
from conftest import rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("H,KH,hd,bs,seqs", [
    (4, 2, 64, 16, [(0, 37)]),                        # first chunk of a prompt
    (15, 5, 64, 16, [(100, 50)]),                     # a later chunk: 100 tokens already cached
    (15, 5, 64, 16, [(30, 20), (199, 1), (0, 5)]),    # mixed batch: chunk, decode row, short prompt
    (8, 1, 128, 16, [(700, 64), (0, 130)]),           # several partitions per row, group 8
])
def test_prefill_attention_matches_oracle(ctx, kb, oracle, torch_cuda, H, KH, hd, bs, seqs):
    torch = torch_cuda
    rng = np.random.Generator(np.random.PCG64(0xB2000E00 + H * 131 + hd + len(seqs)))
    ctx_lens = [sp + ql for sp, ql in seqs]
    NB, tables = permuted_tables(rng, ctx_lens, bs)
    maxb = max(len(t) for t in tables)
    gp, op = kb.KvPool(ctx, 1, NB, bs, KH, hd), oracle.KvPool(1, NB, bs, KH, hd)
    padded = np.array([t + [t[-1]] * (maxb - len(t)) for t in tables], np.uint32)
    for s, c in enumerate(ctx_lens):  # the whole context, the chunk included, is in the pool
        t = np.arange(c)
        slots = (np.asarray(tables[s])[t // bs] * bs + t % bs).astype(np.uint32)
        k = rng.standard_normal((c, KH * hd), dtype=np.float32)
        v = rng.standard_normal((c, KH * hd), dtype=np.float32)
        gp.write_slots(0, dev(torch, slots), dev(torch, k), dev(torch, v), c, slots)
        assert op.write_slots(0, slots, k, v) == 0
    T = sum(ql for _, ql in seqs)
    q = rng.standard_normal((T, H * hd), dtype=np.float32)
    scale = np.float32(1.0) / np.sqrt(np.float32(hd))
    p = kb.PagedAttentionParams(len(seqs), H, KH, hd, bs, maxb, scale)
    out = torch.full((T, H * hd), float("nan"), dtype=torch.float32, device="cuda")
    gp.paged_attention_prefill(0, dev(torch, q), dev(torch, padded.reshape(-1)),
                               np.array(ctx_lens, np.uint32),
                               np.array([ql for _, ql in seqs], np.uint32), out, p)
    ctx.sync()
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    row = 0
    for s, (sp, ql) in enumerate(seqs):
        st, ref = oracle.prefill_attention_int8(op, 0, q[row:row + ql], tables[s], sp, H, scale)
        assert st == 0
        assert rel_err(got[row:row + ql], ref) <= 1e-3, (s, sp, ql)
        row += ql
    # a context shorter than its chunk, or longer than the table, is a shape error
    for bad_ctx in (seqs[0][1] - 1, maxb * bs + 1):
        with pytest.raises(kb.KansoError) as e:
            gp.paged_attention_prefill(0, dev(torch, q), dev(torch, padded.reshape(-1)),
                                       np.array([bad_ctx] + ctx_lens[1:], np.uint32),
                                       np.array([ql for _, ql in seqs], np.uint32), out, p)
        assert e.value.code == kb.ERR_SHAPE
    gp.destroy()


@pytest.mark.filterwarnings("ignore:The CUDA Graph is empty")  # that is the point: nothing enqueued
def test_prefill_attention_refuses_graph_capture(kb, oracle, torch_cuda):
    """The call builds its per-row arrays on the host for each call, so a captured graph would
    replay a copy from memory that is gone: while the stream is being captured it must enqueue
    nothing and say so."""
    torch = torch_cuda
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ctx = kb.Context(0, stream)
        H, KH, hd, bs = 4, 2, 64, 16
        gp = kb.KvPool(ctx, 1, 8, bs, KH, hd)
        q = torch.zeros((5, H * hd), device="cuda")
        out = torch.zeros_like(q)
        tab = torch.zeros(4, dtype=torch.int32, device="cuda")
        p = kb.PagedAttentionParams(1, H, KH, hd, bs, 4, 0.125)
        ctx.sync()
        seen = None
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            try:
                gp.paged_attention_prefill(0, q, tab, np.array([5], np.uint32),
                                           np.array([5], np.uint32), out, p)
            except kb.KansoError as e:
                seen = e.code
        assert seen == kb.ERR_UNSUPPORTED
        # outside a capture the same call works
        gp.paged_attention_prefill(0, q, tab, np.array([5], np.uint32), np.array([5], np.uint32),
                                   out, p)
        ctx.sync()
        gp.destroy()
        ctx.close()
