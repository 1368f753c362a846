"""GPU: streaming GEMV / few-row GEMM against the oracle.

Tolerance: max|y_gpu - y_ref| / max|y_ref| <= 1e-3, the scale-relative form of
the reference's own comparisons (tests/test_quantized_weights.rs:375-397).
"""
import numpy as np
import pytest

from conftest import golden, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-3


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_gemm(ctx, kb, torch, dtype, blocks, x, M, N, K, act=0):
    y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    wb = dev(torch, blocks)
    xd = dev(torch, x.astype(np.float32))
    if dtype == kb.DTYPE_Q8_0:
        if M == 1 and act == 0:
            ctx.gemv_q8_0(wb, xd, y, N, K)
        else:
            ctx.gemm_q8_0(wb, xd, y, M, N, K, act)
    else:
        if M == 1:
            ctx.gemv_q4_k(wb, xd, y, N, K)
        else:
            ctx.gemm_q4_k(wb, xd, y, M, N, K, act)
    ctx.sync()
    return y.cpu().numpy()


def gguf_q8_from_ref(d, qs):
    """Reference-layout blocks (f32 d) -> GGUF bytes (d rounded to f16)."""
    n = d.size
    out = np.zeros((n, 34), np.uint8)
    out[:, :2] = d.astype(np.float16).reshape(-1, 1).view(np.uint8)
    out[:, 2:] = qs.reshape(n, 32).view(np.uint8)
    return out.reshape(-1)


def test_golden_blocks(ctx, kb, oracle, torch_cuda):
    g = golden("gguf_blocks.npz")
    y8 = run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q8_0, g["q8_0"], g["x"][None], 1, 12, 512)
    assert rel_err(y8[0], g["gemv_q8_0"]) <= TOL
    y8q = run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q8_0, g["q8_0"], g["x"][None], 1, 12, 512,
                   kb.ACT_Q8)
    assert rel_err(y8q[0], g["gemv_q8_0_q8"]) <= 1e-5  # same int32 sums, f32 order differs
    y4 = run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q4_K, g["q4_k"], g["x"][None], 1, 12, 512)
    assert rel_err(y4[0], g["gemv_q4_k"]) <= TOL


def test_reference_gemv_patterns(ctx, kb, oracle, torch_cuda):
    # tests/test_neon_simd_gemv.rs:104-143 (Q8_0 64x128) in the f16-scale layout
    g = golden("q8_0_kat.npz")
    blocks = gguf_q8_from_ref(g["gemv_d"].reshape(-1), g["gemv_qs"])
    ref = oracle.gemv_q8_0(blocks, g["gemv_x"], 64, 128)
    got = run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q8_0, blocks, g["gemv_x"][None], 1, 64, 128)
    assert rel_err(got[0], ref) <= TOL
    # tests/test_neon_simd_gemv.rs:146-188 (Q4_K 32x256)
    k = golden("q4_k_kat.npz")
    blk = np.zeros((32, 144), np.uint8)
    blk[:, 0:2] = k["gemv_d"].astype(np.float16).reshape(-1, 1).view(np.uint8)
    blk[:, 2:4] = np.frombuffer(np.float16(k["gemv_dmin"]).tobytes(), np.uint8)
    blk[:, 4:16] = k["gemv_scales"]
    blk[:, 16:] = k["gemv_qs"]
    ref = oracle.gemv_q4_k(blk.reshape(-1), k["gemv_x"], 32, 256)
    got = run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q4_K, blk.reshape(-1), k["gemv_x"][None], 1, 32,
                   256)
    assert rel_err(got[0], ref) <= TOL


@pytest.mark.parametrize("rows,cols", [(2560, 960), (960, 2560), (1, 32), (3, 64), (149, 992),
                                       (300, 4096), (17, 8192), (64, 1056)])
def test_q8_0_gemv_shapes(ctx, kb, oracle, torch_cuda, rows, cols):
    rng = np.random.Generator(np.random.PCG64(0xB2000100 + rows * 31 + cols))
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    x = rng.standard_normal(cols).astype(np.float32)
    blocks = oracle.quantize_weights_q8_0(w)
    ref = oracle.gemv_q8_0(blocks, x, rows, cols)
    got = run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q8_0, blocks, x[None], 1, rows, cols)
    assert rel_err(got[0], ref) <= TOL
    refq = oracle.gemv_q8_0_q8(blocks, x, rows, cols)
    gotq = run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q8_0, blocks, x[None], 1, rows, cols, kb.ACT_Q8)
    assert rel_err(gotq[0], refq) <= 1e-5


@pytest.mark.parametrize("rows,cols", [(14336, 4096), (4096, 14336), (1, 256), (5, 512),
                                       (149, 768), (33, 8192), (9, 28672), (200, 2048)])
def test_q4_k_gemv_shapes(ctx, kb, oracle, torch_cuda, rows, cols):
    rng = np.random.Generator(np.random.PCG64(0xB2000200 + rows * 31 + cols))
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    x = rng.standard_normal(cols).astype(np.float32)
    blocks = oracle.quantize_weights_q4_k(w)
    ref = oracle.gemv_q4_k(blocks, x, rows, cols)
    got = run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q4_K, blocks, x[None], 1, rows, cols)
    assert rel_err(got[0], ref) <= TOL


@pytest.mark.parametrize("M", [2, 3, 4, 7, 8, 13])
def test_few_row_gemm(ctx, kb, oracle, torch_cuda, M):
    rng = np.random.Generator(np.random.PCG64(0xB2000300 + M))
    N, K = 320, 1024
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    b8, b4 = oracle.quantize_weights_q8_0(w), oracle.quantize_weights_q4_k(w)
    assert rel_err(run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q8_0, b8, x, M, N, K),
                   oracle.gemm_q8_0(b8, x, M, N, K)) <= TOL
    assert rel_err(run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q8_0, b8, x, M, N, K, kb.ACT_Q8),
                   oracle.gemm_q8_0(b8, x, M, N, K, 1)) <= 1e-5
    assert rel_err(run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q4_K, b4, x, M, N, K),
                   oracle.gemm_q4_k(b4, x, M, N, K)) <= TOL


@pytest.mark.parametrize("N,K", [(50, 64), (17, 4096), (960, 2560), (2560, 960), (33, 14336)])
@pytest.mark.parametrize("M", [2, 5, 8])
def test_q8_0_tensor_core_gemv_edges(ctx, kb, oracle, torch_cuda, M, N, K):
    """The int8-MMA kernel's corners: row counts that are not a multiple of its 16-row groups,
    rows split across CTAs (K > 1024: partial sums added with atomics), one and two planes."""
    rng = np.random.Generator(np.random.PCG64(0xB2000700 + 131 * M + N + K))
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    b8 = oracle.quantize_weights_q8_0(w)
    assert rel_err(run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q8_0, b8, x, M, N, K),
                   oracle.gemm_q8_0(b8, x, M, N, K)) <= TOL
    assert rel_err(run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q8_0, b8, x, M, N, K, kb.ACT_Q8),
                   oracle.gemm_q8_0(b8, x, M, N, K, 1)) <= 1e-5


@pytest.mark.parametrize("M,N,K", [(1, 512, 14336), (2, 512, 14336), (4, 512, 14336),
                                   (6, 256, 8192), (3, 1192, 4096), (8, 512, 14336),
                                   (7, 320, 4096), (8, 1192, 2048)])
def test_q4_k_ring_depths(ctx, kb, oracle, torch_cuda, M, N, K):
    """The Q4_K tensor-core GEMV sizes its copy rings by the shared memory the activation
    planes leave: long K with several activation rows reaches the shallow rings (and the
    shapes where two CTAs no longer share an SM), short K the deep ones. Seven and eight rows
    go in passes of four."""
    rng = np.random.Generator(np.random.PCG64(0xB2000900 + 977 * M + N + K))
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    b4 = oracle.quantize_weights_q4_k(w)
    assert rel_err(run_gemm(ctx, kb, torch_cuda, kb.DTYPE_Q4_K, b4, x, M, N, K),
                   oracle.gemm_q4_k(b4, x, M, N, K)) <= TOL


def test_k_shard_exchange_on_one_gpu(ctx, kb, oracle, torch_cuda):
    """The two halves of a K-sharded linear, run as two "ranks" on one GPU: each stores its
    partial result into its slice of the shared buffer through the scatter entry point, then
    kanso_cuda_sum_shards adds the slices in rank order."""
    import ctypes as C
    sh = __import__("importlib").import_module("kanso-infer_b200").sharded
    torch = torch_cuda
    rng = np.random.Generator(np.random.PCG64(0xB2000D00))
    rows, cols, world = 264, 1024, 2
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    blocks = oracle.quantize_weights_q4_k(w)
    for M in (1, 3):
        x = rng.standard_normal((M, cols)).astype(np.float32)
        ref = oracle.gemm_q4_k(blocks, x, M, rows, cols)
        xd = dev(torch, x)
        parts = torch.full((M, world * rows), float("nan"), dtype=torch.float32, device="cuda")
        ptrs = (C.c_void_p * 1)(parts.data_ptr())
        keep = []
        for r in range(world):
            shard, cb, cc = sh.k_shard(blocks, kb.DTYPE_Q4_K, rows, cols, r, world)
            wt = kb.Weight(ctx, shard, kb.DTYPE_Q4_K, rows, cc)
            keep.append(wt)
            xs = xd[:, cb:cb + cc].contiguous()
            ctx.call("kanso_cuda_linear_scatter_out", wt.h, kb._ptr(xs), M,
                     C.cast(ptrs, C.c_void_p), 1, world * rows, r * rows, kb.ACT_F32)
        y = torch.empty((M, rows), dtype=torch.float32, device="cuda")
        ctx.call("kanso_cuda_sum_shards", kb._ptr(parts), M, rows, world, kb._ptr(y))
        ctx.sync()
        assert rel_err(y.cpu().numpy(), ref) <= TOL


def test_peer_exchange_single_rank_and_give_up(ctx, kb, torch_cuda):
    """kanso_cuda_peer_exchange on one GPU. With one rank it signals itself: the step counter
    and the flag advance by one per call. With a second rank that never signals (its flag
    array is just a second buffer here) the wait runs out after its 2 s limit: the signal
    was sent, the next sync reports KANSO_ERR_TIMEOUT, and the context stays usable."""
    import ctypes as C
    torch = torch_cuda
    flags = torch.zeros(1, dtype=torch.int64, device="cuda")
    step = torch.zeros(1, dtype=torch.int64, device="cuda")
    ptrs = (C.c_void_p * 1)(flags.data_ptr())
    for _ in range(3):
        ctx.call("kanso_cuda_peer_exchange", C.cast(ptrs, C.c_void_p), kb._ptr(step), 1, 0)
    ctx.sync()
    assert int(step.item()) == 3 and int(flags.item()) == 3

    mine = torch.zeros(2, dtype=torch.int64, device="cuda")
    absent = torch.zeros(2, dtype=torch.int64, device="cuda")
    step.zero_()
    ptrs2 = (C.c_void_p * 2)(mine.data_ptr(), absent.data_ptr())
    ctx.call("kanso_cuda_peer_exchange", C.cast(ptrs2, C.c_void_p), kb._ptr(step), 2, 0)
    with pytest.raises(kb.KansoError) as ei:
        ctx.sync()
    assert ei.value.code == kb.ERR_TIMEOUT
    assert mine.tolist() == [1, 0] and absent.tolist() == [1, 0]
    ctx.call("kanso_cuda_peer_exchange", C.cast(ptrs, C.c_void_p), kb._ptr(step), 1, 0)
    ctx.sync()
    assert int(flags.item()) == 2  # step was 1 after the call that gave up


def test_linearity_at_full_size(ctx, kb, oracle, torch_cuda):
    """Size-independent property at the benchmark shape: W(ax + by) = a Wx + b Wy."""
    torch = torch_cuda
    rows, cols = 14336, 4096
    rng = np.random.Generator(np.random.PCG64(0xB2000400))
    raw = oracle.quantize_weights_q4_k((rng.standard_normal((rows, cols)) * 0.02)
                                       .astype(np.float32))
    wb = dev(torch, raw)
    x1 = torch.randn(cols, device="cuda")
    x2 = torch.randn(cols, device="cuda")
    ys = []
    for x in (x1, x2, 0.5 * x1 - 2.0 * x2):
        y = torch.empty(rows, dtype=torch.float32, device="cuda")
        ctx.gemv_q4_k(wb, x.contiguous(), y, rows, cols)
        ys.append(y)
    ctx.sync()
    comb = 0.5 * ys[0] - 2.0 * ys[1]
    assert float((ys[2] - comb).abs().max() / comb.abs().max()) <= 2e-4


def test_weight_handle_and_host_linear(ctx, kb, oracle, torch_cuda):
    rng = np.random.Generator(np.random.PCG64(0xB2000500))
    N, K, M = 640, 960, 3
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    blocks = oracle.quantize_weights_q8_0(w)
    W = kb.Weight(ctx, blocks, kb.DTYPE_Q8_0, N, K)
    y = np.empty((M, N), np.float32)
    W.forward_host(x, y, M)
    assert rel_err(y, oracle.gemm_q8_0(blocks, x, M, N, K)) <= TOL
    # embed: selected rows, bit-exact dequant (src/weights.rs:50-57)
    ids = np.array([5, 0, 639, 5], np.uint32)
    out = torch_cuda.empty((4, K), dtype=torch_cuda.float32, device="cuda")
    W.embed(dev(torch_cuda, ids), out, 4)
    ctx.sync()
    ref = oracle.dequantize_q8_0(blocks).reshape(N, K)[ids.astype(np.int64)]
    assert out.cpu().numpy().tobytes() == ref.tobytes()
    with pytest.raises(kb.KansoError) as e:
        kb.Weight(ctx, blocks[:-1], kb.DTYPE_Q8_0, N, K)
    assert e.value.code == kb.ERR_SHAPE
    with pytest.raises(kb.KansoError) as e:
        kb.Weight(ctx, blocks, kb.DTYPE_Q4_K, N, K)  # 960 % 256 != 0: a block may not straddle a row
    assert e.value.code == kb.ERR_SHAPE
    W.free()


def test_overlapped_weight_prefetch_gives_same_results(kb, oracle, torch_cuda):
    """With KANSO_OPT_OVERLAP_WEIGHT_PREFETCH consecutive GEMVs may overlap their weight
    fetch with the kernel before them; a chain y1 = W1 x, y2 = W2 y1' must be unchanged."""
    torch = torch_cuda
    stream = torch.cuda.current_stream()
    c2 = kb.Context(0, stream)
    c2.set_option(kb.OPT_OVERLAP_WEIGHT_PREFETCH, 1)
    rng = np.random.Generator(np.random.PCG64(0xB2000600))
    N1, K1, N2 = 2048, 1024, 512
    w1 = oracle.quantize_weights_q4_k((rng.standard_normal((N1, K1)) * 0.02).astype(np.float32))
    w2 = oracle.quantize_weights_q4_k((rng.standard_normal((N2, N1)) * 0.02).astype(np.float32))
    x = rng.standard_normal(K1).astype(np.float32)
    W1 = kb.Weight(c2, w1, kb.DTYPE_Q4_K, N1, K1)
    W2 = kb.Weight(c2, w2, kb.DTYPE_Q4_K, N2, N1)
    xd = torch.from_numpy(x).cuda()
    y1 = torch.empty(N1, dtype=torch.float32, device="cuda")
    y2 = torch.empty(N2, dtype=torch.float32, device="cuda")
    for _ in range(20):  # back to back: the second kernel reads what the first one writes
        W1.forward(xd, y1, 1)
        W2.forward(y1, y2, 1)
    c2.sync()
    r1 = oracle.gemv_q4_k(w1, x, N1, K1)
    assert rel_err(y1.cpu().numpy(), r1) <= TOL
    r2 = oracle.gemv_q4_k(w2, y1.cpu().numpy(), N2, N1)
    assert rel_err(y2.cpu().numpy(), r2) <= TOL
    with pytest.raises(kb.KansoError) as e:
        c2.set_option(99, 1)
    assert e.value.code == kb.ERR_CONFIG
    W1.free()
    W2.free()
    c2.close()
