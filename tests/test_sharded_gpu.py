"""GPU: the sharded layers behind the C ABI against the unsharded oracle.

One test runs the whole protocol on a single GPU as a group of one rank (signal, wait, copy-out
and sum go through the same kernels); the other runs 2 ranks over NCCL (row-sharded with the
gather, row-sharded feeding a K-sharded layer, batches on the tensor-core path, a captured
graph replayed) and is skipped when fewer than 2 GPUs are visible."""
import os
import socket

import numpy as np
import pytest

from conftest import ROOT, package

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import sys
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        from oracle import oracle as O
        pkg = package()
        kb, sh = pkg.backend, pkg.sharded
        stream = torch.cuda.Stream()
        torch.cuda.set_stream(stream)
        ctx = kb.Context(rank, stream)
        rng = np.random.Generator(np.random.PCG64(0xB2000C00))  # same on every rank
        rows, cols = 1024, 2048
        w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
        blocks = O.quantize_weights_q4_k(w)

        def rel(a, b):
            return float(np.max(np.abs(a - b)) / np.max(np.abs(b)))

        for M in (1, 3):
            x = rng.standard_normal((M, cols)).astype(np.float32)
            ref = O.gemm_q4_k(blocks, x, M, rows, cols)
            xd = torch.from_numpy(x).cuda()
            for mode in ("nccl", "fused"):
                lin = sh.RowShardedLinear(ctx, blocks, kb.DTYPE_Q4_K, rows, cols, mode=mode)
                for _ in range(3):  # repeated calls reuse the result buffers
                    y = lin.forward(xd, M)
                    ctx.sync()
                    torch.cuda.synchronize()
                    assert rel(y.cpu().numpy(), ref) <= 1e-3, (mode, M)
                    dist.barrier()
            for mode in ("nccl", "fused"):
                klin = sh.KShardedLinear(ctx, blocks, kb.DTYPE_Q4_K, rows, cols, mode=mode)
                xs = xd[:, klin.col_begin:klin.col_begin + klin.col_count].contiguous()
                for _ in range(3):
                    y = klin.forward(xs, M)
                    ctx.sync()
                    torch.cuda.synchronize()
                    assert rel(y.cpu().numpy(), ref) <= 1e-3, ("k", mode, M)
                    dist.barrier()
        # the FFN pair as it is meant to run: the row-sharded up projection keeps its slice on
        # the rank (no exchange), which is exactly the K slice of the K-sharded down projection
        w2 = (rng.standard_normal((512, rows)) * 0.02).astype(np.float32)
        b2 = O.quantize_weights_q4_k(w2)
        up = sh.RowShardedLinear(ctx, blocks, kb.DTYPE_Q4_K, rows, cols, mode="fused", max_m=64)
        down = sh.KShardedLinear(ctx, b2, kb.DTYPE_Q4_K, 512, rows, mode="fused", max_m=64)
        for M in (1, 64):  # 64 rows take the tensor-core GEMM and the scatter kernel
            x = rng.standard_normal((M, cols)).astype(np.float32)
            h_ref = O.gemm_q4_k(blocks, x, M, rows, cols)
            y_ref = O.gemm_q4_k(b2, h_ref, M, 512, rows)
            xd = torch.from_numpy(x).cuda()
            for _ in range(3):
                h = up.forward(xd, M, local_only=True)
                y = down.forward(h, M)
                ctx.sync()
                torch.cuda.synchronize()
                assert rel(y.cpu().numpy(), y_ref) <= 2e-3, ("pair", M)
                full = up.forward(xd, M)
                ctx.sync()
                torch.cuda.synchronize()
                assert rel(full.cpu().numpy(), h_ref) <= 1e-3, ("gather", M)
            dist.barrier()
        # a captured graph of three pairs replayed: the buffer choice follows the device's step
        # counter, so the replays alternate buffers correctly although the host is not involved
        x = rng.standard_normal((1, cols)).astype(np.float32)
        xd = torch.from_numpy(x).cuda()
        y_ref = O.gemm_q4_k(b2, O.gemm_q4_k(blocks, x, 1, rows, cols), 1, 512, rows)
        ctx.set_option(kb.OPT_OVERLAP_WEIGHT_PREFETCH, 1)
        keep = torch.empty((3, 512), device="cuda")

        def three():
            for i in range(3):
                keep[i].copy_(down.forward(up.forward(xd, 1, local_only=True), 1)[0])
        three()
        ctx.sync()
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            three()
        for _ in range(5):
            g.replay()
        ctx.sync()
        torch.cuda.synchronize()
        for i in range(3):
            assert rel(keep[i].cpu().numpy(), y_ref[0]) <= 2e-3, ("graph", i)
        dist.barrier()
        ctx.set_option(kb.OPT_OVERLAP_WEIGHT_PREFETCH, 0)
        # Q8_0 takes the general path (slice to scratch, then a scatter kernel)
        b8 = O.quantize_weights_q8_0(w[:512])
        x = rng.standard_normal((1, cols)).astype(np.float32)
        lin = sh.RowShardedLinear(ctx, b8, kb.DTYPE_Q8_0, 512, cols, mode="fused")
        y = lin.forward(torch.from_numpy(x).cuda(), 1)
        ctx.sync()
        torch.cuda.synchronize()
        assert rel(y.cpu().numpy()[0], O.gemv_q8_0(b8, x[0], 512, cols)) <= 1e-3
        dist.barrier()
        q.put((rank, "ok"))
    except Exception as e:
        import traceback
        q.put((rank, traceback.format_exc()[-1500:]))
    finally:
        dist.destroy_process_group()


def test_sharded_linear_two_gpus(torch_cuda):
    if torch_cuda.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    procs = [mpc.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_sharded_layers_as_a_group_of_one(ctx, kb, oracle, torch_cuda):
    """The C-ABI objects with world = 1: create / connect / layers / forward. The producing
    kernel signals this rank's own flag, the consumer waits for it and copies or sums, so every
    kernel of the multi-GPU path runs; repeated calls alternate the two exchange buffers."""
    import ctypes as C
    torch = torch_cuda
    sh = package().sharded
    rng = np.random.Generator(np.random.PCG64(0xB2000C10))
    rows, cols = 512, 2048
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    blocks = oracle.quantize_weights_q4_k(w)
    h, handle = C.c_void_p(), (C.c_ubyte * kb.SHARD_HANDLE_BYTES)()
    ctx.call("kanso_cuda_shard_group_create", 0, 1, 32 << 20, C.byref(h), C.cast(handle, C.c_void_p))
    ctx.check(ctx.lib.kanso_cuda_shard_group_connect(h, C.cast(handle, C.c_void_p)))
    layers = {}
    for name, mode in (("rows", kb.SHARD_ROWS), ("k", kb.SHARD_K)):
        lh = C.c_void_p()
        ctx.check(ctx.lib.kanso_cuda_sharded_linear_create(h, blocks.ctypes.data, blocks.nbytes,
                                                           kb.DTYPE_Q4_K, rows, cols, mode, 40,
                                                           C.byref(lh)))
        b, c = C.c_int64(), C.c_int64()
        assert ctx.lib.kanso_cuda_sharded_linear_range(lh, C.byref(b), C.byref(c)) == 0
        assert (b.value, c.value) == ((0, rows) if name == "rows" else (0, cols))
        layers[name] = lh
    for M in (1, 5, 8, 40):
        x = rng.standard_normal((M, cols)).astype(np.float32)
        ref = oracle.gemm_q4_k(blocks, x, M, rows, cols)
        xd = torch.from_numpy(x).cuda()
        for name, lh in layers.items():
            for flags in ((0, kb.SHARD_LOCAL_ONLY) if name == "rows" else (0,)):
                for _ in range(3):
                    out = C.c_void_p()
                    ctx.check(ctx.lib.kanso_cuda_sharded_linear_forward(lh, xd.data_ptr(), M,
                                                                        kb.ACT_F32, flags,
                                                                        C.byref(out)))
                    ctx.sync()
                    got = sh._device_view(torch, out.value, M, rows).cpu().numpy()
                    err = float(np.max(np.abs(got - ref)) / np.max(np.abs(ref)))
                    assert err <= 1e-3, (name, M, flags, err)
    # misuse: too many rows, unknown mode, a region that is too small
    out = C.c_void_p()
    assert ctx.lib.kanso_cuda_sharded_linear_forward(layers["k"], xd.data_ptr(), 41, kb.ACT_F32, 0,
                                                     C.byref(out)) == kb.ERR_SHAPE
    lh = C.c_void_p()
    assert ctx.lib.kanso_cuda_sharded_linear_create(h, blocks.ctypes.data, blocks.nbytes,
                                                    kb.DTYPE_Q4_K, rows, cols, 7, 8,
                                                    C.byref(lh)) == kb.ERR_CONFIG
    assert ctx.lib.kanso_cuda_sharded_linear_create(h, blocks.ctypes.data, blocks.nbytes,
                                                    kb.DTYPE_Q4_K, rows, cols, kb.SHARD_K, 100000,
                                                    C.byref(lh)) == kb.ERR_CONFIG
    for lh in layers.values():
        ctx.lib.kanso_cuda_sharded_linear_destroy(lh)
    ctx.lib.kanso_cuda_shard_group_destroy(h)
