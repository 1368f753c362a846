"""GPU, 2 ranks over NCCL: row-sharded (all-gather, NCCL and fused peer-store) and K-sharded
(all-reduce) GEMV against the unsharded oracle. Skipped when fewer than 2 GPUs are visible."""
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
