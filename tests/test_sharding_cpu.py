"""CPU, world_size 2 over gloo: the sharding arithmetic of the multi-GPU path.

Each rank slices the block bytes with the library's host helpers, computes its shard with the
oracle (standing in for the GPU kernel, test only), and the collective result must equal the
unsharded oracle: concatenation for row sharding, sum for K sharding.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, package


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
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        sh = package().sharded
        kb = package().backend
        rng = np.random.Generator(np.random.PCG64(0xB2000B00))  # same on every rank
        rows, cols = 48, 1024
        w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
        x = rng.standard_normal(cols).astype(np.float32)
        for dtype, quant, gemv in [(kb.DTYPE_Q4_K, O.quantize_weights_q4_k, O.gemv_q4_k),
                                   (kb.DTYPE_Q8_0, O.quantize_weights_q8_0, O.gemv_q8_0)]:
            blocks = quant(w)
            full = gemv(blocks, x, rows, cols)
            # output rows: slices concatenate to the full vector, bit for bit
            shard, rb, rc = sh.row_shard(blocks, dtype, rows, cols, rank, world)
            y_local = torch.from_numpy(gemv(shard, x, rc, cols))
            parts = [torch.empty(sh.shard_range(rows, r, world, 8)[1]) for r in range(world)]
            dist.all_gather(parts, y_local)
            assert np.array_equal(torch.cat(parts).numpy(), full)
            assert np.array_equal(y_local.numpy(), full[rb:rb + rc])
            # K: partial sums add up to the full vector (f32 re-association only)
            kshard, cb, cc = sh.k_shard(blocks, dtype, rows, cols, rank, world)
            y_part = torch.from_numpy(gemv(kshard, x[cb:cb + cc], rows, cc))
            dist.all_reduce(y_part)
            assert np.max(np.abs(y_part.numpy() - full)) <= 1e-5 * np.max(np.abs(full))
        # ranges cover [0, n) without overlap, in aligned pieces; misuse is an error
        cover = [sh.shard_range(28672, r, world, 256) for r in range(world)]
        assert cover[0][0] == 0 and sum(c for _, c in cover) == 28672
        assert all(b % 256 == 0 and c % 256 == 0 for b, c in cover)
        try:
            sh.shard_range(100, rank, world, 8)
        except kb.KansoError as e:
            assert e.code == kb.ERR_SHAPE
        else:
            raise AssertionError("unaligned range accepted")
        q.put((rank, "ok"))
    except Exception as e:  # report instead of hanging the peers
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_sharding_world_size_2():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_shard_helpers_single_process():
    sh, kb = package().sharded, package().backend
    # 3 ranks over 14 groups of 8 rows: 4 + 5 + 5 groups
    ranges = [sh.shard_range(112, r, 3, 8) for r in range(3)]
    assert ranges == [(0, 32), (32, 40), (72, 40)]
    blocks = np.arange(4 * 2 * 144, dtype=np.uint32).astype(np.uint8)  # 4 rows x 2 super-blocks
    shard, cb, cc = sh.k_shard(blocks, kb.DTYPE_Q4_K, 4, 512, 1, 2)
    assert (cb, cc) == (256, 256)
    assert np.array_equal(shard.reshape(4, 144), blocks.reshape(4, 2, 144)[:, 1])
