#!/usr/bin/env python
"""Headline measurement: Q4_K batch-1 decode GEMV, HBM GB/s on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (Llama-3-8B-like FFN shapes): W_up[14336x4096] and W_down[4096x14336], GGUF
Q4_K super-blocks quantised from seeded N(0, 0.02) weights, f32 activations from
N(0, 1), y = W.x. One step = one GEMV over each matrix of a ring of distinct
(up, down) pairs whose total size is several times the 126 MB L2, so every launch
streams its weights from HBM. The step is captured in a CUDA graph so that the
~12 us kernels run back to back instead of at the host's launch rate. The line also
carries `other_paths`: the Q8_0 GEMV, the batched GEMM and the decode step, timed the same way.

Prints ONE JSON line (rank 0). `value` counts algorithmic bytes
(weights once + x + y per launch) over the device time of the timed steps.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

UP = (14336, 4096)    # rows (N), cols (K)
DOWN = (4096, 14336)
Q4K_BYTES, QK_K = 144, 256
SEED = 0xB2000000 + 2 * 100
NCU_DRAM_BYTES_PER_LAUNCH = 33_105_664


def alg_bytes(rows, cols):
    """Weights once + x + y, the byte count the reference's own probe uses
    (src/bench/probes.rs:84-86)."""
    return rows * (cols // QK_K) * Q4K_BYTES + 4 * cols + 4 * rows


def make_weights(oracle, rows, cols, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    return oracle.quantize_weights_q4_k(w)


def ring_of_weights(base, copies, rows, cols, seed):
    """`copies` distinct block matrices: the first is quantised from N(0, 0.02) by the oracle's
    encoder, the others are row rotations of it (different bytes at every address, same
    distribution), which keeps host set-up time short."""
    blocks = base.reshape(rows, -1)
    out = [base]
    rng = np.random.Generator(np.random.PCG64(seed + 7))
    for _ in range(copies - 1):
        out.append(np.ascontiguousarray(np.roll(blocks, int(rng.integers(1, rows)), axis=0))
                   .reshape(-1))
    return out


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.proc, self.lines, self.idx = None, [], gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(self.idx), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(max(mx)) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def cpu_gemv_time(oracle, blocks, x, rows, cols, repeats):
    t0 = time.perf_counter()
    for _ in range(repeats):
        oracle.gemv_q4_k(blocks, x, rows, cols)
    return time.perf_counter() - t0


def cpu_baseline_1core(oracle, up, down, xs):
    """The reference's scalar row loop is single-threaded (src/quant/q4_k.rs:69-93): 1 core."""
    t_once = cpu_gemv_time(oracle, up, xs[0], *UP, 1) + cpu_gemv_time(oracle, down, xs[1], *DOWN, 1)
    passes = max(1, min(200, int(12.0 / max(t_once, 1e-3))))
    t = cpu_gemv_time(oracle, up, xs[0], *UP, passes) + cpu_gemv_time(oracle, down, xs[1], *DOWN,
                                                                      passes)
    nbytes = passes * (alg_bytes(*UP) + alg_bytes(*DOWN))
    return {"value": nbytes / t / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
            "sample": f"{passes} passes of the up and down GEMV ({2 * passes} calls, {t:.1f} s) "
                      "through the scalar restatement of scalar_gemv_q4_k"}


def threaded_cpu_step(oracle, mats, threads):
    """One step on the host: every GEMV split by rows over `threads` threads (ctypes releases
    the GIL). mats: list of (blocks, x, rows, cols)."""
    def work(blocks, x, rows, cols, r0, r1):
        bpr = cols // QK_K * Q4K_BYTES
        oracle.gemv_q4_k(blocks[r0 * bpr:r1 * bpr], x, r1 - r0, cols)

    for blocks, x, rows, cols in mats:
        cuts = [rows * i // threads for i in range(threads + 1)]
        ts = [threading.Thread(target=work, args=(blocks, x, rows, cols, cuts[i], cuts[i + 1]))
              for i in range(threads)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()


def run_reference(args):
    """The reference's CPU path for this workload: scalar_gemv_q4_k restated in oracle/ (the
    reference is a Rust crate and no Rust toolchain exists here, so its own binary cannot
    run). The row loop is split over all host threads; each step is one (up, down) pair."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    O.build()
    cores = os.cpu_count() or 1
    up = make_weights(O, *UP, SEED + 1)
    down = make_weights(O, *DOWN, SEED + 2)
    rng = np.random.Generator(np.random.PCG64(SEED + 3))
    xs = [rng.standard_normal(UP[1]).astype(np.float32),
          rng.standard_normal(DOWN[1]).astype(np.float32)]
    mats = [(up, xs[0], *UP), (down, xs[1], *DOWN)]
    for _ in range(args.warmup):
        threaded_cpu_step(O, mats, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        threaded_cpu_step(O, mats, cores)
    dt = time.perf_counter() - t0
    nbytes = args.steps * (alg_bytes(*UP) + alg_bytes(*DOWN))
    val = nbytes / dt / 1e9
    sample = ("each step = one up GEMV + one down GEMV (1 of the ring's pairs), rows split over "
              f"{cores} threads; the reference's own loop is single-threaded")
    print(json.dumps({
        "impl": "reference", "metric": "Q4_K GEMV HBM GB/s", "value": val, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": "cfg2 Q4_K GEMV batch 1: W_up[14336x4096] + W_down[4096x14336]",
                   "bytes_per_step": alg_bytes(*UP) + alg_bytes(*DOWN)},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def _graph_time_us(torch, stream, fn, calls_per_graph, iters=20):
    """Average device time of one call of a step captured in a CUDA graph (CUDA events)."""
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(iters):
        g.replay()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (iters * calls_per_graph)


def _random_blocks(torch, kb, dtype, rows, cols, copies):
    """Random block bytes with a sane f16 scale: timing only, the values are never checked."""
    blk, per = (34, 32) if dtype == kb.DTYPE_Q8_0 else (144, 256)
    out = []
    for _ in range(copies):
        w = torch.randint(0, 255, (rows * cols // per * blk,), dtype=torch.uint8, device="cuda")
        v = w.view(-1, blk)
        v[:, 1] = 0x1C
        if dtype != kb.DTYPE_Q8_0:
            v[:, 3] = 0x1C
        out.append(w)
    return out


def other_paths(torch, kb, ctx, stream, decode_batches=(1, 8, 32, 64), decode_only=False):
    """The other rows of the hot path, timed the same way (graph + events, weights rotated
    through more than the L2's 126 MB): cfg 1 Q8_0 GEMV, cfg 3 batched GEMM, cfg 4 decode."""
    res = {}
    if decode_only:
        res["cfg4_decode_smollm2_360m_q8_0"] = decode_rates(torch, kb, ctx, stream, decode_batches)
        return res
    gemv = {}
    for rows, cols in ((2560, 960), (960, 2560)):
        nbytes = rows * cols // 32 * 34
        copies = max(2, min(256, int(400e6 / nbytes)))
        ws = _random_blocks(torch, kb, kb.DTYPE_Q8_0, rows, cols, copies)
        x = torch.randn(1, cols, device="cuda")
        y = torch.empty(1, rows, device="cuda")

        def step():
            for w in ws:
                ctx.gemm_q8_0(w, x, y, 1, rows, cols, kb.ACT_F32)
        us = _graph_time_us(torch, stream, step, copies)
        gemv[f"{rows}x{cols}"] = {"us_per_launch": us, "GB/s": nbytes / us / 1e3}
    res["cfg1_q8_0_gemv_batch1"] = gemv
    gemm = {}
    for name, dtype in (("q8_0", kb.DTYPE_Q8_0), ("q4_k", kb.DTYPE_Q4_K)):
        rows, cols = 14336, 4096
        nbytes = rows * cols // (32 if dtype == kb.DTYPE_Q8_0 else 256) * (34 if dtype == kb.DTYPE_Q8_0 else 144)
        copies = max(2, int(300e6 / nbytes))
        ws = _random_blocks(torch, kb, dtype, rows, cols, copies)
        for M in (8, 32, 128):
            x = torch.randn(M, cols, device="cuda")
            y = torch.empty(M, rows, device="cuda")
            f = ctx.gemm_q8_0 if dtype == kb.DTYPE_Q8_0 else ctx.gemm_q4_k

            def step():
                for w in ws:
                    f(w, x, y, M, rows, cols, kb.ACT_F32)
            us = _graph_time_us(torch, stream, step, copies, iters=5)
            gemm[f"{name}_M{M}_N{rows}_K{cols}"] = {
                "us_per_call": us, "TFLOP/s": 2 * M * rows * cols / us / 1e6,
                "weight_GB/s": nbytes / us / 1e3}
    res["cfg3_batched_gemm"] = gemm
    res["cfg4_decode_smollm2_360m_q8_0"] = decode_rates(torch, kb, ctx, stream, decode_batches)
    return res


def decode_rates(torch, kb, ctx, stream, batches=(1, 8, 32, 64)):
    """cfg 4: one decode step of the SmolLM2-360M architecture, Q8_0 weights (random block
    bytes), int8 paged KV with 16-token blocks and permuted block tables, contexts uniform in
    [256, 4096]; tokens per second = sequences / step time."""
    L, hidden, H, KH, inter, vocab, bs = 32, 960, 15, 5, 2560, 49152, 16
    hd = hidden // H
    cfg = kb.ModelConfig(hidden, H, KH, L, inter, vocab, bs, 4352, 1e-5, 100000.0)
    m = kb.Model(ctx, cfg)
    rng = np.random.Generator(np.random.PCG64(SEED + 40))

    def qblocks(rows, cols):
        b = rng.integers(0, 256, size=(rows * cols // 32, 34), dtype=np.uint8)
        b[:, 0] = 0x00
        b[:, 1] = 0x14  # f16 scale ~ 0.00098
        return b.reshape(-1)
    shapes = {0: (H * hd, hidden), 1: (KH * hd, hidden), 2: (KH * hd, hidden), 3: (hidden, H * hd),
              4: (inter, hidden), 5: (inter, hidden), 6: (hidden, inter)}
    for l in range(L):
        for which, (r, c) in shapes.items():
            m.set_weight(l, which, qblocks(r, c), kb.DTYPE_Q8_0, r, c)
        m.set_norm(l, 0, np.ones(hidden, np.float32))
        m.set_norm(l, 1, np.ones(hidden, np.float32))
    m.set_weight(0, 7, qblocks(vocab, hidden), kb.DTYPE_Q8_0, vocab, hidden)
    m.set_norm(0, 2, np.ones(hidden, np.float32))
    out = {}
    for B in batches:
        lens = rng.integers(256, 4097, size=B)
        nblk = [(int(c) + bs - 1) // bs for c in lens]
        NB = sum(nblk) + 8
        pool = kb.KvPool(ctx, L, NB, bs, KH, hd)
        perm = rng.permutation(NB)
        maxb = max(nblk)
        tables = np.zeros((B, maxb), np.uint32)
        used, hist = 0, []
        for i in range(B):
            blocks = perm[used:used + nblk[i]]
            used += nblk[i]
            tables[i, :nblk[i]] = blocks
            tables[i, nblk[i]:] = blocks[-1]
            t = np.arange(int(lens[i]) - 1)
            hist.append((blocks[t // bs] * bs + t % bs).astype(np.uint32))
        hist = np.concatenate(hist)
        hs = torch.from_numpy(hist.astype(np.int64)).to(torch.int32).cuda()
        for l in range(L):
            k = torch.randn(len(hist), KH * hd, device="cuda")
            v = torch.randn(len(hist), KH * hd, device="cuda")
            pool.write_slots(l, hs, k, v, len(hist))
        ctx.sync()
        tok = torch.from_numpy(rng.integers(0, vocab, size=B).astype(np.int32)).cuda()
        pos = torch.from_numpy((lens - 1).astype(np.int32)).cuda()
        slot = torch.from_numpy(np.array(
            [tables[i, (lens[i] - 1) // bs] * bs + (lens[i] - 1) % bs for i in range(B)],
            np.int32)).cuda()
        tb = torch.from_numpy(tables.astype(np.int32)).cuda()
        ln = torch.from_numpy(lens.astype(np.int32)).cuda()
        logits = torch.empty(B, vocab, device="cuda")

        def step():
            m.decode_step_device(pool, tok, pos, slot, tb, ln, B, maxb, int(lens.max()), logits)
        l0 = ctx.launches
        step()
        ctx.sync()
        launches = ctx.launches - l0
        us = _graph_time_us(torch, stream, step, 1)
        out[f"B{B}"] = {"tok/s": B / us * 1e6, "us_per_step": us, "sum_ctx": int(lens.sum()),
                        "launches_per_step": int(launches)}
        pool.destroy()
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        # A rank that never joins (or a stalled exchange) would leave the others waiting for
        # ever: every rank ends itself after a deadline well beyond a normal run.
        deadline = threading.Timer(float(os.environ.get("KANSO_BENCH_DEADLINE_S", "420")),
                                   lambda: (sys.stderr.write("bench: deadline passed, exiting\n"),
                                            os._exit(3)))
        deadline.daemon = True
        deadline.start()
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    kb = importlib.import_module("kanso-infer_b200").backend
    from oracle import oracle as O  # CPU baseline leg + a result check only
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx = kb.Context(local, stream)
    # the weights are uploaded once and never written again: let consecutive GEMVs overlap
    # their weight prefetch with the drain of the kernel before them
    if not os.environ.get("KANSO_BENCH_NO_OVERLAP"):
        ctx.set_option(kb.OPT_OVERLAP_WEIGHT_PREFETCH, 1)

    pairs = args.pairs
    up0 = make_weights(O, *UP, SEED + 1 + 10 * rank)
    down0 = make_weights(O, *DOWN, SEED + 2 + 10 * rank)
    ups = ring_of_weights(up0, pairs, *UP, SEED + 11)
    downs = ring_of_weights(down0, pairs, *DOWN, SEED + 12)
    rng = np.random.Generator(np.random.PCG64(SEED + 3))
    x_up = rng.standard_normal(UP[1]).astype(np.float32)
    x_down = rng.standard_normal(DOWN[1]).astype(np.float32)

    dx_up = torch.from_numpy(x_up).cuda()
    dx_down = torch.from_numpy(x_down).cuda()
    y_up = torch.empty(UP[0], dtype=torch.float32, device="cuda")
    y_down = torch.empty(DOWN[0], dtype=torch.float32, device="cuda")
    if world == 1:
        W_up = [kb.Weight(ctx, b, kb.DTYPE_Q4_K, *UP) for b in ups]
        W_down = [kb.Weight(ctx, b, kb.DTYPE_Q4_K, *DOWN) for b in downs]

        def step():
            for wu, wd in zip(W_up, W_down):
                wu.forward(dx_up, y_up, 1)
                wd.forward(dx_down, y_down, 1)
    else:
        # Weak scaling of the sharded layer pair: every rank keeps config 2's shard sizes.
        # W_up[world*14336 x 4096] is split by output rows, its y gathered by the GEMV kernel's
        # own peer stores; W_down[4096 x world*14336] is split along K, its partial sums
        # exchanged by the same peer stores and added on every rank.
        sh = importlib.import_module("kanso-infer_b200").sharded
        S_up = [sh.RowShardedLinear(ctx, b, kb.DTYPE_Q4_K, world * UP[0], UP[1], mode="fused",
                                    max_m=1, presharded=True) for b in ups]
        S_down = [sh.KShardedLinear(ctx, b, kb.DTYPE_Q4_K, DOWN[0], world * DOWN[1], max_m=1,
                                    presharded=True, mode="fused") for b in downs]
        W_up = [s.weight for s in S_up]
        W_down = [s.weight for s in S_down]
        dx_up2 = dx_up.reshape(1, -1)
        dx_down2 = dx_down.reshape(1, -1)

        def step():
            for su, sd in zip(S_up, S_down):
                y_up_full = su.forward(dx_up2, 1)
                y_dn = sd.forward(dx_down2, 1)
            y_up.copy_(y_up_full[0, su.row_begin:su.row_begin + su.row_count])
            y_down.copy_(y_dn[0])

    # result check against the oracle on the last pair (not timed)
    step()
    ctx.sync()
    ref_up = O.gemv_q4_k(ups[-1], x_up, *UP)  # at N > 1: this rank's slice of the gathered y
    err = float(np.max(np.abs(y_up.cpu().numpy() - ref_up)) / np.max(np.abs(ref_up)))
    if err > 1e-3:
        raise SystemExit(f"bench: GEMV result differs from the oracle by {err:.2e} (> 1e-3)")

    # GEMV launches per step (at N > 1 each pair adds two exchanges and one shard sum)
    launches_per_step = 2 * pairs

    class _Eager:  # same interface as a captured graph, for steps that cannot be captured
        def replay(self):
            step()

    if world == 1 or not os.environ.get("KANSO_BENCH_EAGER"):
        # at N > 1 the step holds only this library's kernels (the cross-GPU exchange is one of
        # them and keeps its step number on the device), so it is captured like the N = 1 step
        launch_mode = "CUDA graph of the step"
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
    else:
        graph, launch_mode = _Eager(), "eager launches"
    for _ in range(max(3, args.warmup)):
        graph.replay()
    torch.cuda.synchronize()
    if world > 1 and launch_mode.startswith("CUDA graph"):
        # a rank whose exchange gave up its bounded wait during the warm-up replays reports it
        # here; then every rank goes back to eager launches instead of failing the run
        ok = 1
        try:
            ctx.sync()
        except kb.KansoError as e:
            ok = 0
            print(f"bench: rank {rank}: graph replay failed ({e}); eager launches", file=sys.stderr)
        t = torch.tensor([ok], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        if int(t.item()) == 0:
            graph, launch_mode = _Eager(), "eager launches (the graph replay failed)"
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        graph.replay()
    e1.record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # keep sampling for a moment so that short timed regions still get samples
    clocks = None
    if world == 1:
        t_end = time.time() + 1.0
        while time.time() < t_end:
            graph.replay()
    else:  # every rank must take part in the collectives: a fixed number of extra steps
        for _ in range(200):
            graph.replay()
    torch.cuda.synchronize()
    if rank == 0:
        clocks = sampler.stop()

    step_bytes = pairs * (alg_bytes(*UP) + alg_bytes(*DOWN))
    value = world * step_bytes * args.steps / (ms * 1e-3) / 1e9
    us_per_launch = ms * 1e3 / (args.steps * launches_per_step)

    # end to end through the host-buffer call: x from host memory, y back to host memory
    e2e = None
    if True:
        yh_up = np.empty(UP[0], np.float32)
        yh_down = np.empty(DOWN[0], np.float32)

        def host_step():
            for wu, wd in zip(W_up, W_down):
                wu.forward_host(x_up, yh_up, 1)
                wd.forward_host(x_down, yh_down, 1)

        host_step()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        n_e2e = max(1, min(args.steps, 20))
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            host_step()
        dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        e2e = {"value": world * step_bytes * n_e2e / dt / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": pairs * 4 * (UP[1] + DOWN[1]),
               "d2h_bytes_per_step": pairs * 4 * (UP[0] + DOWN[0]),
               "steps": n_e2e, "us_per_call": dt / (n_e2e * launches_per_step) * 1e6}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    per_launch_bytes = (alg_bytes(*UP) + alg_bytes(*DOWN)) / 2
    achieved = per_launch_bytes / (us_per_launch * 1e-6) / 1e9
    # dram__bytes_read + dram__bytes_write of one launch, from the ncu capture summarised in
    # profiles/gemv_q4k_mma_cfg2.md (a profiler figure: it is not re-measured by this run)
    traffic = NCU_DRAM_BYTES_PER_LAUNCH

    cpu = cpu_baseline_1core(O, up0, down0, [x_up, x_down]) if (world == 1 and not os.environ.get("KANSO_BENCH_SKIP_CPU")) else None
    line = {
        "metric": "Q4_K GEMV HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
        "data": "synthetic",
        "config": {"workload": "cfg2 Q4_K GEMV batch 1: W_up[14336x4096] + W_down[4096x14336]",
                   "ring_pairs": pairs, "bytes_per_step": step_bytes,
                   "l2": f"inputs larger than L2: {step_bytes / 1e6:.0f} MB of distinct weights "
                         "per step vs 126 MB L2",
                   "launch": launch_mode, "parallelism": (f"shards{world}" if world == 1 else f"row-shard all-gather + K-shard all-reduce, both through the GEMV kernel's peer stores, over {world} GPUs"),
                   "check_vs_oracle_rel_err": err},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_source": peak_src, "traffic": traffic,
                     "kernel": "gemv_q4k_mma_kernel", "us_per_launch": us_per_launch,
                     "alg_bytes_per_launch": per_launch_bytes},
        "e2e": e2e, "gpu_launches": (launches_per_step if world == 1 else 5 * pairs) * args.steps, "clocks": clocks,
    }
    if cpu:
        line["cpu_baseline"] = cpu
    if world == 1 and not os.environ.get("KANSO_BENCH_SKIP_EXTRAS"):
        # not part of the headline value: the remaining rows of the path, for the record
        line["other_paths"] = other_paths(torch, kb, ctx, stream)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--pairs", type=int, default=8, help="distinct (up, down) pairs in the ring")
    ap.add_argument("--decode-only", default=None, metavar="B[,B...]",
                    help="time only the decode step at these batch sizes (1 GPU) and print them; "
                         "for profiler captures of that path")
    ap.add_argument("--gemm-only", default=None, metavar="FMT,M",
                    help="run only the cfg 3 GEMM (q8_0 or q4_k, N=14336, K=4096) with M activation "
                         "rows over four weight copies, eagerly; for profiler captures of that path")
    args = ap.parse_args()
    if args.gemm_only:
        import torch
        kb = importlib.import_module("kanso-infer_b200").backend
        torch.cuda.set_device(0)
        stream = torch.cuda.Stream()
        torch.cuda.set_stream(stream)
        ctx = kb.Context(0, stream)
        fmt, M = args.gemm_only.split(",")
        M = int(M)
        dtype = kb.DTYPE_Q8_0 if fmt == "q8_0" else kb.DTYPE_Q4_K
        ws = _random_blocks(torch, kb, dtype, 14336, 4096, 4)
        x = torch.randn(M, 4096, device="cuda")
        y = torch.empty(M, 14336, device="cuda")
        for w in ws:
            (ctx.gemm_q8_0 if dtype == kb.DTYPE_Q8_0 else ctx.gemm_q4_k)(w, x, y, M, 14336, 4096,
                                                                         kb.ACT_F32)
        ctx.sync()
        print(json.dumps({"gemm_only": args.gemm_only, "launches": int(ctx.launches)}))
        return
    if args.decode_only:
        import torch
        kb = importlib.import_module("kanso-infer_b200").backend
        torch.cuda.set_device(0)
        stream = torch.cuda.Stream()
        torch.cuda.set_stream(stream)
        ctx = kb.Context(0, stream)
        ctx.set_option(kb.OPT_OVERLAP_WEIGHT_PREFETCH, 1)
        batches = tuple(int(b) for b in args.decode_only.split(","))
        print(json.dumps(other_paths(torch, kb, ctx, stream, batches, decode_only=True)))
        return
    if args.impl == "reference":
        if args.steps > 50:
            args.steps = 50  # bounded sample: the CPU step takes ~0.1 s
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
