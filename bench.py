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
# dram__bytes_read + dram__bytes_write of one launch of the headline kernel on the 14336 x 4096
# matrix: the mean of the two launches of the ncu capture summarised under profiles/
NCU_DRAM_BYTES_PER_LAUNCH = 33_110_016


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
    run). The row loop is split over all host threads; a step covers the same ring of (up, down)
    pairs as the GPU arm's step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    O.build()
    cores = os.cpu_count() or 1
    up = make_weights(O, *UP, SEED + 1)
    down = make_weights(O, *DOWN, SEED + 2)
    ups = ring_of_weights(up, args.pairs, *UP, SEED + 11)
    downs = ring_of_weights(down, args.pairs, *DOWN, SEED + 12)
    rng = np.random.Generator(np.random.PCG64(SEED + 3))
    xs = [rng.standard_normal(UP[1]).astype(np.float32),
          rng.standard_normal(DOWN[1]).astype(np.float32)]
    mats = []
    for u, d in zip(ups, downs):
        mats += [(u, xs[0], *UP), (d, xs[1], *DOWN)]
    for _ in range(args.warmup):
        threaded_cpu_step(O, mats, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        threaded_cpu_step(O, mats, cores)
    dt = time.perf_counter() - t0
    step_bytes = args.pairs * (alg_bytes(*UP) + alg_bytes(*DOWN))
    val = args.steps * step_bytes / dt / 1e9
    workload = "cfg2 Q4_K GEMV batch 1: W_up[14336x4096] + W_down[4096x14336]"
    if args.gpus > 1:
        # the GPU arm's weak-scaling step holds this same ring of pairs PER GPU (one shard of the
        # N-times-larger FFN pair each); the host has one set of cores, so it is timed on one
        # GPU's share: the same bytes per pair, GB/s comparable per byte
        workload = (f"one GPU's share of the sharded FFN pair (W_up[{args.gpus * UP[0]}x{UP[1]}] by "
                    f"rows, W_down[{DOWN[0]}x{args.gpus * DOWN[1]}] along K): " + workload)
    sample = (f"each step = the ring of {args.pairs} (up, down) pairs, every GEMV's rows split over "
              f"{cores} threads; the reference's own loop is single-threaded")
    print(json.dumps({
        "impl": "reference", "metric": "Q4_K GEMV HBM GB/s", "value": val, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": workload, "ring_pairs": args.pairs,
                   "bytes_per_step": step_bytes},
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


def _peaks():
    """(HBM GB/s, sustained bf16 TFLOP/s, source): the measured figures of this pool's B200s when
    the driver has written them, else the fallback measurement."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", 1400.0)), "measured"
    return 6650.0, 1400.0, "fallback"


def _weight_bytes(kb, dtype, rows, cols):
    return rows * cols // 32 * 34 if dtype == kb.DTYPE_Q8_0 else rows * cols // 256 * 144


def gemm_legs(torch, kb, O, ctx, stream):
    """cfg 3: y[M,N] = x[M,4096] @ W[N,4096]^T for M in {8, 32, 128, 512}, N in {4096, 14336},
    Q8_0 and Q4_K. Each format is first CHECKED on weights quantised from N(0, 0.02): a seeded
    sample of output columns of the M = 32 and M = 512 products at N = 14336 against the oracle
    (<= 1e-3 of the output scale), then timed over a ring of weight copies larger than L2. Each
    shape reports the fraction of the bound that applies to it: HBM below the ridge of the
    measured peaks, the sustained bf16 tensor rate above it."""
    hbm, tf, src = _peaks()
    ridge = tf * 1e12 / (hbm * 1e9)
    K = 4096
    res = {"peaks": {"hbm_GB/s": hbm, "bf16_TFLOP/s_sustained": tf, "source": src}}
    for name, dtype in (("q8_0", kb.DTYPE_Q8_0), ("q4_k", kb.DTYPE_Q4_K)):
        f = ctx.gemm_q8_0 if dtype == kb.DTYPE_Q8_0 else ctx.gemm_q4_k
        rng = np.random.Generator(np.random.PCG64(SEED + 30 + dtype))
        w = rng.standard_normal((14336, K), dtype=np.float32) * np.float32(0.02)
        quant, gemm = ((O.quantize_weights_q8_0, O.gemm_q8_0) if dtype == kb.DTYPE_Q8_0
                       else (O.quantize_weights_q4_k, O.gemm_q4_k))
        blocks = quant(w)
        wd = torch.from_numpy(blocks).cuda()
        rows2d = blocks.reshape(14336, -1)
        worst = 0.0
        for M in (32, 512):
            x = rng.standard_normal((M, K), dtype=np.float32)
            y = torch.empty(M, 14336, device="cuda")
            f(wd, torch.from_numpy(x).cuda(), y, M, 14336, K, kb.ACT_F32)
            ctx.sync()
            got = y.cpu().numpy()
            pick = np.unique(np.concatenate([[0, 127, 128, 14335], rng.integers(0, 14336, 28)]))
            ref = gemm(np.ascontiguousarray(rows2d[pick]).reshape(-1), x, M, pick.size, K)
            err = float(np.max(np.abs(got[:, pick] - ref)) / np.max(np.abs(got)))
            if not err <= 1e-3:
                raise SystemExit(f"bench: cfg3 {name} M={M} differs from the oracle by {err:.2e}")
            worst = max(worst, err)
        res[f"{name}_check_vs_oracle_rel_err"] = worst
        del wd
        for rows in (14336, 4096):
            nbytes = _weight_bytes(kb, dtype, rows, K)
            copies = max(2, int(300e6 / nbytes))
            ws = _random_blocks(torch, kb, dtype, rows, K, copies)
            for M in (8, 32, 128, 512):
                x = torch.randn(M, K, device="cuda")
                y = torch.empty(M, rows, device="cuda")

                def step():
                    for w_ in ws:
                        f(w_, x, y, M, rows, K, kb.ACT_F32)
                us = _graph_time_us(torch, stream, step, copies, iters=5)
                ctx.sync()
                flops, byts = 2.0 * M * rows * K, nbytes + 4.0 * M * (K + rows)
                bound = "hbm" if flops / byts < ridge else "tensor"
                frac = (byts / us / 1e3 / hbm) if bound == "hbm" else (flops / us / 1e6 / tf)
                res[f"{name}_M{M}_N{rows}_K{K}"] = {
                    "us_per_call": us, "TFLOP/s": flops / us / 1e6, "GB/s": byts / us / 1e3,
                    "bound": bound, "frac_of_bound": frac}
                if dtype == kb.DTYPE_Q8_0 and rows == 14336 and M in (32, 128):
                    # the bit-exact mode: activations quantised per 32 (quantize_row_q8_0), int32
                    # block sums on tcgen05 kind::i8
                    def step_q8():
                        for w_ in ws:
                            f(w_, x, y, M, rows, K, kb.ACT_Q8)
                    us8 = _graph_time_us(torch, stream, step_q8, copies, iters=5)
                    ctx.sync()
                    res[f"q8_0_act_q8_M{M}_N{rows}_K{K}"] = {
                        "us_per_call": us8, "TOP/s": flops / us8 / 1e6, "GB/s": byts / us8 / 1e3,
                        "frac_of_hbm": byts / us8 / 1e3 / hbm}
            del ws
    return res


def gemv_legs(torch, kb, ctx, stream):
    """Batch-1 GEMVs beside the headline: cfg 1 (Q8_0, SmolLM2-360M FFN shapes, 2.6 MB each:
    latency-bound, cycled through 400 MB of copies), an HBM-bound Q8_0 matrix of cfg 2's shape
    with its roofline fraction, and the plain 128-bit read of cfg 2's Q4_K buffers: the floor
    under the headline kernel in the same kind of captured sequence."""
    hbm, _, _ = _peaks()
    res = {}
    for rows, cols in ((2560, 960), (960, 2560), (14336, 4096), (4096, 14336)):
        nbytes = _weight_bytes(kb, kb.DTYPE_Q8_0, rows, cols)
        copies = max(2, min(256, int(400e6 / nbytes)))
        ws = _random_blocks(torch, kb, kb.DTYPE_Q8_0, rows, cols, copies)
        x = torch.randn(1, cols, device="cuda")
        y = torch.empty(1, rows, device="cuda")

        def step():
            for w_ in ws:
                ctx.gemm_q8_0(w_, x, y, 1, rows, cols, kb.ACT_F32)
        us = _graph_time_us(torch, stream, step, copies)
        ctx.sync()
        byts = nbytes + 4 * (rows + cols)
        res[f"q8_0_{rows}x{cols}"] = {"us_per_launch": us, "GB/s": byts / us / 1e3,
                                      "frac_of_hbm": byts / us / 1e3 / hbm}
        del ws
    nb = UP[0] * UP[1] // QK_K * Q4K_BYTES
    bufs = _random_blocks(torch, kb, kb.DTYPE_Q4_K, UP[0], UP[1], 16)

    def floor_step():
        for b in bufs:
            ctx.call("kanso_cuda_probe_read", b.data_ptr(), nb)
    us = _graph_time_us(torch, stream, floor_step, len(bufs))
    ctx.sync()
    res["read_floor_33MB"] = {"us_per_launch": us, "GB/s": nb / us / 1e3,
                              "what": "one launch that only reads a 33 MB Q4_K buffer with "
                                      "128-bit loads, 16 distinct buffers per captured step"}
    return res


def decode_legs(torch, kb, O, ctx, stream, batches=(1, 8, 32, 64), check=True):
    """cfg 4: one decode step of the SmolLM2-360M architecture (32 layers, hidden 960, 15 query /
    5 KV heads, head_dim 64, SwiGLU 2560, vocab 49152, RoPE theta 100000, tied lm_head), every
    projection Q8_0 from seeded N(0, 0.02), int8 paged KV with 16-token blocks and permuted
    block tables, contexts uniform in [256, 4096]. With `check`, a batch of 8 is first compared
    with the oracle engine through the host-array call (logits within 1e-2, same greedy token;
    the full 32 layers). Per batch: device-resident step time under a captured graph, the
    fraction of the HBM roofline (weights once + the int8 history read once), and the same step
    end to end through kanso_cuda_decode_step (host arrays in, logits back to the host)."""
    hbm, _, _ = _peaks()
    L, hidden, H, KH, inter, vocab, bs = 32, 960, 15, 5, 2560, 49152, 16
    hd = hidden // H
    cfg = kb.ModelConfig(hidden, H, KH, L, inter, vocab, bs, 4352, 1e-5, 100000.0)
    m = kb.Model(ctx, cfg)
    om = O.Model(O.ModelConfig(hidden, H, KH, L, inter, vocab, bs, 4352, 1e-5, 100000.0)) if check else None
    rng = np.random.Generator(np.random.PCG64(SEED + 40))
    shapes = {0: (H * hd, hidden), 1: (KH * hd, hidden), 2: (KH * hd, hidden), 3: (hidden, H * hd),
              4: (inter, hidden), 5: (inter, hidden), 6: (hidden, inter)}
    weight_bytes = 0

    def put(l, which, r, c):
        nonlocal weight_bytes
        b = O.quantize_weights_q8_0(rng.standard_normal((r, c), dtype=np.float32) * np.float32(0.02))
        m.set_weight(l, which, b, kb.DTYPE_Q8_0, r, c)
        if om is not None:
            om.set_weight(l, which, b, r, c)
        weight_bytes += b.nbytes
    for l in range(L):
        for which, (r, c) in shapes.items():
            put(l, which, r, c)
        for which in (0, 1):
            nw = (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
            m.set_norm(l, which, nw)
            if om is not None:
                om.set_norm(l, which, nw)
    put(0, 7, vocab, hidden)
    fn = (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
    m.set_norm(0, 2, fn)
    if om is not None:
        om.set_norm(0, 2, fn)
    out = {"weights": "Q8_0 from N(0, 0.02), norm weights 1 + 0.1 N(0,1)"}
    todo = list(batches)
    if check and 8 not in todo:
        todo.append(8)
    # (batch, fp8 pool?): every batch on the int8 pool, then batch 8 (checked) and the largest
    # batch on the fp8 pool (E4M3 bytes, power-of-two scales)
    runs = [(B, False) for B in sorted(set(todo), key=lambda b: (b != 8, b))]  # checked batch first
    if check:
        runs += [(8, True)] + ([(max(batches), True)] if max(batches) != 8 else [])
    for B, fp8 in runs:
        lens = rng.integers(256, 4097, size=B)
        nblk = [(int(c) + bs - 1) // bs for c in lens]
        NB = sum(nblk) + 8
        pool = kb.KvPool(ctx, L, NB, bs, KH, hd, kb.KV_FP8 if fp8 else kb.KV_INT8)
        opool = O.KvPool(L, NB, bs, KH, hd, fp8=fp8) if (check and B == 8) else None
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
            if opool is not None:
                k = rng.standard_normal((len(hist), KH * hd), dtype=np.float32)
                v = rng.standard_normal((len(hist), KH * hd), dtype=np.float32)
                opool.write_slots(l, hist, k, v)
                pool.write_slots(l, hs, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(),
                                 len(hist))
            else:
                pool.write_slots(l, hs, torch.randn(len(hist), KH * hd, device="cuda"),
                                 torch.randn(len(hist), KH * hd, device="cuda"), len(hist))
        ctx.sync()
        tok_h = rng.integers(0, vocab, size=B).astype(np.uint32)
        pos_h = (lens - 1).astype(np.uint32)
        slot_h = np.array([tables[i, (lens[i] - 1) // bs] * bs + (lens[i] - 1) % bs
                           for i in range(B)], np.uint32)
        lens_h = lens.astype(np.uint32)
        logits_h = np.empty((B, vocab), np.float32)
        entry = {"sum_ctx": int(lens.sum())}
        if opool is not None:
            st, ref = om.decode_step(opool, tok_h, pos_h, slot_h, tables.reshape(-1), lens_h, maxb)
            m.decode_step(pool, tok_h, pos_h, slot_h, tables.reshape(-1), lens_h, maxb, logits_h)
            err = float(np.max(np.abs(logits_h - ref)))
            same = [int(np.argmax(r)) for r in logits_h] == [O.greedy_token(r) for r in ref]
            if st != 0 or not err <= 1e-2 or not same:
                raise SystemExit(f"bench: cfg4 B=8 (fp8 pool: {fp8}) differs from the oracle engine: max |dlogit| "
                                 f"{err:.2e}, same greedy tokens {same}")
            entry["check_vs_oracle_max_abs_dlogit"] = err
            # the step above stored the newest token: write a fresh history row over it so that
            # the timed steps below see the same state as the other batches
        if B in batches or fp8:
            tok, pos, slot = (torch.from_numpy(a.astype(np.int32)).cuda()
                              for a in (tok_h, pos_h, slot_h))
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
            ctx.sync()
            byts = weight_bytes + 680 * L * int(lens.sum()) + 4 * B * vocab
            for _ in range(2):
                m.decode_step(pool, tok_h, pos_h, slot_h, tables.reshape(-1), lens_h, maxb, logits_h)
            t0 = time.perf_counter()
            n_e2e = 10
            for _ in range(n_e2e):
                m.decode_step(pool, tok_h, pos_h, slot_h, tables.reshape(-1), lens_h, maxb, logits_h)
            e2e_us = (time.perf_counter() - t0) / n_e2e * 1e6
            entry.update({"tok/s": B / us * 1e6, "us_per_step": us,
                          "launches_per_step": int(launches), "alg_bytes_per_step": byts,
                          "GB/s": byts / us / 1e3, "frac_of_hbm": byts / us / 1e3 / hbm,
                          "e2e_host_call": {"us_per_step": e2e_us, "tok/s": B / e2e_us * 1e6,
                                            "h2d_bytes": int(4 * (4 * B + B * maxb)),
                                            "d2h_bytes": int(4 * B * vocab)}})
        out[f"B{B}_fp8_pool" if fp8 else f"B{B}"] = entry
        pool.destroy()
    m.destroy()
    return out


def prefill_attention_leg(torch, kb, O, ctx, stream):
    """Chunked-prefill attention over the int8 pool (SmolLM2-360M heads: 15 query / 5 KV heads of
    64, 16-token blocks, permuted tables). First a small mixed batch (a 48-token chunk on 80 cached
    tokens and a whole 33-token prompt) against the oracle's restatement of the reference's masked
    dense attention, then 4 sequences with 512-token chunks on 1536 cached tokens each, timed over
    three layers of records (3 x 28 MB of cache, contexts walked once per query row)."""
    H, KH, hd, bs = 15, 5, 64, 16
    scale = float(1.0 / np.sqrt(np.float32(hd)))
    rng = np.random.Generator(np.random.PCG64(SEED + 60))

    def build(ctx_lens, layers, with_oracle):
        nblk = [(c + bs - 1) // bs for c in ctx_lens]
        NB = sum(nblk) + 4
        perm = rng.permutation(NB)
        maxb = max(nblk)
        tab = np.zeros((len(ctx_lens), maxb), np.uint32)
        u = 0
        for i, nb in enumerate(nblk):
            tab[i, :nb] = perm[u:u + nb]
            tab[i, nb:] = tab[i, nb - 1]
            u += nb
        pool = kb.KvPool(ctx, layers, NB, bs, KH, hd)
        opool = O.KvPool(layers, NB, bs, KH, hd) if with_oracle else None
        for i, c in enumerate(ctx_lens):
            t = np.arange(c)
            slots = (tab[i][t // bs] * bs + t % bs).astype(np.uint32)
            sd = torch.from_numpy(slots.astype(np.int64)).to(torch.int32).cuda()
            for l in range(layers):
                k = rng.standard_normal((c, KH * hd), dtype=np.float32)
                v = rng.standard_normal((c, KH * hd), dtype=np.float32)
                pool.write_slots(l, sd, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), c)
                if opool is not None:
                    opool.write_slots(l, slots, k, v)
        return pool, opool, tab, maxb

    # check
    seqs = [(80, 48), (0, 33)]
    ctx_lens = [a + b for a, b in seqs]
    pool, opool, tab, maxb = build(ctx_lens, 1, True)
    T = sum(b for _, b in seqs)
    q = rng.standard_normal((T, H * hd), dtype=np.float32)
    out = torch.empty(T, H * hd, device="cuda")
    p = kb.PagedAttentionParams(len(seqs), H, KH, hd, bs, maxb, scale)
    pool.paged_attention_prefill(0, torch.from_numpy(q).cuda(), torch.from_numpy(tab.reshape(-1).astype(np.int32)).cuda(),
                                 np.array(ctx_lens, np.uint32), np.array([b for _, b in seqs], np.uint32),
                                 out, p)
    ctx.sync()
    got = out.cpu().numpy()
    err, row = 0.0, 0
    for i, (sp, ql) in enumerate(seqs):
        nb = (ctx_lens[i] + bs - 1) // bs
        st, ref = O.prefill_attention_int8(opool, 0, q[row:row + ql], tab[i, :nb], sp, H, scale)
        err = max(err, float(np.max(np.abs(got[row:row + ql] - ref)) / np.max(np.abs(ref))))
        row += ql
    if not err <= 1e-3:
        raise SystemExit(f"bench: prefill attention differs from the oracle: {err:.2e}")
    pool.destroy()
    # timing
    S, chunk, cached, layers = 4, 512, 1536, 3
    ctx_lens = [cached + chunk] * S
    pool, _, tab, maxb = build(ctx_lens, layers, False)
    T = S * chunk
    qd = torch.randn(T, H * hd, device="cuda")
    out = torch.empty(T, H * hd, device="cuda")
    td = torch.from_numpy(tab.reshape(-1).astype(np.int32)).cuda()
    p = kb.PagedAttentionParams(S, H, KH, hd, bs, maxb, scale)
    cl, ql = np.array(ctx_lens, np.uint32), np.full(S, chunk, np.uint32)

    def step():
        for l in range(layers):
            pool.paged_attention_prefill(l, qd, td, cl, ql, out, p)
    # the call builds per-call row arrays on the host, so it is timed as plain launches (it
    # refuses to be captured in a graph)
    for _ in range(3):
        step()
    ctx.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iters = 10
    e0.record(stream)
    for _ in range(iters):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (iters * layers)
    # every query row walks its causal prefix: the records one launch touches, counted per row
    row_tokens = sum(int(c) - chunk + i + 1 for c in ctx_lens for i in range(chunk))
    flops = 4.0 * row_tokens * H * hd  # QK and PV
    res = {"check_vs_oracle_rel_err": err, "sequences": S, "chunk": chunk, "cached": cached,
           "us_per_launch": us, "query_rows_per_s": T / us * 1e6,
           "cache_GB/s_per_row_walk": row_tokens * KH * (2 * hd + 8) / us / 1e3,
           "GFLOP/s": flops / us / 1e3}
    pool.destroy()
    return res


def other_paths(torch, kb, O, ctx, stream, decode_batches=(1, 8, 32, 64), decode_only=False):
    """The other rows of the hot path, timed the same way as the headline (captured graph, CUDA
    events, weights rotated through more than the L2's 126 MB) and checked against the oracle
    before they are timed."""
    if decode_only:
        return {"cfg4_decode_smollm2_360m_q8_0": decode_legs(torch, kb, O, ctx, stream,
                                                              decode_batches, check=False)}
    return {"gemv": gemv_legs(torch, kb, ctx, stream),
            "cfg3_batched_gemm": gemm_legs(torch, kb, O, ctx, stream),
            "prefill_attention": prefill_attention_leg(torch, kb, O, ctx, stream),
            "cfg4_decode_smollm2_360m_q8_0": decode_legs(torch, kb, O, ctx, stream, decode_batches)}


CFG5_UP = (28672, 8192)    # rows (N), cols (K): Llama-3-70B-like FFN, BASELINE.json configs[4]
CFG5_DOWN = (8192, 28672)
CFG5_BLOCK = 3584          # rows of W_up / columns of W_down per generation block (1/8)


def _cfg5_blocks(oracle, rank, world):
    """This rank's shards of the cfg 5 matrices, generated in eighths seeded by their position
    in the full matrix, so that every N sees the same W_up and W_down."""
    per = 8 // world
    ups, downs = [], []
    for b in range(rank * per, (rank + 1) * per):
        rng = np.random.Generator(np.random.PCG64(SEED + 500 + b))
        ups.append(oracle.quantize_weights_q4_k(
            rng.standard_normal((CFG5_BLOCK, CFG5_UP[1]), dtype=np.float32) * np.float32(0.02)))
        d = oracle.quantize_weights_q4_k(
            rng.standard_normal((CFG5_DOWN[0], CFG5_BLOCK), dtype=np.float32) * np.float32(0.02))
        downs.append(d.reshape(CFG5_DOWN[0], -1))
    return np.concatenate(ups), np.ascontiguousarray(np.concatenate(downs, axis=1)).reshape(-1)


def _rotations(base, rows, copies, seed):
    """`copies` distinct block matrices: the base and row rotations of it (timing only)."""
    blocks = base.reshape(rows, -1)
    rng = np.random.Generator(np.random.PCG64(seed))
    return [base] + [np.ascontiguousarray(np.roll(blocks, int(rng.integers(1, rows)), axis=0))
                     .reshape(-1) for _ in range(copies - 1)]


def _event_time_us(torch, dist, stream, graph, iters, world):
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(iters):
        graph.replay()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms * 1e3 / iters


def _capture(torch, stream, fn):
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        fn()
    return g


def sharded_pair_check(torch, dist, kb, O, ctx, up, down, up_blocks, down_blocks, x, rows_total,
                       what):
    """The whole result of a sharded (up, down) pair against the oracle, on every rank: each
    rank computes ITS OWN contribution with the oracle (its rows of h = W_up.x, its partial of
    y = W_down.h) and the contributions are combined with NCCL collectives, independent of the
    library's own exchange. A mismatch ends the run."""
    M = x.shape[0]
    xd = torch.from_numpy(x).cuda()
    h_loc = up.forward(xd, M, local_only=True)
    y = down.forward(h_loc, M).clone()
    h_full = up.forward(xd, M).clone()
    ctx.sync()
    torch.cuda.synchronize()
    ref_h = O.gemm_q4_k(up_blocks, x, M, up.row_count, up.cols)
    ref_p = O.gemm_q4_k(down_blocks, ref_h, M, down.rows, down.col_count)
    parts = [torch.empty((M, up.row_count), device="cuda") for _ in range(up.world)]
    dist.all_gather(parts, torch.from_numpy(ref_h).cuda())
    ref_h_full = torch.cat(parts, dim=1)
    ref_y = torch.from_numpy(ref_p).cuda()
    dist.all_reduce(ref_y)
    e_h = float((h_full - ref_h_full).abs().max() / ref_h_full.abs().max())
    e_y = float((y - ref_y).abs().max() / ref_y.abs().max())
    if not (e_h <= 1e-3 and e_y <= 2e-3):
        raise SystemExit(f"bench: {what}: sharded result differs from the oracle "
                         f"(gathered up {e_h:.2e}, summed down {e_y:.2e})")
    return {"gathered_up_rel_err": e_h, "summed_down_rel_err": e_y}


def cfg5_sharded(torch, dist, kb, sh, O, ctx, stream, rank, world):
    """BASELINE.json configs[4]: W_up[28672x8192] split by output rows, W_down[8192x28672] split
    along K, Q4_K from N(0, 0.02), M in {1, 64}, strong scaling over this run's GPUs. Per M:
    microseconds per (up, down) pair, aggregate algorithmic GB/s, the same shards run without
    any exchange (what the exchange costs), the BASELINE wording with the gather of the up
    projection's output, and the full-size pair on one GPU of this run for the efficiency."""
    up0, down0 = _cfg5_blocks(O, rank, world)
    pair_bytes_rank = up0.nbytes + down0.nbytes
    copies = max(2, int(np.ceil(300e6 / pair_bytes_rank)))
    ups = _rotations(up0, CFG5_UP[0] // world, copies, SEED + 601)
    downs = _rotations(down0, CFG5_DOWN[0], copies, SEED + 602)
    region = 2 * copies * 64 * (CFG5_UP[0] + world * CFG5_DOWN[0]) * 4 + (8 << 20)
    S_up = [sh.RowShardedLinear(ctx, b, kb.DTYPE_Q4_K, *CFG5_UP, mode="fused", max_m=64,
                                presharded=True, region_bytes=region) for b in ups]
    S_down = [sh.KShardedLinear(ctx, b, kb.DTYPE_Q4_K, *CFG5_DOWN, mode="fused", max_m=64,
                                presharded=True, region_bytes=region) for b in downs]
    rng = np.random.Generator(np.random.PCG64(SEED + 603))
    out = {"shapes": "W_up[28672x8192] rows/N, W_down[8192x28672] K/N, Q4_K", "ring_pairs": copies}
    x1 = rng.standard_normal((1, CFG5_UP[1]), dtype=np.float32)
    out["check_M1"] = sharded_pair_check(torch, dist, kb, O, ctx, S_up[0], S_down[0], up0, down0,
                                         x1, CFG5_UP[0], "cfg5 M=1")
    alg = lambda M: (2 * CFG5_UP[0] * CFG5_UP[1] // QK_K * Q4K_BYTES +
                     4 * M * (CFG5_UP[1] + 2 * CFG5_UP[0] + CFG5_DOWN[0]))
    for M in (1, 64):
        x = rng.standard_normal((M, CFG5_UP[1]), dtype=np.float32)
        xd = torch.from_numpy(x).cuda()
        if M == 64:
            # rows of the batched result equal the single-row results (which are oracle-checked)
            yb = S_down[0].forward(S_up[0].forward(xd, M, local_only=True), M).clone()
            for m in (0, 31, 63):
                y1 = S_down[0].forward(S_up[0].forward(xd[m:m + 1], 1, local_only=True), 1)
                ctx.sync()
                e = float((yb[m] - y1[0]).abs().max() / y1.abs().max())
                if e > 2e-3:
                    raise SystemExit(f"bench: cfg5 M=64 row {m} differs from its GEMV by {e:.2e}")

        def pair_chain():
            for su, sd in zip(S_up, S_down):
                sd.forward(su.forward(xd, M, local_only=True), M)

        def pair_gather():
            for su, sd in zip(S_up, S_down):
                h = su.forward(xd, M)
                sd.forward(h[:, su.row_begin:su.row_begin + su.row_count].contiguous()
                           if world > 1 else h, M)

        W = [(kb.Weight(ctx, u, kb.DTYPE_Q4_K, CFG5_UP[0] // world, CFG5_UP[1]),
              kb.Weight(ctx, d, kb.DTYPE_Q4_K, CFG5_DOWN[0], CFG5_DOWN[1] // world))
             for u, d in zip(ups, downs)]
        h_l = torch.empty((M, CFG5_UP[0] // world), device="cuda")
        y_l = torch.empty((M, CFG5_DOWN[0]), device="cuda")

        def pair_local():
            for wu, wd in W:
                wu.forward(xd, h_l, M)
                wd.forward(h_l, y_l, M)

        res = {}
        for name, fn in (("chain", pair_chain), ("gather", pair_gather), ("no_exchange", pair_local)):
            g = _capture(torch, stream, fn)
            res[name] = _event_time_us(torch, dist, stream, g, 10, world) / copies
            ctx.sync()
        for wu, wd in W:
            wu.free()
            wd.free()
        out[f"M{M}"] = {
            "us_per_pair": res["chain"], "aggregate_GB/s": alg(M) / res["chain"] / 1e3,
            "us_per_pair_with_up_gather": res["gather"],
            "us_per_pair_no_exchange": res["no_exchange"],
            "exchange_share": max(0.0, 1.0 - res["no_exchange"] / res["chain"]),
        }
    # the full-size pair on ONE GPU of this run, for the strong-scaling efficiency
    if world > 1:
        full_bytes = world * pair_bytes_rank
        n1 = max(2, int(np.ceil(300e6 / full_bytes)))
        fu = [torch.randint(0, 255, (CFG5_UP[0] * CFG5_UP[1] // QK_K * Q4K_BYTES,),
                            dtype=torch.uint8, device="cuda") for _ in range(n1)]
        fd = [torch.randint(0, 255, (CFG5_UP[0] * CFG5_UP[1] // QK_K * Q4K_BYTES,),
                            dtype=torch.uint8, device="cuda") for _ in range(n1)]
        for t in fu + fd:
            v = t.view(-1, Q4K_BYTES)
            v[:, 1] = 0x1C
            v[:, 3] = 0x1C
        for M in (1, 64):
            xd = torch.randn(M, CFG5_UP[1], device="cuda")
            hf = torch.empty((M, CFG5_UP[0]), device="cuda")
            yf = torch.empty((M, CFG5_DOWN[0]), device="cuda")

            def full_pair():
                for a_, b_ in zip(fu, fd):
                    ctx.gemm_q4_k(a_, xd, hf, M, *CFG5_UP)
                    ctx.gemm_q4_k(b_, hf, yf, M, *CFG5_DOWN)
            g = _capture(torch, stream, full_pair)
            t1 = _event_time_us(torch, dist, stream, g, 10, world) / n1
            ctx.sync()
            out[f"M{M}"]["us_per_pair_1gpu_unsharded"] = t1
            out[f"M{M}"]["strong_scaling_efficiency"] = t1 / (world * out[f"M{M}"]["us_per_pair"])
        del fu, fd
    for s in S_up + S_down:
        s.destroy()
    return out


def run_sharded(args, torch, dist, kb, O, ctx, stream, rank, world, local):
    """N > 1: the sharded FFN pair. Headline = weak scaling at config 2's per-GPU shard sizes:
    W_up[N*14336 x 4096] split by output rows, W_down[4096 x N*14336] split along K, the up
    projection's slice staying on its rank as the K slice of the down projection (one exchange
    per pair, inside the library's kernels). The line also carries config 5 as BASELINE.json
    states it (strong scaling, M in {1, 64}) under `cfg5_sharded`."""
    sh = importlib.import_module("kanso-infer_b200").sharded
    sh.ShardGroup.get(ctx, dist.group.WORLD, region_bytes=3 << 29)
    pairs = args.pairs
    up0 = make_weights(O, *UP, SEED + 1 + 10 * rank)
    down0 = make_weights(O, *DOWN, SEED + 2 + 10 * rank)
    ups = ring_of_weights(up0, pairs, *UP, SEED + 11)
    downs = ring_of_weights(down0, pairs, *DOWN, SEED + 12)
    S_up = [sh.RowShardedLinear(ctx, b, kb.DTYPE_Q4_K, world * UP[0], UP[1], mode="fused", max_m=1,
                                presharded=True) for b in ups]
    S_down = [sh.KShardedLinear(ctx, b, kb.DTYPE_Q4_K, DOWN[0], world * DOWN[1], max_m=1,
                                presharded=True, mode="fused") for b in downs]
    rng = np.random.Generator(np.random.PCG64(SEED + 3))
    x = rng.standard_normal((1, UP[1]), dtype=np.float32)
    check = sharded_pair_check(torch, dist, kb, O, ctx, S_up[0], S_down[0], up0, down0, x,
                               world * UP[0], "headline pair")
    xd = torch.from_numpy(x).cuda()

    def step():
        for su, sd in zip(S_up, S_down):
            sd.forward(su.forward(xd, 1, local_only=True), 1)

    graph = _capture(torch, stream, step)
    for _ in range(max(3, args.warmup)):
        graph.replay()
    ctx.sync()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # The clock sampler needs a moment to start; the GPUs stay busy meanwhile (untimed replays, the
    # same count on every rank because the ranks' steps wait for one another), so that the timed
    # steps do not begin on GPUs that have just idled.
    for _ in range(1000):
        graph.replay()
    ctx.sync()
    us_step = _event_time_us(torch, dist, stream, graph, args.steps, world)
    for _ in range(200):  # keep the GPUs busy while the clock sampler collects
        graph.replay()
    ctx.sync()
    clocks = sampler.stop() if rank == 0 else None
    step_bytes = pairs * (alg_bytes(*UP) + alg_bytes(*DOWN))  # per rank
    value = world * step_bytes / us_step / 1e3

    # end to end through the sharded layers: x from pinned host memory, y back to host memory,
    # every pair synchronised, all ranks in step
    xh = torch.from_numpy(x).pin_memory()
    yh = torch.empty((1, DOWN[0]), dtype=torch.float32).pin_memory()
    x_stage = torch.empty_like(xd)

    def host_step():
        for su, sd in zip(S_up, S_down):
            x_stage.copy_(xh, non_blocking=True)
            yh.copy_(sd.forward(su.forward(x_stage, 1, local_only=True), 1), non_blocking=True)
            ctx.sync()

    host_step()
    dist.barrier()
    n_e2e = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        host_step()
    dt = time.perf_counter() - t0
    t = torch.tensor([dt], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dt = float(t.item())
    e2e = {"value": world * step_bytes * n_e2e / dt / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": world * pairs * 4 * UP[1],
           "d2h_bytes_per_step": world * pairs * 4 * DOWN[0], "steps": n_e2e,
           "us_per_pair": dt / (n_e2e * pairs) * 1e6,
           "path": "pinned x -> up (row shard, slice stays local) -> down (K shard, exchange + "
                   "sum) -> pinned y, one sync per pair, on every rank"}
    for s in S_up + S_down:
        s.destroy()
    cfg5 = None
    if not os.environ.get("KANSO_BENCH_SKIP_EXTRAS"):
        cfg5 = cfg5_sharded(torch, dist, kb, sh, O, ctx, stream, rank, world)
    if rank != 0:
        return
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    us_per_gemv = us_step / (2 * pairs)  # exchange and sum run inside the down GEMV's last CTA
    per_launch_bytes = (alg_bytes(*UP) + alg_bytes(*DOWN)) / 2
    achieved = per_launch_bytes / us_per_gemv / 1e3
    line = {
        "metric": "Q4_K GEMV HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": us_step / 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
        "data": "synthetic",
        "config": {
            "workload": f"sharded FFN pair, Q4_K batch 1, cfg2 shard sizes per GPU: "
                        f"W_up[{world * UP[0]}x{UP[1]}] split by rows over {world} GPUs -> "
                        f"W_down[{DOWN[0]}x{world * DOWN[1]}] split along K, partial sums "
                        "exchanged by peer stores and added on every rank",
            "ring_pairs": pairs, "bytes_per_step_per_gpu": step_bytes,
            "l2": f"inputs larger than L2: {step_bytes / 1e6:.0f} MB of distinct weights per "
                  "GPU per step vs 126 MB L2",
            "launch": "CUDA graph of the step (2 kernels per pair: up GEMV; down GEMV whose last "
                      "CTA stores its partial sums to every rank, signals, waits for the peers "
                      "and adds)",
            "parallelism": f"row shard -> K shard over {world} GPUs, no NCCL call on the data path",
            "pre_timing": "after the warm-up steps every rank replays the graph 1000 times "
                          "(untimed) while the clock sampler starts",
            "check_vs_oracle": check},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_source": peak_src, "traffic": None,
                     "kernel": "gemv_q4k_mma_kernel (exchange fused into its last CTA)",
                     "us_per_launch": us_per_gemv, "alg_bytes_per_launch": per_launch_bytes},
        "e2e": e2e, "gpu_launches": 2 * pairs * args.steps, "clocks": clocks,
    }
    if cfg5:
        line["cfg5_sharded"] = cfg5
    print(json.dumps(line))


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG", "WARN")  # NCCL's version banner goes to stdout
        # A rank that never joins (or a stalled exchange) would leave the others waiting for
        # ever: every rank ends itself after a deadline well beyond a normal run.
        deadline = threading.Timer(float(os.environ.get("KANSO_BENCH_DEADLINE_S", "600")),
                                   lambda: (sys.stderr.write("bench: deadline passed, exiting\n"),
                                            os._exit(3)))
        deadline.daemon = True
        deadline.start()
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    kb = importlib.import_module("kanso-infer_b200").backend
    from oracle import oracle as O  # the checker and the CPU baseline leg only
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx = kb.Context(local, stream)
    # the weights are uploaded once and never written again: let consecutive GEMVs overlap
    # their weight prefetch with the drain of the kernel before them
    if not os.environ.get("KANSO_BENCH_NO_OVERLAP"):
        ctx.set_option(kb.OPT_OVERLAP_WEIGHT_PREFETCH, 1)
    if world > 1:
        try:
            run_sharded(args, torch, dist, kb, O, ctx, stream, rank, world, local)
        finally:
            dist.destroy_process_group()
        return

    pairs = args.pairs
    up0 = make_weights(O, *UP, SEED + 1)
    down0 = make_weights(O, *DOWN, SEED + 2)
    ups = ring_of_weights(up0, pairs, *UP, SEED + 11)
    downs = ring_of_weights(down0, pairs, *DOWN, SEED + 12)
    rng = np.random.Generator(np.random.PCG64(SEED + 3))
    x_up = rng.standard_normal(UP[1]).astype(np.float32)
    x_down = rng.standard_normal(DOWN[1]).astype(np.float32)
    dx_up = torch.from_numpy(x_up).cuda()
    dx_down = torch.from_numpy(x_down).cuda()
    y_up = torch.empty(UP[0], dtype=torch.float32, device="cuda")
    y_down = torch.empty(DOWN[0], dtype=torch.float32, device="cuda")
    W_up = [kb.Weight(ctx, b, kb.DTYPE_Q4_K, *UP) for b in ups]
    W_down = [kb.Weight(ctx, b, kb.DTYPE_Q4_K, *DOWN) for b in downs]

    def step():
        for wu, wd in zip(W_up, W_down):
            wu.forward(dx_up, y_up, 1)
            wd.forward(dx_down, y_down, 1)

    # result check against the oracle on the last pair, both matrices (not timed)
    step()
    ctx.sync()
    errs = []
    for got, blocks, x, shape in ((y_up, ups[-1], x_up, UP), (y_down, downs[-1], x_down, DOWN)):
        ref = O.gemv_q4_k(blocks, x, *shape)
        errs.append(float(np.max(np.abs(got.cpu().numpy() - ref)) / np.max(np.abs(ref))))
    if max(errs) > 1e-3:
        raise SystemExit(f"bench: GEMV result differs from the oracle by {max(errs):.2e} (> 1e-3)")

    launches_per_step = 2 * pairs
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        step()
    for _ in range(max(3, args.warmup)):
        graph.replay()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    # The clock sampler needs a moment to start; the GPU stays busy meanwhile (untimed replays), so
    # that the timed steps do not begin on a GPU that has just idled for 0.3 s.
    t_busy = time.time() + 0.3
    while time.time() < t_busy:
        for _ in range(20):
            graph.replay()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        graph.replay()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    t_end = time.time() + 1.0  # keep the GPU busy while the sampler collects a few more rows
    while time.time() < t_end:
        graph.replay()
    torch.cuda.synchronize()
    clocks = sampler.stop()

    step_bytes = pairs * (alg_bytes(*UP) + alg_bytes(*DOWN))
    value = step_bytes * args.steps / (ms * 1e-3) / 1e9
    us_per_launch = ms * 1e3 / (args.steps * launches_per_step)

    # end to end through the host-buffer call: x from host memory, y back to host memory
    yh_up = np.empty(UP[0], np.float32)
    yh_down = np.empty(DOWN[0], np.float32)

    def host_step():
        for wu, wd in zip(W_up, W_down):
            wu.forward_host(x_up, yh_up, 1)
            wd.forward_host(x_down, yh_down, 1)

    host_step()
    host_step()
    if np.max(np.abs(yh_up - y_up.cpu().numpy())) > 1e-6 * np.max(np.abs(yh_up)):
        raise SystemExit("bench: the host-buffer call and the device call disagree")
    n_e2e = max(1, min(args.steps, 50))
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        host_step()
    dt = time.perf_counter() - t0
    e2e = {"value": step_bytes * n_e2e / dt / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": pairs * 4 * (UP[1] + DOWN[1]),
           "d2h_bytes_per_step": pairs * 4 * (UP[0] + DOWN[0]),
           "steps": n_e2e, "us_per_call": dt / (n_e2e * launches_per_step) * 1e6}

    peak, _, peak_src = _peaks()
    per_launch_bytes = (alg_bytes(*UP) + alg_bytes(*DOWN)) / 2
    achieved = per_launch_bytes / (us_per_launch * 1e-6) / 1e9
    cpu = (cpu_baseline_1core(O, up0, down0, [x_up, x_down])
           if not os.environ.get("KANSO_BENCH_SKIP_CPU") else None)
    line = {
        "metric": "Q4_K GEMV HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
        "data": "synthetic",
        "config": {"workload": "cfg2 Q4_K GEMV batch 1: W_up[14336x4096] + W_down[4096x14336]",
                   "ring_pairs": pairs, "bytes_per_step": step_bytes,
                   "l2": f"inputs larger than L2: {step_bytes / 1e6:.0f} MB of distinct weights "
                         "per step vs 126 MB L2",
                   "launch": "CUDA graph of the step", "parallelism": "shards1",
                   "pre_timing": "after the warm-up steps the graph keeps replaying (untimed) for "
                                 "0.3 s while the clock sampler starts",
                   "check_vs_oracle_rel_err": {"up": errs[0], "down": errs[1]}},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_source": peak_src,
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "kernel": "gemv_q4k_mma_kernel",
                     "us_per_launch": us_per_launch, "alg_bytes_per_launch": per_launch_bytes},
        "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
    }
    if cpu:
        line["cpu_baseline"] = cpu
    for w_ in W_up + W_down:
        w_.free()
    if not os.environ.get("KANSO_BENCH_SKIP_EXTRAS"):
        # not part of the headline value: the remaining rows of the path, for the record
        line["other_paths"] = other_paths(torch, kb, O, ctx, stream)
    print(json.dumps(line))


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
                    help="run only the cfg 3 GEMM (q8_0, q4_k, or q8_0_q8 for Q8 activations; N=14336, K=4096) with M activation "
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
        act = kb.ACT_Q8 if fmt.endswith("_q8") else kb.ACT_F32  # q8_0_q8: Q8 activations
        fmt = fmt[:-3] if fmt.endswith("_q8") else fmt
        dtype = kb.DTYPE_Q8_0 if fmt == "q8_0" else kb.DTYPE_Q4_K
        ws = _random_blocks(torch, kb, dtype, 14336, 4096, 4)
        x = torch.randn(M, 4096, device="cuda")
        y = torch.empty(M, 14336, device="cuda")
        for w in ws:
            (ctx.gemm_q8_0 if dtype == kb.DTYPE_Q8_0 else ctx.gemm_q4_k)(w, x, y, M, 14336, 4096,
                                                                         act)
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
        from oracle import oracle as O
        print(json.dumps(other_paths(torch, kb, O, ctx, stream, batches, decode_only=True)))
        return
    if args.impl == "reference":
        if args.steps > 50:
            args.steps = 50  # bounded sample: one CPU step over the ring takes a fraction of a second
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
