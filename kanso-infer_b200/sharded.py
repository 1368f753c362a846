"""One linear layer sharded over the GPUs of a node: one process per GPU, NCCL for plumbing.

Row sharding (W_up): rank r holds a contiguous range of output rows; y is assembled either by
an NCCL all-gather ("nccl") or by the matmul kernel itself storing its slice into every
peer's result buffer over NVLink ("fused", symmetric memory + one cross-GPU barrier).
K sharding (W_down): rank r holds the blocks of a contiguous range of columns, re-packed;
partial results are summed with an NCCL all-reduce ("nccl") or exchanged by the matmul
kernel's own peer stores and added locally in rank order ("fused").

The fused modes alternate between two symmetric buffers: a rank that is one call ahead of a
peer then never stores into the buffer that peer is still reading.

This module holds no arithmetic: slicing of block bytes and calls into the C ABI.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import backend as kb

_BLOCK = {kb.DTYPE_Q8_0: (32, kb.Q8_BYTES), kb.DTYPE_Q4_K: (256, kb.Q4K_BYTES)}


def shard_range(n: int, rank: int, world: int, align: int):
    """(begin, count) of rank's part of [0, n), in multiples of `align`."""
    b, c = C.c_int64(0), C.c_int64(0)
    st = kb.load().kanso_cuda_shard_range(n, rank, world, align, C.byref(b), C.byref(c))
    if st != kb.OK:
        raise kb.KansoError(st, f"shard_range: {n} is not a multiple of {align}, or bad rank "
                                f"{rank}/{world}")
    return b.value, c.value


def row_shard(blocks: np.ndarray, dtype: int, rows: int, cols: int, rank: int, world: int):
    """Bytes of rank's output rows: (shard_bytes, row_begin, row_count). Rows go in groups of 8."""
    blk, bb = _BLOCK[dtype]
    begin, count = shard_range(rows, rank, world, 8)
    row_bytes = cols // blk * bb
    return (np.ascontiguousarray(blocks[begin * row_bytes:(begin + count) * row_bytes]), begin,
            count)


def k_shard(blocks: np.ndarray, dtype: int, rows: int, cols: int, rank: int, world: int):
    """Rank's columns of every row, re-packed: (shard_bytes, col_begin, col_count)."""
    blk, bb = _BLOCK[dtype]
    begin, count = shard_range(cols, rank, world, blk)
    out = np.empty(rows * (count // blk) * bb, np.uint8)
    blocks = np.ascontiguousarray(blocks, np.uint8)
    st = kb.load().kanso_cuda_shard_k_repack(blocks.ctypes.data, dtype, rows, cols, begin, count,
                                             out.ctypes.data, out.nbytes)
    if st != kb.OK:
        raise kb.KansoError(st, "shard_k_repack: column range does not fall on block boundaries")
    return out, begin, count


class PeerExchange:
    """The flag arrays and step counter of kanso_cuda_peer_exchange for one process group:
    the cross-GPU barrier of the fused sharded layers as a kernel on the context's stream."""

    _by_group = {}

    @classmethod
    def get(cls, ctx, group):
        key = (id(ctx), group.group_name)
        if key not in cls._by_group:
            cls._by_group[key] = cls(ctx, group)
        return cls._by_group[key]

    def __init__(self, ctx, group):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.ctx = ctx
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise kb.KansoError(kb.ERR_UNSUPPORTED, "peer exchange: at most 8 ranks")
        self.flags = symm.empty((self.world,), dtype=torch.int64, device="cuda")
        self.flags.zero_()
        self._hdl = symm.rendezvous(self.flags, group.group_name)
        self._ptrs = (C.c_void_p * self.world)(*[int(p) for p in self._hdl.buffer_ptrs])
        self.step = torch.zeros(1, dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        dist.barrier(group=group)  # every rank's flags are zero before anyone signals

    def __call__(self):
        self.ctx.call("kanso_cuda_peer_exchange", C.cast(self._ptrs, C.c_void_p),
                      kb._ptr(self.step), self.world, self.rank)


class RowShardedLinear:
    """W[rows x cols] split by output rows; forward returns the full y on every rank."""

    def __init__(self, ctx: kb.Context, blocks, dtype, rows, cols, group=None, mode="fused",
                 max_m=8, presharded=False):
        """blocks: the whole [rows x cols] block matrix, or with presharded=True only this
        rank's rows (rows is always the total)."""
        import torch
        import torch.distributed as dist
        self.ctx, self.rows, self.cols, self.mode = ctx, rows, cols, mode
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if presharded:
            self.row_begin, self.row_count = shard_range(rows, self.rank, self.world, 8)
            shard = blocks
        else:
            shard, self.row_begin, self.row_count = row_shard(blocks, dtype, rows, cols,
                                                              self.rank, self.world)
        self.weight = kb.Weight(ctx, shard, dtype, self.row_count, cols)
        self.max_m = max_m
        counts = [shard_range(rows, r, self.world, 8)[1] for r in range(self.world)]
        self.even = len(set(counts)) == 1
        if mode == "fused":
            import torch.distributed._symmetric_memory as symm
            self._bufs, self._hdls, self._ptrs, self._turn = [], [], [], 0
            for _ in range(2):
                buf = symm.empty((max_m, rows), dtype=torch.float32, device="cuda")
                hdl = symm.rendezvous(buf, self.group.group_name)
                self._bufs.append(buf)
                self._hdls.append(hdl)
                self._ptrs.append((C.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs]))
            self.y_full = self._bufs[0]
            self._exchange = PeerExchange.get(ctx, self.group)
        elif mode == "nccl":
            self.y_full = torch.empty((max_m, rows), dtype=torch.float32, device="cuda")
            self.y_local = torch.empty((max_m, self.row_count), dtype=torch.float32, device="cuda")
        else:
            raise ValueError(mode)

    def forward(self, x, M=1, act_mode=kb.ACT_F32):
        """x: device f32 [M, cols]. Returns a view f32 [M, rows] valid on this rank."""
        import torch.distributed as dist
        if M > self.max_m:
            raise kb.KansoError(kb.ERR_SHAPE, f"M {M} exceeds the buffers sized for {self.max_m}")
        if self.mode == "fused":
            # every rank stores its slice into every rank's y_full, then one exchange
            t = self._turn
            self._turn ^= 1
            self.ctx.call("kanso_cuda_linear_scatter_out", self.weight.h, kb._ptr(x), M,
                          C.cast(self._ptrs[t], C.c_void_p), self.world, self.rows,
                          self.row_begin, act_mode)
            self._exchange()
            self.y_full = self._bufs[t]
            return self.y_full[:M]
        y_local = self.y_local[:M]
        self.weight.forward(x, y_local, M, act_mode)
        if M == 1 and self.even:
            dist.all_gather_into_tensor(self.y_full[0], y_local[0], group=self.group)
        else:
            parts = [self.y_full.new_empty((M, shard_range(self.rows, r, self.world, 8)[1]))
                     for r in range(self.world)]
            dist.all_gather(parts, y_local.contiguous(), group=self.group)
            off = 0
            for p in parts:
                self.y_full[:M, off:off + p.shape[1]] = p
                off += p.shape[1]
        return self.y_full[:M]


class KShardedLinear:
    """W[rows x cols] split along K; forward takes this rank's slice of x and returns the
    summed y on every rank (all-reduce)."""

    def __init__(self, ctx: kb.Context, blocks, dtype, rows, cols, group=None, max_m=8,
                 presharded=False, mode="nccl"):
        """blocks: the whole block matrix, or with presharded=True this rank's re-packed
        [rows x cols/world] columns (cols is always the total)."""
        import torch
        import torch.distributed as dist
        self.ctx, self.rows, self.cols, self.mode = ctx, rows, cols, mode
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if presharded:
            self.col_begin, self.col_count = shard_range(cols, self.rank, self.world,
                                                         _BLOCK[dtype][0])
            shard = blocks
        else:
            shard, self.col_begin, self.col_count = k_shard(blocks, dtype, rows, cols, self.rank,
                                                            self.world)
        self.weight = kb.Weight(ctx, shard, dtype, rows, self.col_count)
        self.y = torch.empty((max_m, rows), dtype=torch.float32, device="cuda")
        self.max_m = max_m
        if mode == "fused":
            if self.world > 8:
                raise kb.KansoError(kb.ERR_UNSUPPORTED, "fused K sharding: at most 8 ranks")
            import torch.distributed._symmetric_memory as symm
            self._bufs, self._hdls, self._ptrs, self._turn = [], [], [], 0
            for _ in range(2):
                buf = symm.empty((max_m, self.world * rows), dtype=torch.float32, device="cuda")
                hdl = symm.rendezvous(buf, self.group.group_name)
                self._bufs.append(buf)
                self._hdls.append(hdl)
                self._ptrs.append((C.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs]))
            self._exchange = PeerExchange.get(ctx, self.group)
        elif mode != "nccl":
            raise ValueError(mode)

    def forward(self, x_slice, M=1, act_mode=kb.ACT_F32):
        """x_slice: device f32 [M, col_count] = columns [col_begin, col_begin + col_count) of x."""
        import torch.distributed as dist
        y = self.y[:M]
        if self.mode == "fused":
            # every rank stores its partial y into its slice of every rank's buffer; after
            # one exchange each rank adds the slices itself, in rank order
            t = self._turn
            self._turn ^= 1
            self.ctx.call("kanso_cuda_linear_scatter_out", self.weight.h, kb._ptr(x_slice), M,
                          C.cast(self._ptrs[t], C.c_void_p), self.world, self.world * self.rows,
                          self.rank * self.rows, act_mode)
            self._exchange()
            self.ctx.call("kanso_cuda_sum_shards", kb._ptr(self._bufs[t]), M, self.rows,
                          self.world, kb._ptr(y))
            return y
        self.weight.forward(x_slice, y, M, act_mode)
        dist.all_reduce(y, group=self.group)
        return y
