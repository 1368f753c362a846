"""Test and measurement binding of the sharded layers: one process per GPU.

Everything that matters lives behind the C ABI (kanso_cuda_shard_group_*,
kanso_cuda_sharded_linear_*: peer-visible memory, the two-buffer exchange protocol, the
forward call). This module only (1) carries the 64-byte memory handles between the ranks
with torch.distributed, which is the one thing the library leaves to its caller, (2) slices
block bytes with the library's host helpers, and (3) keeps an NCCL form of the same layers
(mode="nccl": local matmul + all_gather / all_reduce) as the baseline to compare with.

Row sharding (W_up): rank r holds a contiguous range of output rows. K sharding (W_down): rank r
holds the blocks of a contiguous range of columns, re-packed; partial results are summed.
No arithmetic here.
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


class ShardGroup:
    """kanso_cuda_shard_group for a torch.distributed process group."""

    _by_group = {}

    @classmethod
    def get(cls, ctx, group, region_bytes=256 << 20):
        key = (id(ctx), group.group_name)
        if key not in cls._by_group:
            cls._by_group[key] = cls(ctx, group, region_bytes)
        return cls._by_group[key]

    def __init__(self, ctx, group, region_bytes=256 << 20):
        import torch
        import torch.distributed as dist
        self.ctx, self.group = ctx, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        h = C.c_void_p()
        mine = (C.c_ubyte * kb.SHARD_HANDLE_BYTES)()
        ctx.call("kanso_cuda_shard_group_create", self.rank, self.world, region_bytes,
                 C.byref(h), C.cast(mine, C.c_void_p))
        self.h = h
        # the caller's part: every rank learns every rank's handle
        t = torch.tensor(list(mine), dtype=torch.uint8)
        if dist.get_backend(group) == "nccl":
            t = t.cuda()
        gathered = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(gathered, t, group=group)
        blob = bytes(torch.cat([g.cpu() for g in gathered]).tolist())
        self._blob = C.create_string_buffer(blob, len(blob))
        ctx.check(ctx.lib.kanso_cuda_shard_group_connect(self.h, C.cast(self._blob, C.c_void_p)))
        dist.barrier(group=group)  # every rank has mapped its peers before anyone stores

    def destroy(self):
        if getattr(self, "h", None):
            self.ctx.lib.kanso_cuda_shard_group_destroy(self.h)
            self.h = None


class _ShardedBase:
    def _create(self, ctx, shard, dtype, rows, cols, mode_c, max_m, group, region_bytes):
        self.sg = ShardGroup.get(ctx, group, region_bytes)
        h = C.c_void_p()
        shard = np.ascontiguousarray(shard, np.uint8)
        ctx.check(ctx.lib.kanso_cuda_sharded_linear_create(
            self.sg.h, shard.ctypes.data, shard.nbytes, dtype, rows, cols, mode_c, max_m,
            C.byref(h)))
        self.h = h

    def _forward(self, x, M, act_mode, flags, width):
        import torch
        out = C.c_void_p()
        self.ctx.check(self.ctx.lib.kanso_cuda_sharded_linear_forward(
            self.h, kb._ptr(x), M, act_mode, flags, C.byref(out)))
        return _device_view(torch, out.value, M, width)

    def destroy(self):
        if getattr(self, "h", None):
            self.ctx.lib.kanso_cuda_sharded_linear_destroy(self.h)
            self.h = None


def _device_view(torch, ptr, rows, cols):
    """A torch view of rows x cols f32 at a device address the library owns."""
    class _Arr:
        __cuda_array_interface__ = {"shape": (rows, cols), "typestr": "<f4", "data": (ptr, False),
                                    "version": 3}
    return torch.as_tensor(_Arr(), device="cuda")


class RowShardedLinear(_ShardedBase):
    """W[rows x cols] split by output rows; forward returns the full y on every rank, or with
    local_only=True this rank's rows only (no exchange)."""

    def __init__(self, ctx: kb.Context, blocks, dtype, rows, cols, group=None, mode="fused",
                 max_m=8, presharded=False, region_bytes=256 << 20):
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
        self.max_m = max_m
        counts = [shard_range(rows, r, self.world, 8)[1] for r in range(self.world)]
        self.even = len(set(counts)) == 1
        if mode == "fused":
            self._create(ctx, shard, dtype, rows, cols, kb.SHARD_ROWS, max_m, self.group,
                         region_bytes)
        elif mode == "nccl":
            self.weight = kb.Weight(ctx, shard, dtype, self.row_count, cols)
            self.y_full = torch.empty((max_m, rows), dtype=torch.float32, device="cuda")
            self.y_local = torch.empty((max_m, self.row_count), dtype=torch.float32, device="cuda")
        else:
            raise ValueError(mode)

    def forward(self, x, M=1, act_mode=kb.ACT_F32, local_only=False):
        """x: device f32 [M, cols]. Returns a view f32 [M, rows] (or [M, row_count])."""
        import torch.distributed as dist
        if M > self.max_m:
            raise kb.KansoError(kb.ERR_SHAPE, f"M {M} exceeds the buffers sized for {self.max_m}")
        if self.mode == "fused":
            if local_only:
                return self._forward(x, M, act_mode, kb.SHARD_LOCAL_ONLY, self.row_count)
            return self._forward(x, M, act_mode, 0, self.rows)
        y_local = self.y_local[:M]
        self.weight.forward(x, y_local, M, act_mode)
        if local_only:
            return y_local
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


class KShardedLinear(_ShardedBase):
    """W[rows x cols] split along K; forward takes this rank's slice of x and returns the
    summed y on every rank."""

    def __init__(self, ctx: kb.Context, blocks, dtype, rows, cols, group=None, max_m=8,
                 presharded=False, mode="nccl", region_bytes=256 << 20):
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
        self.max_m = max_m
        if mode == "fused":
            self._create(ctx, shard, dtype, rows, cols, kb.SHARD_K, max_m, self.group,
                         region_bytes)
        elif mode == "nccl":
            self.weight = kb.Weight(ctx, shard, dtype, rows, self.col_count)
            self.y = torch.empty((max_m, rows), dtype=torch.float32, device="cuda")
        else:
            raise ValueError(mode)

    def forward(self, x_slice, M=1, act_mode=kb.ACT_F32):
        """x_slice: device f32 [M, col_count] = columns [col_begin, col_begin + col_count) of x."""
        import torch.distributed as dist
        if self.mode == "fused":
            return self._forward(x_slice, M, act_mode, 0, self.rows)
        y = self.y[:M]
        self.weight.forward(x_slice, y, M, act_mode)
        dist.all_reduce(y, group=self.group)
        return y
