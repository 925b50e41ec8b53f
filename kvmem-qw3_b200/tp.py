"""Tensor-parallel FFN pair: shard planning and the group object over qb_tp_*.

The FFN dimension F is split over `world` ranks in whole Q8_0 blocks: rank r owns gate/up rows
[r*F/world, (r+1)*F/world) (column-parallel, fused as [gate_r; up_r]) and the matching K slice of down
(row-parallel).  The [M][n_out] results of the ranks are added in rank order by the library's one-shot
all-reduce over peer memory (see include/qw3b200.h, "tensor-parallel FFN pair").

Plumbing only lives here: the IPC handles of the receive areas travel through torch.distributed
(all_gather_object), everything on the data path is the CUDA library.
"""
import ctypes as C

import numpy as np

from . import binding as B

Q8_BLOCK = 34    # bytes of one Q8_0 block (fp16 scale + 32 int8)


def shard_bounds(F, world, rank):
    """Rows [lo, hi) of the FFN dimension owned by `rank`; F/world must be a whole number of 128-row tiles."""
    if F % world or (F // world) % 128:
        raise ValueError("FFN dimension %d does not split into %d shards of whole 128-row tiles" % (F, world))
    f = F // world
    return rank * f, (rank + 1) * f


def shard_blocks(gate, up, down, F, H, n_out, world, rank):
    """Host Q8_0 blocks (uint8 arrays: gate/up [F][H/32][34], down [n_out][F/32][34]) of one rank's shard:
    returns (gate_up_shard [2f][H/32][34], down_shard [n_out][f/32][34])."""
    lo, hi = shard_bounds(F, world, rank)
    g = np.asarray(gate, np.uint8).reshape(F, H // 32, Q8_BLOCK)
    u = np.asarray(up, np.uint8).reshape(F, H // 32, Q8_BLOCK)
    d = np.asarray(down, np.uint8).reshape(n_out, F // 32, Q8_BLOCK)
    gu = np.ascontiguousarray(np.concatenate([g[lo:hi], u[lo:hi]], axis=0))
    dn = np.ascontiguousarray(d[:, lo // 32:hi // 32])
    return gu, dn


class TpGroup:
    """One rank's end of the tensor-parallel FFN.  recv_ptrs: device pointers (ints or c_void_p) of every rank's
    receive area, this rank's own at index `rank`."""

    def __init__(self, ctx, rank, world, recv_ptrs, max_rows, n_in, f_shard, n_out):
        self.ctx, self.rank, self.world = ctx, rank, world
        self.max_rows, self.n_in, self.f_shard, self.n_out = max_rows, n_in, f_shard, n_out
        arr = (B.vp * world)(*[p if isinstance(p, B.vp) else B.vp(p) for p in recv_ptrs])
        h = B.vp()
        B.check(B.lib().qb_tp_group_create(ctx.h, rank, world, arr, max_rows, n_in, f_shard, n_out, C.byref(h)))
        self.h = h

    @staticmethod
    def recv_bytes(world, max_rows, n_out, f_shard):
        return int(B.lib().qb_tp_recv_bytes(world, max_rows, n_out, f_shard))

    def push(self, gate_up, down, x_dev, M):
        B.check(B.lib().qb_tp_ffn_push(self.ctx.h, self.h, gate_up.h, down.h, x_dev.ptr, M))

    def reduce(self, M, y_dev):
        B.check(B.lib().qb_tp_ffn_reduce(self.ctx.h, self.h, M, y_dev.ptr, self.n_out))

    def ffn(self, gate_up, down, x_dev, M, y_dev):
        B.check(B.lib().qb_tp_ffn(self.ctx.h, self.h, gate_up.h, down.h, x_dev.ptr, M, y_dev.ptr, self.n_out))

    def close(self):
        if self.h:
            B.lib().qb_tp_group_destroy(self.ctx.h, self.h)
            self.h = None


def local_groups(ctx, world, max_rows, n_in, f_shard, n_out):
    """All ranks of a group inside ONE process on one GPU (tests of the data path and of the summation order:
    every rank's push is queued before any reduce, so no reduce ever waits)."""
    nbytes = TpGroup.recv_bytes(world, max_rows, n_out, f_shard)
    areas = [ctx.empty((nbytes,), np.uint8) for _ in range(world)]
    ptrs = [a.ptr for a in areas]
    return [TpGroup(ctx, r, world, ptrs, max_rows, n_in, f_shard, n_out) for r in range(world)], areas


def ipc_group(ctx, dist, max_rows, n_in, f_shard, n_out):
    """One process per GPU: allocate this rank's receive area, exchange IPC handles through torch.distributed,
    map the peers' areas and create the group.  Returns (group, own_area, peer_ptrs)."""
    rank, world = dist.get_rank(), dist.get_world_size()
    nbytes = TpGroup.recv_bytes(world, max_rows, n_out, f_shard)
    area = ctx.empty((nbytes,), np.uint8)
    handle = (C.c_ubyte * 64)()
    B.check(B.lib().qb_ipc_export(ctx.h, area.ptr, handle))
    handles = [None] * world
    dist.all_gather_object(handles, bytes(handle))
    ptrs, opened = [], []
    for r in range(world):
        if r == rank:
            ptrs.append(area.ptr)
            continue
        p = B.vp()
        buf = (C.c_ubyte * 64).from_buffer_copy(handles[r])
        B.check(B.lib().qb_ipc_open(ctx.h, buf, C.byref(p)))
        ptrs.append(p)
        opened.append(p)
    g = TpGroup(ctx, rank, world, ptrs, max_rows, n_in, f_shard, n_out)
    dist.barrier()      # every rank has zeroed its arrival counters before anyone pushes
    return g, area, opened


def ipc_release(ctx, opened):
    for p in opened:
        B.lib().qb_ipc_close(ctx.h, p)
