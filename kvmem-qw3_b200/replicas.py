"""Host logic of the multi-GPU form of the path: independent request replicas, no data-path collective.

Requests never exchange data, so N GPUs run N replicas of the step (one process per GPU).  The only
communication is bookkeeping: which requests a rank serves, and the whole-job figure (tokens of all ranks
over the slowest rank's device time).
"""
import numpy as np


def shard_requests(n_requests, world, rank):
    """Request ids served by `rank`: contiguous, sizes differ by at most one."""
    base, extra = divmod(n_requests, world)
    start = rank * base + min(rank, extra)
    return list(range(start, start + base + (1 if rank < extra else 0)))


def aggregate(dist, times_ms, counts):
    """max over ranks of every entry of times_ms, sum over ranks of every entry of counts.
    dist is torch.distributed (initialised) or None for a single process."""
    t = np.asarray(times_ms, np.float64)
    c = np.asarray(counts, np.float64)
    if dist is None:
        return t, c
    import torch
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    tt = torch.tensor(t, dtype=torch.float64, device=dev)
    cc = torch.tensor(c, dtype=torch.float64, device=dev)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    dist.all_reduce(cc, op=dist.ReduceOp.SUM)
    return tt.cpu().numpy(), cc.cpu().numpy()


def throughput(total_tokens, max_ms):
    return float(total_tokens) / (float(max_ms) * 1e-3)
