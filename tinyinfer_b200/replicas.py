"""Replica arithmetic for multi-GPU runs: the decode path has no exchange step, so N GPUs are N
independent copies of the model, each with its own share of the requests.  What remains to be agreed
between ranks is bookkeeping: which requests a rank owns, and the job-level time and throughput
(slowest rank's time, sum of all ranks' units).  Works on any torch.distributed backend (NCCL on
GPUs, gloo in the CPU tests)."""
from __future__ import annotations


def shard(items, rank, world):
    """Round-robin ownership: request i belongs to rank i % world (every rank computes the same answer)."""
    if not 0 <= rank < world:
        raise ValueError("rank outside world")
    return list(items)[rank::world]


def job_throughput(local_units, local_seconds, dist=None, device=None):
    """(total units of all ranks, max seconds over ranks, units per second of the whole job)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return local_units, local_seconds, (local_units / local_seconds if local_seconds > 0 else 0.0)
    import torch
    units = torch.tensor([float(local_units)], dtype=torch.float64, device=device)
    seconds = torch.tensor([float(local_seconds)], dtype=torch.float64, device=device)
    dist.all_reduce(units, op=dist.ReduceOp.SUM)
    dist.all_reduce(seconds, op=dist.ReduceOp.MAX)
    total, slowest = float(units.item()), float(seconds.item())
    return total, slowest, (total / slowest if slowest > 0 else 0.0)
