"""Host-side sharding of independent sessions over GPUs (one process per GPU, no data-path collective).

A session's verify step touches only the shared immutable weights and its own KV cache and control block
(ref: docs/architecture.md:83-91), so N GPUs run N replicas of the prepared weights and disjoint sets of
sessions. The only communication is the reduction of the timing results: tokens are summed, times are
maximised, and throughput is total tokens over the slowest rank's time.
"""
from __future__ import annotations


def session_shard(total_sessions: int, world: int, rank: int) -> range:
    """Sessions [begin, end) owned by `rank`: an even split, the remainder going to the lowest ranks."""
    if world < 1 or not 0 <= rank < world or total_sessions < 0:
        raise ValueError("invalid shard request")
    base, extra = divmod(total_sessions, world)
    begin = rank * base + min(rank, extra)
    return range(begin, begin + base + (1 if rank < extra else 0))


def aggregate(dist, torch, counts, times_ms, device):
    """Sum `counts` and maximise `times_ms` over the ranks of `dist` (None = single process).

    Returns (counts, times_ms) as lists of floats, identical on every rank.
    """
    totals = torch.tensor([float(c) for c in counts], dtype=torch.float64, device=device)
    slowest = torch.tensor([float(t) for t in times_ms], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(totals, op=dist.ReduceOp.SUM)
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
    return totals.cpu().tolist(), slowest.cpu().tolist()


def throughput(total_count: float, slowest_ms: float) -> float:
    """Whole-job units per second."""
    if slowest_ms <= 0:
        raise ValueError("elapsed time must be positive")
    return total_count / (slowest_ms * 1e-3)
