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


def plan_sessions(total_sessions: int, world: int, rank: int, stack: int, seed: int, shortest: int, longest: int):
    """The sessions one rank serves and how it stacks them into forwards.

    Every rank derives the same seeded prompt lengths (uniform in [shortest, longest]) for all sessions, takes its
    shard, and groups its sessions into batches of `stack` (the last batch may be smaller) that are verified by
    one forward each. Returns (ids, lengths, batches): ids of the owned sessions, their prompt lengths, and the
    batches as lists of positions into `ids`."""
    import numpy as np

    if stack < 1 or shortest < 1 or longest < shortest:
        raise ValueError("invalid session plan")
    lengths = np.random.default_rng(seed).integers(shortest, longest + 1, size=total_sessions)
    ids = list(session_shard(total_sessions, world, rank))
    batches = [list(range(first, min(first + stack, len(ids)))) for first in range(0, len(ids), stack)]
    return ids, [int(lengths[i]) for i in ids], batches


def simulate_accepts(substituted, rows: int, steps: int, budget: int):
    """Accept lengths of `steps` greedy verify steps whose drafts are the exact greedy continuation except where
    `substituted[i]` is true (position i of the continuation was replaced by a random id). Acceptance then depends
    on the substitution mask alone: a step at continuation offset i emits 1 + the number of leading unsubstituted
    drafts among positions i+1 .. i+rows-1 (a random replacement equals the true token with probability 1 / vocab:
    ignored). `budget` steps are run before the walk rewinds to offset 0, as the benchmark loop does.
    Returns the list of emitted counts."""
    emitted, done = [], 0
    while done < steps:
        offset = 0
        for _ in range(min(steps - done, budget)):
            count = 1
            while count < rows and not substituted[offset + count]:
                count += 1
            emitted.append(count)
            offset += count
            done += 1
    return emitted
