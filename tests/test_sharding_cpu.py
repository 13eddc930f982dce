"""Multi-GPU host logic on CPU: two gloo ranks shard sessions and reduce the timing results the way
bench.py does under torchrun (sum of tokens, maximum of times), with no data-path collective."""
import os
import socket
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank: int, world: int, port: int, results):
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        package = entry.load_package()
        shard = package.sharding.session_shard(7, world, rank)
        ids, lengths, batches = package.sharding.plan_sessions(7, world, rank, 3, 5, 256, 8192)
        assert ids == list(shard) and len(lengths) == len(ids)
        assert [i for batch in batches for i in batch] == list(range(len(ids))) and max(map(len, batches)) <= 3
        # each rank "emits" 10 tokens per owned session and takes (rank + 1) * 100 ms
        counts, times = package.sharding.aggregate(dist, torch, [10 * len(shard), len(shard)], [100.0 * (rank + 1), 1.0],
                                                   "cpu")
        dist.barrier()
        results[rank] = (list(shard), counts, times, package.sharding.throughput(counts[0], times[0]))
    finally:
        dist.destroy_process_group()


def test_session_shard_covers_every_session_once():
    import __graft_entry__ as entry

    sharding = entry.load_package().sharding
    for total in (0, 1, 7, 64):
        for world in (1, 2, 3, 4, 8):
            owned = [i for rank in range(world) for i in sharding.session_shard(total, world, rank)]
            assert owned == list(range(total))
            sizes = [len(sharding.session_shard(total, world, rank)) for rank in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.session_shard(4, 2, 2)
    with pytest.raises(ValueError):
        sharding.throughput(1.0, 0.0)


@pytest.mark.timeout(120)
def test_two_gloo_ranks_reduce_like_the_benchmark():
    import torch.multiprocessing as mp

    world, port = 2, free_port()
    manager = mp.get_context("spawn").Manager()
    results = manager.dict()
    mp.spawn(worker, args=(world, port, results), nprocs=world, join=True)
    assert sorted(results.keys()) == [0, 1]
    shard0, counts0, times0, value0 = results[0]
    shard1, counts1, times1, value1 = results[1]
    assert shard0 == [0, 1, 2, 3] and shard1 == [4, 5, 6]          # the remainder goes to the low rank
    assert counts0 == counts1 == [70.0, 7.0]                       # summed over ranks
    assert times0 == times1 == [200.0, 1.0]                        # the slowest rank's time
    assert value0 == value1 == pytest.approx(70.0 / 0.2)           # whole-job tokens per second


def test_session_plan_is_the_same_on_every_rank_and_acceptance_follows_the_mask():
    import numpy as np

    import __graft_entry__ as entry

    sharding = entry.load_package().sharding
    everything = sharding.plan_sessions(64, 1, 0, 3, 5, 256, 8192)
    assert len(everything[0]) == 64 and min(everything[1]) >= 256 and max(everything[1]) <= 8192
    assert len(everything[2]) == 22 and len(everything[2][-1]) == 1
    seen = {}
    for rank in range(4):
        ids, lengths, batches = sharding.plan_sessions(64, 4, rank, 3, 5, 256, 8192)
        assert len(ids) == 16 and [len(b) for b in batches] == [3, 3, 3, 3, 3, 1]
        for session, length in zip(ids, lengths):
            assert length == everything[1][session]               # the same seeded lengths on every rank
            seen[session] = length
    assert len(seen) == 64
    mask = np.zeros(64, dtype=bool)
    mask[[3, 4, 20]] = True
    # offset 0: drafts 1,2 accepted, 3 substituted -> 3; offset 3: draft 4 substituted -> 1; offset 4: 5..8 fine -> 5
    assert sharding.simulate_accepts(mask, 5, 3, 100) == [3, 1, 5]
    assert sharding.simulate_accepts(mask, 5, 4, 2) == [3, 1, 3, 1]                # rewinds after `budget` steps
    with pytest.raises(ValueError):
        sharding.plan_sessions(4, 1, 0, 0, 1, 1, 2)
