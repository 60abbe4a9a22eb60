"""World-size-2 checks of the multi-GPU host logic on CPU (gloo): partition, gather, max-reduce.
The compute itself has no CPU path; each rank stands in for it with a deterministic stream."""
import os
import socket

import pytest
import torch.multiprocessing as mp

from puppygrad_b200 import sharding


def fake_stream(i):
    return [(i * 7919 + s * 31) % 50257 for s in range(5)]


def _worker(rank, world, port, n_items, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = sharding.partition(n_items, world, rank)
        local = {i: fake_stream(i) for i in mine}
        streams = sharding.gather_streams(local, n_items)
        slowest = sharding.max_over_ranks(1.0 + rank)
        dist.barrier()
        q.put((rank, mine, streams, slowest))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.timeout(120)
def test_two_ranks_partition_gather_and_time():
    world, n_items = 2, 9
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_items, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=90) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    want = [fake_stream(i) for i in range(n_items)]
    seen = []
    for rank, mine, streams, slowest in results:
        assert mine == list(range(rank, n_items, world))
        assert streams == want  # same result as one rank doing everything
        assert slowest == 2.0   # max over ranks
        seen += mine
    assert sorted(seen) == list(range(n_items))


def test_partition_edges():
    assert sharding.partition(0, 4, 1) == []
    assert sharding.partition(3, 8, 5) == []
    assert sharding.partition(64, 8, 7) == list(range(7, 64, 8))
    assert sharding.gather_streams({0: [1], 1: [2]}, 2) == [[1], [2]]
    with pytest.raises(ValueError):
        sharding.partition(4, 2, 2)
    with pytest.raises(ValueError):
        sharding.gather_streams({0: [1]}, 2)
