"""N > 1 host logic on CPU: two gloo ranks reduce their measurements the way bench.py does."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from __graft_entry__ import load_package
    import importlib
    load_package()
    rep = importlib.import_module("glm53f_b200.replicas")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        r = rep.whole_job_rate(units_local=100 + rank, seconds_local=0.5 * (rank + 1), dist=dist)
        mine = rep.shard_requests(11, rank, world)
        q.put((rank, r, list(mine)))
    finally:
        dist.destroy_process_group()


def test_two_ranks_reduce_like_the_bench():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    seen = []
    for rank, r, mine in sorted(got):
        assert r["units"] == 201 and r["seconds"] == 1.0 and r["rate"] == 201.0
        seen += mine
    assert seen == list(range(11))                       # every request once, in order


def test_single_rank_needs_no_process_group(pkg):
    import importlib
    rep = importlib.import_module("glm53f_b200.replicas")
    r = rep.whole_job_rate(8, 2.0, dist=dist)
    assert r == {"units": 8.0, "seconds": 2.0, "rate": 4.0}
    assert list(rep.shard_requests(5, 0, 1)) == [0, 1, 2, 3, 4]
    assert [len(rep.shard_requests(10, r, 4)) for r in range(4)] == [3, 3, 2, 2]
    with pytest.raises(ValueError):
        rep.shard_requests(5, 2, 2)
