"""N > 1 host logic on CPU: two gloo ranks agree on outcomes, reduce measurements and gather
handles the way bench.py and the multi-GPU tests do."""
import os
import socket

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
    rk = importlib.import_module("glm53f_b200.ranks")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        r = rk.Ranks(dist, "cpu")
        res = {"world": r.world, "rank": r.rank,
               "max": r.reduce(0.5 * (rank + 1), "max"), "sum": r.reduce(100 + rank, "sum"),
               "ok_all": r.all_ok(True), "ok_one_failed": r.all_ok(rank != 1),
               "gathered": r.gather(f"handle-{rank}".encode()),
               "rate": rk.strong_scaling_rate(10, 0.5 * (rank + 1), r),
               "mine": list(rk.expert_range(288, rank, world))[:2]}
        r.barrier()
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_agree():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    for rank in range(world):
        r = got[rank]
        assert r["world"] == 2 and r["rank"] == rank
        assert r["max"] == 1.0 and r["sum"] == 201.0
        assert r["ok_all"] is True and r["ok_one_failed"] is False
        assert r["gathered"] == [b"handle-0", b"handle-1"]
        assert r["rate"]["seconds"] == 1.0 and r["rate"]["rate"] == 10.0
    assert got[0]["mine"] == [0, 1] and got[1]["mine"] == [144, 145]


def test_single_rank_needs_no_process_group():
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from __graft_entry__ import load_package
    import importlib
    load_package()
    rk = importlib.import_module("glm53f_b200.ranks")
    r = rk.Ranks(None)
    assert r.world == 1 and r.reduce(3.0, "max") == 3.0 and r.all_ok(True) and r.gather(7) == [7]
    try:
        rk.expert_range(288, 0, 5)
    except ValueError:
        pass
    else:
        raise AssertionError("5 ranks do not divide 288 experts")
