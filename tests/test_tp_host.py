"""CPU-only checks of the tensor-parallel host logic: the shard plan and the id exchange that a
multi-rank launch does before any GPU work (two gloo ranks on 127.0.0.1)."""
import os
import socket

import pytest


def test_tp_share_partitions(pkg):
    for units in (1, 2, 7, 16, 43, 56, 112, 1000):
        for n in (1, 2, 3, 4, 8):
            if units < n:
                continue
            spans = [pkg.api.tp_share(units, n, r) for r in range(n)]
            assert spans[0][0] == 0 and spans[-1][1] == units
            assert all(spans[i][1] == spans[i + 1][0] for i in range(n - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    # the 7B FFN: 43 blocks of 256 do not divide by 2, 4 or 8
    assert [pkg.api.tp_share(43, 4, r) for r in range(4)] == [(0, 11), (11, 22), (22, 33), (33, 43)]
    assert [e - b for b, e in (pkg.api.tp_share(43, 8, r) for r in range(8))] == [6, 6, 6, 5, 5, 5, 5, 5]
    with pytest.raises(pkg.B200Error):
        pkg.api.tp_share(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    import __graft_entry__
    pkg = __graft_entry__.load_package()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # what bench.py does before building the engines: rank 0 owns a 128-byte id, everyone receives it
    blob = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        blob.copy_(torch.arange(128, dtype=torch.uint8) * 3 % 251)
    dist.broadcast(blob, src=0)
    b, e = pkg.api.tp_share(43, world, rank)
    spans = [None] * world
    dist.all_gather_object(spans, (b, e))
    # timing is reported as the max over ranks
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    q.put((rank, bytes(blob.tolist()), spans, float(t.item())))
    dist.destroy_process_group()


def test_two_rank_plan_exchange_over_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert out[0][1] == out[1][1] and out[0][1][1] == 3
    assert out[0][2] == out[1][2] == [(0, 22), (22, 43)]
    assert out[0][3] == out[1][3] == 2.0
