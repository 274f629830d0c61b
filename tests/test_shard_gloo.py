"""The multi-rank plumbing (batch partition + gather of unequal row blocks) on CPU ranks over gloo."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fblt_b200 import shard, workloads


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_partition_covers_every_sequence_once():
    for n in (0, 1, 7, 8, 2048, 2051):
        for w in (1, 2, 3, 4, 8):
            r = shard.partition(n, w)
            assert r[0][0] == 0 and r[-1][1] == n and len(r) == w
            assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
            sizes = [e - b for b, e in r]
            assert max(sizes) - min(sizes) <= 1


def _worker(rank: int, world: int, port: int, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = workloads.c5_prefill(batch=10, with_tensors=False)      # patch structure only
        ranges = shard.partition(10, world)
        rows_per_rank = [int(case.cu_q[e] - case.cu_q[b]) for b, e in ranges]
        E = 8
        # "output rows" a rank would produce: global row index in every column
        b, e = ranges[rank]
        g0, g1 = int(case.cu_q[b]), int(case.cu_q[e])
        local = torch.arange(g0, g1, dtype=torch.float32)[:, None].expand(g1 - g0, E).contiguous()
        gathered, counts = shard.gather_rows(local, rows_per_rank)
        full = shard.unpad(gathered, counts)
        ok = full.shape == (int(case.cu_q[-1]), E) and bool((full[:, 0] == torch.arange(full.shape[0])).all())
        q.put((rank, ok, rows_per_rank))
    finally:
        dist.destroy_process_group()


def test_gather_rows_world_size_2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results)
    assert results[0][2] == results[1][2] and len(set(results[0][2])) == 2   # unequal blocks were exercised


def test_parse_cpulist():
    from fblt_b200 import shard
    assert shard.parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert shard.parse_cpulist("5") == {5}
    assert shard.parse_cpulist("") == set()
