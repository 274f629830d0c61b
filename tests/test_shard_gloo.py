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


def _rdv_worker(rank: int, world: int, path: str, mode: str, q):
    """mode: "ok" = both check in; "late" = rank 1 arrives after the deadline; "fail" = rank 1 announces
    a failure; "absent" = rank 1 never comes."""
    import time
    store = dist.FileStore(path, world)
    # line the processes up first (interpreter start-up differs by seconds under load), so that
    # "late" and "on time" below are measured from a common start
    store.set(f"started/{rank}", b"1")
    store.wait([f"started/{r}" for r in range(world)])
    t0 = time.monotonic()
    try:
        if rank == 1 and mode == "absent":
            q.put((rank, "skipped", 0.0))
            return
        if rank == 1 and mode == "late":
            time.sleep(2.5)
        if rank == 1 and mode == "fail":
            shard.report_failure(store, rank, "step0", "input shard unreadable")
            q.put((rank, "reported", time.monotonic() - t0))
            return
        shard.rendezvous(store, rank, world, "step0", deadline_s=0.5 if mode != "ok" else 20.0)
        q.put((rank, "ok", time.monotonic() - t0))
    except shard.RankTimeout as e:
        q.put((rank, f"timeout{e.missing}", time.monotonic() - t0))
    except shard.RankFailed as e:
        q.put((rank, f"failed{e.rank}:{e.reason}", time.monotonic() - t0))


def _run_rdv(mode: str, tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    path = str(tmp_path / f"store_{mode}")
    procs = [ctx.Process(target=_rdv_worker, args=(r, 2, path, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict()
    for _ in procs:
        rank, what, secs = q.get(timeout=120)
        results[rank] = (what, secs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return results


def test_rendezvous_before_collectives(tmp_path):
    """A rank that is late, absent or has failed is found out on the host, within the deadline, before
    any collective is enqueued (none is: these ranks never create a process group)."""
    r = _run_rdv("ok", tmp_path)
    assert r[0][0] == "ok" and r[1][0] == "ok"
    r = _run_rdv("absent", tmp_path)
    assert r[0][0] == "timeout[1]" and r[0][1] < 10.0
    r = _run_rdv("late", tmp_path)
    assert r[0][0] == "timeout[1]"            # rank 0 gave up at its deadline and said so in the store ...
    assert r[1][0].startswith("failed0:timed out")   # ... so the late rank does not go on alone
    r = _run_rdv("fail", tmp_path)
    assert r[0][0] == "failed1:input shard unreadable" and r[0][1] < 10.0


def test_parse_cpulist():
    from fblt_b200 import shard
    assert shard.parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert shard.parse_cpulist("5") == {5}
    assert shard.parse_cpulist("") == set()
