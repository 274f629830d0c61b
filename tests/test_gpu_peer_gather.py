"""shard.PeerGather and the library's own gather (fblt_gather_*) on two GPUs of one box: every rank's rows
arrive in every rank's buffer.
Skipped on a box with one GPU (the CPU suite covers the partition and the NCCL/gloo gather)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q):
    import datetime
    from fblt_b200 import shard
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
    try:
        rows_per_rank, E = [700, 513], 256
        g = shard.PeerGather(max(rows_per_rank), E, dev)
        n = rows_per_rank[rank]
        local = (torch.arange(n * E, device=dev, dtype=torch.float32).view(n, E) + 1000000.0 * (rank + 1))
        g.buf.fill_(-1.0)
        dist.barrier()                       # nobody writes into a buffer that is still being cleared
        g.put(local, n)
        torch.cuda.synchronize()
        dist.barrier()                       # every rank's copies have landed everywhere
        ok = True
        for r in range(world):
            m = rows_per_rank[r]
            want = torch.arange(m * E, device=dev, dtype=torch.float32).view(m, E) + 1000000.0 * (r + 1)
            ok = ok and bool(torch.equal(g.buf[r, :m], want)) and bool((g.buf[r, m:] == -1.0).all())
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_peer_gather_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(ok for _, ok in results)


def _ipc_worker(rank: int, world: int, path: str, q):
    """The C ABI's own gather: no torch.distributed anywhere; the ranks meet through a directory."""
    import ctypes as C
    from fblt_b200 import lib as L
    from fblt_b200 import shard
    lib = L.load()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)

    def barrier(tag: str):
        buf = C.create_string_buffer(world)
        L.check(lib.fblt_rendezvous_files(path.encode(), tag.encode(), rank, world, b"x", 1, buf, 120000))

    rows_per_rank, E = [700, 513], 256
    g = shard.IpcGather(max(rows_per_rank), E, rank, world, path, "handles")
    n = rows_per_rank[rank]
    local = (torch.arange(n * E, device=dev, dtype=torch.float32).view(n, E) + 1000000.0 * (rank + 1))
    g.buf.fill_(-1.0)
    torch.cuda.synchronize()
    barrier("cleared")                       # nobody writes into a buffer that is still being cleared
    side = torch.cuda.Stream(device=dev)
    g.put(local[: n // 2], stream=side)                                  # in two pieces, as a chunked caller would
    g.put(local[n // 2:], row_offset=n // 2, stream=side)
    torch.cuda.synchronize()
    barrier("landed")                        # every rank's copies have completed everywhere
    ok = True
    for r in range(world):
        m = rows_per_rank[r]
        want = torch.arange(m * E, device=dev, dtype=torch.float32).view(m, E) + 1000000.0 * (r + 1)
        ok = ok and bool(torch.equal(g.buf[r, :m], want)) and bool((g.buf[r, m:] == -1.0).all())
    too_many = lib.fblt_gather_rows(g._h, local.data_ptr(), 701, 0, None)
    barrier("checked")
    g.close()
    q.put((rank, ok and too_many == L.ERR_CAPACITY))


def test_library_gather_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ipc_worker, args=(r, 2, str(tmp_path), q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(ok for _, ok in results)
