"""Host-side pieces of the one-process-per-GPU path that need no GPU: the batch partition and the
file-based check-in with a deadline (fblt_shard_partition, fblt_rendezvous_files). The failures are
made on the host -- a rank that never comes, comes late, or announces a failure -- with CPU
processes; no kernel and no collective is involved."""
import ctypes as C
import multiprocessing as mp
import time

from fblt_b200 import lib as L
from fblt_b200 import shard


def test_partition_matches_python_and_covers_everything():
    lib = L.load()
    for units in (0, 1, 7, 8, 2048, 2051):
        for world in (1, 2, 3, 8):
            want = shard.partition(units, world)
            got = []
            for r in range(world):
                b, e = C.c_int64(), C.c_int64()
                L.check(lib.fblt_shard_partition(units, world, r, C.byref(b), C.byref(e)))
                got.append((b.value, e.value))
            assert got == want
            assert got[0][0] == 0 and got[-1][1] == units and all(a[1] == b[0] for a, b in zip(got, got[1:]))
    b, e = C.c_int64(), C.c_int64()
    assert lib.fblt_shard_partition(8, 2, 2, C.byref(b), C.byref(e)) == L.ERR_ARG


def _worker(rank, world, path, mode, q):
    lib = L.load()
    mine = bytes([rank + 1]) * 64
    everyone = C.create_string_buffer(64 * world)
    # line the processes up first: interpreter start-up differs by seconds under load
    lib.fblt_rendezvous_files(path.encode(), b"start", rank, world, mine, 64, everyone, 120000)
    t0 = time.monotonic()
    if rank == 1 and mode == "absent":
        q.put((rank, "skipped", 0.0, b""))
        return
    if rank == 1 and mode == "late":
        time.sleep(2.5)
    if rank == 1 and mode == "fail":
        lib.fblt_rendezvous_report_failure(path.encode(), b"step0", rank)
        q.put((rank, "reported", 0.0, b""))
        return
    st = lib.fblt_rendezvous_files(path.encode(), b"step0", rank, world, mine, 64, everyone,
                                   500 if mode != "ok" else 60000)
    q.put((rank, st, time.monotonic() - t0, everyone.raw if st == L.OK else lib.fblt_last_error()))


def _run(mode, tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    d = tmp_path / mode
    d.mkdir()
    procs = [ctx.Process(target=_worker, args=(r, 2, str(d), mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    for _ in procs:
        rank, st, secs, payload = q.get(timeout=180)
        res[rank] = (st, secs, payload)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return res


def test_file_rendezvous_outcomes(tmp_path):
    r = _run("ok", tmp_path)
    want = bytes([1]) * 64 + bytes([2]) * 64
    assert r[0][0] == L.OK and r[1][0] == L.OK and r[0][2] == want and r[1][2] == want
    r = _run("absent", tmp_path)
    assert r[0][0] == L.ERR_TIMEOUT and b"rank 1" in r[0][2] and r[0][1] < 10.0
    r = _run("late", tmp_path)
    assert r[0][0] == L.ERR_TIMEOUT              # rank 0 gave up at its deadline and said so ...
    assert r[1][0] == L.ERR_PEER                 # ... so the late rank does not go on alone
    r = _run("fail", tmp_path)
    assert r[0][0] == L.ERR_PEER and b"rank 1" in r[0][2] and r[0][1] < 10.0
