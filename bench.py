"""Benchmark of the attention path on the scaled batch-sharded workload.

One step = one pass of the hot path over the whole batch: block-causal patch-transformer
prefill attention (16 heads x 64, patch structure from the seeded generator) followed by 64
KV-cache decode steps with a block of 4 verify rows (cache 512 -> 768 rows), for 2048
independent sequences sharded by batch over the ranks; when the batch is partitioned the
outputs are gathered over NVLink, by default with the library's own gather (`--gather ipc`:
fblt_gather_* of the C ABI, one-sided copy-engine copies into IPC-mapped peer buffers after a
host-side check-in; no SM is taken from the attention launches), with the same copies over
torch's symmetric memory (`--gather peer`) or with NCCL all-gathers (`--gather nccl`, also the
fallback when the peer set-up fails).

    python bench.py [--gpus N --steps K --warmup W]            # this library
    python bench.py --impl reference [...]                     # reference CPU operator, host cores
    torchrun --nproc-per-node N bench.py --gpus N ...           # one rank per GPU

Prints ONE JSON line (rank 0). `value` is algorithmic attention bytes per second with inputs
resident in HBM; `e2e` is the same metric through the host-buffer C ABI (sessions) with all
host<->device copies inside the timed region.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

_RESULT_FD = 1


def emit(line: dict) -> None:
    os.write(_RESULT_FD, (json.dumps(line) + "\n").encode())


METRIC = "attn_algorithmic_bytes_per_s"
UNIT = "GB/s"
H, HD, E = 16, 64, 1024
N_NEW, BASE_LEN = 4, 512
SCALE = 0.125


# ----------------------------------------------------------------------------- workload arithmetic

def prefill_bytes(rows: int) -> int:
    """Q, K, V rows read once and O rows written once (fp32)."""
    return 4 * E * 4 * rows


def decode_bytes(batch: int, base: int) -> int:
    """One block-verify step: K and V of base + 4 rows per sequence read once, q read, out written."""
    return 4 * E * (2 * batch * (base + N_NEW) + 2 * batch * N_NEW)


def job_bytes(rows: int, batch: int, decode_steps: int) -> int:
    return prefill_bytes(rows) + sum(decode_bytes(batch, BASE_LEN + N_NEW * t) for t in range(decode_steps))


# ----------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            try:
                pw.append(float(f[3]))
            except ValueError:
                pass
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons), "power_w": statistics.median(pw) if pw else None}


# ----------------------------------------------------------------------------- CPU reference legs

def cpu_sample(qkv: np.ndarray, cu: np.ndarray, kc: np.ndarray, vc: np.ndarray, qn: np.ndarray, kn: np.ndarray,
               vn: np.ndarray, step_ids, total_batch: int, total_rows: int, decode_steps: int, threads: int,
               use_ref: bool):
    """Times the reference CPU operator on a bounded sample of the workload and scales it to
    the whole job: `qkv`/`cu` are a sample of prefill sequences, kc/vc/qn/kn/vn a sample of
    decode sequences evaluated at the decode steps in `step_ids`. Returns
    (estimated job seconds, outputs for checking, description)."""
    from oracle import binding as ob
    nb = len(cu) - 1
    t_mask0 = time.perf_counter()
    masks = [ob.build_mask(int(cu[b + 1] - cu[b]), int(cu[b + 1] - cu[b]), is_causal=True, use_ref=use_ref)[0]
             for b in range(nb)]
    t_mask = time.perf_counter() - t_mask0
    out_p, t_pre = ob.batched_attention(qkv, qkv, qkv, cu, cu, H, HD, SCALE, masks, k_col0=E, v_col0=2 * E,
                                        use_ref=use_ref, nthreads=threads)
    db = kc.shape[0]
    outs_d, t_dec = [], 0.0
    for t in step_ids:
        base = BASE_LEN + N_NEW * t
        jobs = ob.HeadJobs()
        out_d = np.zeros((db * N_NEW, E), np.float32)
        mask = np.zeros((N_NEW, base + N_NEW), np.float32)   # block rows see every key
        kk = np.ascontiguousarray(np.concatenate([kc[:, :base], kn.reshape(db, N_NEW, E)], axis=1))
        vv = np.ascontiguousarray(np.concatenate([vc[:, :base], vn.reshape(db, N_NEW, E)], axis=1))
        for b in range(db):
            for h in range(H):
                c = h * HD
                jobs.add(qn, kk[b], vv[b], out_d, col=c, head_dim=HD, q_col=c, k_col=c, v_col=c, scale=SCALE,
                         mask=mask, nq=N_NEW, nk=base + N_NEW, q_row=b * N_NEW)
        t_dec += jobs.run(threads, use_ref)
        outs_d.append(out_d)
    prefill_rows = int(cu[-1])
    est = t_pre * (total_rows / max(prefill_rows, 1)) + \
        (t_dec / max(len(step_ids), 1)) * decode_steps * (total_batch / max(db, 1))
    desc = (f"{nb} of {total_batch} sequences prefill ({prefill_rows} rows, {t_pre:.2f}s) + {db} sequences x "
            f"{len(step_ids)} of {decode_steps} decode steps ({t_dec:.2f}s), scaled linearly; dense mask build "
            f"{t_mask:.2f}s not included")
    return est, out_p, outs_d, desc


def run_reference_arm(args):
    """The reference's own CPU attention operator on the box's host cores, bounded sample per step."""
    from fblt_b200 import workloads
    from oracle import binding as ob
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    use_ref = ob.have_ref()
    threads = ob.host_cores()
    case = workloads.c5_prefill(batch=args.batch, with_tensors=False)
    total_rows = int(case.cu_q[-1])
    nb, db = min(args.cpu_prefill_seqs, args.batch), min(args.cpu_decode_seqs, args.batch)
    cu = (case.cu_q[: nb + 1] - case.cu_q[0]).astype(np.int32)
    rng = np.random.default_rng(4)
    qkv = rng.standard_normal((int(cu[-1]), 3 * E), dtype=np.float32) * 0.125
    rows = BASE_LEN + N_NEW * args.decode_steps
    kc = rng.standard_normal((db, rows, E), dtype=np.float32)
    vc = rng.standard_normal((db, rows, E), dtype=np.float32)
    qn, kn, vn = (rng.standard_normal((db * N_NEW, E), dtype=np.float32) for _ in range(3))
    step_ids = list(range(0, args.decode_steps, max(1, args.decode_steps // args.cpu_decode_steps)))[: args.cpu_decode_steps]
    ests, desc = [], ""
    for it in range(args.warmup + args.steps):
        est, _, _, desc = cpu_sample(qkv, cu, kc, vc, qn, kn, vn, step_ids, args.batch, total_rows, args.decode_steps,
                                     threads, use_ref)
        if it >= args.warmup:
            ests.append(est)
    sec = statistics.mean(ests)
    value = job_bytes(total_rows, args.batch, args.decode_steps) / sec / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, total_rows),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "reference" if use_ref else "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def workload_config(args, total_rows: int) -> dict:
    return {"workload": "scaled batch-sharded prefill+decode (config 5): block-causal patch attention + "
                        f"{args.decode_steps} block-verify decode steps (B=4) over the KV cache",
            "sequences": args.batch, "patch_rows": total_rows, "heads": H, "head_dim": HD, "cache_rows_start": BASE_LEN,
            "block": N_NEW, "decode_steps": args.decode_steps, "parallelism": f"batch-sharded x{args.gpus}",
            "l2": "inputs larger than L2 (>= 8 GB streamed per decode launch set)"}


# ----------------------------------------------------------------------------- GPU arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=2048, help="total sequences over all ranks")
    ap.add_argument("--decode-steps", type=int, default=64)
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--cpu-prefill-seqs", type=int, default=512)
    ap.add_argument("--cpu-decode-seqs", type=int, default=128)
    ap.add_argument("--cpu-decode-steps", type=int, default=8)
    ap.add_argument("--workload", default="scaled", choices=["scaled", "configs", "matmul", "blocks", "long"],
                    help="scaled = the headline job (one JSON line); configs = one line per small benchmark "
                         "configuration (byte self-attention, patch attention, cross-attention, cache decode)")
    ap.add_argument("--matmul-small", action="store_true",
                    help="matmul workload: only the decode-step shapes (8192 rows), for profiler captures")
    ap.add_argument("--gather-chunks", type=int, default=4,
                    help="N > 1: the decode rows of a step are gathered in this many pieces while the launches go on")
    ap.add_argument("--gather", default="ipc", choices=["nccl", "peer", "ipc"],
                    help="N > 1: outputs gathered by the library's own one-sided copy-engine copies into IPC-mapped peer "
                         "buffers (ipc: fblt_gather_* of the C ABI), by the same copies over torch's symmetric memory "
                         "(peer), or by NCCL all-gather kernels (nccl)")
    ap.add_argument("--nccl-max-ctas", type=int, default=0, help="N > 1: cap on the CTAs of an NCCL gather (0 = NCCL's default)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg")
    ap.add_argument("--no-configs", action="store_true", help="skip the small configurations (`configs` key, one GPU)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    # Libraries (NCCL's version banner, for one) write to stdout; keep stdout for the JSON
    # result only and send everything else to stderr.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.workload == "configs":
        run_small_configs(args)
        return
    if args.workload == "matmul":
        run_matmul(args)
        return
    if args.workload == "blocks":
        run_blocks(args)
        return
    if args.workload == "long":
        run_long_prefill(args)
        return

    import torch
    import torch.distributed as dist
    from fblt_b200 import lib as L
    from fblt_b200 import ops, shard, workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the attention path has no CPU fallback")
    lib = L.load()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # one process per GPU: keep each rank and its pinned host buffers on the GPU's own NUMA node
    # (the CPU baseline leg of a single-GPU run gets the full affinity mask back)
    full_affinity = os.sched_getaffinity(0)
    numa = shard.bind_to_device_numa_node(local_rank)
    if world > 1:
        if args.nccl_max_ctas > 0:
            # the gathers share the GPU with the decode launches: fewer NCCL CTAs leave more SMs to them
            os.environ.setdefault("NCCL_MAX_CTAS", str(args.nccl_max_ctas))
        # plain rings / trees for the few collectives this job makes: a rank that leaves early must not
        # be bound to an NVLink multicast object (the gathers themselves are peer copies)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        # a collective that stays enqueued past this deadline is aborted by the process group's watchdog
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
    assert world == args.gpus or world == 1, "launch with torchrun --nproc-per-node N for --gpus N"

    # ---- this rank's shard ---------------------------------------------------
    case = workloads.c5_prefill(batch=args.batch, with_tensors=False)
    total_rows = int(case.cu_q[-1])
    ranges = shard.partition(args.batch, world)
    s0, s1 = ranges[rank]
    B = s1 - s0
    cu = (case.cu_q[s0: s1 + 1] - case.cu_q[s0]).astype(np.int32)
    rows = int(cu[-1])
    rows_per_rank = [int(case.cu_q[e] - case.cu_q[b]) for b, e in ranges]
    cache_rows = BASE_LEN + N_NEW * args.decode_steps
    gen = torch.Generator(device=dev).manual_seed(4 + 1000 * rank)
    qkv = torch.randn((rows, 3 * E), generator=gen, device=dev) * 0.125
    out_p = torch.empty((rows, E), device=dev)
    kc = torch.randn((B, cache_rows, E), generator=gen, device=dev)
    vc = torch.randn((B, cache_rows, E), generator=gen, device=dev)
    qn = torch.randn((B * N_NEW, E), generator=gen, device=dev)
    kn = torch.randn((B * N_NEW, E), generator=gen, device=dev)
    vn = torch.randn((B * N_NEW, E), generator=gen, device=dev)
    # two decode-output buffers: step i's rows are gathered while step i + 1 computes into the other
    out_d2 = [torch.empty((args.decode_steps, B * N_NEW, E), device=dev) for _ in range(2 if world > 1 else 1)]
    out_d = out_d2[0]
    lens_all = (BASE_LEN + N_NEW * torch.arange(args.decode_steps, device=dev, dtype=torch.int32))[:, None] \
        .expand(args.decode_steps, B).contiguous()
    pre = ops.make_batch(qkv[:, 0:E], qkv[:, E:2 * E], qkv[:, 2 * E:], out_p, cu, cu, H, HD, SCALE,
                         ops.MaskConfig(is_causal=True))
    dec2 = [[ops.make_decode(kc, vc, lens_all[t], qn, od[t], H, HD, N_NEW, SCALE, block_mode=True, k_new=kn,
                             v_new=vn, max_len=BASE_LEN + N_NEW * (t + 1)) for t in range(args.decode_steps)]
            for od in out_d2]
    dec = dec2[0]
    ws = ops.decode_workspace(dec[-1])

    main_stream = torch.cuda.Stream(device=dev)
    comm_stream = torch.cuda.Stream(device=dev)
    if world > 1:
        # every rank has built its shard: check in on the HOST before anything collective happens (the
        # gather set-up below, the first all-reduce), so that a rank that died or fell behind while
        # building is named here instead of leaving the others inside a collective
        torch.cuda.synchronize()
        try:
            shard.rendezvous(shard.default_store(), rank, world, "bench-setup", deadline_s=240.0)
        except (shard.RankTimeout, shard.RankFailed) as exc:
            sys.stderr.write(f"rank {rank}: {exc}\n")
            dist.destroy_process_group()
            sys.exit(3)
        store = shard.default_store()
        if rank == 0:
            import tempfile
            base = "/dev/shm" if os.path.isdir("/dev/shm") else None
            store.set("fblt/exchange_dir", tempfile.mkdtemp(prefix="fblt_bench_", dir=base).encode())
        exchange_dir = store.get("fblt/exchange_dir").decode()
        max_rows = max(rows_per_rank)
        pad_p = torch.zeros((max_rows, E), device=dev)
        gath_p = torch.empty((world, max_rows, E), device=dev)
        # the decode rows of a step travel in chunks of a quarter of the decode launches, so that
        # only the last chunk's gather is still under way when the step's compute ends
        n_chunks = args.gather_chunks if args.decode_steps % args.gather_chunks == 0 else 1
        chunk_steps = args.decode_steps // n_chunks
        gath_d = [torch.empty((world, chunk_steps * B * N_NEW, E), device=dev) for _ in range(n_chunks)] \
            if args.gather == "nccl" else None
        peer_p = peer_d = None
        gather_mode = args.gather
        if args.gather in ("ipc", "peer"):
            # set-up; if it fails on any rank, every rank falls back to NCCL all-gathers
            try:
                if args.gather == "ipc":     # the library's own gather: C ABI, IPC-mapped peers, host check-in
                    peer_p = shard.IpcGather(max_rows, E, rank, world, exchange_dir, "prefill")
                    peer_d = [shard.IpcGather(chunk_steps * B * N_NEW, E, rank, world, exchange_dir, f"decode{c}")
                              for c in range(n_chunks)]
                else:                        # torch's symmetric memory + Tensor.copy_
                    peer_p = shard.PeerGather(max_rows, E, dev)
                    peer_d = [shard.PeerGather(chunk_steps * B * N_NEW, E, dev) for _ in range(n_chunks)]
                ok = torch.ones(1, device=dev)
            except Exception as exc:   # noqa: BLE001 - any set-up failure selects the fallback
                sys.stderr.write(f"rank {rank}: peer gather unavailable ({exc}); using NCCL\n")
                ok = torch.zeros(1, device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if float(ok) > 0:
                del gath_p
                gath_p, gath_d = peer_p.buf, [g.buf for g in peer_d]
            else:
                peer_p = peer_d = None
                gather_mode = "nccl (peer set-up failed)"
                gath_d = [torch.empty((world, chunk_steps * B * N_NEW, E), device=dev) for _ in range(n_chunks)]
        ev_chunk = [torch.cuda.Event() for _ in range(n_chunks)]
        equal = len({e - b for b, e in ranges}) == 1
        assert equal, "decode gather assumes equal sequence counts per rank"

    ev_pre_done = torch.cuda.Event()
    ev_dec_done = [torch.cuda.Event() for _ in out_d2]
    ev_gathered = [torch.cuda.Event() for _ in out_d2]   # the buffer's rows have left: it may be overwritten
    ev_pre_gathered = torch.cuda.Event()
    dec_t0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.warmup + args.steps)]
    dec_t1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.warmup + args.steps)]

    pre_t0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.warmup + args.steps)]

    # side-stream duration of the gathers of the last timed step (they overlap the decode launches)
    last_it = args.warmup + args.steps - 1
    g_pre = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    g_dec = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(args.decode_steps)]

    def one_step(it: int):
        with torch.cuda.stream(main_stream):
            buf = it % len(out_d2)
            pre_t0[it].record(main_stream)
            if world > 1 and it > 0:
                main_stream.wait_event(ev_pre_gathered)      # last step's prefill rows have been sent
            ops.attn_forward(pre, main_stream)
            if world > 1:
                ev_pre_done.record(main_stream)
                comm_stream.wait_event(ev_pre_done)
                with torch.cuda.stream(comm_stream):   # prefill rows travel while decode runs
                    if it == last_it:
                        g_pre[0].record(comm_stream)
                    if peer_p is not None:
                        peer_p.put(out_p, rows_per_rank[rank])
                    else:
                        shard.gather_rows(out_p, rows_per_rank, padded=pad_p, gathered=gath_p)
                    ev_pre_gathered.record(comm_stream)
                    if it == last_it:
                        g_pre[1].record(comm_stream)
                if it >= len(out_d2):
                    main_stream.wait_event(ev_gathered[buf])  # this buffer's previous rows have been sent
            dec_t0[it].record(main_stream)
            for t in range(args.decode_steps):
                ops.attn_decode(dec2[buf][t], ws, main_stream)
                if world > 1 and (t + 1) % chunk_steps == 0:   # this chunk's rows travel while decode goes on
                    c = t // chunk_steps
                    ev_chunk[c].record(main_stream)
                    comm_stream.wait_event(ev_chunk[c])
                    with torch.cuda.stream(comm_stream):
                        if it == last_it:
                            g_dec[c][0].record(comm_stream)
                        rows_c = out_d2[buf][c * chunk_steps:(c + 1) * chunk_steps].view(-1, E)
                        if peer_d is not None:
                            peer_d[c].put(rows_c)
                        else:
                            dist.all_gather_into_tensor(gath_d[c].view(-1, E), rows_c)
                        if it == last_it:
                            g_dec[c][1].record(comm_stream)
                        if c == n_chunks - 1:
                            ev_gathered[buf].record(comm_stream)
            dec_t1[it].record(main_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for it in range(args.warmup):
        one_step(it)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = lib.fblt_launch_count()
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin.record(main_stream)
    for it in range(args.steps):
        one_step(args.warmup + it)
    main_stream.wait_stream(comm_stream)   # the timed region ends when the last gather has landed
    t_end.record(main_stream)
    barrier()
    launches = lib.fblt_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    ms = t_begin.elapsed_time(t_end)
    dec_ms = sum(dec_t0[args.warmup + i].elapsed_time(dec_t1[args.warmup + i]) for i in range(args.steps))
    pre_ms = sum(pre_t0[args.warmup + i].elapsed_time(dec_t0[args.warmup + i]) for i in range(args.steps))
    if world > 1:
        tt = torch.tensor([ms, dec_ms, pre_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, dec_ms, pre_ms = float(tt[0]), float(tt[1]), float(tt[2])
        lt = torch.tensor([launches], device=dev, dtype=torch.int64)
        dist.all_reduce(lt)
        launches = int(lt[0])
    gather = None
    if world > 1:
        # every rank's rows must have arrived everywhere: per-slot sums of what this rank holds
        # against the sums the owners computed from their own outputs (after the closing barrier)
        last_buf = out_d2[last_it % len(out_d2)]
        mine = torch.stack([last_buf[c * chunk_steps:(c + 1) * chunk_steps].double().sum() for c in range(n_chunks)]
                           + [out_p.double().sum()])
        sums = torch.empty((world, n_chunks + 1), device=dev, dtype=torch.float64)
        dist.all_gather_into_tensor(sums, mine)
        got = torch.stack([torch.stack([gath_d[c][r].double().sum() for c in range(n_chunks)]
                                       + [gath_p[r, :rows_per_rank[r]].double().sum()]) for r in range(world)])
        gather_ok = bool(torch.allclose(got, sums, rtol=1e-9, atol=1e-6))
        assert gather_ok, "gathered rows differ from what their owners computed"
        gather = {"mode": gather_mode, "checked": "per-rank sums of the gathered rows equal the owners' sums",
                  "prefill_ms": g_pre[0].elapsed_time(g_pre[1]),
                  "decode_chunk_ms": [g_dec[c][0].elapsed_time(g_dec[c][1]) for c in range(n_chunks)],
                  "prefill_bytes_gathered": int(world * max_rows * E * 4),
                  "decode_bytes_gathered_per_chunk": int(world * chunk_steps * B * N_NEW * E * 4),
                  "note": "rank 0, last timed step, on the side stream while the decode launches run"}
    ms_per_step = ms / args.steps
    total_bytes = job_bytes(total_rows, args.batch, args.decode_steps)
    value = total_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- roofline of the dominant kernel (block-verify decode) ------------------
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        peak, peak_src = float(json.loads(peaks_file.read_text())["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    launch_ms = dec_ms / (args.steps * args.decode_steps)
    launch_bytes = sum(decode_bytes(B, BASE_LEN + N_NEW * t) for t in range(args.decode_steps)) / args.decode_steps
    achieved = launch_bytes / (launch_ms * 1e-3) / 1e9
    roofline = {"kernel": "decode_attn_kernel<64,4>", "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_source": peak_src, "launch_ms": launch_ms,
                "algorithmic_bytes_per_launch": launch_bytes, "traffic": NCU_TRAFFIC_PER_ALGORITHMIC_BYTE and
                NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * launch_bytes}

    # secondary kernel: the prefill tile kernel (one launch per step; at N > 1 the time includes
    # enqueueing the overlapped gather)
    pre_launch_ms = pre_ms / args.steps
    pre_bytes = prefill_bytes(rows)
    pre_flops = 4.0 * HD * H * float(sum(int(n) * (int(n) + 1) // 2 for n in np.diff(cu)))  # allowed pairs only
    prefill = {"kernel": "unit5_attn_kernel (tcgen05 + TMA, fp32 by three TF32 passes)", "launch_ms": pre_launch_ms,
               "algorithmic_bytes_per_launch": pre_bytes, "achieved_GBps": pre_bytes / pre_launch_ms / 1e6,
               "frac_of_hbm_peak": pre_bytes / pre_launch_ms / 1e6 / peak,
               "algorithmic_tflops": pre_flops / pre_launch_ms / 1e9}
    # The same launch timed alone (L2 flushed before each of 10 launches, median): launch_ms above is taken
    # inside the step, right after 64 decode launches that hold the GPU at its power cap, and this kernel,
    # unlike the HBM-bound decode stream, runs with the SM clock.
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    alone = []
    for _ in range(10):
        flush.zero_()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record(main_stream)
        ops.attn_forward(pre, main_stream)
        a1.record(main_stream)
        a1.synchronize()
        alone.append(a0.elapsed_time(a1))
    del flush
    alone_ms = sorted(alone)[len(alone) // 2]
    prefill["launch_ms_alone"] = alone_ms
    prefill["frac_of_hbm_peak_alone"] = pre_bytes / alone_ms / 1e6 / peak

    # ---- host-buffer leg (sessions): copies inside the timed region -------------
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, torch, ops, dev, qkv, cu, rows, B, cache_rows, kc, vc, qn, kn, vn, world, total_bytes, barrier)

    # ---- CPU baseline on a bounded sample of the same tensors (rank 0, one GPU) ----
    cpu = None
    os.sched_setaffinity(0, full_affinity)
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = run_cpu_baseline(args, torch, qkv, cu, kc, vc, qn, kn, vn, out_p,
                               out_d2[(args.warmup + args.steps - 1) % len(out_d2)], total_rows)

    # ---- the small configurations at their full sizes (microseconds each; one GPU only) ----
    configs = None
    if rank == 0 and world == 1 and not args.no_configs:
        configs = small_config_lines(args, with_tf32=False)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(args, total_rows),
            "roofline": roofline, "prefill": prefill, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "host_binding": numa,
            "gather": gather,
            "job_bytes": total_bytes,
            "configs": configs,
        }
        emit(line)
    if world > 1:
        barrier()          # nobody frees a receive buffer a peer may still be writing into
        if peer_p is not None and hasattr(peer_p, "close"):
            for g_ in [peer_p] + list(peer_d):
                g_.close()
        dist.destroy_process_group()


def run_small_configs(args):
    """`--workload configs`: one JSON line per small configuration (both precisions) and the decode-step loop."""
    import torch
    from fblt_b200 import ops
    for line in small_config_lines(args, with_tf32=True):
        emit(line)
    run_decode_loop(args, torch, ops, emit)


def small_config_lines(args, with_tf32: bool):
    """Device time, roofline fraction, CPU reference time and max error of every small
    configuration at its full size (inputs from the seeded host generators). L2 is flushed
    between timed iterations because these working sets fit in it. The decode configurations are
    also timed as a run of back-to-back launches over rotating copies of the caches (together
    larger than L2), which is how a decode loop issues them: launch latency then overlaps the
    previous launch."""
    import torch
    sys.path.insert(0, str(ROOT / "tests"))
    from fblt_b200 import lib as L
    from fblt_b200 import ops, workloads
    from gpu_utils import upload_case
    from helpers import oracle_decode, oracle_forward
    from oracle import binding as ob
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_file.read_text())["hbm_gbs"]) if peaks_file.exists() else 6650.0
    flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
    lines = []

    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        times = []
        for _ in range(max(args.steps, 20)):
            flush.zero_()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            fn()
            t1.record()
            torch.cuda.synchronize()
            times.append(t0.elapsed_time(t1))
        times.sort()
        return statistics.median(times), times[min(len(times) - 1, int(0.9 * len(times)))]

    def report(name, t, nbytes, flops, cpu_s, err, extra=None):
        ms, p90 = t
        line = {"workload": name, "ms": ms, "ms_p90": p90, "iterations": max(args.steps, 20),
                "algorithmic_bytes": nbytes, "GB/s": nbytes / ms / 1e6,
                "frac_of_hbm_peak": nbytes / ms / 1e6 / peak, "algorithmic_flops": flops,
                "TFLOP/s": flops / ms / 1e9, "cpu_reference_ms": cpu_s * 1e3,
                "cpu_cores": ob.host_cores(), "max_abs_err": err, "l2": "flushed between iterations"}
        line.update(extra or {})
        lines.append(line)

    fwd = [workloads.c1_byte_self_attention(), workloads.c2_patch_attention(), workloads.c3_cross_attention("enc"),
           workloads.c3_cross_attention("dec_paper"), workloads.c3_cross_attention("dec_leq")]
    for case in fwd:
        q, k, v = upload_case(case)
        out = torch.empty((int(case.cu_q[-1]), case.embed), device="cuda")
        for prec, tag in ((L.PREC_FP32, ""), (L.PREC_TF32, "+tf32"))[: 2 if with_tf32 else 1]:
            b = ops.make_batch(q, k, v, out, case.cu_q, case.cu_k, case.num_heads, case.head_dim, case.scale, case.mask,
                               precision=prec)
            ms = timed(lambda: ops.attn_forward(b))
            if prec == L.PREC_FP32:
                want, masks, cpu_s = oracle_forward(case)
                # 4 x head_dim flop per allowed (query, key) pair and head
                flops = 4 * case.head_dim * case.num_heads * sum(int((m == 0).sum()) for m in masks)
            err = float(np.abs(out.cpu().numpy() - want).max())
            report(case.name + tag, ms, case.algorithmic_bytes(), flops, cpu_s, err)
            if case.mask.group_rule in (L.GROUP_PATCH_ENC, L.GROUP_PATCH_DEC):
                break   # row kernel: one precision
    for case in (workloads.c4_decode(), workloads.c4_block_verify()):
        kc, vc = torch.from_numpy(case.k_cache).cuda(), torch.from_numpy(case.v_cache).cuda()
        base, q = torch.from_numpy(case.base_len).cuda(), torch.from_numpy(case.q).cuda()
        kn, vn = torch.from_numpy(case.k_new).cuda(), torch.from_numpy(case.v_new).cuda()
        out = torch.empty_like(q)
        d = ops.make_decode(kc, vc, base, q, out, case.num_heads, case.head_dim, case.n_new, case.scale,
                            block_mode=case.block_mode, k_new=kn, v_new=vn, max_len=int(case.base_len.max()) + case.n_new)
        ws = ops.decode_workspace(d)
        ms = timed(lambda: ops.attn_decode(d, ws))
        want, cpu_s = oracle_decode(case)
        err = float(np.abs(out.cpu().numpy() - want).max())
        n, lens = case.n_new, case.base_len.astype(np.int64)
        pairs = int(((lens + n) * n).sum()) if case.block_mode else int(sum((lens + r + 1).sum() for r in range(n)))
        # back to back over four copies of the caches (4 x 151 MB > L2), eight launches per timed run
        sets = [(kc, vc)] + [(kc.clone(), vc.clone()) for _ in range(3)]
        descs = [ops.make_decode(k_, v_, base, q, out, case.num_heads, case.head_dim, case.n_new, case.scale,
                                 block_mode=case.block_mode, k_new=kn, v_new=vn,
                                 max_len=int(case.base_len.max()) + case.n_new) for k_, v_ in sets]
        def burst():
            for i in range(8):
                ops.attn_decode(descs[i % 4], ws)
        for _ in range(3):
            burst()
        ts = []
        for _ in range(10):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0.record()
            burst()
            t1.record()
            torch.cuda.synchronize()
            ts.append(t0.elapsed_time(t1) / 8)
        b2b = statistics.median(ts)
        report(case.name, ms, case.algorithmic_bytes(), 4 * case.head_dim * case.num_heads * pairs, cpu_s, err,
               {"splits": int(d.splits), "ms_back_to_back": b2b,
                "frac_of_hbm_peak_back_to_back": case.algorithmic_bytes() / b2b / 1e6 / peak,
                "back_to_back": "8 launches over 4 rotating copies of the caches (larger than L2 together)"})
        del sets, descs
    return lines


def run_decode_loop(args, torch, ops, emit_line):
    """The decode-step block (QKV matmul, rotary + write-through + cache attention, output matmul) at the
    cache-decode configuration (256 sequences, 4 heads x 64, one new row per step), 32 steps in a row:
    launched step by step from the host, and as one captured CUDA graph replayed. Lengths live in
    device memory, so the same graph serves the growing caches."""
    Hc, n, batch, cache_rows, steps = 4, 1, 256, 640, 32
    Ec = Hc * HD
    g = torch.Generator(device="cuda").manual_seed(3)
    kc = torch.randn((batch, cache_rows, Ec), device="cuda", generator=g)
    vc = torch.randn((batch, cache_rows, Ec), device="cuda", generator=g)
    base0 = (64 + torch.randint(0, 449, (batch,), device="cuda", generator=g)).to(torch.int32)
    base = base0.clone()
    w_qkv = ops.PackedWeights(torch.randn((Ec, 3 * Ec), device="cuda", generator=g) / 16.0)
    w_proj = ops.PackedWeights(torch.randn((Ec, Ec), device="cuda", generator=g) / 16.0)
    half = torch.arange(HD // 2, device="cuda", dtype=torch.float32)
    ang = torch.arange(cache_rows, device="cuda", dtype=torch.float32)[:, None] * (500000.0 ** (-2.0 * half / HD))[None, :]
    plan = ops.KvStepPlan(w_qkv, w_proj, kc, vc, base, Hc, n, rope_cos=torch.cos(ang).contiguous(),
                          rope_sin=torch.sin(ang).contiguous())
    plan.x.copy_(torch.randn((batch * n, Ec), device="cuda", generator=g))

    def eager():
        base.copy_(base0)
        for _ in range(steps):
            plan.run()
            base.add_(n)

    eager()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(steps):
                plan.run(side)
                base.add_(n)
    torch.cuda.current_stream().wait_stream(side)

    def replay():
        base.copy_(base0)
        graph.replay()

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(20):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0.record()
            fn()
            t1.record()
            torch.cuda.synchronize()
            ts.append(t0.elapsed_time(t1))
        return statistics.median(ts)

    e_ms, g_ms = timed(eager), timed(replay)
    emit_line({"workload": "c4_decode_step_block_loop", "sequences": batch, "steps": steps, "launches_per_step": 4,
               "host_launched_us_per_step": e_ms * 1e3 / steps, "cuda_graph_us_per_step": g_ms * 1e3 / steps,
               "note": "caches stay in L2 between steps, as in a real decode loop"})


def run_long_prefill(args):
    """Causal byte self-attention over long sequences (16 heads x 64, 65536 rows in all): the shape
    where the prefill is bound by the tensor pipe rather than by HBM. One line per sequence length,
    mask, kernel and precision with device time, TFLOP/s of the allowed (query, key) pairs
    (4 x head_dim flop each) and the fraction of the measured dense bf16 peak. A sample of rows is
    checked against an fp64 softmax of the same tensors computed with torch."""
    import torch
    from fblt_b200 import lib as L
    from fblt_b200 import ops
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    peaks = json.loads(peaks_file.read_text()) if peaks_file.exists() else {}
    bf16 = float(peaks.get("bf16_tflops", 1590.0))
    g = torch.Generator(device="cuda").manual_seed(5)
    total = 65536
    for T, window in ((2048, 0), (8192, 0), (8192, 512)):
        B = total // T
        qkv = torch.randn((total, 3 * E), device="cuda", generator=g) * 0.125
        q, k, v = qkv[:, 0:E], qkv[:, E:2 * E], qkv[:, 2 * E:]
        out = torch.empty((total, E), device="cuda")
        cu = np.arange(B + 1, dtype=np.int32) * T
        w = window if window else T
        pairs = B * (w * (w + 1) // 2 + (T - w) * w)       # keys max(0, i-w+1) .. i for every row i
        flop = 4.0 * HD * pairs * H
        rows = torch.tensor([0, 1, T // 3, T - 1, total - T + 777, total - 1], device="cuda")
        for impl, iname in ((L.IMPL_TCGEN05, "tcgen05"), (L.IMPL_TILE, "mma.sync")):
            for prec, pname in ((L.PREC_FP32, "fp32x3"), (L.PREC_TF32, "tf32")):
                b = ops.make_batch(q, k, v, out, cu, cu, H, HD, SCALE,
                                   ops.MaskConfig(is_causal=True, sliding_window=window), impl=impl, precision=prec)
                for _ in range(3):
                    ops.attn_forward(b)
                n = max(args.steps, 5)
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                t0.record()
                for _ in range(n):
                    ops.attn_forward(b)
                t1.record()
                torch.cuda.synchronize()
                ms = t0.elapsed_time(t1) / n
                err = 0.0
                for r in rows.tolist():
                    s0, i = (r // T) * T, r % T
                    lo = max(0, i - w + 1)
                    kk = k[s0 + lo:s0 + i + 1].double().view(-1, H, HD)
                    vv = v[s0 + lo:s0 + i + 1].double().view(-1, H, HD)
                    sc = torch.einsum("hd,jhd->hj", q[r].double().view(H, HD), kk) * SCALE
                    want = torch.einsum("hj,jhd->hd", torch.softmax(sc, dim=1), vv).reshape(E)
                    err = max(err, float((out[r].double() - want).abs().max()))
                emit({"workload": f"long_prefill_T{T}" + (f"_w{window}" if window else ""), "kernel": iname,
                      "precision": pname, "sequences": B, "ms": ms, "TFLOP/s": flop / ms / 1e9,
                      "frac_of_bf16_peak": flop / ms / 1e9 / bf16, "algorithmic_bytes": 4 * total * E * 4,
                      "GB/s": 4 * total * E * 4 / ms / 1e6, "max_abs_err_sampled_rows": err,
                      "inputs": "1.07 GB, larger than L2"})


def run_matmul(args):
    """The projection GEMMs beside the attention operator (E = 1024: QKV [M,1024]x[1024,3072] and
    output [M,1024]x[1024,1024]) at the row counts of the headline job: one line per shape and
    precision with device time, TFLOP/s, the fraction of the tensor roofline, the same shape
    through torch's fp32 matmul (cuBLAS SGEMM, what the reference calls on CUDA) and the
    reference's CPU loop on a row sample."""
    import torch
    from fblt_b200 import lib as L
    from fblt_b200 import ops
    from oracle import binding as ob
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    peaks = json.loads(peaks_file.read_text()) if peaks_file.exists() else {}
    bf16 = float(peaks.get("bf16_tflops", 1590.0))
    torch.backends.cuda.matmul.allow_tf32 = False
    g = torch.Generator(device="cuda").manual_seed(0)

    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = max(args.steps, 5)
        torch.cuda.synchronize()
        t0.record()
        for _ in range(n):
            fn()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / n

    shapes = (("qkv_prefill", 256508, 1024, 3072), ("proj_prefill", 256508, 1024, 1024),
              ("qkv_decode_step", 8192, 1024, 3072), ("proj_decode_step", 8192, 1024, 1024))
    for name, M, K, N in shapes[2:] if args.matmul_small else shapes:
        a = torch.randn(M, K, device="cuda", generator=g)
        b = torch.randn(K, N, device="cuda", generator=g) / 32.0
        w = ops.PackedWeights(b)
        out = torch.empty(M, N, device="cuda")
        flops = 2.0 * M * K * N
        ms_lib = timed(lambda: torch.matmul(a, b, out=out))
        exact = (a[:64].double() @ b.double())
        lib_err = float((out[:64].double() - exact).abs().max())
        sample = a[:64].cpu().numpy()
        t0 = time.perf_counter()
        cpu_out = ob.matmul(sample, b.cpu().numpy(), use_ref=ob.have_ref())
        cpu_s = time.perf_counter() - t0
        for prec, tag, passes in ((L.PREC_FP32, "fp32 (3xTF32)", 3), (L.PREC_TF32, "tf32", 1)):
            ms = timed(lambda: ops.matmul(a, w, out=out, precision=prec))
            # clocks under this kernel: a second, longer loop with the sampler running
            sampler = ClockSampler(torch.cuda.current_device())
            sampler.start()
            t_end = time.perf_counter() + 0.8
            while time.perf_counter() < t_end:
                for _ in range(8):
                    ops.matmul(a, w, out=out, precision=prec)
                torch.cuda.synchronize()
            clocks = sampler.stop()
            assert L.load().fblt_tcgen05_error() == 0
            err = float((out[:64].double() - exact).abs().max())
            tf = flops / ms / 1e9
            emit({"workload": f"matmul_{name}", "precision": tag, "M": M, "K": K, "N": N, "ms": ms, "TFLOP/s": tf,
                  "tensor_TFLOP/s": tf * passes,
                  "frac_of_tf32_peak": tf * passes / (bf16 / 2.0),
                  "tf32_peak_TFLOP/s": bf16 / 2.0, "peak_source": "measured bf16 cuBLAS figure / 2 (TF32 runs at half the bf16 rate)",
                  "max_abs_err_vs_f64": err, "clocks": clocks, "cublas_sgemm_ms": ms_lib, "cublas_sgemm_TFLOP/s": flops / ms_lib / 1e9,
                  "cublas_sgemm_max_abs_err_vs_f64": lib_err,
                  "cpu_reference": {"rows": 64, "seconds": cpu_s, "GFLOP/s": 2.0 * 64 * K * N / cpu_s / 1e9,
                                    "max_abs_err_vs_f64": float(np.abs(cpu_out - exact.cpu().numpy()).max()), "cores": 1},
                  "l2": "operands larger than L2 for the prefill shapes; decode-step shapes fit in L2"})
        del a, b, w, out


def run_blocks(args):
    """The whole multi-head self-attention block (QKV matmul, rotary attention, output matmul;
    fblt_mha_forward) on the patch-transformer shape of the headline job: 2048 sequences with the
    config-5 patch structure, E = 1024, 16 heads. One line with the device time of the three
    launches, and the reference's own blt_multihead_attention on the CPU for a few sequences."""
    import torch
    from fblt_b200 import lib as L
    from fblt_b200 import ops, workloads
    from fblt_b200.ops import MaskConfig
    from oracle import binding as ob
    H, hd = 16, 64
    E = H * hd
    case = workloads.patch_self_attention(4, args.batch, H, "c5_prefill", with_tensors=False)
    cu = case.cu_q
    rows = int(cu[-1])
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(rows, E, device="cuda", generator=g)
    w_qkv = torch.randn(E, 3 * E, device="cuda", generator=g) / 32.0
    w_proj = torch.randn(E, E, device="cuda", generator=g) / 32.0
    pq, pp = ops.PackedWeights(w_qkv), ops.PackedWeights(w_proj)
    cs, sn = ob.rope_tables(int(np.max(np.diff(cu))), hd, use_ref=ob.have_ref())
    cs_d, sn_d = torch.from_numpy(cs).cuda(), torch.from_numpy(sn).cuda()
    mask = MaskConfig(is_causal=True)
    fn = lambda: ops.mha_forward(x, pq, pp, cu, H, mask, rope_cos=cs_d, rope_sin=sn_d)
    for _ in range(max(3, args.warmup)):
        out = fn()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = max(args.steps, 5)
    torch.cuda.synchronize()
    t0.record()
    for _ in range(n):
        out = fn()
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / n
    assert L.load().fblt_tcgen05_error() == 0
    flops = 2.0 * rows * E * 3 * E + 2.0 * rows * E * E
    line = {"workload": "mha_block_c5_prefill", "sequences": args.batch, "rows": rows, "embed": E, "heads": H,
            "ms": ms, "rows_per_s": rows / ms * 1e3, "matmul_TFLOP/s_equivalent": flops / ms / 1e9,
            "launches": 3, "l2": "operands larger than L2"}
    if ob.have_ref():
        nseq = 4
        xs, wq, wp = x[: int(cu[nseq])].cpu().numpy(), w_qkv.cpu().numpy(), w_proj.cpu().numpy()
        t = time.perf_counter()
        err = 0.0
        for b in range(nseq):
            want = ob.ref_multihead_attention(xs[cu[b]:cu[b + 1]], wq, wp, H, is_causal=True, use_rope=True)
            err = max(err, float(np.abs(out[cu[b]:cu[b + 1]].cpu().numpy() - want).max()))
        cpu_s = time.perf_counter() - t
        line["cpu_reference"] = {"sequences": nseq, "rows": int(cu[nseq]), "seconds": cpu_s,
                                 "rows_per_s": int(cu[nseq]) / cpu_s, "cores": 1, "max_abs_err_vs_gpu": err}
    emit(line)


# dram__bytes_read + dram__bytes_write per algorithmic byte of the decode kernel, from an ncu capture
# of a 256-sequence launch; the traffic of a full launch is scaled from it by the rows processed
# (traffic grows in proportion: every cache row is read once).
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.009


def measure_host_link(torch, dev, barrier, world: int):
    """Ceiling of the host link in this run: every rank copies a 1 GiB pinned buffer to its GPU and back
    with plain asynchronous copies, all ranks at once -- one direction at a time and both together
    (the session overlaps uploads and downloads). GB/s per GPU, the slowest rank's figure."""
    import torch.distributed as dist
    n = 1 << 30
    host_a = torch.empty(n, dtype=torch.uint8, pin_memory=True)
    host_b = torch.empty(n, dtype=torch.uint8, pin_memory=True)
    host_a.fill_(1)
    dev_a = torch.empty(n, dtype=torch.uint8, device=dev)
    dev_b = torch.zeros(n, dtype=torch.uint8, device=dev)
    s_up, s_down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def run(up: bool, down: bool, reps: int = 3) -> float:
        barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            if up:
                with torch.cuda.stream(s_up):
                    dev_a.copy_(host_a, non_blocking=True)
            if down:
                with torch.cuda.stream(s_down):
                    host_b.copy_(dev_b, non_blocking=True)
        torch.cuda.synchronize()
        sec = time.perf_counter() - t0
        if world > 1:
            tt = torch.tensor([sec], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            sec = float(tt[0])
        return reps * n / sec / 1e9

    run(True, True, 1)
    res = {"h2d_GBps_per_gpu": run(True, False), "d2h_GBps_per_gpu": run(False, True)}
    both = run(True, True)
    res["duplex_GBps_per_gpu_each_way"] = both
    res["how"] = "1 GiB pinned <-> device, cudaMemcpyAsync, all ranks concurrently, slowest rank"
    del host_a, host_b, dev_a, dev_b
    return res


def run_e2e(args, torch, ops, dev, qkv, cu, rows, B, cache_rows, kc, vc, qn, kn, vn, world, total_bytes, barrier):
    import torch.distributed as dist
    steps = args.decode_steps
    sess = ops.Session(B, H, HD, max_q_rows=rows, max_k_rows=rows, cache_rows=cache_rows, max_new=N_NEW)
    h_qkv = torch.empty((rows, 3 * E), dtype=torch.float32, pin_memory=True)
    h_qkv.copy_(qkv)
    h_out = torch.empty((rows, E), dtype=torch.float32, pin_memory=True)
    h_kc = torch.empty((B, BASE_LEN, E), dtype=torch.float32, pin_memory=True)
    h_vc = torch.empty((B, BASE_LEN, E), dtype=torch.float32, pin_memory=True)
    h_kc.copy_(kc[:, :BASE_LEN])
    h_vc.copy_(vc[:, :BASE_LEN])
    # every decode step has rows of its own, as a caller's would be: [steps, B * 4, E] in and out
    step_rows = B * N_NEW
    h_new = [torch.empty((steps, step_rows, E), dtype=torch.float32, pin_memory=True) for _ in range(3)]
    gen = torch.Generator(device=dev).manual_seed(77)
    for h in h_new:
        for t in range(steps):
            h[t].copy_(torch.randn((step_rows, E), generator=gen, device=dev))
    h_od = torch.empty((steps, step_rows, E), dtype=torch.float32, pin_memory=True)
    torch.cuda.synchronize()
    lens0 = np.full(B, BASE_LEN, dtype=np.int32)
    q_h, k_h, v_h = h_qkv[:, 0:E], h_qkv[:, E:2 * E], h_qkv[:, 2 * E:]

    def step():
        # the prefill rows come home while the caches go up; everything is back at wait()
        sess.forward(q_h, k_h, v_h, h_out, cu, cu, SCALE, ops.MaskConfig(is_causal=True), q_stride=3 * E,
                     k_stride=3 * E, v_stride=3 * E, out_stride=E, wait=False)
        sess.cache_load(lens0, h_kc, h_vc, BASE_LEN)
        # the steps' rows are known up front here, so copies and kernels may overlap
        sess.decode_steps(B, N_NEW, steps, h_new[0], h_new[1], h_new[2], h_od, SCALE, block_mode=True,
                          in_step_stride=step_rows * E, out_step_stride=step_rows * E)
        sess.wait()

    step()  # warm-up
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        step()
    barrier()
    sec = (time.perf_counter() - t0) / args.e2e_steps
    if world > 1:
        tt = torch.tensor([sec], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        sec = float(tt[0])
    sess.close()
    del h_new, h_od, h_qkv, h_out, h_kc, h_vc
    h2d = 4 * E * (3 * rows + 2 * B * BASE_LEN + 3 * step_rows * steps)
    d2h = 4 * E * (rows + step_rows * steps)
    link = measure_host_link(torch, dev, barrier, world)
    # the copies of a step cannot take less than this on the link as measured (each direction at
    # its own one-way rate, the two fully overlapped: the kindest floor, so the fraction is a lower bound)
    floor_s = max(h2d / (link["h2d_GBps_per_gpu"] * 1e9), d2h / (link["d2h_GBps_per_gpu"] * 1e9))
    return {"value": total_bytes / sec / 1e9, "unit": UNIT, "ms_per_step": sec * 1e3, "timed_steps": args.e2e_steps,
            "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
            "link": link, "link_floor_ms": floor_s * 1e3, "frac_of_link": floor_s / sec,
            "rows": "every decode step uploads and downloads rows of its own (distinct pinned memory per step)",
            "path": "fblt_session_forward_async + fblt_session_cache_load + fblt_session_decode_steps + fblt_session_wait on pinned host buffers"}


def run_cpu_baseline(args, torch, qkv, cu, kc, vc, qn, kn, vn, out_p, out_d, total_rows):
    from oracle import binding as ob
    use_ref = ob.have_ref()
    threads = ob.host_cores()
    nb, db = min(args.cpu_prefill_seqs, len(cu) - 1), min(args.cpu_decode_seqs, kc.shape[0])
    cu_s = cu[: nb + 1].copy()
    qkv_h = qkv[: int(cu_s[-1])].cpu().numpy()
    kc_h, vc_h = kc[:db].cpu().numpy(), vc[:db].cpu().numpy()
    qn_h, kn_h, vn_h = (x[: db * N_NEW].cpu().numpy() for x in (qn, kn, vn))
    step_ids = list(range(0, args.decode_steps, max(1, args.decode_steps // args.cpu_decode_steps)))[: args.cpu_decode_steps]
    est, ref_p, ref_d, desc = cpu_sample(qkv_h, cu_s, kc_h, vc_h, qn_h, kn_h, vn_h, step_ids, args.batch, total_rows,
                                         args.decode_steps, threads, use_ref)
    # the sample doubles as a parity check of the timed GPU outputs (same tensors)
    err_p = float(np.abs(out_p[: int(cu_s[-1])].cpu().numpy() - ref_p).max())
    err_d = max(float(np.abs(out_d[t, : db * N_NEW].cpu().numpy() - r).max()) for t, r in zip(step_ids, ref_d))
    value = job_bytes(total_rows, args.batch, args.decode_steps) / est / 1e9
    return {"value": value, "unit": UNIT, "cores": threads, "kind": "reference" if use_ref else "port", "sample": desc,
            "est_job_seconds": est, "max_abs_err_vs_gpu": {"prefill": err_p, "decode": err_d}}


if __name__ == "__main__":
    main()
