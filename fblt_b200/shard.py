"""Batch sharding of independent sequences over the GPUs of one box.

Attention has no exchange step: every (sequence, head) is independent, so each
rank owns a contiguous range of sequences together with their Q/K/V rows and KV
caches, and the only collective is the gather of finished output rows. The
helpers are backend-agnostic (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import os
import subprocess
from typing import List, Optional, Set, Tuple

import torch
import torch.distributed as dist


def partition(num_sequences: int, world_size: int) -> List[Tuple[int, int]]:
    """Contiguous [begin, end) sequence ranges, sizes differing by at most one."""
    base, extra = divmod(num_sequences, world_size)
    out, start = [], 0
    for r in range(world_size):
        n = base + (1 if r < extra else 0)
        out.append((start, start + n))
        start += n
    return out


def gather_rows(local: torch.Tensor, rows_per_rank: List[int], group=None, padded: torch.Tensor = None,
                gathered: torch.Tensor = None):
    """All-gather of row blocks with unequal row counts.

    `local` is this rank's [rows_per_rank[rank], E] block. Every rank contributes a block
    padded to max(rows_per_rank) rows (all_gather needs equal sizes); the result is the
    [world, max_rows, E] buffer plus the list of valid row counts. `padded` / `gathered` may be
    passed in to avoid allocation inside a timed region.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    max_rows = max(rows_per_rank)
    E = local.shape[1]
    assert local.shape[0] == rows_per_rank[rank]
    if local.shape[0] == max_rows and local.is_contiguous():
        send = local
    else:
        send = padded if padded is not None else local.new_zeros((max_rows, E))
        send[: local.shape[0]].copy_(local)
    if gathered is None:
        gathered = local.new_empty((world, max_rows, E))
    dist.all_gather_into_tensor(gathered.view(world * max_rows, E), send, group=group)
    return gathered, rows_per_rank


class PeerGather:
    """All-gather of row blocks by one-sided copies over NVLink instead of a collective kernel.

    Every rank owns a [world, rows, E] buffer in symmetric memory (peer-mapped by
    torch.distributed._symmetric_memory); put() copies this rank's block into slot [rank] of every
    rank's buffer with plain device-to-device copies, which the driver runs on the copy engines,
    so the gather takes no SM from the attention launches it overlaps with (an NCCL all-gather
    runs as a kernel). Nothing is ever loaded from a peer: data lands in the owner's memory first.

    Completion is one-sided: when put() has finished on this rank's stream, this rank's rows have
    arrived everywhere; a rank's own buffer is complete once every rank has reached that point
    (a barrier, or the max over ranks of a device-timed region). Construction is collective.
    """

    def __init__(self, rows: int, E: int, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm
        # plain peer mappings are all the copies need; ask the allocator not to bind a multicast
        # object as well (a hint: this torch build still reports multicast support on the handle)
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.buf = symm.empty((self.world, rows, E), dtype=torch.float32, device=device)
        self.handle = symm.rendezvous(self.buf, group)
        self.peers = [self.buf if r == self.rank else self.handle.get_buffer(r, (self.world, rows, E), torch.float32)
                      for r in range(self.world)]

    def put(self, local: torch.Tensor, nrows: Optional[int] = None) -> None:
        """Enqueue, on the current stream, the copies of local[:nrows] into slot [rank] of every buffer."""
        n = local.shape[0] if nrows is None else nrows
        src = local[:n]
        for k in range(self.world):            # start with the next rank so that the ranks do not all
            r = (self.rank + 1 + k) % self.world   # write to the same peer at the same time
            self.peers[r][self.rank, :n].copy_(src, non_blocking=True)


class IpcGather:
    """The library's own gather (fblt_gather_* in include/fblt_attn.h) from Python: the same one-sided
    copy-engine copies as PeerGather, but set up and enqueued by the C ABI -- receive buffers from
    cudaMalloc, peers mapped through CUDA IPC handles that the ranks exchange on the host with a
    deadline (fblt_rendezvous_files over `exchange_dir`, a directory all ranks of the box share).
    No torch.distributed call is involved in the set-up or in put()."""

    def __init__(self, rows: int, E: int, rank: int, world: int, exchange_dir: str, tag: str, deadline_s: float = 120.0):
        import ctypes as C
        from . import lib as L
        self._lib, self.rank, self.world, self.rows, self.E = L.load(), rank, world, rows, E
        self._h = C.c_void_p()
        L.check(self._lib.fblt_gather_create(C.byref(self._h), rank, world, rows, E))
        nb = self._lib.fblt_gather_handle_bytes()
        mine = C.create_string_buffer(nb)
        L.check(self._lib.fblt_gather_export(self._h, mine))
        everyone = C.create_string_buffer(nb * world)
        os.makedirs(exchange_dir, exist_ok=True)
        L.check(self._lib.fblt_rendezvous_files(exchange_dir.encode(), tag.encode(), rank, world, mine, nb, everyone,
                                                int(deadline_s * 1000)))
        L.check(self._lib.fblt_gather_connect(self._h, everyone))
        ptr = self._lib.fblt_gather_buffer(self._h)
        # a tensor view of this rank's receive buffer (owned by the library)
        self.buf = _device_view(ptr, (world, rows, E))

    def put(self, local: torch.Tensor, nrows: Optional[int] = None, row_offset: int = 0, stream=None) -> None:
        from . import lib as L
        n = local.shape[0] if nrows is None else nrows
        assert local.is_contiguous() and local.dtype == torch.float32 and local.shape[1] == self.E
        st = (stream or torch.cuda.current_stream()).cuda_stream
        L.check(self._lib.fblt_gather_rows(self._h, local.data_ptr(), n, row_offset, st))

    def close(self) -> None:
        """Only after a barrier of the job: peers write into this rank's buffer until then."""
        if self._h:
            self.buf = None
            self._lib.fblt_gather_destroy(self._h)
            self._h = None


class _CudaArrayView:
    """Minimal __cuda_array_interface__ holder so that torch can view library-owned device memory."""

    def __init__(self, ptr: int, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (int(ptr), False), "version": 3}


def _device_view(ptr: int, shape) -> torch.Tensor:
    return torch.as_tensor(_CudaArrayView(ptr, shape), device="cuda")


def unpad(gathered: torch.Tensor, rows_per_rank: List[int]) -> torch.Tensor:
    """Concatenate the valid rows of a gather_rows() result in rank order."""
    return torch.cat([gathered[r, :n] for r, n in enumerate(rows_per_rank)], dim=0)


# ---- host-side check-in before collectives ------------------------------------------------------
# The reference has no failure handling beyond exit(1) (core/backend.h:13-31). With one process per
# GPU a rank that died, raised or fell behind must be noticed on the HOST, before the others enqueue
# a gather that would wait for it on the device: every rank checks in through the job's key-value
# store and waits, with a deadline, for the others. No kernel or collective is involved.

class RankTimeout(RuntimeError):
    """Some ranks did not check in before the deadline. `.missing` lists them."""

    def __init__(self, tag: str, missing: List[int], waited_s: float):
        super().__init__(f"rendezvous '{tag}': ranks {missing} did not check in within {waited_s:.1f} s")
        self.missing = missing


class RankFailed(RuntimeError):
    """A rank announced a failure (report_failure) instead of checking in. `.rank`, `.reason`."""

    def __init__(self, tag: str, rank: int, reason: str):
        super().__init__(f"rendezvous '{tag}': rank {rank} failed: {reason}")
        self.rank, self.reason = rank, reason


def _key(tag: str, kind: str, rank: int) -> str:
    return f"fblt/{tag}/{kind}/{rank}"


def report_failure(store, rank: int, tag: str, reason: str) -> None:
    """Called by a rank that cannot go on (exception, bad input): the others' rendezvous(tag) raises
    RankFailed at once instead of waiting for the deadline."""
    store.set(_key(tag, "failed", rank), reason.encode()[:512] or b"?")


def rendezvous(store, rank: int, world_size: int, tag: str, deadline_s: float = 30.0, poll_s: float = 0.005) -> None:
    """Check in under `tag` and return once every rank has checked in AND has seen everyone else do so.

    Two phases over any torch.distributed store shared by the ranks (the process group's own, a
    TCPStore, a FileStore): every rank publishes `ready`, waits for the others' `ready`, publishes
    `go`, waits for the others' `go`. A rank that gives up publishes `failed` first, so the outcome
    is the same on every rank: a rank that arrives after another one's deadline finds that rank's
    `failed` key and raises RankFailed instead of going on alone towards a peer that has left.
    Raises RankFailed as soon as any rank has announced a failure (report_failure, or a timeout
    elsewhere), RankTimeout (naming the absent ranks) when this rank's own deadline passes. The
    second phase has a deadline of its own: by then every rank was alive a moment ago. Tags must not
    be reused within a job."""
    import time
    others = [r for r in range(world_size) if r != rank]

    def wait_for(kind: str, limit_s: float) -> None:
        t0 = time.monotonic()
        while True:
            for r in others:
                if store.check([_key(tag, "failed", r)]):
                    raise RankFailed(tag, r, store.get(_key(tag, "failed", r)).decode(errors="replace"))
            missing = [r for r in others if not store.check([_key(tag, kind, r)])]
            if not missing:
                return
            waited = time.monotonic() - t0
            if waited >= limit_s:
                report_failure(store, rank, tag, f"timed out after {waited:.1f} s waiting for ranks {missing} ({kind})")
                raise RankTimeout(tag, missing, waited)
            time.sleep(poll_s)

    store.set(_key(tag, "ready", rank), b"1")
    wait_for("ready", deadline_s)
    store.set(_key(tag, "go", rank), b"1")
    wait_for("go", max(deadline_s, 5.0))


def default_store():
    """The key-value store of the default process group."""
    return dist.distributed_c10d._get_default_store()


def parse_cpulist(text: str) -> Set[int]:
    """'0-3,8,10-11' -> {0, 1, 2, 3, 8, 10, 11} (the format of /sys/devices/system/node/*/cpulist)."""
    cpus: Set[int] = set()
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-", 1)
            cpus.update(range(int(lo), int(hi) + 1))
        else:
            cpus.add(int(part))
    return cpus


def _pci_address(device_index: int) -> Optional[str]:
    props = torch.cuda.get_device_properties(device_index)
    if all(hasattr(props, a) for a in ("pci_domain_id", "pci_bus_id", "pci_device_id")):
        return f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
    try:
        out = subprocess.run(["nvidia-smi", f"--id={device_index}", "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20).stdout.strip()
        return out[-12:].lower() if out else None  # '00000000:1B:00.0' -> '0000:1b:00.0'
    except (OSError, subprocess.SubprocessError):
        return None


def bind_to_device_numa_node(device_index: int) -> dict:
    """Restrict this process to the CPUs of the NUMA node its GPU is attached to.

    Pinned host buffers allocated afterwards are first touched on that node, and the thread that
    issues the copies runs there, so host<->device traffic of a rank does not cross the socket
    interconnect. Every rank of a one-process-per-GPU job calls this before it allocates host
    memory. Returns what was done -- and, when nothing could be bound, why (`why_not`): the topology
    comes from sysfs first and from the driver (NVML's CPU affinity of the device) second."""
    info = {"numa_node": None, "cpus": None, "source": None, "why_not": None}
    allowed = os.sched_getaffinity(0)
    # 1) sysfs: the PCI device's NUMA node and that node's CPU list
    try:
        addr = _pci_address(device_index)
        if not addr:
            info["why_not"] = "no PCI address for the device"
        else:
            node = int(open(f"/sys/bus/pci/devices/{addr}/numa_node").read().strip())
            if node < 0:
                info["why_not"] = f"sysfs reports numa_node {node} for {addr} (no affinity exposed to this container)"
            else:
                cpus = parse_cpulist(open(f"/sys/devices/system/node/node{node}/cpulist").read())
                target = cpus & allowed
                if target:
                    os.sched_setaffinity(0, target)
                    info.update(numa_node=node, cpus=len(target), source="sysfs", why_not=None)
                    return info
                info["why_not"] = f"node {node}'s CPUs are outside this process's affinity mask"
    except (OSError, ValueError) as exc:
        info["why_not"] = f"sysfs: {type(exc).__name__}: {exc}"
    # 2) the driver's own answer (NVML: the CPUs closest to the device), read-only
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            props = torch.cuda.get_device_properties(device_index)
            handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(props.uuid)).encode()) if hasattr(props, "uuid") \
                else pynvml.nvmlDeviceGetHandleByIndex(device_index)
            words = (max(allowed | {0}) // 64) + 1
            mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
            cpus = {w * 64 + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1}
            target = cpus & allowed
            if target and target != allowed:
                os.sched_setaffinity(0, target)
                info.update(cpus=len(target), source="nvml cpu affinity", why_not=None)
            elif target == allowed:
                info["why_not"] = (info["why_not"] or "") + "; nvml: the device's CPU set is the whole affinity mask"
        finally:
            pynvml.nvmlShutdown()
    except Exception as exc:   # noqa: BLE001 - NVML absent or refusing is not an error for the caller
        info["why_not"] = (info["why_not"] or "") + f"; nvml: {type(exc).__name__}: {exc}"
    return info
