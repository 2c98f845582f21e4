"""Host-side plumbing for minibatch-sharded (data-parallel) runs: one process
per GPU, launched by ``torch.distributed.run``.

The gradient exchange itself happens inside the library (peer-memory or NCCL all-reduce on its
own stream, started from backward()).  ``torch.distributed`` is only the
rendezvous: it carries the 128-byte NCCL id from rank 0 to the others, provides
the barrier around timed regions and the max-over-ranks of a timing.
"""
from __future__ import annotations

import os


def shard_rows(total_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Rows [begin, end) of a global batch owned by ``rank``.  Contiguous blocks;
    the first ``total_rows % world`` ranks hold one extra row."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(total_rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def bind_near_gpu(device_index: int) -> dict:
    """Restricts this process to the CPUs of the NUMA node its GPU hangs off, so that
    pinned staging buffers allocated afterwards are local to that GPU's PCIe root
    (eight ranks staging through one socket's memory share its bandwidth).  Uses
    only what the process is already allowed to run on; returns what was done."""
    info = {"numa_node": None, "bound": False, "cpus": len(os.sched_getaffinity(0))}
    try:
        import pynvml
        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(device_index)).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        # NVML prints an 8-digit PCI domain, sysfs a 4-digit one
        dom, rest = bus.split(":", 1)
        sysfs = f"/sys/bus/pci/devices/{dom[-4:].lower()}:{rest.lower()}"
        with open(os.path.join(sysfs, "numa_node")) as f:
            info["numa_node"] = int(f.read().strip())
        with open(os.path.join(sysfs, "local_cpulist")) as f:
            local = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                local.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & local
        if allowed and allowed != os.sched_getaffinity(0):
            os.sched_setaffinity(0, allowed)
            info["bound"] = True
        info["cpus"] = len(os.sched_getaffinity(0))
    except Exception as exc:  # no NVML, no sysfs entry, or not permitted: stay as launched
        info["note"] = f"{type(exc).__name__}: {exc}"[:120]
    return info


def env_rank_world() -> tuple[int, int, int]:
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def broadcast_bytes(payload: bytes | None, nbytes: int, src: int = 0) -> bytes:
    """Broadcast a small byte string over the default torch.distributed group."""
    import torch
    import torch.distributed as dist
    buf = torch.zeros(nbytes, dtype=torch.uint8)
    if dist.get_rank() == src:
        buf = torch.frombuffer(bytearray(payload), dtype=torch.uint8).clone()
    if dist.get_backend() == "nccl":
        buf = buf.cuda()
    dist.broadcast(buf, src=src)
    return bytes(buf.cpu().numpy().tobytes())


def init_comm(api) -> tuple[int, int]:
    """Bring up the library's NCCL communicator across the torch.distributed
    group (which must already be initialised).  Returns (rank, world)."""
    import torch.distributed as dist
    rank, world = dist.get_rank(), dist.get_world_size()
    if world == 1:
        return rank, world
    uid = api.comm_unique_id() if rank == 0 else None
    uid = broadcast_bytes(uid, 128, src=0)
    api.comm_init(uid, rank, world)
    return rank, world


def max_over_ranks(value: float) -> float:
    import torch
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64)
    if dist.get_backend() == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
