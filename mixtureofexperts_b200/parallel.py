"""Host-side plumbing of the expert-parallel layer (no counterpart in the reference, which has
no communication layer): expert partition, NCCL unique-id exchange, and the row layout of the
all-to-all exchange."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib


def expert_partition(num_experts: int, world: int, rank: int) -> range:
    """Experts are block-partitioned: rank r owns [r*E/world, (r+1)*E/world)."""
    if num_experts % world:
        raise _lib.MoEError(_lib.ERR_INVALID, f"num_experts ({num_experts}) must be divisible by world ({world})")
    per = num_experts // world
    return range(rank * per, (rank + 1) * per)


def _parse_cpulist(text: str) -> set:
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_to_gpu_numa_node(pci_bus_id: str, sysfs: str = "/sys") -> dict:
    """Pin the calling process to the CPUs of the NUMA node its GPU hangs off, so that the pinned
    host buffers it allocates next are first-touched in the memory closest to that GPU's PCIe
    root.  With one process per GPU and all GPUs copying at once, buffers on the far socket halve
    the host-copy rate.  ``pci_bus_id`` is "domain:bus:device.function" as CUDA reports it.

    Returns {"node": n, "cpus": count} on success; {"node": -1, "why": ...} and no change when the
    node is unknown (virtualised PCI topology), the CPU list is empty, or the process may not use
    those CPUs (a cgroup cpuset)."""
    import os

    dev = pci_bus_id.lower()
    if dev.count(":") == 1:
        dev = "0000:" + dev
    if len(dev.split(":")[0]) > 4:      # CUDA prints an 8-digit domain, sysfs a 4-digit one
        dev = dev.split(":")[0][-4:] + dev[dev.index(":"):]
    try:
        with open(f"{sysfs}/bus/pci/devices/{dev}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return {"node": -1, "why": "sysfs reports no NUMA node for the GPU"}
        with open(f"{sysfs}/devices/system/node/node{node}/cpulist") as f:
            cpus = _parse_cpulist(f.read())
    except (OSError, ValueError) as exc:
        return {"node": -1, "why": f"{type(exc).__name__}: {exc}"}
    allowed = cpus & os.sched_getaffinity(0)
    if not allowed:
        return {"node": -1, "why": "none of the node's CPUs are in this process's affinity mask"}
    os.sched_setaffinity(0, allowed)
    return {"node": node, "cpus": len(allowed)}


def new_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    _lib.check(_lib.lib.moe_ep_unique_id(buf))
    return buf.raw


def broadcast_unique_id(dist, rank: int, device=None, make_id=new_unique_id) -> bytes:
    """Rank 0 draws an NCCL unique id and ships it to every rank of the default
    torch.distributed group (any backend); returns the 128 bytes."""
    import torch

    t = torch.zeros(128, dtype=torch.uint8, device=device)
    if rank == 0:
        t.copy_(torch.frombuffer(bytearray(make_id()), dtype=torch.uint8))
    dist.broadcast(t, src=0)
    return bytes(t.cpu().numpy().tobytes())


def exchange_layout(counts, rank: int, tile_m: int):
    """Row layout of one rank's dispatch/combine, from the all-gathered pair counts
    ``counts[world][E]`` -- the host arithmetic a forward call runs (moe_ep_layout of the C ABI).

    Returns (send_off[E+1], recv_off[per][world], local_off[per+1], tile_prefix[per+1], rows):
    rows this rank sends to expert e start at send_off[e] of its permuted buffer; rows it
    receives from rank r for its local expert el land at recv_off[el][r]; local_off/tile_prefix
    describe the received rows grouped by local expert for the grouped GEMM."""
    counts = np.ascontiguousarray(counts, dtype=np.int32)
    world, E = counts.shape
    per = E // world
    send_off = np.zeros(E + 1, dtype=np.int64)
    recv_off = np.zeros((per, world), dtype=np.int64)
    local_off = np.zeros(per + 1, dtype=np.int32)
    tile_prefix = np.zeros(per + 1, dtype=np.int32)
    rows = _lib.lib.moe_ep_layout(counts.ctypes.data, world, E, int(rank), int(tile_m), send_off.ctypes.data,
                                  recv_off.ctypes.data, local_off.ctypes.data, tile_prefix.ctypes.data)
    if rows < 0:
        _lib.check(int(rows))
    return send_off, recv_off, local_off, tile_prefix, int(rows)


def all_gather_counts(dist, counts, rank: int, timeout_s: float = 30.0):
    """All-gather of the per-expert pair counts over the default torch.distributed group for callers
    that run the exchange themselves (the library's own forward exchanges them on the device).
    Bounded like the library's collectives: a rank that never posts its counts ends the wait with
    MoEError(ERR_TIMEOUT) after ``timeout_s`` instead of hanging, and a gathered table whose own
    row differs from what this rank posted, or that holds a negative count, raises
    MoEError(ERR_NCCL).  Returns ``counts[world][E]`` (int32)."""
    import datetime

    import torch

    mine = torch.from_numpy(np.ascontiguousarray(counts, dtype=np.int32))
    world = dist.get_world_size()
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    try:
        work = dist.all_gather(gathered, mine, async_op=True)
        done = work.wait(timeout=datetime.timedelta(seconds=timeout_s))
    except Exception as exc:  # noqa: BLE001  (gloo reports a missing peer as a RuntimeError)
        raise _lib.MoEError(_lib.ERR_TIMEOUT, f"a rank did not post its routing counts within {timeout_s} s: {exc}") from None
    if done is False:
        raise _lib.MoEError(_lib.ERR_TIMEOUT, f"a rank did not post its routing counts within {timeout_s} s")
    cnt = np.stack([g.numpy() for g in gathered]).astype(np.int32)
    if not np.array_equal(cnt[rank], mine.numpy()) or (cnt < 0).any():
        raise _lib.MoEError(_lib.ERR_NCCL, "the gathered routing counts do not match this rank's own (corrupted exchange)")
    return cnt
