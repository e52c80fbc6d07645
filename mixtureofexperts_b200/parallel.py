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
    ``counts[world][E]`` (the same arithmetic libmoe_b200 runs on the host inside a forward).

    Returns (send_off[E+1], recv_off[per][world], local_off[per+1], tile_prefix[per+1]):
    rows this rank sends to expert e start at send_off[e] of its permuted buffer; rows it
    receives from rank r for its local expert el land at recv_off[el][r]; local_off/tile_prefix
    describe the received rows grouped by local expert for the grouped GEMM."""
    counts = np.asarray(counts, dtype=np.int64)
    world, E = counts.shape
    per = E // world
    send_off = np.zeros(E + 1, dtype=np.int64)
    send_off[1:] = np.cumsum(counts[rank])
    recv_off = np.zeros((per, world), dtype=np.int64)
    local_off = np.zeros(per + 1, dtype=np.int64)
    tile_prefix = np.zeros(per + 1, dtype=np.int64)
    rows = 0
    tiles = 0
    for el in range(per):
        local_off[el] = rows
        tile_prefix[el] = tiles
        n_e = 0
        for r in range(world):
            recv_off[el, r] = rows + n_e
            n_e += counts[r, rank * per + el]
        rows += n_e
        tiles += (n_e + tile_m - 1) // tile_m
    local_off[per] = rows
    tile_prefix[per] = tiles
    return send_off, recv_off, local_off, tile_prefix
