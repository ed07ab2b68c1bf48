"""Host-side partition for the one-process-per-GPU launch (torchrun).

The library itself drives every GPU of the box from one process, as the reference does.
When a launcher starts one process per GPU instead, each rank calls the library on the
part of the problem its GPU would own in-process: the C block of its cell in the
D1 x D2 device grid for GEMM (no exchange between ranks), a contiguous chunk for the
level-1 routines (one scalar all-reduce for DDOT). This module holds that arithmetic;
it needs no GPU.

Reference: grid rule Autotuner/src/Subkernel_distributions.cpp:325-336, owner of a C
tile :399, DDOT's final sum Library_scheduler/src/Functions/ddot.cpp:431.
"""
from __future__ import annotations

import math


def device_grid(units: int) -> tuple[int, int]:
    """Most-square factorisation units = d1*d2 found by the reference's scan."""
    d1 = int(math.sqrt(units))
    if d1 == 0:
        return 1, units
    g = d1 + 1
    while g > 0 and units % g:
        g -= 1
    if g == 0:
        return units, 1
    return g, units // g


def _split(n: int, parts: int, idx: int, quantum: int = 1) -> tuple[int, int]:
    """[lo, hi) of part idx when n is cut into `parts` runs of whole quanta, the first
    runs one quantum longer when it does not divide."""
    q = -(-n // quantum)
    base, extra = divmod(q, parts)
    lo = idx * base + min(idx, extra)
    hi = lo + base + (1 if idx < extra else 0)
    return min(lo * quantum, n), min(hi * quantum, n)


def gemm_block(rank: int, world: int, M: int, N: int, quantum: int = 1):
    """Rows [m0, m1) and columns [n0, n1) of C that `rank` computes; rank = r*d2 + c."""
    d1, d2 = device_grid(world)
    r, c = divmod(rank, d2)
    m0, m1 = _split(M, d1, r, quantum)
    n0, n1 = _split(N, d2, c, quantum)
    return (m0, m1), (n0, n1), (r, c), (d1, d2)


def vector_chunk(rank: int, world: int, N: int, quantum: int = 1) -> tuple[int, int]:
    """Contiguous run [lo, hi) of a length-N vector owned by `rank`."""
    return _split(N, world, rank, quantum)


def allreduce_sum(value: float, device=None) -> float:
    """Sum of one double over all ranks (DDOT's cross-GPU reduction; the reference adds the
    per-tile partials on the host in tile order, ddot.cpp:431). The rank partials are
    gathered (NCCL on GPUs, gloo on CPUs) and added in rank order on every rank, so all
    ranks return the same bits and a rerun reproduces them; a reducing collective would
    leave the order of the additions to the backend. With torch.distributed not
    initialised the value is returned unchanged."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    mine = torch.tensor([value], dtype=torch.float64, device=device)
    parts = [torch.empty_like(mine) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, mine)
    total = 0.0
    for p in parts:            # rank order
        total += float(p.item())
    return total


def ddot_tiles_in_order(tile_sums, start: float = 0.0, device=None) -> float:
    """DDOT across ranks, bit-equal to the single-process result. Every rank holds a contiguous
    run of WHOLE tiles of the vectors (``vector_chunk`` with quantum = the tile length) and
    passes the per-tile sums of its run (``ddot_tiles``). The runs are gathered in rank order,
    which is the global tile order, and added one tile after the other to ``start`` on every
    rank -- exactly the sequence of additions the library performs when one process owns the
    whole vector (reference: the host-side sum in tile order, ddot.cpp:431)."""
    import torch
    import torch.distributed as dist

    mine = [float(v) for v in tile_sums]
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        runs = [mine]
    else:
        world = dist.get_world_size()
        n = torch.tensor([len(mine)], dtype=torch.int64, device=device)
        counts = [torch.empty_like(n) for _ in range(world)]
        dist.all_gather(counts, n)
        longest = max(int(c.item()) for c in counts)
        pad = torch.zeros(max(longest, 1), dtype=torch.float64, device=device)
        if mine:
            pad[:len(mine)] = torch.tensor(mine, dtype=torch.float64, device=device)
        parts = [torch.empty_like(pad) for _ in range(world)]
        dist.all_gather(parts, pad)
        runs = [p[:int(c.item())].tolist() for p, c in zip(parts, counts)]
    acc = float(start)
    for run in runs:              # rank order = global tile order
        for v in run:
            acc += v
    return acc
