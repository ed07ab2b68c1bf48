"""DAXPY and DDOT with the vectors pre-split across the GPUs, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 \
        paralia-framework_b200/level1_ranks.py [--n 1073741824] [--tile 8388608] [--iters 5]

Rank r holds the contiguous run ``ranks.vector_chunk(r, G, N, quantum=tile)`` of x and y in
the memory of its own GPU (generated there from the global seeds 42 / 43, so the union of the
chunks is the same vector a single process would fill). DAXPY (alpha = -0.5) needs no exchange
at all; DDOT gathers the per-tile sums of all ranks and adds them in global tile order
(``ranks.ddot_tiles_in_order``), which reproduces the bits of a one-process call with the same
tile length. Rank 0 prints one JSON line: aggregate GB/s over all GPUs (24 B per element for
DAXPY, 16 B for DDOT; device time = CUDA events around the calls, max over the ranks).

Reference: the reference splits level-1 work into tiles dealt to the GPUs and sums the DDOT
partials on the host in tile order (Library_scheduler/src/Functions/daxpy.cpp:200-469,
ddot.cpp:201-469,431); it has no multi-process mode.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent


def _pkg():
    name = "paralia_framework_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, PKG_DIR / "__init__.py",
                                                  submodule_search_locations=[str(PKG_DIR)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=1 << 30)
    ap.add_argument("--tile", type=int, default=1 << 23)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args(argv)
    import importlib
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dev = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(dev)
    cuda = f"cuda:{dev}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(cuda))
    pl = _pkg()
    pl.init()
    ranks = importlib.import_module("paralia_framework_b200.ranks")
    lo, hi = ranks.vector_chunk(rank, world, a.n, quantum=a.tile)
    m = hi - lo
    x = torch.empty(m, dtype=torch.float64, device=cuda)
    y = torch.empty(m, dtype=torch.float64, device=cuda)
    # element i of the global vector depends on (seed, i) only: generate the prefix [0, hi) of
    # the global vector on this GPU and keep the chunk (a temporary of at most 8 * N bytes)
    for (vec, seed) in ((x, 42), (y, 43)):
        full = torch.empty(hi, dtype=torch.float64, device=cuda)
        pl.fill_f64(full, hi, seed, 0, dev)
        vec.copy_(full[lo:hi])
        del full
    ctl = pl.make_ctl(T=a.tile, units=[dev])

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = None
        for _ in range(a.iters):
            out = fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / a.iters], dtype=torch.float64, device=cuda)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() * 1e-3, out

    t_dot, sums = timed(lambda: pl.ddot_tiles(m, x, 1, y, 1, locx=dev, locy=dev, ctl=ctl)[0])
    dot = ranks.ddot_tiles_in_order(sums, start=0.0, device=cuda)
    t_axpy, _ = timed(lambda: pl.daxpy(m, -0.5, x, 1, y, 1, locx=dev, locy=dev, ctl=ctl))
    if rank == 0:
        print(json.dumps({"routine": "level1 pre-split", "n": a.n, "gpus": world, "tile": a.tile,
                          "ddot_gbs": 16.0 * a.n / t_dot / 1e9, "daxpy_gbs": 24.0 * a.n / t_axpy / 1e9,
                          "ddot": dot, "per_rank_elements": m}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
