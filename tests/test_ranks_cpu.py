"""The one-process-per-GPU partition, exercised with world_size 2 and 4 on the CPU
(gloo): every rank computes its C block / vector chunk with the CPU oracle, the blocks
are gathered and must equal the whole-problem result; DDOT partials meet in one
all-reduce."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, M, N, K, nvec, out_dir):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    entry.load_package()
    import importlib
    ranks = importlib.import_module("paralia_framework_b200.ranks")
    orc = entry.load_oracle()

    A = orc.matrix_f64(M, K, 42)
    B = orc.matrix_f64(K, N, 43)
    C = orc.matrix_f64(M, N, 44)
    (m0, m1), (n0, n1), _, _ = ranks.gemm_block(rank, world, M, N, quantum=16)
    blk = np.asfortranarray(C[m0:m1, n0:n1])
    if m1 > m0 and n1 > n0:
        orc.dgemm_tiled("N", "N", m1 - m0, n1 - n0, K, 1.25, A[m0:, :], M, B[:, n0:], K, 0.75,
                        blk, m1 - m0, 32)
    # gather the blocks on rank 0
    full = torch.zeros(M, N, dtype=torch.float64)
    full[m0:m1, n0:n1] = torch.from_numpy(np.ascontiguousarray(blk))
    dist.all_reduce(full)          # blocks are disjoint, the sum places them
    # DDOT: chunk partials -> one all-reduce
    x = orc.uniform_f64(nvec, 42)
    y = orc.uniform_f64(nvec, 43)
    lo, hi = ranks.vector_chunk(rank, world, nvec, quantum=64)
    part, _ = orc.ddot_tiled(hi - lo, x[lo:], 1, y[lo:], 1, 128, 0.0)
    total = ranks.allreduce_sum(part)
    np.save(os.path.join(out_dir, f"dot_rank{rank}.npy"), np.array([part, total]))
    # the bit-exact form: runs of whole tiles per rank, per-tile sums combined in tile order
    T = 128
    tlo, thi = ranks.vector_chunk(rank, world, nvec, quantum=T)
    sums = []
    for s0 in range(tlo, thi, T):
        n_t = min(T, thi - s0)
        v, _ = orc.ddot_tiled(n_t, x[s0:], 1, y[s0:], 1, T, 0.0)
        sums.append(v)
    exact = ranks.ddot_tiles_in_order(sums, start=0.25)
    np.save(os.path.join(out_dir, f"dot_exact_rank{rank}.npy"), np.array([exact]))
    cover = torch.zeros(nvec, dtype=torch.int32)
    cover[lo:hi] += 1
    dist.all_reduce(cover)
    if rank == 0:
        np.save(os.path.join(out_dir, "C.npy"), full.numpy())
        np.save(os.path.join(out_dir, "dot.npy"), np.array([total]))
        np.save(os.path.join(out_dir, "cover.npy"), cover.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_rank_partition_reassembles_whole_problem(orc, tmp_path, world):
    import torch.multiprocessing as mp
    M, N, K, nvec = 200, 136, 96, 10007
    port = 29500 + os.getpid() % 2000 + world
    mp.spawn(_worker, args=(world, port, M, N, K, nvec, str(tmp_path)), nprocs=world, join=True)
    got = np.load(tmp_path / "C.npy")
    A = orc.matrix_f64(M, K, 42)
    B = orc.matrix_f64(K, N, 43)
    want = orc.matrix_f64(M, N, 44)
    orc.dgemm_tiled("N", "N", M, N, K, 1.25, A, M, B, K, 0.75, want, M, 32)
    assert orc.normwise_rel_err(got, want) <= 8 * K * 2.0 ** -52
    x = orc.uniform_f64(nvec, 42)
    y = orc.uniform_f64(nvec, 43)
    dot, mag = orc.ddot_tiled(nvec, x, 1, y, 1, 128, 0.0)
    assert abs(np.load(tmp_path / "dot.npy")[0] - dot) <= nvec * 2.0 ** -52 * mag
    assert (np.load(tmp_path / "cover.npy") == 1).all()   # every element owned exactly once
    # the rank partials are added in rank order on every rank: same bits everywhere
    per_rank = [np.load(tmp_path / f"dot_rank{r}.npy") for r in range(world)]
    ordered = 0.0
    for part, _ in per_rank:
        ordered += float(part)
    assert all(float(total) == ordered for _, total in per_rank)
    # per-tile sums combined in the global tile order: the single-process bits, on every rank
    whole, _ = orc.ddot_tiled(nvec, x, 1, y, 1, 128, 0.25)
    for r in range(world):
        assert float(np.load(tmp_path / f"dot_exact_rank{r}.npy")[0]) == whole


def test_gemm_block_grid_matches_library(pl):
    import importlib
    ranks = importlib.import_module("paralia_framework_b200.ranks")
    for world in (1, 2, 3, 4, 6, 8):
        d1, d2 = ranks.device_grid(world)
        _, ld1, ld2 = pl.distribute_2d(world, 8 * d1, 8 * d2, 1)
        assert (d1, d2) == (ld1, ld2)
        # the rank's block is exactly the set of C tiles the library gives unit `rank`
        owner, _, _ = pl.distribute_2d(world, 8 * d1, 8 * d2, 1)
        T = 16
        for rank in range(world):
            (m0, m1), (n0, n1), _, _ = ranks.gemm_block(rank, world, 8 * d1 * T, 8 * d2 * T, T)
            tiles = {(mi, ni) for mi in range(m0 // T, m1 // T) for ni in range(n0 // T, n1 // T)}
            lib_tiles = {(sk // (8 * d2), sk % (8 * d2)) for sk, u in enumerate(owner) if u == rank}
            assert tiles == lib_tiles
