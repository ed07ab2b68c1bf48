"""In-process multi-GPU path (the library drives several GPUs from one process, like
the reference): 2D block ownership of C, home-GPU host fetch plus NVLink forwarding,
operands spread over different GPUs. Needs at least two GPUs."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
EPS64 = 2.0 ** -52
ROOT = Path(__file__).resolve().parent.parent


def _ngpu():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


need2 = pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
need4 = pytest.mark.skipif(_ngpu() < 4, reason="needs four GPUs")


def _dev(t, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(t.T)).to(f"cuda:{dev}")


@need2
@pytest.mark.parametrize("ta,tb", [("N", "N"), ("T", "N"), ("N", "T")])
@pytest.mark.parametrize("peer", [True, False])
def test_dgemm_two_gpus_host_resident(pl, orc, ta, tb, peer):
    M, N, K, T = 1024, 768, 512, 256
    ar, ac = (K, M) if ta == "T" else (M, K)
    br, bc = (N, K) if tb == "T" else (K, N)
    A = orc.matrix_f64(ar, ac, 42)
    B = orc.matrix_f64(br, bc, 43)
    C = orc.matrix_f64(M, N, 44)
    want = C.copy(order="F")
    orc.dgemm_tiled(ta, tb, M, N, K, 1.23, A, ar, B, br, 0.9876, want, M, T)
    flags = 0 if peer else pl.FLAG_NO_PEER_FETCH
    rep = pl.dgemm(ta, tb, M, N, K, 1.23, A, ar, B, br, 0.9876, C, M,
                   ctl=pl.make_ctl(T=T, units=[0, 1], flags=flags))
    assert orc.normwise_rel_err(C, want) <= 8 * K * EPS64
    assert rep.active_unit_num == 2 and (rep.grid_d1, rep.grid_d2) == (2, 1)
    assert list(rep.subkernels_per_unit[:2]) == [rep.subkernel_num // 2] * 2
    szA, szB, szC = M * K * 8, K * N * 8, M * N * 8
    if peer:
        # grid 2 x 1: each GPU owns half of the tile rows; B is read by both -> every B tile
        # crosses the host link once and NVLink once; A tiles are private to a GPU
        assert rep.h2d_bytes == szA + szB + szC
        assert rep.p2p_bytes == szB
    else:
        assert rep.h2d_bytes == szA + 2 * szB + szC
        assert rep.p2p_bytes == 0
    assert rep.d2h_bytes == szC


@need2
def test_dgemm_two_gpus_bitwise_equal_to_one_gpu(pl, orc):
    # the arithmetic of a C tile does not depend on which GPU runs it
    M = N = K = 1024
    A = orc.matrix_f64(M, K, 42)
    B = orc.matrix_f64(K, N, 43)
    C0 = orc.matrix_f64(M, N, 44)
    C1, C2 = C0.copy(order="F"), C0.copy(order="F")
    pl.dgemm("N", "N", M, N, K, 1.23, A, M, B, K, 0.9876, C1, M, ctl=pl.make_ctl(T=256, units=[0]))
    pl.dgemm("N", "N", M, N, K, 1.23, A, M, B, K, 0.9876, C2, M, ctl=pl.make_ctl(T=256, units=[0, 1]))
    assert np.array_equal(C1, C2)
    C3 = C0.copy(order="F")
    pl.dgemm("N", "N", M, N, K, 1.23, A, M, B, K, 0.9876, C3, M, ctl=pl.make_ctl(T=256, units=[1, 0]))
    assert np.array_equal(C1, C3)


@need2
def test_dgemm_operands_on_different_gpus(pl, orc):
    # the placement of BASELINE config 3: A (transposed) on GPU 0, B on GPU 1, C on the host, beta = 0
    import torch
    M, N, K, T = 1024, 1024, 256, 256
    A = orc.matrix_f64(K, M, 42)   # stored K x M, ldA = K
    B = orc.matrix_f64(K, N, 43)
    C = orc.matrix_f64(M, N, 44)
    want = C.copy(order="F")
    orc.dgemm_tiled("T", "N", M, N, K, 1.0, A, K, B, K, 0.0, want, M, T)
    dA, dB = _dev(A, 0), _dev(B, 1)
    rep = pl.dgemm("T", "N", M, N, K, 1.0, dA, K, dB, K, 0.0, C, M, ctl=pl.make_ctl(T=T, units=[0, 1]))
    assert orc.normwise_rel_err(C, want) <= 8 * K * EPS64
    assert rep.h2d_bytes == 0 and rep.d2h_bytes == M * N * 8 and rep.p2p_bytes > 0


@need2
def test_dgemm_c_on_other_gpu(pl, orc):
    import torch
    M, N, K, T = 512, 512, 512, 256
    A = orc.matrix_f64(M, K, 42)
    B = orc.matrix_f64(K, N, 43)
    C = orc.matrix_f64(M, N, 44)
    want = C.copy(order="F")
    orc.dgemm_tiled("N", "N", M, N, K, 1.23, A, M, B, K, 0.9876, want, M, T)
    dC = _dev(C, 1)
    pl.dgemm("N", "N", M, N, K, 1.23, A, M, B, K, 0.9876, dC, M, ctl=pl.make_ctl(T=T, units=[0]))
    torch.cuda.synchronize(1)
    got = np.asfortranarray(dC.cpu().numpy().T)
    assert orc.normwise_rel_err(got, want) <= 8 * K * EPS64


@need2
def test_level1_two_gpus(pl, orc):
    n = (1 << 21) + 5
    x = orc.uniform_f64(n, 42)
    y = orc.uniform_f64(n, 43)
    want_y = y.copy()
    orc.daxpy_tiled(n, -0.5, x, 1, want_y, 1, n)
    want_dot, mag = orc.ddot_tiled(n, x, 1, y, 1, 1 << 16, 0.0)
    dot, rep = pl.ddot(n, x, 1, y, 1, 0.0, ctl=pl.make_ctl(T=1 << 16, units=[0, 1]))
    assert rep.active_unit_num == 2
    assert abs(dot - want_dot) <= n * EPS64 * mag
    dot1, _ = pl.ddot(n, x, 1, y, 1, 0.0, ctl=pl.make_ctl(T=1 << 16, units=[0]))
    assert dot == dot1      # same tiles, same order of the final sum: bit-identical
    pl.daxpy(n, -0.5, x, 1, y, 1, ctl=pl.make_ctl(T=1 << 16, units=[0, 1]))
    assert np.array_equal(y, want_y)


@need2
def test_dgemm_two_gpus_bounded_cache(pl, orc):
    M, N, K, T = 1024, 1024, 768, 256
    A = orc.matrix_f64(M, K, 42)
    B = orc.matrix_f64(K, N, 43)
    C = orc.matrix_f64(M, N, 44)
    want = C.copy(order="F")
    orc.dgemm_tiled("N", "N", M, N, K, 1.23, A, M, B, K, 0.9876, want, M, T)
    rep = pl.dgemm("N", "N", M, N, K, 1.23, A, M, B, K, 0.9876, C, M,
                   ctl=pl.make_ctl(T=T, units=[0, 1], cache_limit=8 * T * T * 8))
    assert orc.normwise_rel_err(C, want) <= 8 * K * EPS64
    assert rep.p2p_bytes == 0 and rep.h2d_bytes > (M * K + K * N + M * N) * 8


@need2
def test_sgemm_two_gpus(pl, orc):
    M, N, K, T = 1024, 768, 512, 256
    A = orc.uniform_f32(M * K, 42).reshape((M, K), order="F")
    B = orc.uniform_f32(K * N, 43).reshape((K, N), order="F")
    C = orc.uniform_f32(M * N, 44).reshape((M, N), order="F")
    want = 1.25 * (A.astype(np.float64) @ B.astype(np.float64)) + 0.75 * C.astype(np.float64)
    C1 = C.copy(order="F")
    pl.sgemm("N", "N", M, N, K, 1.25, A, M, B, K, 0.75, C1, M, ctl=pl.make_ctl(T=T, units=[0]))
    rep = pl.sgemm("N", "N", M, N, K, 1.25, A, M, B, K, 0.75, C, M, ctl=pl.make_ctl(T=T, units=[0, 1]))
    assert orc.normwise_rel_err(C, want) <= 4 * K * 2.0 ** -23
    assert np.array_equal(C, C1)          # same bits on one and on two GPUs
    assert rep.h2d_bytes == (M * K + K * N + M * N) * 4 and rep.p2p_bytes > 0


@need4
def test_dgemm_four_gpus_grid(pl, orc):
    M, N, K, T = 1024, 1024, 512, 256
    A = orc.matrix_f64(M, K, 42)
    B = orc.matrix_f64(K, N, 43)
    C = orc.matrix_f64(M, N, 44)
    want = C.copy(order="F")
    orc.dgemm_tiled("N", "N", M, N, K, 1.23, A, M, B, K, 0.9876, want, M, T)
    rep = pl.dgemm("N", "N", M, N, K, 1.23, A, M, B, K, 0.9876, C, M,
                   ctl=pl.make_ctl(T=T, units=[0, 1, 2, 3]))
    assert orc.normwise_rel_err(C, want) <= 8 * K * EPS64
    assert (rep.grid_d1, rep.grid_d2) == (2, 2)
    szA, szB, szC = M * K * 8, K * N * 8, M * N * 8
    assert rep.h2d_bytes == szA + szB + szC      # every host tile crosses a host link once
    assert rep.p2p_bytes == szA + szB            # and is forwarded to one grid neighbour


def _l1_rank(rank, world, port, n, T, out_dir):
    """One process per GPU over NCCL: vectors pre-split across the GPUs (BASELINE configs[4])."""
    sys.path.insert(0, str(ROOT))
    import importlib
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    pl = entry.load_package()
    ranks = importlib.import_module("paralia_framework_b200.ranks")
    lo, hi = ranks.vector_chunk(rank, world, n, quantum=T)
    m = hi - lo
    # the rank's chunk of the seeded global vectors, resident on its own GPU
    x = torch.empty(n, dtype=torch.float64, device=f"cuda:{rank}")
    y = torch.empty(n, dtype=torch.float64, device=f"cuda:{rank}")
    pl.fill_f64(x, n, 42, 0, rank)
    pl.fill_f64(y, n, 43, 0, rank)
    xc, yc = x[lo:hi].clone(), y[lo:hi].clone()
    ctl = pl.make_ctl(T=T, units=[rank])
    sums, _ = pl.ddot_tiles(m, xc, 1, yc, 1, locx=rank, locy=rank, ctl=ctl)
    dot = ranks.ddot_tiles_in_order(sums, start=0.0, device=f"cuda:{rank}")
    pl.daxpy(m, -0.5, xc, 1, yc, 1, locx=rank, locy=rank, ctl=ctl)
    torch.cuda.synchronize()
    np.save(os.path.join(out_dir, f"l1_{rank}.npy"), np.array([dot, lo, hi]))
    np.save(os.path.join(out_dir, f"y_{rank}.npy"), yc.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_level1_presplit_ranks_bit_equal_to_one_gpu(pl, tmp_path):
    """DAXPY and DDOT with the vectors pre-split over one process per GPU: the chunk results
    and the dot product, combined in global tile order, equal the one-GPU call bit for bit."""
    import torch
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    n, T = (1 << 24) + 12345, 1 << 20
    port = 29700 + os.getpid() % 2000
    mp.spawn(_l1_rank, args=(world, port, n, T, str(tmp_path)), nprocs=world, join=True)
    x = torch.empty(n, dtype=torch.float64, device="cuda:0")
    y = torch.empty(n, dtype=torch.float64, device="cuda:0")
    pl.fill_f64(x, n, 42, 0, 0)
    pl.fill_f64(y, n, 43, 0, 0)
    ctl = pl.make_ctl(T=T, units=[0])
    want_dot, _ = pl.ddot(n, x, 1, y, 1, 0.0, locx=0, locy=0, ctl=ctl)
    pl.daxpy(n, -0.5, x, 1, y, 1, locx=0, locy=0, ctl=ctl)
    want_y = y.cpu().numpy()
    for r in range(world):
        dot, lo, hi = np.load(tmp_path / f"l1_{r}.npy")
        assert float(dot) == want_dot                      # every rank holds the same, exact bits
        assert np.array_equal(np.load(tmp_path / f"y_{r}.npy"), want_y[int(lo):int(hi)])
