"""One process per GPU (PARALiA_group_*): the ranks of a group share host-resident tiles
over NVLink through CUDA IPC. Spawns one process per GPU; needs at least two GPUs."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
EPS64 = 2.0 ** -52


def _ngpu():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _worker(rank, world, name, M, N, K, T, ta, share, steps, out_dir):
    sys.path.insert(0, str(ROOT))
    import importlib
    import __graft_entry__ as entry
    pl = entry.load_package()
    ranks = importlib.import_module("paralia_framework_b200.ranks")
    orc = entry.load_oracle()
    pl.group_init(name, rank, world, rank)
    (m0, m1), (n0, n1), _, _ = ranks.gemm_block(rank, world, M, N, quantum=T)
    Mloc, Nloc = m1 - m0, n1 - n0
    if ta == "N":
        A = orc.matrix_f64(M, K, 42)
        Ap = np.asfortranarray(A[m0:m1, :]); lda = Mloc
    else:
        A = orc.matrix_f64(K, M, 42)
        Ap = np.asfortranarray(A[:, m0:m1]); lda = K
    B = orc.matrix_f64(K, N, 43)
    Bp = np.asfortranarray(B[:, n0:n1])
    C = orc.matrix_f64(M, N, 44)
    flags = 0 if share else pl.FLAG_NO_PEER_FETCH
    tot = {"h2d": 0, "p2p": 0, "d2h": 0}
    for _ in range(steps):
        Cb = np.asfortranarray(C[m0:m1, n0:n1])
        rep = pl.group_dgemm(ta, "N", Mloc, Nloc, K, 1.23, Ap, lda, Bp, K, 0.9876, Cb, Mloc,
                             ctl=pl.make_ctl(T=T, flags=flags))
        tot["h2d"] += rep.h2d_bytes; tot["p2p"] += rep.p2p_bytes; tot["d2h"] += rep.d2h_bytes
    np.save(os.path.join(out_dir, f"C_{rank}.npy"), Cb)
    np.save(os.path.join(out_dir, f"bytes_{rank}.npy"),
            np.array([tot["h2d"], tot["p2p"], tot["d2h"], m0, m1, n0, n1]))
    pl.group_finalize()


def _run(world, M, N, K, T, ta, share, steps, tmp_path, orc):
    import torch.multiprocessing as mp
    name = f"t{os.getpid()}_{world}_{int(share)}_{ta}_{M}"
    mp.spawn(_worker, args=(world, name, M, N, K, T, ta, share, steps, str(tmp_path)),
             nprocs=world, join=True)
    A = orc.matrix_f64(M, K, 42) if ta == "N" else orc.matrix_f64(K, M, 42)
    B = orc.matrix_f64(K, N, 43)
    want = orc.matrix_f64(M, N, 44)
    orc.dgemm_tiled(ta, "N", M, N, K, 1.23, A, A.shape[0], B, K, 0.9876, want, M, T)
    got = np.zeros_like(want)
    h2d = p2p = d2h = 0
    for r in range(world):
        b = np.load(tmp_path / f"bytes_{r}.npy")
        m0, m1, n0, n1 = (int(v) for v in b[3:7])
        got[m0:m1, n0:n1] = np.load(tmp_path / f"C_{r}.npy")
        h2d += int(b[0]); p2p += int(b[1]); d2h += int(b[2])
    assert orc.normwise_rel_err(got, want) <= 8 * K * EPS64
    return h2d // steps, p2p // steps, d2h // steps


@pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("ta", ["N", "T"])
def test_group_two_ranks_share_b_tiles(orc, tmp_path, ta):
    M, N, K, T = 1024, 768, 512, 256
    h2d, p2p, d2h = _run(2, M, N, K, T, ta, True, 2, tmp_path, orc)
    szA, szB, szC = M * K * 8, K * N * 8, M * N * 8
    # grid 2 x 1: both ranks read all of B -> each B tile crosses the host link once and
    # NVLink once; A and C are private to a rank
    assert h2d == szA + szB + szC
    assert p2p == szB
    assert d2h == szC


@pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
def test_group_two_ranks_without_sharing(orc, tmp_path):
    M, N, K, T = 1024, 768, 512, 256
    h2d, p2p, d2h = _run(2, M, N, K, T, "N", False, 1, tmp_path, orc)
    szA, szB, szC = M * K * 8, K * N * 8, M * N * 8
    assert h2d == szA + 2 * szB + szC and p2p == 0


@pytest.mark.skipif(_ngpu() < 4, reason="needs four GPUs")
def test_group_four_ranks_share_a_and_b(orc, tmp_path):
    M, N, K, T = 1024, 1024, 768, 256
    h2d, p2p, d2h = _run(4, M, N, K, T, "N", True, 2, tmp_path, orc)
    szA, szB, szC = M * K * 8, K * N * 8, M * N * 8
    assert h2d == szA + szB + szC
    assert p2p == szA + szB


def _sgemm_worker(rank, world, name, M, N, K, T, out_dir):
    sys.path.insert(0, str(ROOT))
    import importlib
    import __graft_entry__ as entry
    pl = entry.load_package()
    ranks = importlib.import_module("paralia_framework_b200.ranks")
    orc = entry.load_oracle()
    pl.group_init(name, rank, world, rank)
    (m0, m1), (n0, n1), _, _ = ranks.gemm_block(rank, world, M, N, quantum=T)
    A = orc.uniform_f32(M * K, 42).reshape((M, K), order="F")
    B = orc.uniform_f32(K * N, 43).reshape((K, N), order="F")
    C = orc.uniform_f32(M * N, 44).reshape((M, N), order="F")
    Ap, Bp = np.asfortranarray(A[m0:m1, :]), np.asfortranarray(B[:, n0:n1])
    Cb = np.asfortranarray(C[m0:m1, n0:n1])
    rep = pl.group_sgemm("N", "N", m1 - m0, n1 - n0, K, 1.25, Ap, m1 - m0, Bp, K, 0.75, Cb, m1 - m0,
                         ctl=pl.make_ctl(T=T))
    np.save(os.path.join(out_dir, f"S_{rank}.npy"), Cb)
    np.save(os.path.join(out_dir, f"sb_{rank}.npy"), np.array([rep.h2d_bytes, rep.p2p_bytes, m0, m1, n0, n1]))
    pl.group_finalize()


@pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
def test_group_sgemm_two_ranks(orc, tmp_path):
    import torch.multiprocessing as mp
    M, N, K, T = 1024, 768, 512, 256
    mp.spawn(_sgemm_worker, args=(2, f"s{os.getpid()}", M, N, K, T, str(tmp_path)), nprocs=2, join=True)
    A = orc.uniform_f32(M * K, 42).reshape((M, K), order="F")
    B = orc.uniform_f32(K * N, 43).reshape((K, N), order="F")
    C = orc.uniform_f32(M * N, 44).reshape((M, N), order="F")
    want = 1.25 * (A.astype(np.float64) @ B.astype(np.float64)) + 0.75 * C.astype(np.float64)
    got = np.zeros((M, N))
    h2d = p2p = 0
    for r in range(2):
        b = np.load(tmp_path / f"sb_{r}.npy")
        m0, m1, n0, n1 = (int(v) for v in b[2:6])
        got[m0:m1, n0:n1] = np.load(tmp_path / f"S_{r}.npy")
        h2d += int(b[0]); p2p += int(b[1])
    assert orc.normwise_rel_err(got, want) <= 4 * K * 2.0 ** -23
    assert h2d == (M * K + K * N + M * N) * 4     # every host tile crosses the host link once
    assert p2p > 0                                # B tiles reach the other rank packed, over NVLink
