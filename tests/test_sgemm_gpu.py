"""Parity of the CUDA SGEMM path (3xTF32 on tcgen05) through the C ABI.

The oracle is the FP64 product of the same FP32 inputs (so the bound is measured against
a result more accurate than any FP32 GEMM); tolerance stated by the task: normwise
relative error <= 4*K*eps32. OpenBLAS sgemm results are checked as golden vectors too."""
import sys, pathlib
import numpy as np
import pytest

sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent / "golden"))
from gen_golden import SGEMM_CASES, stored_shape  # noqa: E402

pytestmark = pytest.mark.gpu
EPS32 = 2.0 ** -23


def tol(K):
    return 4 * max(K, 1) * EPS32


def _inputs(orc, ta, tb, M, N, K, pad=0, normal=False):
    ar, ac = stored_shape(ta, M, K)
    br, bc = stored_shape(tb, K, N)
    gen = (lambda n, s: orc.normal_f64(n, s).astype(np.float32)) if normal else orc.uniform_f32
    A = gen((ar + pad) * ac, 42).reshape((ar + pad, ac), order="F")
    B = gen((br + pad) * bc, 43).reshape((br + pad, bc), order="F")
    C = gen((M + pad) * N, 44).reshape((M + pad, N), order="F")
    return A, B, C, ar, br


def _want(ta, tb, M, N, K, alpha, beta, A, B, C, ar, br):
    a = A[:ar, :].astype(np.float64)
    b = B[:br, :].astype(np.float64)
    opa = a.T if ta == "T" else a
    opb = b.T if tb == "T" else b
    return alpha * (opa @ opb) + beta * C[:M, :].astype(np.float64)


def _dev(t, dev=0):
    import torch
    return torch.from_numpy(np.ascontiguousarray(t.T)).to(f"cuda:{dev}")


@pytest.mark.parametrize("ta,tb", [("N", "N"), ("T", "N"), ("N", "T"), ("T", "T")])
@pytest.mark.parametrize("dims", [(128, 256, 16), (256, 512, 256), (100, 36, 50), (289, 353, 307),
                                  (1, 1, 1), (130, 2, 3), (1024, 1024, 1024)])
def test_tile_sgemm_vs_fp64(pl, orc, ta, tb, dims):
    import torch
    M, N, K = dims
    A, B, C, ar, br = _inputs(orc, ta, tb, M, N, K)
    want = _want(ta, tb, M, N, K, 1.25, 0.75, A, B, C, ar, br)
    dA, dB, dC = _dev(A), _dev(B), _dev(C)
    pl.tile_sgemm(0, ta, tb, M, N, K, 1.25, dA, ar, dB, br, 0.75, dC, M)
    torch.cuda.synchronize()
    got = dC.cpu().numpy().T
    err = orc.normwise_rel_err(got, want)
    assert err <= tol(K)
    # the split keeps FP32-level accuracy: far inside the allowed budget
    assert err <= 64 * EPS32 * max(1.0, K ** 0.5) / 8


@pytest.mark.parametrize("idx", range(len(SGEMM_CASES)))
def test_sgemm_host_vs_openblas_golden(pl, orc, golden_dir, idx):
    gold = np.load(golden_dir / "blas_openblas.npz")
    ta, tb, M, N, K, alpha, beta, pad = SGEMM_CASES[idx]
    A, B, C, ar, br = _inputs(orc, ta, tb, M, N, K, pad)
    before = C.copy(order="F")
    rep = pl.sgemm(ta, tb, M, N, K, alpha, A, ar + pad, B, br + pad, beta, C, M + pad,
                   ctl=pl.make_ctl(T=16, units=[0]))
    assert orc.normwise_rel_err(C[:M, :], gold[f"sgemm_{idx}"]) <= tol(K)
    assert np.array_equal(C[M:, :], before[M:, :])
    assert rep.kernel_launches > 0 and rep.d2h_bytes == M * N * 4


@pytest.mark.parametrize("ta,tb", [("N", "N"), ("T", "N"), ("N", "T"), ("T", "T")])
@pytest.mark.parametrize("dims,T", [((512, 512, 512), 256), ((289, 353, 307), 128),
                                    ((1024, 256, 768), 256), ((1156, 1412, 1228), 512)])
def test_sgemm_host_resident_vs_fp64(pl, orc, ta, tb, dims, T):
    M, N, K = dims
    A, B, C, ar, br = _inputs(orc, ta, tb, M, N, K, normal=True)
    want = _want(ta, tb, M, N, K, 1.23, 0.9876, A, B, C, ar, br)
    rep = pl.sgemm(ta, tb, M, N, K, 1.23, A, ar, B, br, 0.9876, C, M,
                   ctl=pl.make_ctl(T=T, units=[0]))
    assert orc.normwise_rel_err(C, want) <= tol(K)
    assert rep.h2d_bytes == (M * K + K * N + M * N) * 4
    assert rep.d2h_bytes == M * N * 4


def test_sgemm_device_resident_and_deterministic(pl, orc):
    import torch
    M, N, K, T = 768, 640, 1024, 256
    A, B, C, ar, br = _inputs(orc, "N", "N", M, N, K, normal=True)
    want = _want("N", "N", M, N, K, 1.0, 0.0, A, B, C, ar, br)
    outs = []
    for _ in range(2):
        dA, dB, dC = _dev(A), _dev(B), _dev(C)
        rep = pl.sgemm("N", "N", M, N, K, 1.0, dA, ar, dB, br, 0.0, dC, M,
                       ctl=pl.make_ctl(T=T, units=[0]))
        torch.cuda.synchronize()
        outs.append(dC.cpu().numpy().T.copy())
        assert rep.h2d_bytes == 0 and rep.d2h_bytes == 0
    assert orc.normwise_rel_err(outs[0], want) <= tol(K)
    assert np.array_equal(outs[0], outs[1])
    # host-resident run of the same problem and T: identical bits for A/B placement
    Ch = np.asfortranarray(C.copy())
    dC = _dev(C)
    pl.sgemm("N", "N", M, N, K, 1.0, A, ar, B, br, 0.0, Ch, M, ctl=pl.make_ctl(T=T, units=[0]))
    Cd = np.asfortranarray(C.copy())
    pl.sgemm("N", "N", M, N, K, 1.0, _dev(A), ar, _dev(B), br, 0.0, Cd, M,
             ctl=pl.make_ctl(T=T, units=[0]))
    assert np.array_equal(Ch, Cd)


def test_sgemm_large_k_accuracy(pl, orc):
    # K as deep as one tile column of BASELINE config 4, normal(0,1) entries
    import torch
    M, N, K = 256, 256, 40960
    A, B, C, ar, br = _inputs(orc, "N", "N", M, N, K, normal=True)
    want = _want("N", "N", M, N, K, 1.0, 0.0, A, B, C, ar, br)
    rep = pl.sgemm("N", "N", M, N, K, 1.0, A, ar, B, br, 0.0, C, M, ctl=pl.make_ctl(T=4096, units=[0]))
    err = orc.normwise_rel_err(C, want)
    assert err <= tol(K)
    # the tensor core accumulates FP32 without round-to-nearest, so the error grows roughly
    # like K*2^-24 rather than sqrt(K)*2^-24: about 1e-4 here, 200x inside the budget
    assert err <= 5e-4


def test_sgemm_k_zero(pl, orc):
    M, N = 64, 48
    C = orc.uniform_f32(M * N, 44).reshape((M, N), order="F")
    want = C * np.float32(0.5)
    A = np.zeros((M, 1), dtype=np.float32, order="F")
    B = np.zeros((1, N), dtype=np.float32, order="F")
    pl.sgemm("N", "N", M, N, 0, 1.0, A, M, B, 1, 0.5, C, M, ctl=pl.make_ctl(units=[0]))
    np.testing.assert_allclose(C, want, rtol=1e-6)


def test_sgemm_bounded_cache(pl, orc):
    M, N, K, T = 1024, 768, 1024, 256
    A, B, C, ar, br = _inputs(orc, "N", "T", M, N, K)
    want = _want("N", "T", M, N, K, 1.25, 0.75, A, B, C, ar, br)
    blk = 2 * 256 * 256 * 4          # packed FP32 tile (hi + lo planes)
    rep = pl.sgemm("N", "T", M, N, K, 1.25, A, ar, B, br, 0.75, C, M,
                   ctl=pl.make_ctl(T=T, units=[0], cache_limit=6 * blk))
    assert orc.normwise_rel_err(C, want) <= tol(K)
    assert rep.h2d_bytes > (M * K + K * N + M * N) * 4
