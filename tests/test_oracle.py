"""The CPU oracle against the committed golden vectors (OpenBLAS results, the
reference's own distribution output) and against OpenBLAS run live. No GPU needed."""
import json

import numpy as np
import pytest

import sys, pathlib
sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent / "golden"))
from gen_golden import DGEMM_CASES, L1_CASES, SGEMM_CASES, stored_shape

EPS64 = 2.0 ** -52
EPS32 = 2.0 ** -23


@pytest.fixture(scope="module")
def blas_golden(golden_dir):
    return np.load(golden_dir / "blas_openblas.npz")


def test_rng_golden(orc, golden_dir):
    vec = json.loads((golden_dir / "rng_vectors.json").read_text())
    assert [float(v).hex() for v in orc.uniform_f64(8, 42)] == vec["uniform_f64_seed42"]
    assert [float(v).hex() for v in orc.uniform_f64(8, 43)] == vec["uniform_f64_seed43"]
    assert [float(v).hex() for v in orc.uniform_f32(8, 42)] == vec["uniform_f32_seed42"]
    np.testing.assert_allclose(orc.normal_f64(8, 44), vec["normal_f64_seed44"], rtol=1e-14)


def test_rng_distribution(orc):
    u = orc.uniform_f64(1 << 18, 7)
    assert u.min() >= -1.0 and u.max() < 1.0
    assert abs(u.mean()) < 5e-3 and abs(u.var() - 1.0 / 3.0) < 5e-3
    n = orc.normal_f64(1 << 18, 7)
    assert abs(n.mean()) < 1e-2 and abs(n.std() - 1.0) < 1e-2


@pytest.mark.parametrize("idx", range(len(DGEMM_CASES)))
@pytest.mark.parametrize("T", [16, 24, 1000])
def test_dgemm_oracle_vs_openblas_golden(orc, blas_golden, idx, T):
    ta, tb, M, N, K, alpha, beta, pad = DGEMM_CASES[idx]
    ar, ac = stored_shape(ta, M, K)
    br, bc = stored_shape(tb, K, N)
    A = orc.matrix_f64(ar, ac, 42, ar + pad)
    B = orc.matrix_f64(br, bc, 43, br + pad)
    Cm = orc.matrix_f64(M, N, 44, M + pad)
    before = Cm.copy(order="F")
    orc.dgemm_tiled(ta, tb, M, N, K, alpha, A, ar + pad, B, br + pad, beta, Cm, M + pad, T)
    want = blas_golden[f"dgemm_{idx}"]
    assert orc.normwise_rel_err(Cm[:M, :], want) <= 8 * K * EPS64
    # rows of the buffer below the matrix (leading-dimension padding) are untouched
    assert np.array_equal(Cm[M:, :], before[M:, :])


@pytest.mark.parametrize("idx", range(len(SGEMM_CASES)))
def test_sgemm_oracle_vs_openblas_golden(orc, blas_golden, idx):
    ta, tb, M, N, K, alpha, beta, pad = SGEMM_CASES[idx]
    ar, ac = stored_shape(ta, M, K)
    br, bc = stored_shape(tb, K, N)
    A = orc.uniform_f32((ar + pad) * ac, 42).reshape((ar + pad, ac), order="F")
    B = orc.uniform_f32((br + pad) * bc, 43).reshape((br + pad, bc), order="F")
    Cm = orc.uniform_f32((M + pad) * N, 44).reshape((M + pad, N), order="F")
    orc.sgemm_tiled(ta, tb, M, N, K, alpha, A, ar + pad, B, br + pad, beta, Cm, M + pad, 16)
    assert orc.normwise_rel_err(Cm[:M, :], blas_golden[f"sgemm_{idx}"]) <= 4 * K * EPS32


@pytest.mark.parametrize("idx", range(len(L1_CASES)))
def test_level1_oracle_vs_openblas_golden(orc, blas_golden, idx):
    n, incx, incy, alpha = L1_CASES[idx]
    x = orc.uniform_f64(1 + (n - 1) * incx, 42)
    y = orc.uniform_f64(1 + (n - 1) * incy, 43)
    dot, mag = orc.ddot_tiled(n, x, incx, y, incy, 256, 0.0)
    assert abs(dot - blas_golden[f"ddot_{idx}"][0]) <= n * EPS64 * mag
    # *result is accumulated into, not overwritten (ddot.cpp:431)
    dot2, _ = orc.ddot_tiled(n, x, incx, y, incy, 256, 10.0)
    assert abs(dot2 - 10.0 - dot) <= 16 * EPS64 * (10.0 + abs(dot))
    yy = y.copy()
    orc.daxpy_tiled(n, alpha, x, incx, yy, incy, 300)
    np.testing.assert_allclose(yy[::incy], blas_golden[f"daxpy_{idx}"], rtol=0, atol=2 * EPS64 * 4)
    if incy > 1:  # elements between the strides are untouched
        mask = np.ones(len(y), bool)
        mask[::incy] = False
        assert np.array_equal(yy[mask], y[mask])


def test_dgemm_oracle_vs_openblas_live(orc):
    M, N, K = 289, 353, 307   # the reference's odd-size family (dgemm_tester.cpp:133-152)
    A = orc.matrix_f64(M, K, 42)
    B = orc.matrix_f64(K, N, 43)
    Cm = orc.matrix_f64(M, N, 44)
    want = orc.openblas_dgemm("N", "N", 1.23, A, B, 0.9876, Cm)
    orc.dgemm_tiled("N", "N", M, N, K, 1.23, A, M, B, K, 0.9876, Cm, M, 128)
    assert orc.normwise_rel_err(Cm, want) <= 8 * K * EPS64


def test_distribution_oracle_vs_reference_golden(orc, golden_dir):
    cases = json.loads((golden_dir / "distribution_ref.json").read_text())["cases"]
    assert len(cases) > 100
    for c in cases:
        active, owner, d1, d2 = orc.distribute_2d(c["units"], c["Mt"], c["Nt"], c["Kt"])
        assert active == c["active"], c
        assert owner == c["owner"], (c["units"], c["Mt"], c["Nt"], c["Kt"])
        assert d1 * d2 == c["units"]


def test_device_grid_rule(orc):
    # most-square factorisation found by the reference's scan
    # (Subkernel_distributions.cpp:325-336): not monotone in orientation
    want = {1: (1, 1), 2: (2, 1), 3: (1, 3), 4: (2, 2), 6: (3, 2), 8: (2, 4)}
    for u, g in want.items():
        _, _, d1, d2 = orc.distribute_2d(u, 8, 8, 1)
        assert (d1, d2) == g


def test_tile_score_worked_example(orc):
    # N = 32768 on 8 units: T = 4096 scores 2/64, T = 2048 scores 2/512 and wins
    assert orc.tile_slowdowns(32768, 32768, 32768, 4096, 8)[0] == pytest.approx(2 / 64)
    assert orc.tile_slowdowns(32768, 32768, 32768, 2048, 8)[0] == pytest.approx(2 / 512)
    T, sl = orc.optimize_tile(32768, 32768, 32768, 8)
    assert T == 2048 and sl[0] == pytest.approx(2 / 512)


@pytest.mark.parametrize("ta", ["N", "T"])
@pytest.mark.parametrize("dims", [(64, 48), (37, 53), (1, 70), (70, 1), (300, 200)])
def test_dgemv_oracle_vs_openblas_live(orc, ta, dims):
    M, N = dims
    A = orc.matrix_f64(M, N, 42, M + 3)
    in_len, out_len = (M, N) if ta == "T" else (N, M)
    x = orc.uniform_f64(in_len, 43)
    y = orc.uniform_f64(out_len, 44)
    want = orc.openblas_dgemv(ta, 1.23, A[:M, :], x, 0.9876, y)
    orc.dgemv(ta, M, N, 1.23, A, M + 3, x, 1, 0.9876, y, 1)
    assert orc.normwise_rel_err(y, want) <= 8 * in_len * EPS64


def test_dgemv_oracle_vs_openblas_golden(orc, golden_dir):
    from gen_golden import DGEMV_CASES, dgemv_inputs
    gold = np.load(golden_dir / "blas_openblas_dgemv.npz")
    for i, case in enumerate(DGEMV_CASES):
        ta, M, N, alpha, beta, pad, incx, incy = case
        A, x, y = dgemv_inputs(case)
        before = y.copy()
        orc.dgemv(ta, M, N, alpha, A, M + pad, x, incx, beta, y, incy)
        in_len = M if ta == "T" else N
        assert orc.normwise_rel_err(y[::incy], gold[f"dgemv_{i}"]) <= 8 * in_len * EPS64, case
        if incy > 1:      # elements between the strides are untouched
            mask = np.ones(len(y), bool); mask[::incy] = False
            assert np.array_equal(y[mask], before[mask])
