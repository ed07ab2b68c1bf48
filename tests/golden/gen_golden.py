"""Generates the committed golden fixtures of this directory. Run from the repo root in
the build container (needs the reference checkout for the distribution fixture):

    python tests/golden/gen_golden.py

* ``distribution_ref.json`` -- output of the REFERENCE's own subkernel distribution
  (Autotuner/src/Subkernel_distributions.cpp, compiled by ``make -C oracle _ref``) for a
  list of (units, Mt, Nt, Kt) cases: the owner unit of every subkernel id.
* ``blas_openblas.npz`` -- results of OpenBLAS cblas_dgemm / sgemm / daxpy / ddot (the
  routines the reference uses on its CPU path) on seeded inputs produced by the oracle's
  counter-based generator; inputs are regenerated from the seeds by the tests.
* ``blas_openblas_dgemv.npz`` -- the same for OpenBLAS cblas_dgemv (kept in a file of its own
  so that adding it did not rewrite the older fixtures).
* ``rng_vectors.json`` -- first values of the input generator for fixed seeds.
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402

OUT = Path(__file__).resolve().parent

DIST_CASES = [(u, m, n, k)
              for u in (1, 2, 3, 4, 5, 6, 7, 8)
              for (m, n, k) in ((1, 1, 1), (2, 2, 1), (4, 4, 2), (8, 8, 2), (5, 7, 3), (3, 2, 2),
                                (7, 1, 1), (1, 5, 1), (2, 9, 2), (16, 16, 1), (9, 4, 2),
                                (6, 6, 6), (16, 16, 4), (3, 3, 3))]

# (ta, tb, M, N, K, alpha, beta, extra leading-dimension padding)
DGEMM_CASES = [
    ("N", "N", 64, 48, 40, 1.25, 0.75, 0),
    ("N", "N", 37, 53, 29, 1.23, 0.9876, 3),
    ("T", "N", 48, 32, 56, 1.0, 0.0, 0),
    ("N", "T", 33, 65, 17, -0.5, 1.0, 5),
    ("T", "T", 41, 39, 43, 1.23, 0.9876, 1),
    ("N", "N", 1, 70, 9, 2.0, -1.0, 0),
    ("N", "N", 70, 1, 9, 2.0, -1.0, 0),
]
SGEMM_CASES = [
    ("N", "N", 64, 48, 40, 1.0, 0.0, 0),
    ("T", "N", 37, 53, 29, 1.25, 0.75, 3),
    ("N", "T", 33, 65, 17, -0.5, 1.0, 0),
]
# (ta, M, N, alpha, beta, extra leading-dimension padding, incx, incy)
DGEMV_CASES = [
    ("N", 64, 48, 1.25, 0.75, 0, 1, 1),
    ("T", 64, 48, 1.25, 0.75, 0, 1, 1),
    ("N", 37, 53, 1.23, 0.9876, 3, 2, 3),
    ("T", 37, 53, -0.5, 0.0, 3, 3, 2),
    ("N", 1, 70, 2.0, -1.0, 0, 1, 1),
    ("T", 70, 1, 2.0, -1.0, 1, 1, 1),
    ("N", 513, 257, 1.0, 1.0, 1, 1, 1),
]
L1_CASES = [(1000, 1, 1, -0.5), (777, 2, 3, 1.5), (4096, 1, 1, 0.25), (1, 1, 1, 3.0)]


def stored_shape(t, rows, cols):
    return (cols, rows) if t == "T" else (rows, cols)


def gen_distribution():
    cases = []
    for (u, m, n, k) in DIST_CASES:
        try:
            active, owner = oracle.ref_distribute(u, m, n, k)
            cases.append({"units": u, "Mt": m, "Nt": n, "Kt": k, "active": active, "owner": owner})
        except Exception:
            cases.append({"units": u, "Mt": m, "Nt": n, "Kt": k, "active": -1, "owner": []})
    (OUT / "distribution_ref.json").write_text(json.dumps({"cases": cases}))
    print("distribution cases:", len(cases), "aborted:", sum(c["active"] < 0 for c in cases))


def gen_blas():
    out = {}
    for i, (ta, tb, M, N, K, alpha, beta, pad) in enumerate(DGEMM_CASES):
        ar, ac = stored_shape(ta, M, K)
        br, bc = stored_shape(tb, K, N)
        A = oracle.matrix_f64(ar, ac, 42, ar + pad)
        B = oracle.matrix_f64(br, bc, 43, br + pad)
        Cm = oracle.matrix_f64(M, N, 44, M + pad)
        res = oracle.openblas_dgemm(ta, tb, alpha, A[:ar, :], B[:br, :], beta, Cm[:M, :])
        out[f"dgemm_{i}"] = np.asfortranarray(res)
    for i, (ta, tb, M, N, K, alpha, beta, pad) in enumerate(SGEMM_CASES):
        ar, ac = stored_shape(ta, M, K)
        br, bc = stored_shape(tb, K, N)
        A = oracle.uniform_f32((ar + pad) * ac, 42).reshape((ar + pad, ac), order="F")
        B = oracle.uniform_f32((br + pad) * bc, 43).reshape((br + pad, bc), order="F")
        Cm = oracle.uniform_f32((M + pad) * N, 44).reshape((M + pad, N), order="F")
        res = oracle.openblas_sgemm(ta, tb, alpha, A[:ar, :], B[:br, :], beta, Cm[:M, :])
        out[f"sgemm_{i}"] = np.asfortranarray(res)
    for i, (n, incx, incy, alpha) in enumerate(L1_CASES):
        x = oracle.uniform_f64(1 + (n - 1) * incx, 42)
        y = oracle.uniform_f64(1 + (n - 1) * incy, 43)
        out[f"daxpy_{i}"] = oracle.openblas_daxpy(alpha, x[::incx], y[::incy])
        out[f"ddot_{i}"] = np.array([oracle.openblas_ddot(x[::incx], y[::incy])])
    np.savez_compressed(OUT / "blas_openblas.npz", **out)
    print("blas fixtures:", len(out))


def dgemv_inputs(case):
    ta, M, N, alpha, beta, pad, incx, incy = case
    in_len, out_len = (M, N) if ta == "T" else (N, M)
    A = oracle.matrix_f64(M, N, 42, M + pad)
    x = oracle.uniform_f64(1 + (in_len - 1) * incx, 43)
    y = oracle.uniform_f64(1 + (out_len - 1) * incy, 44)
    return A, x, y


def gen_dgemv():
    out = {}
    for i, case in enumerate(DGEMV_CASES):
        ta, M, N, alpha, beta, pad, incx, incy = case
        A, x, y = dgemv_inputs(case)
        out[f"dgemv_{i}"] = oracle.openblas_dgemv(ta, alpha, A[:M, :], x[::incx].copy(), beta,
                                                  y[::incy].copy())
    np.savez_compressed(OUT / "blas_openblas_dgemv.npz", **out)
    print("dgemv fixtures:", len(out))


def gen_rng():
    vec = {
        "uniform_f64_seed42": [float(v).hex() for v in oracle.uniform_f64(8, 42)],
        "uniform_f64_seed43": [float(v).hex() for v in oracle.uniform_f64(8, 43)],
        "uniform_f32_seed42": [float(v).hex() for v in oracle.uniform_f32(8, 42)],
        "normal_f64_seed44": [float(v) for v in oracle.normal_f64(8, 44)],
    }
    (OUT / "rng_vectors.json").write_text(json.dumps(vec, indent=1))


if __name__ == "__main__":
    gen_distribution()
    gen_blas()
    gen_dgemv()
    gen_rng()
