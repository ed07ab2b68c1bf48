"""The reference's own acceptance check, re-created: the library's GEMM against whole-problem
cuBLASXt on the same seeded inputs (Benchmarking/CuCuBLAS/src/PARALia/dgemm_runner.cpp:94-99
demands at least 9 agreeing digits; cuBLASXt configured as in
Benchmarking/CuCuBLAS/src/cuBLASXt/cuBLASXtWrappers.cpp:49-60).

Both results are also held against the CPU oracle. cuBLASXt is a vendor library used here
only as a second checker; the library under test never calls it."""
import pathlib
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "paralia-framework_b200"))
EPS64, EPS32 = 2.0 ** -52, 2.0 ** -23


def _xt():
    import comparators
    try:
        comparators.cublas().cublasXtDgemm
    except (OSError, AttributeError) as e:   # no cuBLAS in the image: nothing to compare with
        pytest.skip(f"cuBLASXt not available: {e}")
    return comparators


@pytest.mark.parametrize("ta,tb", [("N", "N"), ("T", "N"), ("N", "T")])
def test_dgemm_agrees_with_cublasxt(pl, orc, ta, tb):
    xt = _xt()
    M, N, K = 3000, 2504, 2048
    ar, ac = (K, M) if ta == "T" else (M, K)
    br, bc = (N, K) if tb == "T" else (K, N)
    A = orc.matrix_f64(ar, ac, 42, ar)
    B = orc.matrix_f64(br, bc, 43, br)
    C0 = orc.matrix_f64(M, N, 44, M)
    alpha, beta = 1.2345, 1.1154
    mine = C0.copy(order="F")
    pl.dgemm(ta, tb, M, N, K, alpha, A, ar, B, br, beta, mine, M, ctl=pl.make_ctl(T=1024, units=[0]))
    theirs = C0.copy(order="F")
    xt.cublasxt_gemm(8, ta, tb, M, N, K, alpha, A.ctypes.data, ar, B.ctypes.data, br, beta,
                     theirs.ctypes.data, M, T=1024, dev_ids=[0])
    # at least 9 agreeing digits, as the reference's runner requires
    assert orc.normwise_rel_err(mine, theirs) <= 1e-9
    # and within the stated bound of each other (both are within 8*K*eps of the exact result)
    assert orc.normwise_rel_err(mine, theirs) <= 2 * 8 * K * EPS64
    opA = A.T if ta == "T" else A
    opB = B.T if tb == "T" else B
    want = alpha * (opA @ opB) + beta * C0
    assert orc.normwise_rel_err(mine, want) <= 8 * K * EPS64
    assert orc.normwise_rel_err(theirs, want) <= 8 * K * EPS64


def test_sgemm_agrees_with_cublasxt(pl, orc):
    xt = _xt()
    M, N, K = 2048, 1536, 4096
    A = np.asfortranarray(orc.normal_f64(M * K, 42).astype(np.float32).reshape((M, K), order="F"))
    B = np.asfortranarray(orc.normal_f64(K * N, 43).astype(np.float32).reshape((K, N), order="F"))
    mine = np.zeros((M, N), dtype=np.float32, order="F")
    pl.sgemm("N", "N", M, N, K, 1.0, A, M, B, K, 0.0, mine, M, ctl=pl.make_ctl(T=1024, units=[0]))
    theirs = np.zeros((M, N), dtype=np.float32, order="F")
    xt.cublasxt_gemm(4, "N", "N", M, N, K, 1.0, A.ctypes.data, M, B.ctypes.data, K, 0.0,
                     theirs.ctypes.data, M, T=1024, dev_ids=[0])
    want = A.astype(np.float64) @ B.astype(np.float64)
    bound = 4 * K * EPS32
    assert orc.normwise_rel_err(mine, want) <= bound
    assert orc.normwise_rel_err(theirs, want) <= bound
    assert orc.normwise_rel_err(mine, theirs) <= 2 * bound
