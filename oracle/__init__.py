"""CPU oracle for the tiled BLAS hot path -- TEST INFRASTRUCTURE ONLY.

Two tiers, both on the host:

* ``liboracle.so`` (``paralia_oracle.c``): a plain-C restatement of the reference's
  per-call arithmetic and planning rules, each function citing the reference lines it
  follows.
* OpenBLAS (the ILP64 build bundled with numpy/scipy, reached through
  ``scipy.linalg.blas``): ``cblas_dgemm/sgemm/daxpy/ddot`` are the routines the reference
  itself runs on its CPU path and as validation comparator
  (``Benchmarking/CuCuBLAS/src/cuBLASXt/cuBLASXtWrappers.cpp:15-28``,
  ``Database_builder/CuCuBLAS/src/dgemm_microbench.cu:118,145``).

Parity is pinned relative to those OpenBLAS routines and to the reference's own
distribution code (``_ref/ref_distribute``); the reference has no absolute golden
vectors for this path, so absolute parity is unpinned.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this
package. The shipped library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

ORACLE_DIR = Path(__file__).resolve().parent
LIB_PATH = ORACLE_DIR / "liboracle.so"
REF_DISTRIBUTE = ORACLE_DIR / "_ref" / "ref_distribute"

_lib = None


def build() -> Path:
    """Compile liboracle.so (and the reference distribution driver when the reference
    checkout is present)."""
    subprocess.run(["make", "-C", str(ORACLE_DIR), "liboracle.so"], check=True,
                   capture_output=True)
    ref = os.environ.get("PARALIA_REFERENCE_DIR", "")
    if ref and (Path(ref) / "Autotuner/src/Subkernel_distributions.cpp").exists():
        subprocess.run(["make", "-C", str(ORACLE_DIR), "_ref", f"REF={ref}"], check=True,
                       capture_output=True)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        h = C.CDLL(str(LIB_PATH))
        i64, dbl, flt, vp = C.c_int64, C.c_double, C.c_float, C.c_void_p
        h.oracle_fill_uniform_f64.argtypes = [vp, i64, C.c_uint64]
        h.oracle_fill_uniform_f32.argtypes = [vp, i64, C.c_uint64]
        h.oracle_fill_normal_f64.argtypes = [vp, i64, C.c_uint64]
        h.oracle_dgemm_tiled.argtypes = [C.c_int, C.c_int, i64, i64, i64, dbl, vp, i64, vp, i64,
                                         dbl, vp, i64, i64]
        h.oracle_sgemm_tiled.argtypes = [C.c_int, C.c_int, i64, i64, i64, flt, vp, i64, vp, i64,
                                         flt, vp, i64, i64]
        h.oracle_daxpy_tiled.argtypes = [i64, dbl, vp, i64, vp, i64, i64]
        h.oracle_ddot_tiled.argtypes = [i64, vp, i64, vp, i64, i64, C.POINTER(dbl), C.POINTER(dbl)]
        h.oracle_dgemv.argtypes = [C.c_int, i64, i64, dbl, vp, i64, vp, i64, dbl, vp, i64]
        h.oracle_tile_slowdowns.argtypes = [i64, i64, i64, i64, C.c_int, C.POINTER(dbl)]
        h.oracle_optimize_tile.argtypes = [i64, i64, i64, C.c_int, i64, C.POINTER(dbl)]
        h.oracle_optimize_tile.restype = i64
        h.oracle_distribute_2d.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int,
                                           C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                           C.POINTER(C.c_int32)]
        _lib = h
    return _lib


# ---------------------------------------------------------------- inputs
def uniform_f64(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float64)
    lib().oracle_fill_uniform_f64(out.ctypes.data, n, seed)
    return out


def uniform_f32(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().oracle_fill_uniform_f32(out.ctypes.data, n, seed)
    return out


def normal_f64(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float64)
    lib().oracle_fill_normal_f64(out.ctypes.data, n, seed)
    return out


def matrix_f64(rows: int, cols: int, seed: int, ld: int | None = None) -> np.ndarray:
    """Column-major rows x cols matrix inside an ld x cols buffer (Fortran order)."""
    ld = rows if ld is None else ld
    buf = uniform_f64(ld * cols, seed).reshape((ld, cols), order="F")
    return buf


# ---------------------------------------------------------------- C restatement
def _t(ch: str) -> int:
    return 1 if ch.upper() in ("T", "C") else 0


def dgemm_tiled(ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, Cm, ldc, T) -> None:
    """In place on Cm (Fortran-ordered float64 buffers)."""
    rc = lib().oracle_dgemm_tiled(_t(ta), _t(tb), M, N, K, alpha, A.ctypes.data, lda,
                                  B.ctypes.data, ldb, beta, Cm.ctypes.data, ldc, T)
    assert rc == 0


def sgemm_tiled(ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, Cm, ldc, T) -> None:
    rc = lib().oracle_sgemm_tiled(_t(ta), _t(tb), M, N, K, alpha, A.ctypes.data, lda,
                                  B.ctypes.data, ldb, beta, Cm.ctypes.data, ldc, T)
    assert rc == 0


def daxpy_tiled(N, alpha, x, incx, y, incy, T) -> None:
    rc = lib().oracle_daxpy_tiled(N, alpha, x.ctypes.data, incx, y.ctypes.data, incy, T)
    assert rc == 0


def ddot_tiled(N, x, incx, y, incy, T, result: float = 0.0):
    """Returns (result + x.y, sum |x_i y_i|)."""
    res, mag = C.c_double(result), C.c_double(0.0)
    rc = lib().oracle_ddot_tiled(N, x.ctypes.data, incx, y.ctypes.data, incy, T, C.byref(res),
                                 C.byref(mag))
    assert rc == 0
    return res.value, mag.value


def dgemv(ta, M, N, alpha, A, lda, x, incx, beta, y, incy) -> None:
    """In place on y."""
    rc = lib().oracle_dgemv(_t(ta), M, N, alpha, A.ctypes.data, lda, x.ctypes.data, incx, beta,
                            y.ctypes.data, incy)
    assert rc == 0


def tile_slowdowns(D1, D2, D3, T, units) -> list[float]:
    sl = (C.c_double * 6)()
    lib().oracle_tile_slowdowns(D1, D2, D3, T, units, sl)
    return list(sl)


def optimize_tile(D1, D2, D3, units, step=1):
    sl = (C.c_double * 6)()
    T = lib().oracle_optimize_tile(D1, D2, D3, units, step, sl)
    return int(T), list(sl)


def distribute_2d(units, Mt, Nt, Kt):
    owner = (C.c_int32 * (Mt * Nt * Kt))()
    d1, d2 = C.c_int32(), C.c_int32()
    active = lib().oracle_distribute_2d(units, Mt, Nt, Kt, owner, C.byref(d1), C.byref(d2))
    return active, list(owner), d1.value, d2.value


def ref_distribute(units, Mt, Nt, Kt):
    """The reference's own distribution code (only where _ref was built)."""
    out = subprocess.run([str(REF_DISTRIBUTE), str(units), str(Mt), str(Nt), str(Kt)],
                         check=True, capture_output=True, text=True).stdout.split()
    vals = [int(v) for v in out]
    return vals[0], vals[1:]


# ---------------------------------------------------------------- OpenBLAS tier
def openblas_dgemm(ta, tb, alpha, A, B, beta, Cm) -> np.ndarray:
    """cblas_dgemm through scipy; A, B, Cm are Fortran-ordered views of the logical
    (untransposed-storage) matrices. Returns a new array."""
    from scipy.linalg import blas
    return blas.dgemm(alpha, A, B, beta=beta, c=Cm, trans_a=_t(ta), trans_b=_t(tb),
                      overwrite_c=False)


def openblas_sgemm(ta, tb, alpha, A, B, beta, Cm) -> np.ndarray:
    from scipy.linalg import blas
    return blas.sgemm(alpha, A, B, beta=beta, c=Cm, trans_a=_t(ta), trans_b=_t(tb),
                      overwrite_c=False)


def openblas_dgemv(ta, alpha, A, x, beta, y) -> np.ndarray:
    from scipy.linalg import blas
    return blas.dgemv(alpha, A, x, beta=beta, y=y.copy(), trans=_t(ta))


def openblas_daxpy(alpha, x, y) -> np.ndarray:
    from scipy.linalg import blas
    return blas.daxpy(x, y.copy(), a=alpha)


def openblas_ddot(x, y) -> float:
    from scipy.linalg import blas
    return float(blas.ddot(x, y))


def normwise_rel_err(got: np.ndarray, want: np.ndarray) -> float:
    """||got - want||_F / ||want||_F"""
    d = np.linalg.norm((got.astype(np.float64) - want.astype(np.float64)).ravel())
    n = np.linalg.norm(want.astype(np.float64).ravel())
    return float(d / n) if n > 0 else float(d)
