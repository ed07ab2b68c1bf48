"""Python face of libparalia.so: a ctypes mirror of ``include/paralia_c.h``.

This module holds no arithmetic. Every call goes through the C ABI into the CUDA
library; if ``lib/libparalia.so`` is missing the import of the library fails loudly
(``LibraryMissing``) -- there is no fallback path of any kind.

Operands may be given as raw integer addresses, numpy arrays (host memory) or objects
with a ``data_ptr()`` method (torch tensors on the host or on a GPU).
Matrices are column-major as in BLAS and in the reference
(``Library_scheduler/include/PARALiA.hpp:33-72``).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "lib" / "libparalia.so"

MAX_UNITS = 16
LOC_HOST = -1
LOC_AUTO = -100

FLAG_NO_PEER_FETCH = 1
FLAG_KEEP_PINNED = 2
FLAG_NO_METADATA_REUSE = 4
FLAG_BETA_ZERO = 8          # autotune_gemm only: model the call with beta == 0

OK = 0
ERR_INVALID_ARG = 1
ERR_OUT_OF_MEMORY = 2
ERR_CUDA = 3
ERR_TIMEOUT = 4
ERR_NO_PEER_ACCESS = 5
ERR_DB_MISSING = 6
ERR_NO_DEVICE = 7
ERR_UNSUPPORTED = 8
ERR_GROUP_FAILED = 9


class LibraryMissing(RuntimeError):
    pass


class ParaliaError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"libparalia error {code}: {msg}")
        self.code = code


class Ctl(C.Structure):
    """``paralia_ctl``: caller-fixed control values (reference: the predefined ATC of
    ``PARALiADgemmControled``, dgemm.cpp:697-705)."""
    _fields_ = [
        ("T", C.c_int64),
        ("active_unit_num", C.c_int32),
        ("active_unit_id_list", C.c_int32 * MAX_UNITS),
        ("cache_limit", C.c_int64),
        ("exec_streams", C.c_int32),
        ("flags", C.c_int32),
    ]


class Report(C.Structure):
    """``paralia_report``: what a call chose and measured (reference: the returned ATC)."""
    _fields_ = [
        ("T", C.c_int64),
        ("active_unit_num", C.c_int32),
        ("active_unit_id_list", C.c_int32 * MAX_UNITS),
        ("active_unit_score", C.c_double * MAX_UNITS),
        ("cache_limit", C.c_int64),
        ("subkernel_num", C.c_int64),
        ("subkernels_per_unit", C.c_int32 * MAX_UNITS),
        ("pred_t", C.c_double),
        ("pred_J", C.c_double),
        ("T_slowdowns", C.c_double * 6),
        ("device_ms", C.c_double),
        ("host_ms", C.c_double),
        ("plan_ms", C.c_double),
        ("pin_ms", C.c_double),
        ("alloc_ms", C.c_double),
        ("h2d_bytes", C.c_int64),
        ("d2h_bytes", C.c_int64),
        ("p2p_bytes", C.c_int64),
        ("d2d_bytes", C.c_int64),
        ("kernel_launches", C.c_int64),
        ("metadata_reused", C.c_int32),
        ("grid_d1", C.c_int32),
        ("grid_d2", C.c_int32),
        ("fill_ms", C.c_double),
        ("exec_end_ms", C.c_double),
        ("h2d_end_ms", C.c_double),
    ]

    def as_dict(self) -> dict:
        n = max(self.active_unit_num, 0)
        return {
            "T": self.T, "active_unit_num": self.active_unit_num,
            "active_unit_id_list": list(self.active_unit_id_list[:n]),
            "subkernel_num": self.subkernel_num,
            "subkernels_per_unit": list(self.subkernels_per_unit[:n]),
            "pred_t": self.pred_t, "T_slowdowns": list(self.T_slowdowns),
            "device_ms": self.device_ms, "host_ms": self.host_ms, "plan_ms": self.plan_ms,
            "pin_ms": self.pin_ms, "alloc_ms": self.alloc_ms,
            "h2d_bytes": self.h2d_bytes, "d2h_bytes": self.d2h_bytes,
            "p2p_bytes": self.p2p_bytes, "d2d_bytes": self.d2d_bytes,
            "kernel_launches": self.kernel_launches, "grid": (self.grid_d1, self.grid_d2),
            "metadata_reused": self.metadata_reused,
            "fill_ms": self.fill_ms, "exec_end_ms": self.exec_end_ms, "h2d_end_ms": self.h2d_end_ms,
        }


_i64, _i32, _dbl, _flt, _vp, _chr = C.c_int64, C.c_int32, C.c_double, C.c_float, C.c_void_p, C.c_char
_ctl_p, _rep_p = C.POINTER(Ctl), C.POINTER(Report)

# name -> (restype, argtypes); the list of symbols include/paralia_c.h declares
SIGNATURES = {
    "PARALiA_init": (C.c_int, []),
    "PARALiA_finalize": (C.c_int, []),
    "PARALiA_device_count": (C.c_int, []),
    "PARALiA_last_error": (C.c_char_p, []),
    "PARALiA_dev_cache_free": (C.c_int, [C.c_int]),
    "PARALiA_dgemm": (C.c_int, [_chr, _chr, _i64, _i64, _i64, _dbl, _vp, _i64, C.c_int, _vp, _i64,
                                C.c_int, _dbl, _vp, _i64, C.c_int, _ctl_p, _rep_p]),
    "PARALiA_sgemm": (C.c_int, [_chr, _chr, _i64, _i64, _i64, _flt, _vp, _i64, C.c_int, _vp, _i64,
                                C.c_int, _flt, _vp, _i64, C.c_int, _ctl_p, _rep_p]),
    "PARALiA_dgemv": (C.c_int, [_chr, _i64, _i64, _dbl, _vp, _i64, C.c_int, _vp, _i64, C.c_int, _dbl,
                                _vp, _i64, C.c_int, _ctl_p, _rep_p]),
    "PARALiA_daxpy": (C.c_int, [_i64, _dbl, _vp, _i64, C.c_int, _vp, _i64, C.c_int, _ctl_p, _rep_p]),
    "PARALiA_ddot": (C.c_int, [_i64, _vp, _i64, C.c_int, _vp, _i64, C.c_int, C.POINTER(_dbl),
                               _ctl_p, _rep_p]),
    "PARALiA_ddot_tiles": (C.c_int, [_i64, _vp, _i64, C.c_int, _vp, _i64, C.c_int, C.POINTER(_dbl), _i64,
                                     C.POINTER(_i64), _ctl_p, _rep_p]),
    "PARALiA_group_init": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.c_int]),
    "PARALiA_group_finalize": (C.c_int, []),
    "PARALiA_group_dgemm": (C.c_int, [_chr, _chr, _i64, _i64, _i64, _dbl, _vp, _i64, C.c_int, _vp,
                                      _i64, C.c_int, _dbl, _vp, _i64, C.c_int, _ctl_p, _rep_p]),
    "PARALiA_group_sgemm": (C.c_int, [_chr, _chr, _i64, _i64, _i64, _flt, _vp, _i64, C.c_int, _vp,
                                      _i64, C.c_int, _flt, _vp, _i64, C.c_int, _ctl_p, _rep_p]),
    "PARALiA_selftest_bounded_wait": (C.c_int, [C.c_int, _dbl]),
    "PARALiA_tile_status": (C.c_int, [C.c_int]),
    "PARALiA_tile_dgemm": (C.c_int, [C.c_int, _vp, _chr, _chr, _i64, _i64, _i64, _dbl, _vp, _i64,
                                     _vp, _i64, _dbl, _vp, _i64]),
    "PARALiA_tile_sgemm": (C.c_int, [C.c_int, _vp, _chr, _chr, _i64, _i64, _i64, _flt, _vp, _i64,
                                     _vp, _i64, _flt, _vp, _i64]),
    "PARALiA_tile_daxpy": (C.c_int, [C.c_int, _vp, _i64, _dbl, _vp, _i64, _vp, _i64]),
    "PARALiA_tile_ddot_scratch_bytes": (_i64, [_i64]),
    "PARALiA_tile_ddot": (C.c_int, [C.c_int, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp]),
    "PARALiA_tile_dgemv_scratch_bytes": (_i64, [_chr, _i64, _i64]),
    "PARALiA_tile_dgemv": (C.c_int, [C.c_int, _vp, _chr, _i64, _i64, _dbl, _vp, _i64, _vp, _i64,
                                     _dbl, _vp, _i64, _vp]),
    "PARALiA_tile_ddot_noalloc_max_n": (_i64, []),
    "PARALiA_tile_ddot_noalloc": (C.c_int, [C.c_int, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "PARALiA_malloc": (C.c_int, [C.POINTER(_vp), _i64, C.c_int]),
    "PARALiA_free": (C.c_int, [_vp, C.c_int]),
    "PARALiA_memcpy": (C.c_int, [_vp, C.c_int, _vp, C.c_int, _i64]),
    "PARALiA_fill_f64": (C.c_int, [_vp, _i64, C.c_uint64, C.c_int, C.c_int]),
    "PARALiA_fill_f32": (C.c_int, [_vp, _i64, C.c_uint64, C.c_int, C.c_int]),
    "PARALiA_autotune_gemm": (C.c_int, [C.c_int, _chr, _chr, _i64, _i64, _i64, C.c_int, C.c_int,
                                        C.c_int, _ctl_p, _rep_p]),
    "PARALiA_tile_slowdowns": (C.c_int, [_i64, _i64, _i64, _i64, C.c_int, C.POINTER(_dbl)]),
    "PARALiA_distribute_2d": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(_i32),
                                        C.POINTER(_i32), C.POINTER(_i32)]),
    "PARALiA_plan_gemm": (C.c_int, [_i64, _i64, _i64, _i64, C.c_int, C.c_int, C.POINTER(_i32), _i64,
                                    C.POINTER(_i64), C.POINTER(_i32), C.POINTER(_i32)]),
    "PARALiA_load_database": (C.c_int, [C.c_char_p]),
    "PARALiA_bench_dmma_peak": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(_dbl)]),
    "PARALiA_bench_tile_dgemm": (C.c_int, [C.c_int, _chr, _chr, _i64, C.c_int, C.POINTER(_dbl)]),
    "PARALiA_bench_tile_dgemm_chain": (C.c_int, [C.c_int, _chr, _chr, _i64, C.c_int, C.c_int,
                                                 C.POINTER(_dbl)]),
    "PARALiA_bench_tile_sgemm": (C.c_int, [C.c_int, _i64, C.c_int, C.POINTER(_dbl)]),
    "PARALiA_bench_tf32_peak": (C.c_int, [C.c_int, C.c_int, C.POINTER(_dbl)]),
    "PARALiA_bench_tf32_peak_random": (C.c_int, [C.c_int, C.c_int, C.POINTER(_dbl)]),
    "PARALiA_selftest_join_deadline": (C.c_int, [C.c_int, _dbl, _dbl]),
    "PARALiA_selftest_group_rendezvous": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                                    C.c_int, C.c_int, C.POINTER(_dbl)]),
    "PARALiA_bench_tile_daxpy": (C.c_int, [C.c_int, _i64, C.c_int, C.POINTER(_dbl)]),
    "PARALiA_bench_tile_ddot": (C.c_int, [C.c_int, _i64, C.c_int, C.POINTER(_dbl)]),
    "PARALiA_bench_tile_dgemv": (C.c_int, [C.c_int, _chr, _i64, C.c_int, C.POINTER(_dbl)]),
    "PARALiA_bench_host_aggregate": (C.c_int, [C.c_int, C.c_int, _i64, C.c_int, C.POINTER(_dbl)]),
    "PARALiA_autotune_vec": (C.c_int, [C.c_int, _i64, C.c_int, C.c_int, _ctl_p, _rep_p]),
    "PARALiA_model_host_link": (C.c_int, [C.c_int, C.c_int, _i64, C.c_int, C.c_int, C.POINTER(_i32),
                                          C.c_int, C.POINTER(_dbl), C.POINTER(_i32)]),
    "PARALiA_bench_link": (C.c_int, [C.c_int, C.c_int, _i64, C.c_int, C.POINTER(_dbl)]),
    "PARALiA_bench_link_overlap": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, _i64, C.c_int,
                                             C.POINTER(_dbl), C.POINTER(_dbl)]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded shared library; raises LibraryMissing if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise LibraryMissing(
                f"{LIB_PATH} not found: build it with `python {PKG_DIR / 'build.py'}` "
                "(there is no fallback implementation)")
        handle = C.CDLL(str(LIB_PATH), mode=getattr(os, "RTLD_NOW", 2))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if a declared symbol is missing
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def _check(rc: int) -> None:
    if rc != OK:
        msg = lib().PARALiA_last_error()
        raise ParaliaError(rc, msg.decode() if msg else "")


def _ptr(x) -> int:
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    if hasattr(x, "ctypes"):
        return int(x.ctypes.data)
    raise TypeError(f"cannot take the address of {type(x)!r}")


def _c(ch: str) -> bytes:
    return ch.encode()[:1]


def make_ctl(T: int = 0, units=None, cache_limit: int = 0, exec_streams: int = 0,
             flags: int = 0) -> Ctl:
    ctl = Ctl()
    ctl.T = int(T)
    ctl.cache_limit = int(cache_limit)
    ctl.exec_streams = int(exec_streams)
    ctl.flags = int(flags)
    if units is not None:
        units = list(units)
        ctl.active_unit_num = len(units)
        for i, u in enumerate(units):
            ctl.active_unit_id_list[i] = int(u)
    return ctl


DEFAULT_DB = PKG_DIR / "db_b200"   # measured on this pool's B200s by db_builder.py


def init(load_default_db: bool = True) -> None:
    _check(lib().PARALiA_init())
    if load_default_db and "PARALIA_DB" not in os.environ and (DEFAULT_DB / "Processed").is_dir():
        load_database(str(DEFAULT_DB))


def finalize() -> None:
    _check(lib().PARALiA_finalize())


def device_count() -> int:
    return int(lib().PARALiA_device_count())


def dev_cache_free(loc: int) -> None:
    """Reference: PARALiADevCacheFree (Subkernel.cpp:488-495)."""
    _check(lib().PARALiA_dev_cache_free(int(loc)))


def dgemm(TransA, TransB, M, N, K, alpha, A, ldA, B, ldB, beta, Cm, ldC,
          locA=LOC_AUTO, locB=LOC_AUTO, locC=LOC_AUTO, ctl: Ctl | None = None) -> Report:
    """Reference: PARALiADgemm / PARALiADgemmControled (dgemm.cpp:318-705)."""
    rep = Report()
    _check(lib().PARALiA_dgemm(_c(TransA), _c(TransB), M, N, K, alpha, _ptr(A), ldA, locA,
                               _ptr(B), ldB, locB, beta, _ptr(Cm), ldC, locC,
                               C.byref(ctl) if ctl is not None else None, C.byref(rep)))
    return rep


def group_init(name: str, rank: int, world: int, dev: int) -> None:
    """Join the one-process-per-GPU group `name` as `rank` of `world`, driving GPU `dev`."""
    _check(lib().PARALiA_group_init(name.encode(), rank, world, dev))


def group_finalize() -> None:
    _check(lib().PARALiA_group_finalize())


def group_dgemm(TransA, TransB, Mloc, Nloc, K, alpha, A, ldA, B, ldB, beta, Cm, ldC,
                locA=LOC_AUTO, locB=LOC_AUTO, locC=LOC_AUTO, ctl: Ctl | None = None) -> Report:
    """Collective DGEMM of a process group: this rank's row panel of A, column panel of B
    and block of C (see ``ranks.gemm_block``)."""
    rep = Report()
    _check(lib().PARALiA_group_dgemm(_c(TransA), _c(TransB), Mloc, Nloc, K, alpha, _ptr(A), ldA,
                                     locA, _ptr(B), ldB, locB, beta, _ptr(Cm), ldC, locC,
                                     C.byref(ctl) if ctl is not None else None, C.byref(rep)))
    return rep


def group_sgemm(TransA, TransB, Mloc, Nloc, K, alpha, A, ldA, B, ldB, beta, Cm, ldC,
                locA=LOC_AUTO, locB=LOC_AUTO, locC=LOC_AUTO, ctl: Ctl | None = None) -> Report:
    rep = Report()
    _check(lib().PARALiA_group_sgemm(_c(TransA), _c(TransB), Mloc, Nloc, K, alpha, _ptr(A), ldA,
                                     locA, _ptr(B), ldB, locB, beta, _ptr(Cm), ldC, locC,
                                     C.byref(ctl) if ctl is not None else None, C.byref(rep)))
    return rep


def selftest_bounded_wait(dev: int = 0, budget_ms: float = 1.0) -> None:
    """Runs a kernel whose wait can never be satisfied; raises ParaliaError(ERR_TIMEOUT)
    when the bounded wait gave up and reported to the host, as it must."""
    _check(lib().PARALiA_selftest_bounded_wait(dev, budget_ms))


def sgemm(TransA, TransB, M, N, K, alpha, A, ldA, B, ldB, beta, Cm, ldC,
          locA=LOC_AUTO, locB=LOC_AUTO, locC=LOC_AUTO, ctl: Ctl | None = None) -> Report:
    """Reference: PARALiASgemm / PARALiASgemmControled (sgemm.cpp:296-...)."""
    rep = Report()
    _check(lib().PARALiA_sgemm(_c(TransA), _c(TransB), M, N, K, alpha, _ptr(A), ldA, locA,
                               _ptr(B), ldB, locB, beta, _ptr(Cm), ldC, locC,
                               C.byref(ctl) if ctl is not None else None, C.byref(rep)))
    return rep


def dgemv(TransA, M, N, alpha, A, ldA, x, incx, beta, y, incy, locA=LOC_AUTO, locx=LOC_AUTO,
          locy=LOC_AUTO, ctl: Ctl | None = None) -> Report:
    """Reference: PARALiADgemv (dgemv.cpp:288). ctl.T = columns of A per tile."""
    rep = Report()
    _check(lib().PARALiA_dgemv(_c(TransA), M, N, alpha, _ptr(A), ldA, locA, _ptr(x), incx, locx,
                               beta, _ptr(y), incy, locy,
                               C.byref(ctl) if ctl is not None else None, C.byref(rep)))
    return rep


def daxpy(N, alpha, x, incx, y, incy, locx=LOC_AUTO, locy=LOC_AUTO,
          ctl: Ctl | None = None) -> Report:
    """Reference: PARALiADaxpy (daxpy.cpp:200-469)."""
    rep = Report()
    _check(lib().PARALiA_daxpy(N, alpha, _ptr(x), incx, locx, _ptr(y), incy, locy,
                               C.byref(ctl) if ctl is not None else None, C.byref(rep)))
    return rep


def ddot(N, x, incx, y, incy, result: float = 0.0, locx=LOC_AUTO, locy=LOC_AUTO,
         ctl: Ctl | None = None):
    """Reference: PARALiADdot (ddot.cpp:201-469). Returns (result_in + x.y, report)."""
    rep = Report()
    res = C.c_double(result)
    _check(lib().PARALiA_ddot(N, _ptr(x), incx, locx, _ptr(y), incy, locy, C.byref(res),
                              C.byref(ctl) if ctl is not None else None, C.byref(rep)))
    return res.value, rep


def ddot_tiles(N, x, incx, y, incy, locx=LOC_AUTO, locy=LOC_AUTO, ctl: Ctl | None = None):
    """Per-tile sums of a DDOT in tile order (``PARALiA_ddot_tiles``). Returns (list, report)."""
    rep = Report()
    cap = max(1, -(-N // (ctl.T if ctl is not None and ctl.T > 0 else 1 << 16)))
    buf = (C.c_double * cap)()
    cnt = _i64()
    _check(lib().PARALiA_ddot_tiles(N, _ptr(x), incx, locx, _ptr(y), incy, locy, buf, cap, C.byref(cnt),
                                    C.byref(ctl) if ctl is not None else None, C.byref(rep)))
    if cnt.value > cap:
        raise ParaliaError(ERR_INVALID_ARG, f"{cnt.value} tiles do not fit the buffer of {cap}")
    return list(buf[:cnt.value]), rep


def tile_dgemm(dev, TransA, TransB, M, N, K, alpha, A, ldA, B, ldB, beta, Cm, ldC,
               stream: int = 0) -> None:
    """Reference: backend_run_operation(params, "Dgemm", queue) (Subkernel.cpp:168,228)."""
    _check(lib().PARALiA_tile_dgemm(dev, stream, _c(TransA), _c(TransB), M, N, K, alpha, _ptr(A),
                                    ldA, _ptr(B), ldB, beta, _ptr(Cm), ldC))


def tile_status(dev) -> None:
    """Raises ParaliaError(ERR_TIMEOUT) if a tile kernel on `dev` gave up on a wait."""
    _check(lib().PARALiA_tile_status(dev))


def tile_sgemm(dev, TransA, TransB, M, N, K, alpha, A, ldA, B, ldB, beta, Cm, ldC,
               stream: int = 0) -> None:
    _check(lib().PARALiA_tile_sgemm(dev, stream, _c(TransA), _c(TransB), M, N, K, alpha, _ptr(A),
                                    ldA, _ptr(B), ldB, beta, _ptr(Cm), ldC))


def tile_daxpy(dev, N, alpha, x, incx, y, incy, stream: int = 0) -> None:
    _check(lib().PARALiA_tile_daxpy(dev, stream, N, alpha, _ptr(x), incx, _ptr(y), incy))


def tile_ddot_scratch_bytes(N: int) -> int:
    return int(lib().PARALiA_tile_ddot_scratch_bytes(N))


def tile_ddot(dev, N, x, incx, y, incy, partials, result_dev, stream: int = 0) -> None:
    _check(lib().PARALiA_tile_ddot(dev, stream, N, _ptr(x), incx, _ptr(y), incy, _ptr(partials),
                                   _ptr(result_dev)))


def tile_dgemv_scratch_bytes(TransA, M, N) -> int:
    return int(lib().PARALiA_tile_dgemv_scratch_bytes(_c(TransA), M, N))


def tile_dgemv(dev, TransA, M, N, alpha, A, ldA, x, incx, beta, y, incy, scratch=None,
               stream: int = 0) -> None:
    """Per-tile DGEMV on the caller's stream (reference: the "Dgemv" backend operation)."""
    _check(lib().PARALiA_tile_dgemv(dev, stream, _c(TransA), M, N, alpha, _ptr(A), ldA, _ptr(x), incx,
                                    beta, _ptr(y), incy, _ptr(scratch)))


def tile_ddot_noalloc_max_n() -> int:
    return int(lib().PARALiA_tile_ddot_noalloc_max_n())


def tile_ddot_noalloc(dev, N, x, incx, y, incy, result_dev, stream: int = 0) -> None:
    """Dot product that allocates nothing: for callers that cannot call cudaMalloc (a
    latency-critical loop, a plugin with a fixed memory budget) and so cannot supply the
    scratch ``tile_ddot`` needs. The partial sums live in a fixed array inside the
    library; N is limited to ``tile_ddot_noalloc_max_n()``; calls that may overlap on
    one GPU race on that array. No counterpart in the reference."""
    _check(lib().PARALiA_tile_ddot_noalloc(dev, stream, N, _ptr(x), incx, _ptr(y), incy,
                                           _ptr(result_dev)))


def malloc(nbytes: int, loc: int) -> int:
    """Reference: CoCoMalloc(bytes, loc, ...) (dgemm_runner.cpp:55-57)."""
    p = C.c_void_p()
    _check(lib().PARALiA_malloc(C.byref(p), nbytes, loc))
    return int(p.value or 0)


def free(ptr: int, loc: int) -> None:
    _check(lib().PARALiA_free(ptr, loc))


def memcpy(dst, loc_dst, src, loc_src, nbytes) -> None:
    _check(lib().PARALiA_memcpy(_ptr(dst), loc_dst, _ptr(src), loc_src, nbytes))


def fill_f64(ptr, n, seed, dist=0, loc=LOC_HOST) -> None:
    """Reference: CoCoVecInit(ptr, n, seed, loc) (dgemm_runner.cpp:64-66)."""
    _check(lib().PARALiA_fill_f64(_ptr(ptr), n, seed, dist, loc))


def fill_f32(ptr, n, seed, dist=0, loc=LOC_HOST) -> None:
    _check(lib().PARALiA_fill_f32(_ptr(ptr), n, seed, dist, loc))


def autotune_gemm(elem_size, TransA, TransB, M, N, K, locA, locB, locC,
                  ctl: Ctl | None = None) -> Report:
    """Reference: ATC::autotune_problem (Autotuner.cpp:279-560)."""
    rep = Report()
    _check(lib().PARALiA_autotune_gemm(elem_size, _c(TransA), _c(TransB), M, N, K, locA, locB, locC,
                                       C.byref(ctl) if ctl is not None else None, C.byref(rep)))
    return rep


def autotune_vec(is_dot: bool, N, locx, locy, ctl: Ctl | None = None) -> Report:
    """Reference: ATC::autotune_problem for the level-1 models (ModelLvl1.cpp:19-144)."""
    rep = Report()
    _check(lib().PARALiA_autotune_vec(int(bool(is_dot)), N, locx, locy,
                                      C.byref(ctl) if ctl is not None else None, C.byref(rep)))
    return rep


def model_host_link(dev, to_gpu: bool, nbytes, n_active, both_directions=False, active_devs=None):
    """Seconds the shared host-link model predicts, and whether write-backs are deferred with
    ``n_active`` GPUs. Reference: t_com_predict_shared (CoModel.cpp:120-140)."""
    sec, defer = _dbl(), _i32()
    arr, n = None, 0
    if active_devs is not None:
        n = len(active_devs)
        arr = (_i32 * max(n, 1))(*active_devs)
    _check(lib().PARALiA_model_host_link(dev, int(bool(to_gpu)), int(nbytes), n_active,
                                         int(bool(both_directions)), arr, n, C.byref(sec), C.byref(defer)))
    return sec.value, bool(defer.value)


def tile_slowdowns(M, N, K, T, units) -> list[float]:
    """Reference: ATC::get_T_slowdowns (Autotuner.cpp:571-603)."""
    sl = (C.c_double * 6)()
    _check(lib().PARALiA_tile_slowdowns(M, N, K, T, units, sl))
    return list(sl)


def distribute_2d(units, Mt, Nt, Kt):
    """Reference: CoCoDistributeSubkernels2DBlockCyclic (Subkernel_distributions.cpp:315-485).
    Returns (owner unit of every subkernel id, d1, d2)."""
    arr = (C.c_int32 * (Mt * Nt * Kt))()
    d1, d2 = C.c_int32(), C.c_int32()
    _check(lib().PARALiA_distribute_2d(units, Mt, Nt, Kt, arr, C.byref(d1), C.byref(d2)))
    return list(arr), d1.value, d2.value


def plan_gemm(M, N, K, T, units, bounded_cache: bool = False):
    """Launch plan of a tiled GEMM: list of (unit, mi, ni, ki0, ki1) in enqueue order, and the
    device grid. Reference: chosen at run time by SubkernelSelect (Subkernel.cpp:384-449)."""
    n = C.c_int64()
    d1, d2 = C.c_int32(), C.c_int32()
    _check(lib().PARALiA_plan_gemm(M, N, K, T, units, int(bounded_cache), None, 0, C.byref(n),
                                   C.byref(d1), C.byref(d2)))
    arr = (C.c_int32 * (5 * max(n.value, 1)))()
    _check(lib().PARALiA_plan_gemm(M, N, K, T, units, int(bounded_cache), arr, n.value, C.byref(n),
                                   C.byref(d1), C.byref(d2)))
    flat = list(arr)[:5 * n.value]
    return [tuple(flat[i:i + 5]) for i in range(0, len(flat), 5)], (d1.value, d2.value)


def load_database(path: str) -> None:
    _check(lib().PARALiA_load_database(str(path).encode()))


def bench_dmma_peak(dev=0, shape=1688, iters=20000) -> float:
    v = C.c_double()
    _check(lib().PARALiA_bench_dmma_peak(dev, shape, iters, C.byref(v)))
    return v.value


def bench_tile_dgemm_chain(dev, TransA, TransB, T, chain, reps) -> float:
    v = _dbl()
    _check(lib().PARALiA_bench_tile_dgemm_chain(dev, _c(TransA), _c(TransB), T, chain, reps, C.byref(v)))
    return v.value


def bench_tile_dgemv(dev, trans, T, reps=8) -> float:
    """Mean seconds of one square T x T DGEMV tile on device-resident operands."""
    v = _dbl()
    _check(lib().PARALiA_bench_tile_dgemv(dev, _c(trans), int(T), int(reps), C.byref(v)))
    return v.value


def bench_tf32_peak(dev, stages, random_operands=False) -> float:
    """Dense TF32 TFLOP/s of the tcgen05 instruction shape the FP32 kernel issues, on operands
    of ones (the issue rate) or drawn from uniform(-1, 1) (what the power limit allows)."""
    v = _dbl()
    fn = lib().PARALiA_bench_tf32_peak_random if random_operands else lib().PARALiA_bench_tf32_peak
    _check(fn(dev, int(stages), C.byref(v)))
    return v.value


def selftest_join_deadline(dev, kernel_ms, deadline_ms) -> None:
    _check(lib().PARALiA_selftest_join_deadline(dev, float(kernel_ms), float(deadline_ms)))


def selftest_group_rendezvous(name, rank, world, rounds, fail_rank=-1, fail_round=0, fail_mode=0):
    """Returns (status code, milliseconds spent in the failing barrier); never raises."""
    w = _dbl()
    rc = lib().PARALiA_selftest_group_rendezvous(name.encode(), rank, world, rounds, fail_rank,
                                                 fail_round, fail_mode, C.byref(w))
    return int(rc), w.value


def bench_tile_daxpy(dev, N, reps) -> float:
    v = _dbl()
    _check(lib().PARALiA_bench_tile_daxpy(dev, N, reps, C.byref(v)))
    return v.value


def bench_tile_ddot(dev, N, reps) -> float:
    v = _dbl()
    _check(lib().PARALiA_bench_tile_ddot(dev, N, reps, C.byref(v)))
    return v.value


def bench_host_aggregate(ngpu, mode, nbytes, reps) -> float:
    """Aggregate GB/s per direction; mode 0 host->GPU, 1 GPU->host, 2 both together."""
    v = _dbl()
    _check(lib().PARALiA_bench_host_aggregate(ngpu, mode, int(nbytes), reps, C.byref(v)))
    return v.value


def bench_tile_dgemm(dev, TransA, TransB, T, reps) -> float:
    v = C.c_double()
    _check(lib().PARALiA_bench_tile_dgemm(dev, _c(TransA), _c(TransB), T, reps, C.byref(v)))
    return v.value


def bench_tile_sgemm(dev, T, reps) -> float:
    v = C.c_double()
    _check(lib().PARALiA_bench_tile_sgemm(dev, T, reps, C.byref(v)))
    return v.value


def bench_link(dst_loc, src_loc, dim, reps) -> float:
    v = C.c_double()
    _check(lib().PARALiA_bench_link(dst_loc, src_loc, dim, reps, C.byref(v)))
    return v.value


def bench_link_overlap(dst_loc, src_loc, odst_loc, osrc_loc, dim, reps):
    """(t_alone, t_shared) of link dst<-src while link odst<-osrc is kept busy."""
    a, b = C.c_double(), C.c_double()
    _check(lib().PARALiA_bench_link_overlap(dst_loc, src_loc, odst_loc, osrc_loc, dim, reps,
                                            C.byref(a), C.byref(b)))
    return a.value, b.value
