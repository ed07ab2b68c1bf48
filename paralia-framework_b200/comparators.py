"""The reference's own GPU comparators, for measurements and tests on the GPU box.

The reference validates and compares its GEMM against whole-problem cuBLASXt, configured
as in ``Benchmarking/CuCuBLAS/src/cuBLASXt/cuBLASXtWrappers.cpp:30-75`` (block dimension T,
CPU ratio 0, pinning enabled, an explicit device list), and its per-tile compute call is a
plain cuBLAS GEMM on device-resident tiles (``Library_scheduler/src/Subkernel.cpp:168,228``
through the backend). Both are bound here through ``ctypes`` on the CUDA toolkit's
``libcublas`` so that they can be timed beside this library's kernels and used as the second
checker of its results (the reference's runner does the same,
``Benchmarking/CuCuBLAS/src/PARALia/dgemm_runner.cpp:94-99``).

Nothing in the library's compute path imports this module: it calls vendor library kernels
and exists only as a yardstick.
"""
from __future__ import annotations

import ctypes as C
import glob
import os
import time

_OP = {"N": 0, "T": 1, "C": 2}
_XT_GEMM = 0                 # cublasXtBlasOp_t: CUBLASXT_GEMM
_XT_FLOAT, _XT_DOUBLE = 0, 1  # cublasXtOpType_t
_XT_PINNING_ENABLED = 1
CBLASXT_MAX_SAFE_TILE = 10000   # dgemm_runner.cpp:14

_lib = None


def cublas() -> C.CDLL:
    """libcublas of the CUDA toolkit in this image (the copy torch ships, else the system one)."""
    global _lib
    if _lib is not None:
        return _lib
    # torch's loader brings in the toolkit libraries libcublas depends on in a consistent
    # set; loaded on its own, the same libcublas answers CUBLAS_STATUS_INVALID_VALUE to
    # every cublasXt GEMM on this image.
    import torch  # noqa: F401
    cands = ["libcublas.so.12", "libcublas.so"]
    try:
        import nvidia.cublas  # type: ignore
        for base in list(getattr(nvidia.cublas, "__path__", [])):
            cands = sorted(glob.glob(os.path.join(base, "lib", "libcublas.so*"))) + cands
    except Exception:
        pass
    cands += sorted(glob.glob("/usr/local/cuda/lib64/libcublas.so*"))
    err = None
    for c in cands:
        try:
            _lib = C.CDLL(c, mode=C.RTLD_GLOBAL)
            break
        except OSError as e:
            err = e
    if _lib is None:
        raise OSError(f"libcublas not found: {err}")
    return _lib


def _ok(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what} failed with cuBLAS status {status}")


class ComparatorRefused(ValueError):
    """The requested comparator run would hand a vendor kernel memory of another GPU."""


def check_xt_placement(dev_ids, locs) -> None:
    """cuBLASXt runs vendor GEMM kernels on every GPU of ``dev_ids``. Those kernels must never
    be given an operand that lives on a different GPU, so a run is allowed only if every
    operand is in host memory, or there is exactly one GPU and every GPU-resident operand
    lives on it. Anything else raises ``ComparatorRefused`` before any CUDA call."""
    devs = list(dev_ids)
    if not devs:
        raise ComparatorRefused("empty device list")
    on_gpu = [int(l) for l in locs if int(l) >= 0]
    if not on_gpu:
        return
    if len(devs) > 1:
        raise ComparatorRefused(
            f"cuBLASXt on {len(devs)} GPUs needs all three operands in host memory; "
            f"operand locations were {tuple(int(l) for l in locs)}")
    if any(l != devs[0] for l in on_gpu):
        raise ComparatorRefused(
            f"cuBLASXt on GPU {devs[0]} cannot take an operand that lives on another GPU; "
            f"operand locations were {tuple(int(l) for l in locs)}")


def cublasxt_gemm(elem_size: int, TransA: str, TransB: str, M: int, N: int, K: int, alpha: float,
                  A: int, ldA: int, B: int, ldB: int, beta: float, Cm: int, ldC: int,
                  T: int = 0, dev_ids=(0,), pinning: bool = True, locs=(-1, -1, -1)) -> float:
    """One blocking cublasXt{D,S}gemm on raw pointers (host or device); returns wall seconds
    of the call including handle set-up, as the reference's wrapper does. ``pinning`` =
    False for operands that are already page-locked (asking the library to pin them again
    makes the call fail with CUBLAS_STATUS_INVALID_VALUE on this toolkit). ``locs`` are the
    location ids of A, B and C (-1 host, else the GPU): see ``check_xt_placement``."""
    check_xt_placement(dev_ids, locs)
    lib = cublas()
    if T <= 0:    # the reference's choice when it validates (dgemm_runner.cpp:97)
        T = int(min(min(M, N, K) // 2, CBLASXT_MAX_SAFE_TILE))
    T = max(T, 1)
    t0 = time.perf_counter()
    h = C.c_void_p()
    _ok(lib.cublasXtCreate(C.byref(h)), "cublasXtCreate")
    try:
        ids = (C.c_int * len(dev_ids))(*dev_ids)
        _ok(lib.cublasXtDeviceSelect(h, C.c_int(len(dev_ids)), ids), "cublasXtDeviceSelect")
        _ok(lib.cublasXtSetBlockDim(h, C.c_int(T)), "cublasXtSetBlockDim")
        typ = _XT_DOUBLE if elem_size == 8 else _XT_FLOAT
        _ok(lib.cublasXtSetCpuRatio(h, C.c_int(_XT_GEMM), C.c_int(typ), C.c_float(0.0)),
            "cublasXtSetCpuRatio")
        _ok(lib.cublasXtSetPinningMemMode(h, C.c_int(_XT_PINNING_ENABLED if pinning else 0)), "cublasXtSetPinningMemMode")
        sz = C.c_size_t
        if elem_size == 8:
            a, b = C.c_double(alpha), C.c_double(beta)
            fn = lib.cublasXtDgemm
        else:
            a, b = C.c_float(alpha), C.c_float(beta)
            fn = lib.cublasXtSgemm
        fn.restype = C.c_int
        fn.argtypes = [C.c_void_p, C.c_int, C.c_int, sz, sz, sz, C.c_void_p, C.c_void_p, sz,
                       C.c_void_p, sz, C.c_void_p, C.c_void_p, sz]
        _ok(fn(h, _OP[TransA.upper()], _OP[TransB.upper()], M, N, K, C.byref(a), C.c_void_p(A), ldA,
               C.c_void_p(B), ldB, C.byref(b), C.c_void_p(Cm), ldC), "cublasXt gemm")
    finally:
        lib.cublasXtDestroy(h)
    return time.perf_counter() - t0


def cublas_tile_gemm_tflops(elem_size: int, T: int, reps: int = 10, dev: int = 0,
                            TransA: str = "N", TransB: str = "N") -> float:
    """TFLOP/s of cublas{D,S}gemm on one T x T x T tile resident in HBM: the call the
    reference issues per subkernel. Device-timed with CUDA events on the launching stream."""
    import torch
    lib = cublas()
    torch.cuda.set_device(dev)
    dt = torch.float64 if elem_size == 8 else torch.float32
    g = torch.Generator(device="cuda").manual_seed(42)
    A = torch.rand(T, T, dtype=dt, device="cuda", generator=g) * 2 - 1
    B = torch.rand(T, T, dtype=dt, device="cuda", generator=g) * 2 - 1
    Cm = torch.zeros(T, T, dtype=dt, device="cuda")
    h = C.c_void_p()
    _ok(lib.cublasCreate_v2(C.byref(h)), "cublasCreate")
    try:
        stream = torch.cuda.current_stream()
        _ok(lib.cublasSetStream_v2(h, C.c_void_p(stream.cuda_stream)), "cublasSetStream")
        if elem_size == 8:
            a, b, fn = C.c_double(1.0), C.c_double(0.0), lib.cublasDgemm_v2
        else:
            a, b, fn = C.c_float(1.0), C.c_float(0.0), lib.cublasSgemm_v2
        fn.restype = C.c_int
        fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                       C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int]

        def call():
            _ok(fn(h, _OP[TransA], _OP[TransB], T, T, T, C.byref(a), C.c_void_p(A.data_ptr()), T,
                   C.c_void_p(B.data_ptr()), T, C.byref(b), C.c_void_p(Cm.data_ptr()), T), "cublas gemm")
        for _ in range(3):
            call()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(reps):
            call()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
    finally:
        lib.cublasDestroy_v2(h)
    return 2.0 * T * T * T / (ms * 1e-3) / 1e12
