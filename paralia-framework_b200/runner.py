"""Timed runners for the four routines: the harness of the reference re-created over the
C ABI (reference: ``Benchmarking/CuCuBLAS/src/PARALia/{dgemm,daxpy,ddot}_runner.cpp``,
``sgemm_tester.cpp``, argument parsing ``Benchmarking/CuCuBLAS/src/testing.cpp:273-329``,
log rows ``testing.cpp:420-428``).

Level 3 (same argument order as the reference's runners)::

    python runner.py dgemm|sgemm active_unit_num dev_ids T cache_limit TransA TransB alpha beta M N K locA locB locC outloc
    python runner.py daxpy|ddot  active_unit_num dev_ids T cache_limit alpha N incx incy locx locy
    python runner.py dgemv       active_unit_num dev_ids T cache_limit TransA alpha beta M N incx incy locA locx locy
    python runner.py dgemm_predict|sgemm_predict  (level-3 arguments)   # autotuner only, nothing runs on a GPU stream
    python runner.py cublasxt_dgemm|cublasxt_sgemm (level-3 arguments)  # the reference's comparator, same protocol

``active_unit_num < 0`` = autotuned unit set; ``dev_ids`` is the reference's decimal mask
(``0101`` = GPUs 0 and 2); ``T <= 0`` = autotuned tile; locations: -1 pinned host, >= 0 GPU.
Protocol of the reference's runner: one cold call, warm-up calls (10, or 2 for problems of
20000^3 and more), then 10 timed calls; wall clock around the blocking call; one CSV row
per timed call appended to ``--log`` in the reference's schema
``T,ndev,devmask,cache_limit, TA,TB,alpha,beta,M,N,K,locA,locB,locC,locOut, t,pred_t,pred_J``.
Inputs are seeded (42/43/44) like the reference's runner (dgemm_runner.cpp:64-66).
Validation (``--validate``): the first result is compared with the FP64 product computed on
the host by numpy (which calls OpenBLAS, the reference's CPU comparator) on problems small
enough for the host, else on sampled rows and columns in FP64.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import sys
import time
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
ROOT = PKG_DIR.parent


def _pkg():
    name = "paralia_framework_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, PKG_DIR / "__init__.py",
                                                  submodule_search_locations=[str(PKG_DIR)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def parse_mask(num: int, token: str) -> list[int] | None:
    """Reference convention: decimal digits, digit i (from the right) set = GPU i."""
    if num < 0:
        return None
    ids = [i for i, ch in enumerate(reversed(token.strip())) if ch == "1"]
    if len(ids) != num:
        raise SystemExit(f"dev_ids {token!r} names {len(ids)} devices, active_unit_num says {num}")
    return ids


def csv_control(rep) -> str:
    n = max(rep.active_unit_num, 0)
    mask = sum(10 ** int(rep.active_unit_id_list[i]) for i in range(n))
    return f"{rep.T},{rep.active_unit_num},{mask},{rep.cache_limit}"


def run_level3(pl, a, routine: str) -> dict:
    import numpy as np
    esz = 8 if routine == "dgemm" else 4
    fill = pl.fill_f64 if esz == 8 else pl.fill_f32
    sys.path.insert(0, str(PKG_DIR))
    M, N, K = a.M, a.N, a.K
    ar, ac = (K, M) if a.TransA == "T" else (M, K)
    br, bc = (N, K) if a.TransB == "T" else (K, N)
    dist = 1 if routine == "sgemm" else 0     # normal(0,1) for SGEMM, uniform[-1,1) for DGEMM
    bufs = []
    for (rows, cols, seed, loc) in ((ar, ac, 42, a.locA), (br, bc, 43, a.locB), (M, N, 44, a.locC)):
        p = pl.malloc(rows * cols * esz, loc)
        if loc >= 0:
            fill(p, rows * cols, seed, dist, loc)
        else:                                # generate on a GPU, copy to the pinned host buffer
            tmp = pl.malloc(rows * cols * esz, 0)
            fill(tmp, rows * cols, seed, dist, 0)
            pl.memcpy(p, -1, tmp, 0, rows * cols * esz)
            pl.free(tmp, 0)
        bufs.append(p)
    A, B, C = bufs
    units = parse_mask(a.active_unit_num, a.dev_ids)
    ctl = pl.make_ctl(T=max(a.T, 0), units=units, cache_limit=max(a.cache_limit, 0))
    if getattr(a, "comparator", False):
        # whole-problem cuBLASXt as the reference runs it (cuBLASXt_dgemm_runner): block
        # dimension T (default min(M,N,K)/2 capped at 10000), device list from the mask
        import comparators
        # every GPU when all operands are in host memory; one GPU (the one that holds the
        # operands) otherwise -- a vendor kernel is never given another GPU's memory
        locs = (a.locA, a.locB, a.locC)
        on_gpu = sorted({l for l in locs if l >= 0})
        devs = units if units else ([on_gpu[0]] if on_gpu else list(range(pl.device_count())))
        comparators.check_xt_placement(devs, locs)
        rep_like = pl.autotune_gemm(esz, a.TransA, a.TransB, M, N, K, a.locA, a.locB, a.locC, ctl)

        def call():
            comparators.cublasxt_gemm(esz, a.TransA, a.TransB, M, N, K, a.alpha, A, ar, B, br,
                                      a.beta, C, M, T=a.T, dev_ids=devs, pinning=False, locs=locs)
            rep_like.device_ms = float("nan")
            return rep_like
    else:
        gemm = pl.dgemm if esz == 8 else pl.sgemm
        call = lambda: gemm(a.TransA, a.TransB, M, N, K, a.alpha, A, ar, B, br, a.beta, C, M,
                            locA=a.locA, locB=a.locB, locC=a.locC, ctl=ctl)
    out = {"routine": ("cublasxt_" if getattr(a, "comparator", False) else "") + routine}
    if a.validate:
        out["validation"] = validate_level3(pl, a, routine, A, B, C, ar, br, call)
        fill_c = C
        # restore C for the timed runs
        if a.locC >= 0:
            fill(fill_c, M * N, 44, dist, a.locC)
    t0 = time.perf_counter()
    rep = call()
    first = time.perf_counter() - t0
    warm = 2 if (M >= 20000 and N >= 20000 and K >= 20000) else 10
    for _ in range(warm if a.warmup < 0 else a.warmup):
        call()
    times, dev_ms = [], []
    for _ in range(a.iters):
        t0 = time.perf_counter()
        rep = call()
        times.append(time.perf_counter() - t0)
        dev_ms.append(rep.device_ms)
        if a.log:
            with open(a.log, "a") as f:
                f.write(f"{csv_control(rep)}, {a.TransA},{a.TransB},{a.alpha:.5f},{a.beta:.5f},"
                        f"{M},{N},{K},{a.locA},{a.locB},{a.locC},{a.outloc}, "
                        f"{times[-1]:e},{rep.pred_t:e},{rep.pred_J:e}\n")
    flops = 2.0 * M * N * K
    out.update(control=csv_control(rep), first_s=first, avg_s=sum(times) / len(times),
               min_s=min(times), max_s=max(times),
               device_ms_min=min(dev_ms), tflops_avg=flops / (sum(times) / len(times)) / 1e12,
               tflops_best=flops / min(times) / 1e12,
               tflops_device_best=flops / (min(dev_ms) * 1e-3) / 1e12,
               h2d_bytes=rep.h2d_bytes, d2h_bytes=rep.d2h_bytes, p2p_bytes=rep.p2p_bytes,
               launches=rep.kernel_launches, pred_t=rep.pred_t, grid=[rep.grid_d1, rep.grid_d2],
               phases_ms={"fill": rep.fill_ms, "last_kernel_end": rep.exec_end_ms,
                          "h2d_end": rep.h2d_end_ms, "device": rep.device_ms})
    for p, loc in zip(bufs, (a.locA, a.locB, a.locC)):
        pl.free(p, loc)
    return out


def run_predict(pl, a, routine: str) -> dict:
    """Autotune-only run: the model's choice of tile, unit set and its time prediction for a
    problem, without moving or computing anything (reference:
    ``Benchmarking/CuCuBLAS/src/PARALia/dgemm_predictor.cpp:16-93``)."""
    esz = 8 if routine.startswith("d") else 4
    units = parse_mask(a.active_unit_num, a.dev_ids)
    ctl = pl.make_ctl(T=max(a.T, 0), units=units, cache_limit=max(a.cache_limit, 0))
    t0 = time.perf_counter()
    rep = pl.autotune_gemm(esz, a.TransA, a.TransB, a.M, a.N, a.K, a.locA, a.locB, a.locC, ctl)
    t_auto = time.perf_counter() - t0
    if a.log:
        with open(a.log, "a") as f:
            f.write(f"{csv_control(rep)}, {a.TransA},{a.TransB},{a.alpha:.5f},{a.beta:.5f},"
                    f"{a.M},{a.N},{a.K},{a.locA},{a.locB},{a.locC},{a.outloc}, "
                    f"{t_auto:e},{rep.pred_t:e},{rep.pred_J:e}\n")
    n = max(rep.active_unit_num, 0)
    return {"routine": routine, "control": csv_control(rep), "t_autotune_ms": t_auto * 1e3,
            "T": rep.T, "units": [int(rep.active_unit_id_list[i]) for i in range(n)],
            "grid": [rep.grid_d1, rep.grid_d2], "subkernels": rep.subkernel_num,
            "pred_t": rep.pred_t, "pred_tflops": 2.0 * a.M * a.N * a.K / max(rep.pred_t, 1e-30) / 1e12,
            "T_slowdowns": [float(v) for v in rep.T_slowdowns]}


def validate_level3(pl, a, routine, A, B, C, ar, br, call) -> dict:
    """First call vs the CPU: full OpenBLAS product when M*N*K <= 2^36, else 8 sampled rows
    and 8 sampled columns of C in FP64."""
    import ctypes
    import numpy as np
    esz = 8 if routine == "dgemm" else 4
    dt = np.float64 if esz == 8 else np.float32
    M, N, K = a.M, a.N, a.K
    ac = M if a.TransA == "T" else K
    bc = K if a.TransB == "T" else N

    def to_host(ptr, rows, cols, loc):
        h = np.empty((rows, cols), dtype=dt, order="F")
        pl.memcpy(h, -1, ptr, loc, rows * cols * esz)
        return h
    hA, hB, hC0 = to_host(A, ar, ac, a.locA), to_host(B, br, bc, a.locB), to_host(C, M, N, a.locC)
    call()
    hC = to_host(C, M, N, a.locC)
    opA = hA.T if a.TransA == "T" else hA
    opB = hB.T if a.TransB == "T" else hB
    eps = 2.0 ** -52 if esz == 8 else 2.0 ** -23
    bound = (8 if esz == 8 else 4) * K * eps
    if M * N * K <= 2 ** 36:
        want = a.alpha * (opA.astype(np.float64) @ opB.astype(np.float64)) + a.beta * hC0
        den = float(np.linalg.norm(want.astype(np.float64)))
        err = float(np.linalg.norm(hC.astype(np.float64) - want)) / (den if den > 0 else 1.0)
        mode = "full"
    else:
        rs = np.random.default_rng(0)
        rows = rs.integers(0, M, 8)
        cols = rs.integers(0, N, 8)
        num = den = 0.0
        for i in rows:
            w = a.alpha * (opA[i, :].astype(np.float64) @ opB.astype(np.float64)) + a.beta * hC0[i, :]
            num += float(np.sum((hC[i, :] - w) ** 2)); den += float(np.sum(w ** 2))
        for j in cols:
            w = a.alpha * (opA.astype(np.float64) @ opB[:, j].astype(np.float64)) + a.beta * hC0[:, j]
            num += float(np.sum((hC[:, j] - w) ** 2)); den += float(np.sum(w ** 2))
        err = (num / den) ** 0.5
        mode = "sampled 8 rows + 8 columns"
    # put the original C back so that timed runs start from the same data
    pl.memcpy(C, a.locC, hC0, -1, M * N * esz)
    return {"mode": mode, "normwise_rel_err": err, "bound": bound, "ok": bool(err <= bound)}


def run_level1(pl, a, routine: str) -> dict:
    import numpy as np
    n = a.N
    bufs = []
    for (inc, seed, loc) in ((a.incx, 42, a.locx), (a.incy, 43, a.locy)):
        cnt = 1 + (n - 1) * inc
        p = pl.malloc(cnt * 8, loc)
        if loc >= 0:
            pl.fill_f64(p, cnt, seed, 0, loc)
        else:
            tmp = pl.malloc(cnt * 8, 0)
            pl.fill_f64(tmp, cnt, seed, 0, 0)
            pl.memcpy(p, -1, tmp, 0, cnt * 8)
            pl.free(tmp, 0)
        bufs.append(p)
    x, y = bufs
    units = parse_mask(a.active_unit_num, a.dev_ids)
    ctl = pl.make_ctl(T=max(a.T, 0), units=units)
    if routine == "daxpy":
        call = lambda: pl.daxpy(n, a.alpha, x, a.incx, y, a.incy, locx=a.locx, locy=a.locy, ctl=ctl)
        nbytes = 24.0 * n
    else:
        call = lambda: pl.ddot(n, x, a.incx, y, a.incy, 0.0, locx=a.locx, locy=a.locy, ctl=ctl)[1]
        nbytes = 16.0 * n
    t0 = time.perf_counter()
    rep = call()
    first = time.perf_counter() - t0
    for _ in range(10 if a.warmup < 0 else a.warmup):
        call()
    times, dev_ms = [], []
    for _ in range(a.iters):
        t0 = time.perf_counter()
        rep = call()
        times.append(time.perf_counter() - t0)
        dev_ms.append(rep.device_ms)
        if a.log:
            with open(a.log, "a") as f:
                f.write(f"{csv_control(rep)}, {a.alpha:.5f},{n},{a.incx},{a.incy},{a.locx},{a.locy},"
                        f"{a.locx},{a.locy}, {times[-1]:e}\n")
    out = {"routine": routine, "control": csv_control(rep), "first_s": first,
           "avg_s": sum(times) / len(times), "min_s": min(times),
           "gbs_avg": nbytes / (sum(times) / len(times)) / 1e9,
           "gbs_device_best": nbytes / (min(dev_ms) * 1e-3) / 1e9,
           "h2d_bytes": rep.h2d_bytes, "d2h_bytes": rep.d2h_bytes, "launches": rep.kernel_launches}
    for p, loc in zip(bufs, (a.locx, a.locy)):
        pl.free(p, loc)
    return out


def run_dgemv(pl, a) -> dict:
    M, N = a.M, a.N
    in_len, out_len = (M, N) if a.TransA == "T" else (N, M)
    specs = ((M * N, 42, a.locA), (1 + (in_len - 1) * a.incx, 43, a.locx),
             (1 + (out_len - 1) * a.incy, 44, a.locy))
    bufs = []
    for (cnt, seed, loc) in specs:
        p = pl.malloc(cnt * 8, loc)
        if loc >= 0:
            pl.fill_f64(p, cnt, seed, 0, loc)
        else:
            tmp = pl.malloc(cnt * 8, 0)
            pl.fill_f64(tmp, cnt, seed, 0, 0)
            pl.memcpy(p, -1, tmp, 0, cnt * 8)
            pl.free(tmp, 0)
        bufs.append(p)
    A, x, y = bufs
    ctl = pl.make_ctl(T=max(a.T, 0), units=parse_mask(a.active_unit_num, a.dev_ids))
    call = lambda: pl.dgemv(a.TransA, M, N, a.alpha, A, M, x, a.incx, a.beta, y, a.incy,
                            locA=a.locA, locx=a.locx, locy=a.locy, ctl=ctl)
    t0 = time.perf_counter()
    rep = call()
    first = time.perf_counter() - t0
    for _ in range(10 if a.warmup < 0 else a.warmup):
        call()
    times, dev_ms = [], []
    for _ in range(a.iters):
        t0 = time.perf_counter()
        rep = call()
        times.append(time.perf_counter() - t0)
        dev_ms.append(rep.device_ms)
        if a.log:
            with open(a.log, "a") as f:   # level-2 row of the reference (testing.cpp StoreLogLvl2)
                f.write(f"{csv_control(rep)}, {a.TransA},{a.alpha:.5f},{a.beta:.5f},{M},{N},{a.incx},"
                        f"{a.incy},{a.locA},{a.locx},{a.locy},{a.locy}, {times[-1]:e},{rep.pred_t:e},"
                        f"{rep.pred_J:e}\n")
    nbytes = 8.0 * M * N
    out = {"routine": "dgemv", "control": csv_control(rep), "first_s": first,
           "avg_s": sum(times) / len(times), "min_s": min(times),
           "gbs_avg": nbytes / (sum(times) / len(times)) / 1e9,
           "gbs_device_best": nbytes / (min(dev_ms) * 1e-3) / 1e9,
           "h2d_bytes": rep.h2d_bytes, "d2h_bytes": rep.d2h_bytes, "launches": rep.kernel_launches}
    for p, loc in zip(bufs, (a.locA, a.locx, a.locy)):
        pl.free(p, loc)
    return out


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("routine", choices=["dgemm", "sgemm", "dgemv", "daxpy", "ddot", "dgemm_predict", "sgemm_predict", "cublasxt_dgemm", "cublasxt_sgemm"])
    ap.add_argument("active_unit_num", type=int)
    ap.add_argument("dev_ids")
    ap.add_argument("T", type=int)
    ap.add_argument("cache_limit", type=int)
    ap.add_argument("rest", nargs="+")
    ap.add_argument("--log", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=-1)
    ap.add_argument("--validate", action="store_true")
    a = ap.parse_args(argv)
    r = a.rest
    pl = _pkg()
    try:
        pl.init()
    except pl.ParaliaError:
        # the predictor needs no GPU when the unit list is given: the model runs on the host
        if not (a.routine.endswith("_predict") and a.active_unit_num > 0):
            raise
        if (pl.DEFAULT_DB / "Processed").is_dir():
            pl.load_database(str(pl.DEFAULT_DB))
    a.comparator = a.routine.startswith("cublasxt_")
    if a.comparator:
        a.routine = a.routine[len("cublasxt_"):]
    if a.routine in ("dgemm", "sgemm", "dgemm_predict", "sgemm_predict"):
        if len(r) != 11:
            raise SystemExit("level 3 needs: TransA TransB alpha beta M N K locA locB locC outloc")
        a.TransA, a.TransB = r[0].upper(), r[1].upper()
        a.alpha, a.beta = float(r[2]), float(r[3])
        a.M, a.N, a.K = int(r[4]), int(r[5]), int(r[6])
        a.locA, a.locB, a.locC, a.outloc = (int(v) for v in r[7:11])
        out = run_predict(pl, a, a.routine) if a.routine.endswith("_predict") else run_level3(pl, a, a.routine)
    elif a.routine == "dgemv":
        if len(r) != 10:
            raise SystemExit("level 2 needs: TransA alpha beta M N incx incy locA locx locy")
        a.TransA = r[0].upper()
        a.alpha, a.beta = float(r[1]), float(r[2])
        a.M, a.N, a.incx, a.incy = (int(v) for v in r[3:7])
        a.locA, a.locx, a.locy = (int(v) for v in r[7:10])
        out = run_dgemv(pl, a)
    else:
        if len(r) != 6:
            raise SystemExit("level 1 needs: alpha N incx incy locx locy")
        a.alpha, a.N, a.incx, a.incy = float(r[0]), int(r[1]), int(r[2]), int(r[3])
        a.locx, a.locy = int(r[4]), int(r[5])
        out = run_level1(pl, a, a.routine)
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
