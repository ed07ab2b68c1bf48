"""Calibration database builder: the install-time microbenchmarks of the reference
re-run against this library's own kernels and this box's links.

Reference: ``Deploy.in:14-18`` -> ``Database_builder/RunMicrobenchmarks.in:37-59``
(``Database_builder/CuCuBLAS/src/dgemm_microbench.cu:125-187`` tile sweep with a
Student-t 95 % confidence stop rule, ``transfer_link_microbench.cu:119-153,186-218`` link
sweep and link-sharing slowdowns) -> ``ProcessDatabase.in:22-42``
(``Python-DataManage/BenchToLookupTables.py.in:30-56`` lookup tables,
``LinkPreprocessing.py.in:31-62`` least-squares link model).

Output files keep the reference's names and row formats so that the autotuner's readers
(``PARALiA_load_database``; reference ``GPUexec_lookup.cpp:79-81``, ``CoModel.cpp:26-38``)
parse them unchanged::

    <db>/Benchmark-Results/cublasDgemm_dev-<d>_TransA-<c>_TransB-<c>_<ver>.log   M,N,K, mean_t,W,J,err,samples,bench_t
    <db>/Benchmark-Results/CuCuBLAS_link_benchmark_loc_dest-<d>_loc_src-<s>_<ver>.log   dim,dim, mean_t,err,samples, bench_t
    <db>/Benchmark-Results/CuCuBLAS_link_overlap_benchmark_loc_dest-<d>_loc_src-<s>_<ver>.log  other_dest,other_src, t_alone,t_shared,10, bench_t
    <db>/Processed/<Func>_lookup-table_dev-<d>.log     TransA,TransB,T,T,T,mean_t,W,J,err,samples,bench_t
    <db>/Processed/Link-Stats_loc_dest-<d>_loc_src-<s>.log   Intercept / Coefficient / Slowdown([s']->[d']) lines
    <db>/Benchmark-Results/cublasDaxpy_dev-<d>_<ver>.log, cublasDdot_...   N, mean_t,W,J,err,samples,bench_t
    <db>/Processed/Daxpy_lookup-table_dev-<d>.log, Ddot_...    N,mean_t,W,J,err,samples,bench_t
    <db>/Processed/Host-Link-Aggregate.log    "H2D|D2H|BIDIR <gpus> <aggregate GB/s per direction>"
                                              (no counterpart in the reference)

Energy columns (W, J) are written as 0: power measurement is not built.

    python db_builder.py <db dir> [--gpus N] [--quick]
"""
from __future__ import annotations

import argparse
import math
import sys
import time
from pathlib import Path

VERSION = "b200-1"
# two-sided Student-t 97.5 % quantiles for small sample counts (index = degrees of freedom)
_T975 = [0, 12.706, 4.303, 3.182, 2.776, 2.571, 2.447, 2.365, 2.306, 2.262, 2.228, 2.201, 2.179,
         2.160, 2.145, 2.131, 2.120, 2.110, 2.101, 2.093, 2.086]


def _pkg():
    import importlib.util
    name = "paralia_framework_b200"
    if name in sys.modules:
        return sys.modules[name]
    pkg_dir = Path(__file__).resolve().parent
    spec = importlib.util.spec_from_file_location(name, pkg_dir / "__init__.py",
                                                  submodule_search_locations=[str(pkg_dir)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def sample_until_confident(fn, min_samples=5, max_samples=30, rel=0.05, budget_s=3.0):
    """Repeat fn() (seconds) until the 95 % confidence interval of the mean is within `rel`
    of the mean (the reference's stop rule, dgemm_microbench.cu:155-159) or the budget ends.
    Returns (mean, margin, samples, bench_time)."""
    xs = []
    t0 = time.perf_counter()
    while True:
        xs.append(fn())
        n = len(xs)
        mean = sum(xs) / n
        if n >= 2:
            var = sum((x - mean) ** 2 for x in xs) / (n - 1)
            t = _T975[n - 1] if n - 1 < len(_T975) else 1.96
            margin = t * math.sqrt(var / n)
        else:
            margin = float("inf")
        done = n >= min_samples and margin <= rel * mean
        if done or n >= max_samples or time.perf_counter() - t0 > budget_s:
            return mean, (margin if margin != float("inf") else 0.0), n, time.perf_counter() - t0


def tile_sizes(quick: bool):
    if quick:
        return [512, 1024, 2048, 4096]
    # the reference sweeps 256, 512, ... in steps of 256 for 16 steps, then doubles the step
    out, t, step = [], 256, 256
    while t <= 8192:
        out.append(t)
        if len(out) % 16 == 0:
            step *= 2
        t += step
    return out


_SG_BUFS = {}


def pipeline_tile_sgemm(pl, dev: int, T: int) -> float:
    """Seconds per T x T x T subkernel of a device-resident 2T x 2T x 4T SGEMM run through the
    whole executor with tile edge T."""
    M, N, K = 2 * T, 2 * T, 4 * T
    key = (dev, T)
    if key not in _SG_BUFS:
        for (_d, _t), bufs in list(_SG_BUFS.items()):
            for p in bufs:
                pl.free(p, dev)
            del _SG_BUFS[(_d, _t)]
        bufs = [pl.malloc(M * K * 4, dev), pl.malloc(K * N * 4, dev), pl.malloc(M * N * 4, dev)]
        pl.fill_f32(bufs[0], M * K, 42, 1, dev)
        pl.fill_f32(bufs[1], K * N, 43, 1, dev)
        pl.fill_f32(bufs[2], M * N, 44, 1, dev)
        _SG_BUFS[key] = bufs
        ctl = pl.make_ctl(T=T, units=[dev])
        pl.sgemm("N", "N", M, N, K, 1.0, bufs[0], M, bufs[1], K, 0.0, bufs[2], M,
                 locA=dev, locB=dev, locC=dev, ctl=ctl)          # warm-up: slab, plan
    A, B, Cm = _SG_BUFS[key]
    rep = pl.sgemm("N", "N", M, N, K, 1.0, A, M, B, K, 0.0, Cm, M, locA=dev, locB=dev, locC=dev,
                   ctl=pl.make_ctl(T=T, units=[dev]))
    return rep.device_ms * 1e-3 / 16.0


def build_exec(pl, db: Path, dev: int, quick: bool):
    raw = db / "Benchmark-Results"
    rows = {"Dgemm": [], "Sgemm": []}
    for ta in "NT":
        for tb in "NT":
            lines = []
            for T in tile_sizes(quick):
                # the time of one k tile inside the launches the executor issues: chains of
                # four k tiles per C tile, eight launches over four streams
                mean, err, n, bt = sample_until_confident(
                    lambda: pl.bench_tile_dgemm_chain(dev, ta, tb, T, 4, 8))
                lines.append(f"{T},{T},{T}, {mean:e},0,0,{err:e},{n},{bt:e}")
                rows["Dgemm"].append((ta, tb, T, mean, err, n, bt))
            (raw / f"cublasDgemm_dev-{dev}_TransA-{ta}_TransB-{tb}_{VERSION}.log").write_text(
                "\n".join(lines) + "\n")
    # the FP32 kernel reads packed operands: one curve serves every transpose pair. The tile time
    # is taken the way the executor runs tiles -- pack kernels on their own stream, launches of
    # different C tiles in flight on four streams, one k tile per launch: a device-resident
    # 2T x 2T x 4T product through the library, device time divided by its 16 subkernels.
    lines = []
    for T in tile_sizes(quick):
        mean, err, n, bt = sample_until_confident(lambda: pipeline_tile_sgemm(pl, dev, T), min_samples=3,
                                                  budget_s=2.0)
        lines.append(f"{T},{T},{T}, {mean:e},0,0,{err:e},{n},{bt:e}")
        for ta in "NT":
            for tb in "NT":
                rows["Sgemm"].append((ta, tb, T, mean, err, n, bt))
    for ta in "NT":
        for tb in "NT":
            (raw / f"cublasSgemm_dev-{dev}_TransA-{ta}_TransB-{tb}_{VERSION}.log").write_text(
                "\n".join(lines) + "\n")
    for func, rs in rows.items():
        rs.sort(key=lambda r: (r[0], r[1], r[2]))
        text = "".join(f"{ta},{tb},{T},{T},{T},{m:e},0.000000e+00,0.000000e+00,{e:e},{n},{bt:e}\n"
                       for (ta, tb, T, m, e, n, bt) in rs)
        (db / "Processed" / f"{func}_lookup-table_dev-{dev}.log").write_text(text)


def vector_lengths(quick: bool):
    if quick:
        return [1 << 16, 1 << 18, 1 << 20, 1 << 22, 1 << 24]
    # the reference starts at 4096 with a step of 4096 that doubles every 16 steps
    # (daxpy_microbench.cu:109-111); tiles the executor uses lie between 2^16 and 2^25
    out, n, step = [], 1 << 16, 1 << 16
    while n <= (1 << 25):
        out.append(n)
        if n >= step * 16:
            step *= 2
        n += step
    return out


def build_level1(pl, db: Path, dev: int, quick: bool):
    """Daxpy / Ddot tile tables (daxpy_microbench.cu:26-231, ddot_microbench.cu:26-228)."""
    raw = db / "Benchmark-Results"
    for func, fn in (("Daxpy", pl.bench_tile_daxpy), ("Ddot", pl.bench_tile_ddot)):
        raw_lines, rows = [], []
        for n in vector_lengths(quick):
            mean, err, cnt, bt = sample_until_confident(lambda: fn(dev, n, 8), budget_s=0.5)
            raw_lines.append(f"{n}, {mean:e},0,0,{err:e},{cnt},{bt:e}")
            rows.append(f"{n},{mean:e},0.000000e+00,0.000000e+00,{err:e},{cnt},{bt:e}")
        (raw / f"cublas{func}_dev-{dev}_{VERSION}.log").write_text("\n".join(raw_lines) + "\n")
        (db / "Processed" / f"{func}_lookup-table_dev-{dev}.log").write_text("\n".join(rows) + "\n")


def build_level2(pl, db: Path, dev: int, quick: bool):
    """Dgemv tile tables, one file per transpose as the reference writes them
    (dgemv_microbench.cu:19-24,56-58,127-190): rows ``M,N, mean_t,W,J,margin,samples,bench_t``."""
    raw = db / "Benchmark-Results"
    rows = []
    for trans in ("N", "T"):
        raw_lines = []
        for T in ((4096, 16384) if quick else range(2048, 32768 + 1, 2048)):
            mean, err, cnt, bt = sample_until_confident(lambda: pl.bench_tile_dgemv(dev, trans, T, 8),
                                                        budget_s=0.5)
            raw_lines.append(f"{T},{T}, {mean:e},0,0,{err:e},{cnt},{bt:e}")
            rows.append(f"{trans},{T},{T},{mean:e},0.000000e+00,0.000000e+00,{err:e},{cnt},{bt:e}")
        (raw / f"cublasDgemv_dev-{dev}_TransA-{trans}_{VERSION}.log").write_text("\n".join(raw_lines) + "\n")
    (db / "Processed" / f"Dgemv_lookup-table_dev-{dev}.log").write_text("\n".join(rows) + "\n")


def build_host_aggregate(pl, db: Path, ngpu: int, quick: bool):
    """Aggregate host-link bandwidth against the number of GPUs copying at once."""
    counts = sorted({c for c in (1, 2, 4, 8, ngpu) if c <= ngpu})
    nbytes = (128 if quick else 512) << 20
    lines = []
    for mode, tag in ((0, "H2D"), (1, "D2H"), (2, "BIDIR")):
        for c in counts:
            lines.append(f"{tag} {c} {pl.bench_host_aggregate(c, mode, nbytes, 3):e}")
    (db / "Processed" / "Host-Link-Aggregate.log").write_text("\n".join(lines) + "\n")


def linear_fit(xs, ys):
    """Least squares y = a + b x (LinkPreprocessing.py.in:45-48)."""
    n = len(xs)
    mx, my = sum(xs) / n, sum(ys) / n
    sxx = sum((x - mx) ** 2 for x in xs)
    b = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / sxx if sxx > 0 else 0.0
    return my - b * mx, b


def build_links(pl, db: Path, locs: list[int], quick: bool):
    raw = db / "Benchmark-Results"
    dims = [256, 512, 1024, 2048, 4096] if quick else [256, 512, 1024, 1536, 2048, 3072, 4096, 6144, 8192]
    for d in locs:
        for s in locs:
            if d == s:
                continue
            if d == -1 and s == -1:
                continue
            lines, xs, ys = [], [], []
            for dim in dims:
                mean, err, n, bt = sample_until_confident(lambda: pl.bench_link(d, s, dim, 2), budget_s=1.0)
                lines.append(f"{dim},{dim}, {mean:e},{err:e},{n}, {bt:e}")
                xs.append(dim * dim * 8.0)
                ys.append(mean)
            (raw / f"CuCuBLAS_link_benchmark_loc_dest-{d}_loc_src-{s}_{VERSION}.log").write_text(
                "\n".join(lines) + "\n")
            ti, tb = linear_fit(xs, ys)
            # slowdown of this link by traffic on every other link
            slow, olines = [], []
            for od in locs:
                for os_ in locs:
                    if od == os_ or (od == d and os_ == s) or (od == -1 and os_ == -1):
                        continue
                    # behind NVSwitch every GPU pair has its own path: only host links can
                    # contend, so only pairs of host links are probed
                    if not ((d == -1 or s == -1) and (od == -1 or os_ == -1)):
                        continue
                    t0 = time.perf_counter()
                    ta_, ts_ = pl.bench_link_overlap(d, s, od, os_, 2048 if quick else 4096, 3)
                    olines.append(f"{od},{os_}, {ta_:e},{ts_:e},10, {time.perf_counter() - t0:e}")
                    slow.append((os_, od, ts_ / ta_ if ta_ > 0 else 1.0))
            (raw / f"CuCuBLAS_link_overlap_benchmark_loc_dest-{d}_loc_src-{s}_{VERSION}.log").write_text(
                "\n".join(olines) + "\n")
            text = f"Intercept: {max(ti, 0.0):e}\nCoefficient: {tb:e}\n"
            text += "".join(f"Slowdown([{a}]->[{b}]): {v:e}\n" for (a, b, v) in slow)
            (db / "Processed" / f"Link-Stats_loc_dest-{d}_loc_src-{s}.log").write_text(text)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("db")
    ap.add_argument("--gpus", type=int, default=0, help="GPUs to calibrate links for (0 = all)")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--tables-only", action="store_true",
                    help="measure only the kernel tables of GPU 0 (no links)")
    ap.add_argument("--links-only", action="store_true",
                    help="measure only the links and the host aggregate (the tile tables of "
                         "one GPU serve every identical GPU)")
    a = ap.parse_args(argv)
    pl = _pkg()
    pl.init()
    db = Path(a.db)
    (db / "Benchmark-Results").mkdir(parents=True, exist_ok=True)
    (db / "Processed").mkdir(parents=True, exist_ok=True)
    ngpu = pl.device_count() if a.gpus <= 0 else min(a.gpus, pl.device_count())
    if not a.links_only:
        build_exec(pl, db, 0, a.quick)      # identical GPUs: device 0's curve serves all
        build_level1(pl, db, 0, a.quick)
        build_level2(pl, db, 0, a.quick)
    if not a.tables_only:
        build_links(pl, db, [-1] + list(range(ngpu)), a.quick)
        build_host_aggregate(pl, db, ngpu, a.quick)
    peak = max(pl.bench_dmma_peak(0, s, 20000) for s in (884, 1688, 16816))
    (db / "Processed" / "fp64_tensor_peak_dev-0.log").write_text(f"{peak:e}\n")
    # TF32 tcgen05 issue rate of the SGEMM kernel's MMA shape; the 3xTF32 kernel's roofline
    # is a third of it
    tf32 = max(pl.bench_tf32_peak(0, 20000) for _ in range(3))
    (db / "Processed" / "tf32_tensor_peak_dev-0.log").write_text(f"{tf32:e}\n")
    # the same loop on uniform(-1, 1) operands, run for about a second: what the board's power
    # limit leaves of the issue rate for a real product (the second of two runs is steady)
    tf32_real = [pl.bench_tf32_peak(0, 1500000, random_operands=True) for _ in range(2)][-1]
    (db / "Processed" / "tf32_tensor_peak_random_dev-0.log").write_text(f"{tf32_real:e}\n")
    print(f"database written to {db} ({ngpu} GPU(s))")


if __name__ == "__main__":
    main()
