"""Operand-placement sweep for the level-3 routines: the evaluation matrix of the reference
(``Benchmarking/Full_performance_evaluation.in:37-163``) driven through ``runner.py``.

Ten placement scenarios (where A, B and C live: pinned host = -1, or a GPU id) times three
shape families (mid-sized squares; thin K = MN/{2,8,32}; fat K = {2,8,32}*MN), each problem run
twice: unit set chosen by the autotuner, and all GPUs forced (the reference's ``8 11111111``).
alpha = 1.2345, beta = 1.1154 as in the reference's script. Every timed call appends one row in
the reference's log schema (``Benchmarking/CuCuBLAS/src/testing.cpp:420-428``) to ``--log``, so
the reference's plot scripts can read it; the summary printed at the end compares the
autotuner's predicted time with the measured one (the role of the reference's
``Benchmarking/Full_model_validation.in``).

The reference's scenarios name GPUs 0..7. On a box with fewer GPUs an id is folded with
``id % gpus`` (the scenario keeps its shape: operands on distinct GPUs stay distinct while
enough GPUs exist).

    python sweep.py --routine dgemm --log sweep.csv                 # the full matrix
    python sweep.py --quick --scenarios Full_offload,Device_only_offload_mixed1
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
import runner  # noqa: E402

ALPHA, BETA = 1.2345, 1.1154

# scenario -> (locA, locB, locC), Full_performance_evaluation.in:39-91
SCENARIOS = {
    "Full_offload": (-1, -1, -1),
    "Partial_offload_result": (0, 0, -1),
    "Partial_offload_result_mixed_in": (4, 2, -1),
    "Partial_offload_in": (-1, -1, 0),
    "Partial_offload_mixed": (-1, 0, 5),
    "Device_only_offload": (0, 0, 0),
    "Device_only_offload_mixed1": (0, 1, 2),
    "Device_only_offload_mixed2": (0, 3, 6),
    "Device_only_offload_mixed3": (4, 2, 5),
    "Device_only_offload_mixed4": (1, 6, 7),
}


class BufferPool:
    """Stand-in for the package inside a sweep: operand buffers are kept and handed out again
    instead of being allocated and page-locked anew for every problem (a pinned allocation of
    a few GiB costs more than most of the problems it would serve)."""

    def __init__(self, pl):
        self._pl = pl
        self._free: dict[int, list[tuple[int, int]]] = {}   # loc -> [(bytes, ptr)]
        self._size: dict[tuple[int, int], int] = {}          # (loc, ptr) -> bytes

    def __getattr__(self, name):
        return getattr(self._pl, name)

    def malloc(self, nbytes: int, loc: int) -> int:
        lst = self._free.setdefault(loc, [])
        best = None
        for i, (b, _p) in enumerate(lst):
            if b >= nbytes and (best is None or b < lst[best][0]):
                best = i
        if best is not None:
            return lst.pop(best)[1]
        ptr = self._pl.malloc(nbytes, loc)
        self._size[(loc, ptr)] = nbytes
        return ptr

    def free(self, ptr: int, loc: int) -> None:
        self._free.setdefault(loc, []).append((self._size[(loc, ptr)], ptr))

    def release(self) -> None:
        for loc, lst in self._free.items():
            for (_b, ptr) in lst:
                self._pl.free(ptr, loc)
                self._size.pop((loc, ptr), None)
        self._free.clear()


def fold(loc: int, gpus: int) -> int:
    return loc if loc < 0 else loc % gpus


def shapes(family: str, quick: bool) -> list[tuple[int, int, int]]:
    """(M, N, K) lists of the reference's three families (Full_performance_evaluation.in:94,
    136-162); ``quick`` keeps three members of each."""
    out = []
    if family == "square":
        dims = (4096, 8192, 16384) if quick else range(2048, 22528 + 1, 1024)
        out = [(d, d, d) for d in dims]
    elif family == "thin":           # K < M = N
        mns = (8192, 16384) if quick else range(8192, 32768 + 1, 4096)
        ratios = (8,) if quick else (2, 8, 32)
        out = [(mn, mn, mn // r) for r in ratios for mn in mns]
    elif family == "fat":            # K > M = N
        ks = (16384, 32768) if quick else range(12288, 36864 + 1, 4096)
        ratios = (8,) if quick else (2, 8, 32)
        out = [(k // r, k // r, k) for r in ratios for k in ks]
    else:
        raise SystemExit(f"unknown family {family!r}")
    return out


def main(argv=None) -> list[dict]:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--routine", choices=["dgemm", "sgemm"], default="dgemm")
    ap.add_argument("--scenarios", default="all", help="comma-separated names, or 'all'")
    ap.add_argument("--families", default="square,thin,fat")
    ap.add_argument("--quick", action="store_true", help="three shapes per family")
    ap.add_argument("--units", default="auto,all", help="'auto' (autotuned set), 'all' (every GPU), or both")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--log", default="", help="CSV rows in the reference's schema are appended here")
    ap.add_argument("--summary", default="", help="write the per-problem summary as JSON lines here")
    a = ap.parse_args(argv)

    pl = runner._pkg()
    pl.init()
    gpus = pl.device_count()
    pl = BufferPool(pl)
    names = list(SCENARIOS) if a.scenarios == "all" else a.scenarios.split(",")
    results = []
    for name in names:
        if name not in SCENARIOS:
            raise SystemExit(f"unknown scenario {name!r}; known: {', '.join(SCENARIOS)}")
        la, lb, lc = (fold(v, gpus) for v in SCENARIOS[name])
        for fam in a.families.split(","):
            for (M, N, K) in shapes(fam, a.quick):
                for mode in a.units.split(","):
                    ns = argparse.Namespace(
                        active_unit_num=-1 if mode == "auto" else gpus,
                        dev_ids="0" if mode == "auto" else "1" * gpus, T=-1, cache_limit=-1,
                        TransA="N", TransB="N", alpha=ALPHA, beta=BETA, M=M, N=N, K=K,
                        locA=la, locB=lb, locC=lc, outloc=lc, log=a.log, iters=a.iters,
                        warmup=a.warmup, validate=False)
                    r = runner.run_level3(pl, ns, a.routine)
                    row = {"scenario": name, "family": fam, "units": mode, "M": M, "N": N, "K": K,
                           "loc": [la, lb, lc], "control": r["control"], "t_avg": r["avg_s"],
                           "t_min": r["min_s"], "pred_t": r["pred_t"], "tflops": r["tflops_avg"],
                           "pred_over_measured": r["pred_t"] / r["avg_s"] if r["avg_s"] > 0 else None}
                    results.append(row)
                    print(json.dumps(row), flush=True)
                    if a.summary:
                        with open(a.summary, "a") as f:
                            f.write(json.dumps(row) + "\n")
    pl.release()
    ratios = [r["pred_over_measured"] for r in results if r["pred_over_measured"]]
    if ratios:
        errs = [abs(x - 1.0) for x in ratios]
        tf = [r["tflops"] for r in results if r["tflops"] > 0]
        # mean and harmonic mean of the rates: the two statistics the reference's evaluation reports
        print(json.dumps({"problems": len(results), "gpus": gpus,
                          "tflops_mean": statistics.fmean(tf), "tflops_harmonic_mean": statistics.harmonic_mean(tf),
                          "pred_over_measured_median": statistics.median(ratios),
                          "abs_rel_error_median": statistics.median(errs),
                          "abs_rel_error_max": max(errs)}))
    return results


if __name__ == "__main__":
    main()
