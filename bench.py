#!/usr/bin/env python
"""Benchmark of the tiled multi-GPU DGEMM hot path (BASELINE config 2).

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One "step" is one square DGEMM M=N=K=32768 (alpha=beta=1, column-major, entries
uniform[-1,1) from fixed seeds) through ``PARALiA_dgemm`` with HOST-resident (pinned)
operands, as the workload is stated: every step streams A, B and C host->device and C
device->host inside the timed region.

* ``value``  -- TFLOP/s = 2*M*N*K / the library's device time of a step (CUDA events from
                the first enqueue to the last write-back, max over the GPUs), whole job;
* ``e2e``    -- the same steps timed around the blocking calls;
* ``hbm_resident`` -- for comparison, the same call with the operands already in HBM;
* ``parity_check`` -- after the timed region, outside it: Freivalds' check of every rank's
                C block against C0 + calls*A*B (the script exits non-zero if it fails);
* ``inproc_e2e``   -- N > 1 only: one process (rank 0) drives all N GPUs through a single
                ``PARALiA_dgemm`` call, the reference's own launch model.

With N > 1 the launch is one process per GPU (torchrun). C is partitioned over the
D1 x D2 device grid exactly as the library partitions it in-process
(Subkernel_distributions.cpp:325-336,399): rank (r, c) computes the C block of tile rows r
and tile columns c from its A row panel and B column panel; the ranks form a library group
so that a host-resident tile crosses the host link once and reaches the other ranks over
NVLink. No data-path collective is needed; the ranks only meet in barriers and in the MAX
of the timings. Total work is fixed, so scaling is "strong".

``--impl reference`` times the reference's CPU implementation of the same routine --
OpenBLAS ``cblas_dgemm`` (the library the reference calls on its CPU path) -- on the host
cores, on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FULL_N = 32768
METRIC = "DGEMM TFLOP/s (device-timed, whole box) at 1/2/4/8 B200 and % of roofline"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--n", type=int, default=FULL_N, help="problem edge (default 32768)")
    ap.add_argument("--tile", type=int, default=0, help="tile edge T (0 = autotuned)")
    ap.add_argument("--no-hbm", action="store_true", help="skip the HBM-resident comparison leg")
    ap.add_argument("--no-inproc", action="store_true",
                    help="N > 1: skip the single-process run over all GPUs on rank 0")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--inproc", action="store_true",
                    help="one process drives all --gpus GPUs through the library (the "
                         "reference's own execution model) instead of one process per GPU")
    return ap.parse_args()


# ------------------------------------------------------------------ clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown",
                                      "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), samples=len(sm))
        out["reasons"] = sorted(reasons)
        return out


# ------------------------------------------------------------------ CPU arm
def _use_all_host_threads() -> int:
    """Launchers set OMP_NUM_THREADS=1 per rank; the CPU arm runs on rank 0 alone and may use
    every core the job has."""
    try:
        cores = len(os.sched_getaffinity(0))
    except Exception:
        cores = os.cpu_count() or 1
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[var] = str(cores)
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=cores)
    except Exception:
        pass
    return cores


def cpu_dgemm_sample(target_s: float = 12.0, repeats: int = 1, warm: int = 0):
    """OpenBLAS cblas_dgemm on all host cores, NN, alpha=beta=1, seeded uniform inputs, on
    the largest square sample of the workload that takes about target_s seconds per call
    (small samples run OpenBLAS well below its large-matrix rate, so the sample is as large
    as the time allows, up to 12288^3). Returns (TFLOP/s, cores, n, seconds per call)."""
    cores = _use_all_host_threads()
    import oracle

    def make(n):
        return (oracle.uniform_f64(n * n, 42).reshape((n, n), order="F"),
                oracle.uniform_f64(n * n, 43).reshape((n, n), order="F"),
                oracle.uniform_f64(n * n, 44).reshape((n, n), order="F"))

    def run(ops):
        t0 = time.perf_counter()
        oracle.openblas_dgemm("N", "N", 1.0, ops[0], ops[1], 1.0, ops[2])
        return time.perf_counter() - t0

    run(make(1024))                 # warm the thread pool
    t = run(make(2048))
    rate = 2.0 * 2048 ** 3 / t      # flop/s estimate
    n = int((rate * target_s / 2.0) ** (1.0 / 3.0)) // 1024 * 1024
    n = max(2048, min(n, 12288))
    ops = make(n)
    for _ in range(warm):
        run(ops)
    t = sum(run(ops) for _ in range(max(repeats, 1))) / max(repeats, 1)
    return 2.0 * n ** 3 / t / 1e12, cores, n, t


def run_reference_arm(args, rank):
    if rank != 0:
        return
    steps, warm = args.steps, args.warmup
    # bounded sample per step, chosen by the same rule as the cpu_baseline leg of the library
    # arm; the per-step budget shrinks with the step count so that the run ends within minutes
    per_step = max(2.0, min(12.0, 90.0 / max(steps + warm, 1)))
    tf, cores, n, dt = cpu_dgemm_sample(per_step, repeats=steps, warm=warm)
    sample = (f"OpenBLAS cblas_dgemm NN alpha=beta=1 on a {n}^3 sample of the {args.n}^3 workload, "
              f"{dt:.2f} s per step, {cores} host threads; OpenBLAS is the routine the reference "
              f"runs on its CPU path")
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": f"DGEMM FP64 NN M=N=K={args.n} alpha=1 beta=1 (BASELINE configs[1])",
                   "sample": f"{n}^3"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm
def freivalds(torch, dA, dB, dC0, dC, calls, K, dev):
    """Randomised check of C = C0 + calls * A*B without forming the product: for two seeded
    vectors x, compare C*x with C0*x + calls * A*(B*x). dA (m x K), dB (K x n), dC0 and dC
    (m x n) are column-major FP64 buffers on the GPU; the matrix-vector products are torch's.
    Returns the larger normwise relative error and the bound 8*K*eps."""
    m, n = dC.numel() // (dB.numel() // K), dB.numel() // K
    A = dA.view(K, m).t()       # column-major m x K seen as a strided torch matrix
    B = dB.view(n, K).t()
    C0 = dC0.view(n, m).t()
    C = dC.view(n, m).t()
    worst = 0.0
    g = torch.Generator(device=dev).manual_seed(2024)
    for kind in range(2):
        if kind == 0:
            x = (torch.randint(0, 2, (n,), generator=g, device=dev, dtype=torch.int64) * 2 - 1).to(torch.float64)
        else:
            x = torch.rand(n, generator=g, device=dev, dtype=torch.float64) * 2 - 1
        want = torch.mv(C0, x) + float(calls) * torch.mv(A, torch.mv(B, x))
        got = torch.mv(C, x)
        err = (torch.linalg.norm(got - want) / torch.linalg.norm(want)).item()
        worst = max(worst, err)
    return worst, 8.0 * K * 2.0 ** -52


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    # one process per GPU: rank i drives GPU i (LOCAL_RANK) and touches no other GPU
    dev = local_rank if world > 1 else 0
    phys = dev
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        try:
            phys = int(visible.split(",")[dev])
        except (ValueError, IndexError):
            phys = dev

    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    pl = entry.load_package()
    pl.lib()   # fails loudly if the CUDA library is missing
    torch.cuda.set_device(dev)
    cuda = f"cuda:{dev}"
    pl.init()
    host_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(cuda))
        # a second, host-side group: ranks that only wait must not keep a kernel on their GPU
        host_group = dist.new_group(backend="gloo")
        # the ranks form a library group: host-resident tiles are shared over NVLink (CUDA IPC)
        token = [f"{os.environ.get('MASTER_PORT', '0')}_{os.getpid()}"]
        dist.broadcast_object_list(token, src=0)
        try:
            pl.group_init(token[0], rank, world, dev)
            joined = 1
        except pl.ParaliaError as exc:      # e.g. no POSIX shared memory in this container
            print(f"rank {rank}: no process group ({exc}); every rank fetches for itself",
                  file=sys.stderr, flush=True)
            joined = 0
        flag = torch.tensor([joined], device=cuda)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        use_group = bool(flag.item())
        if joined and not use_group:
            pl.group_finalize()
    else:
        use_group = False

    import importlib
    ranks = importlib.import_module("paralia_framework_b200.ranks")
    n = args.n
    # rank (r, c) of the D1 x D2 device grid computes its block of C
    (m0, m1), (n0, n1), (r, c), (d1, d2) = ranks.gemm_block(rank, world, n, n, quantum=128)
    Mloc, Nloc, K = m1 - m0, n1 - n0, n
    flops_total = 2.0 * n * n * n
    ctl = pl.make_ctl(T=args.tile, units=[dev])
    if args.inproc:
        assert world == 1, "--inproc is a single-process mode"
        ngpu = min(args.gpus, pl.device_count())
        ctl = pl.make_ctl(T=args.tile, units=list(range(ngpu)))
        d1, d2 = ranks.device_grid(ngpu)

    # ---- operands: generated on the GPU by the counter-based generator (same bits as the
    # host generator); the rank's panels are independent seeded streams
    nA, nB, nC = Mloc * K, K * Nloc, Mloc * Nloc
    dA = torch.empty(nA, dtype=torch.float64, device=cuda)
    dB = torch.empty(nB, dtype=torch.float64, device=cuda)
    dC = torch.empty(nC, dtype=torch.float64, device=cuda)
    seeds = (42 + 1000 * r, 43 + 1000 * c, 44 + 1000 * rank)
    pl.fill_f64(dA, nA, seeds[0], 0, dev)
    pl.fill_f64(dB, nB, seeds[1], 0, dev)
    pl.fill_f64(dC, nC, seeds[2], 0, dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    gemm = pl.group_dgemm if use_group else pl.dgemm

    def run_leg(A, B, C, steps, warm, call=None, call_ctl=None, dims=None):
        call = call or gemm
        call_ctl = call_ctl or ctl
        m, nn = dims or (Mloc, Nloc)
        launches = h2d = d2h = 0
        dev_ms = 0.0
        phases = [0.0, 0.0, 0.0]
        for _ in range(warm):
            call("N", "N", m, nn, K, 1.0, A, m, B, K, 1.0, C, m, ctl=call_ctl)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            rep = call("N", "N", m, nn, K, 1.0, A, m, B, K, 1.0, C, m, ctl=call_ctl)
            launches += rep.kernel_launches
            h2d += rep.h2d_bytes
            d2h += rep.d2h_bytes
            dev_ms += rep.device_ms
            phases = [phases[0] + rep.fill_ms, phases[1] + rep.exec_end_ms, phases[2] + rep.h2d_end_ms]
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1), dev_ms] + phases, dtype=torch.float64, device=cuda)
        cnt = torch.tensor([launches, h2d, d2h], dtype=torch.int64, device=cuda)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.all_reduce(cnt, op=dist.ReduceOp.SUM)
        per = (ms / steps).tolist()
        return {"ms": per[0], "dev_ms": per[1], "fill_ms": per[2], "exec_end_ms": per[3],
                "h2d_end_ms": per[4], "launches": cnt[0].item(), "h2d": cnt[1].item(),
                "d2h": cnt[2].item(), "rep": rep}

    # ---- FP64 tensor-core peak of this GPU, measured now (register-only DMMA loop)
    peak_tf = max(pl.bench_dmma_peak(dev, 1688, 20000), pl.bench_dmma_peak(dev, 16816, 10000))

    # ---- the workload as BASELINE states it: host-resident pinned operands through the
    # public entry point; every step streams A, B and C in and C out inside the timed region
    hA, hB, hC = pl.malloc(nA * 8, -1), pl.malloc(nB * 8, -1), pl.malloc(nC * 8, -1)
    pl.memcpy(hA, -1, dA, dev, nA * 8)
    pl.memcpy(hB, -1, dB, dev, nB * 8)
    pl.memcpy(hC, -1, dC, dev, nC * 8)
    sampler = ClockSampler(phys)
    if rank == 0:
        sampler.start()
    host = run_leg(hA, hB, hC, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else {}
    rep = host["rep"]
    value = flops_total / (host["dev_ms"] * 1e-3) / 1e12
    e2e = {"value": flops_total / (host["ms"] * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": host["h2d"] // args.steps, "d2h_bytes_per_step": host["d2h"] // args.steps,
           "ms_per_step": host["ms"], "gpu_launches": host["launches"]}

    # ---- untimed: is the result of the timed region right? Each rank checks its own block.
    # After the warm-up and timed calls C = C0 + calls * A*B (alpha = beta = 1).
    calls = args.steps + args.warmup
    pl.fill_f64(dC, nC, seeds[2], 0, dev)                 # C0 again, from its seed
    dCres = torch.empty(nC, dtype=torch.float64, device=cuda)
    pl.memcpy(dCres, dev, hC, -1, nC * 8)
    err, bound = freivalds(torch, dA, dB, dC, dCres, calls, K, cuda)
    del dCres
    errs = torch.tensor([err], dtype=torch.float64, device=cuda)
    if world > 1:
        dist.all_reduce(errs, op=dist.ReduceOp.MAX)
    parity = {"check": "Freivalds, two seeded vectors per rank block, C = C0 + calls*A*B",
              "calls": calls, "rel_err": errs.item(), "bound": bound,
              "ok": bool(errs.item() <= bound)}
    for p in (hA, hB, hC):
        pl.free(p, -1)

    # ---- for comparison: the same call with the operands already in HBM (no host traffic)
    hbm = None
    if not args.no_hbm:
        h = run_leg(dA, dB, dC, min(args.steps, 3), 1)
        hbm = {"value": flops_total / (h["dev_ms"] * 1e-3) / 1e12, "unit": "TFLOP/s",
               "ms_per_step": h["ms"], "placement": "operands resident in HBM (location id = the GPU)"}

    tile_sharing = bool(use_group)
    # ---- N > 1: the drop-in call itself -- ONE process driving all N GPUs -- on rank 0,
    # host-resident operands, while the other ranks hold no GPU work (they wait on the host)
    inproc = None
    if world > 1 and not args.no_inproc:
        del dA, dB, dC
        torch.cuda.empty_cache()
        if use_group:
            pl.group_finalize()
            use_group = False
        pl.dev_cache_free(dev)
        torch.cuda.synchronize()
        dist.barrier(group=host_group)
        if rank == 0:
            inproc = run_inproc(pl, torch, args, world, n, freivalds)
        dist.barrier(group=host_group)

    if rank == 0:
        # dominant kernel: the DMMA tile GEMM. Algorithmic flops per launch = 2*m*n*k of the
        # tiles that launch covers; with every launch of a step doing equal work that is
        # flops_total / launches. Launches on the library's execution streams overlap, so
        # the per-launch duration is the device time of the timed region (CUDA events on
        # the library's own streams) divided by the launches in it.
        # GPUs the launches are spread over: the ranks, or the units one process drives
        nu = max(int(ctl.active_unit_num), 1) if args.inproc else world
        launches = host["launches"]
        per_launch_flop = flops_total * args.steps / max(launches, 1)
        per_launch_s = host["dev_ms"] * 1e-3 * args.steps / max(launches / nu, 1)
        achieved = per_launch_flop / per_launch_s / 1e12
        # the path's roofline: the slower of compute at peak and the host-link bytes over the
        # host links of nu GPUs (the calibration database's shared-link model)
        t_compute = flops_total / (nu * peak_tf * 1e12)
        bytes_in, bytes_out = e2e["h2d_bytes_per_step"], e2e["d2h_bytes_per_step"]
        t_in, defer = pl.model_host_link(0, True, bytes_in // nu, nu)
        t_out, _ = pl.model_host_link(0, False, bytes_out // nu, nu)
        t_link = t_in + t_out if defer else max(t_in, t_out)
        t_roof = max(t_compute, t_link)
        cpu = None
        if not args.no_cpu and world == 1:
            tf, cores, ns, ts = cpu_dgemm_sample()
            cpu = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                   "sample": (f"OpenBLAS cblas_dgemm (the routine the reference runs on its CPU "
                              f"path) NN alpha=beta=1 on a {ns}^3 sample of the workload, "
                              f"{ts:.1f} s, {cores} threads")}
        per_step_launches = max(launches // max(args.steps, 1), 1)
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s",
            "n_gpus": nu,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": host["ms"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f64", "data": "synthetic",
            "config": {
                "workload": f"DGEMM FP64 NN M=N=K={n} alpha=1 beta=1, column-major, operands "
                            f"host-resident (pinned), C written back to the host (BASELINE configs[1])",
                "tile": int(rep.T), "device_grid": [d1, d2],
                "per_rank_block": [Mloc, Nloc, K],
                "l2": "operands (>= 3 GiB per GPU) are far larger than the 126 MB L2",
                "value_timing": "library device time: CUDA events from the first enqueue to the "
                                "last write-back, max over the GPUs, summed over the steps",
                "e2e_timing": "CUDA events around the blocking calls of the timed region",
                "launch": "inproc" if args.inproc else "one process per GPU",
                "tile_sharing_between_ranks": tile_sharing,
            },
            "roofline": {
                "bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                "frac": achieved / peak_tf if peak_tf else None,
                # DRAM bytes per launch: algorithmic bytes of an average launch = (one A and one
                # B tile read per (mi, ni, ki) step, plus one C tile read and written per launch,
                # summed over the step's launches on all GPUs) / launches per step,
                # times the 2.03 ratio of measured to algorithmic bytes from the ncu capture
                # of the same kernel on a small case
                "traffic": 2.03 * 8.0 * (2.0 * float(n) ** 3 / max(rep.T, 1)
                                         + 2.0 * float(rep.T) ** 2 * per_step_launches) / per_step_launches,
                "traffic_source": "algorithmic bytes x 2.03 (ncu dram__bytes of this kernel on "
                                  "4096-wide tiles with 4096-deep k parts, "
                                  "profiles/dgemm_tile_kernel_T4096_ncu_full.md)",
                "peak_source": "FP64 DMMA register-loop microbenchmark run in this process "
                               "(MEASURED_PEAKS.json holds no FP64 figure)",
                "kernel": "dgemm_tile_kernel", "launches": launches,
            },
            "path_roofline": {
                "t_compute_s": t_compute, "t_host_link_s": t_link, "t_roof_s": t_roof,
                "t_measured_s": host["dev_ms"] * 1e-3, "frac": t_roof / (host["dev_ms"] * 1e-3),
                "host_link_model": "calibration database: aggregate host bandwidth with n GPUs "
                                   "active; write-backs after the inputs" if defer else
                                   "calibration database: aggregate host bandwidth with n GPUs active",
            },
            "phases_ms": {"fill": host["fill_ms"], "last_kernel_end": host["exec_end_ms"],
                          "h2d_end": host["h2d_end_ms"], "device": host["dev_ms"],
                          "drain": host["dev_ms"] - host["exec_end_ms"]},
            "parity_check": parity,
            "cpu_baseline": cpu,
            "e2e": e2e,
            "hbm_resident": hbm,
            "inproc_e2e": inproc,
            "gpu_launches": launches,
            "clocks": clocks,
            "library_device_ms_per_step": host["dev_ms"],
        }
        print(json.dumps(line), flush=True)
    ok = parity["ok"] and (inproc is None or inproc.get("parity_check", {}).get("ok", True))
    if world > 1:
        if use_group:
            pl.group_finalize()
        dist.destroy_process_group()
    if not ok:
        sys.exit(3)


def run_inproc(pl, torch, args, ngpu, n, check):
    """One PARALiA_dgemm call driving `ngpu` GPUs from this process (the reference's own
    launch model), host-resident pinned operands; returns the e2e record."""
    nn = n * n
    cuda = "cuda:0"
    dA = torch.empty(nn, dtype=torch.float64, device=cuda)
    dB = torch.empty(nn, dtype=torch.float64, device=cuda)
    dC0 = torch.empty(nn, dtype=torch.float64, device=cuda)
    hA, hB, hC = pl.malloc(nn * 8, -1), pl.malloc(nn * 8, -1), pl.malloc(nn * 8, -1)
    for (d, h, seed) in ((dA, hA, 42), (dB, hB, 43), (dC0, hC, 44)):
        pl.fill_f64(d, nn, seed, 0, 0)
        pl.memcpy(h, -1, d, 0, nn * 8)
    ctl = pl.make_ctl(T=args.tile, units=list(range(ngpu)))
    steps, warm = min(args.steps, 3), 2
    for _ in range(warm):
        pl.dgemm("N", "N", n, n, n, 1.0, hA, n, hB, n, 1.0, hC, n, ctl=ctl)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    dev_ms = 0.0
    launches = h2d = d2h = 0
    for _ in range(steps):
        rep = pl.dgemm("N", "N", n, n, n, 1.0, hA, n, hB, n, 1.0, hC, n, ctl=ctl)
        dev_ms += rep.device_ms
        launches += rep.kernel_launches
        h2d += rep.h2d_bytes
        d2h += rep.d2h_bytes
    wall = (time.perf_counter() - t0) / steps
    flops = 2.0 * n ** 3
    dC = torch.empty(nn, dtype=torch.float64, device=cuda)
    pl.memcpy(dC, 0, hC, -1, nn * 8)
    err, bound = check(torch, dA, dB, dC0, dC, steps + warm, n, cuda)
    for p in (hA, hB, hC):
        pl.free(p, -1)
    return {"value": flops / wall / 1e12, "unit": "TFLOP/s", "ms_per_step": wall * 1e3,
            "device_value": flops / (dev_ms / steps * 1e-3) / 1e12, "steps": steps, "warmup": warm,
            "tile": int(rep.T), "device_grid": [rep.grid_d1, rep.grid_d2],
            "h2d_bytes_per_step": h2d // steps, "d2h_bytes_per_step": d2h // steps,
            "gpu_launches": launches, "p2p_bytes_per_step": int(rep.p2p_bytes),
            "last_call_ms": {"host": rep.host_ms, "device": rep.device_ms, "plan": rep.plan_ms,
                             "pin": rep.pin_ms, "alloc": rep.alloc_ms},
            "phases_ms": {"fill": rep.fill_ms, "last_kernel_end": rep.exec_end_ms,
                          "h2d_end": rep.h2d_end_ms, "device": rep.device_ms},
            "timing": "wall clock around the blocking calls (one process drives all GPUs)",
            "parity_check": {"rel_err": err, "bound": bound, "ok": bool(err <= bound)}}


if __name__ == "__main__":
    main()
