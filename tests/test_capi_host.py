"""Host-side checks of libparalia.so that need no GPU: the library loads, exports every
symbol the header declares, and its planner (tile score, tile choice, 2D block
distribution, autotune with a fixed unit list) agrees with the oracle and with the
reference's own distribution output."""
import json
import re
import subprocess

import pytest


def test_header_symbols_exported(pl):
    header = (pl.PKG_DIR.parent / "include" / "paralia_c.h").read_text()
    declared = set(re.findall(r"\b(PARALiA_\w+)\s*\(", header))
    assert len(declared) >= 25
    assert declared == set(pl.SIGNATURES), declared ^ set(pl.SIGNATURES)
    out = subprocess.run(["nm", "-D", "--defined-only", str(pl.LIB_PATH)], check=True,
                         capture_output=True, text=True).stdout
    exported = set(re.findall(r" T (PARALiA_\w+)", out))
    assert declared <= exported, declared - exported
    handle = pl.lib()
    for name in declared:
        assert getattr(handle, name) is not None


def test_cpp_compat_symbols_exported(pl):
    out = subprocess.run(["nm", "-D", "-C", "--defined-only", str(pl.LIB_PATH)], check=True,
                         capture_output=True, text=True).stdout
    for name in ("PARALiADgemm(", "PARALiADgemmControled(", "PARALiASgemm(", "PARALiADaxpy(",
                 "PARALiADdot(", "PARALiADdotControled(", "PARALiADevCacheFree(short)",
                 "ATC::print_csv()"):
        assert name in out, name


def test_struct_layout_matches_header(pl):
    # compile a tiny C program against the header and compare sizeof with ctypes
    import ctypes, tempfile, os
    src = ('#include <stdio.h>\n#include "paralia_c.h"\n'
           'int main(){printf("%zu %zu\\n", sizeof(paralia_ctl), sizeof(paralia_report));return 0;}\n')
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "t.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "t")
        subprocess.run(["/usr/bin/gcc", "-I", str(pl.PKG_DIR.parent / "include"), c, "-o", exe],
                       check=True)
        a, b = map(int, subprocess.run([exe], check=True, capture_output=True,
                                       text=True).stdout.split())
    assert ctypes.sizeof(pl.Ctl) == a
    assert ctypes.sizeof(pl.Report) == b


@pytest.mark.parametrize("dims", [(32768, 32768, 32768), (4096, 4096, 4096), (65536, 65536, 2048),
                                  (289, 353, 307), (8192, 1024, 4096), (19457, 19457, 19457)])
@pytest.mark.parametrize("units", [1, 2, 4, 8])
def test_tile_slowdowns_match_oracle(pl, orc, dims, units):
    M, N, K = dims
    for T in (128, 256, 1024, 2048, 2816, 4096, 6144, min(dims)):
        if T > min(dims):
            continue
        got = pl.tile_slowdowns(M, N, K, T, units)
        want = orc.tile_slowdowns(M, N, K, T, units)
        assert got == want, (T, got, want)


def test_distribution_matches_reference_golden(pl, golden_dir):
    cases = json.loads((golden_dir / "distribution_ref.json").read_text())["cases"]
    for c in cases:
        owner, d1, d2 = pl.distribute_2d(c["units"], c["Mt"], c["Nt"], c["Kt"])
        assert owner == c["owner"], (c["units"], c["Mt"], c["Nt"], c["Kt"])
        assert d1 * d2 == c["units"]


def test_distribution_matches_oracle_large(pl, orc):
    for units, Mt, Nt, Kt in [(8, 16, 16, 16), (8, 32, 32, 1), (4, 10, 10, 3), (6, 13, 7, 2)]:
        owner, d1, d2 = pl.distribute_2d(units, Mt, Nt, Kt)
        active, want, od1, od2 = orc.distribute_2d(units, Mt, Nt, Kt)
        assert owner == want and (d1, d2) == (od1, od2)
        # every k of a C tile on the same unit
        for ct in range(Mt * Nt):
            assert len(set(owner[ct * Kt:(ct + 1) * Kt])) == 1


def test_autotune_fixed_units_no_gpu(pl, orc):
    # the model alone, with a caller-fixed unit list: no GPU is touched
    ctl = pl.make_ctl(units=list(range(8)))
    rep = pl.autotune_gemm(8, "N", "N", 32768, 32768, 32768, -1, -1, -1, ctl)
    assert rep.T in (2048, 4096)
    # the reference's tile score of the chosen tile is still reported (Autotuner.cpp:571-603)
    assert list(rep.T_slowdowns) == orc.tile_slowdowns(32768, 32768, 32768, rep.T, 8)
    assert rep.active_unit_num == 8 and (rep.grid_d1, rep.grid_d2) == (2, 4)
    nt = 32768 // rep.T
    assert rep.subkernel_num == nt ** 3
    assert list(rep.subkernels_per_unit[:8]) == [nt ** 3 // 8] * 8
    assert rep.pred_t > 0
    # a caller-fixed T is kept
    rep = pl.autotune_gemm(8, "N", "N", 32768, 32768, 32768, -1, -1, -1,
                           pl.make_ctl(T=4096, units=[0, 1]))
    assert rep.T == 4096 and rep.active_unit_num == 2


@pytest.mark.parametrize("esz,dims,locs,units", [
    (8, (32768, 32768, 32768), (-1, -1, -1), 1), (8, (32768, 32768, 32768), (-1, -1, -1), 8),
    (8, (32768, 32768, 32768), (-1, -1, -1), 4), (8, (4096, 4096, 4096), (-1, -1, -1), 1),
    (8, (65536, 65536, 2048), (0, 1, -1), 2), (4, (40960, 40960, 40960), (-1, -1, -1), 8),
    (8, (8192, 8192, 8192), (0, 0, 0), 1), (8, (1156, 1412, 1228), (-1, -1, -1), 3),
])
def test_tile_is_the_argmin_of_the_predicted_time(pl, esz, dims, locs, units):
    # the tile edge is chosen by the model: no forced tile size predicts a shorter time
    M, N, K = dims
    us = list(range(units))
    chosen = pl.autotune_gemm(esz, "N", "N", M, N, K, *locs, pl.make_ctl(units=us))
    assert chosen.T % 16 == 0 or chosen.T == min(dims)
    for T in (256, 512, 1024, 2048, 3072, 4096, 5120, 8192):
        if T > min(dims):
            continue
        forced = pl.autotune_gemm(esz, "N", "N", M, N, K, *locs, pl.make_ctl(T=T, units=us))
        assert chosen.pred_t <= forced.pred_t * (1 + 1e-9), (T, chosen.T, chosen.pred_t, forced.pred_t)


def test_beta_zero_flag_drops_the_fetch_of_c(pl):
    # write-back-bound shape of BASELINE configs[2]: with beta == 0 C crosses the host link once
    args = (8, "T", "N", 65536, 65536, 2048, 0, 1, -1)
    with_c = pl.autotune_gemm(*args, pl.make_ctl(T=2048, units=[0, 1]))
    without = pl.autotune_gemm(*args, pl.make_ctl(T=2048, units=[0, 1], flags=pl.FLAG_BETA_ZERO))
    assert without.pred_t < 0.75 * with_c.pred_t


def _write_db(tmp_path, links, aggregate=None):
    proc = tmp_path / "Processed"
    proc.mkdir(parents=True, exist_ok=True)
    for (dst, src), (ti, tb, slow) in links.items():
        text = f"Intercept: {ti:e}\nCoefficient: {tb:e}\n"
        text += "".join(f"Slowdown([{s}]->[{d}]): {r:e}\n" for (d, s, r) in slow)
        (proc / f"Link-Stats_loc_dest-{dst}_loc_src-{src}.log").write_text(text)
    if aggregate is not None:
        (proc / "Host-Link-Aggregate.log").write_text(
            "".join(f"{k} {n} {v:e}\n" for (k, n, v) in aggregate))
    return str(tmp_path)


def test_shared_host_link_model(pl, tmp_path):
    # reference: Slowdown lines CoModel.cpp:32-55, shared prediction CoModel.cpp:120-140
    tb = 1.0 / 50e9
    links = {
        (0, -1): (0.0, tb, [(1, -1, 1.6), (-1, 0, 1.25), (2, -1, 1.02), (3, -1, 3.0)]),
        (1, -1): (0.0, tb, []), (2, -1): (0.0, tb, []), (3, -1): (0.0, tb, []),
        (-1, 0): (0.0, tb, []),
    }
    agg = [("H2D", 1, 50.0), ("H2D", 2, 100.0), ("H2D", 4, 120.0), ("D2H", 1, 50.0), ("D2H", 4, 120.0),
           ("BIDIR", 1, 45.0), ("BIDIR", 2, 90.0), ("BIDIR", 4, 50.0)]
    try:
        pl.load_database(_write_db(tmp_path, links, agg))
        gb = 10 ** 9
        alone, _ = pl.model_host_link(0, True, gb, 1)
        assert alone == pytest.approx(1 / 50.0)
        # a busy partner link slows this one by its measured ratio
        t, _ = pl.model_host_link(0, True, gb, 2, active_devs=[0, 1])
        assert t == pytest.approx(1.6 / 50.0)
        # ratios within 5 % of 1 are dropped; ratios above 2 are clamped to 2
        t, _ = pl.model_host_link(0, True, gb, 2, active_devs=[0, 2])
        assert t == pytest.approx(1 / 50.0)
        t, _ = pl.model_host_link(0, True, gb, 2, active_devs=[0, 3])
        assert t == pytest.approx(2.0 / 50.0)
        # the opposite direction of the same GPU counts only when it is busy
        t, _ = pl.model_host_link(0, True, gb, 1, both_directions=True, active_devs=[0])
        assert t == pytest.approx(max(1.25 / 50.0, 1 / 45.0))
        # the aggregate caps what four GPUs get together: 120 / 4 = 30 GB/s each
        t, defer4 = pl.model_host_link(2, True, gb, 4, active_devs=[0, 1, 2, 3])
        assert t == pytest.approx(1 / 30.0)
        # three GPUs: between the measured points 2 -> 100 and 4 -> 120
        t, _ = pl.model_host_link(2, True, gb, 3, active_devs=[1, 2, 3])
        assert t == pytest.approx(3 / 110.0)
        # write-backs are deferred where both directions together deliver less than one
        # after the other: 2 x 50 < 0.92 x 120 at four GPUs, 2 x 90 > 100 at two
        _, defer2 = pl.model_host_link(0, True, gb, 2)
        assert defer4 is True and defer2 is False
    finally:
        pl.load_database(str(pl.DEFAULT_DB))


def test_level1_model_picks_units_and_tile(pl):
    n = 1 << 30
    # host-resident vectors: every GPU brings its own host link, so all of them are used
    rep = pl.autotune_vec(False, n, -1, -1, pl.make_ctl(units=list(range(8))))
    assert rep.active_unit_num == 8 and (1 << 16) <= rep.T <= (1 << 25) and rep.pred_t > 0
    one = pl.autotune_vec(False, n, -1, -1, pl.make_ctl(units=[0]))
    assert rep.pred_t < one.pred_t
    # a caller-fixed tile length is kept; DDOT moves less than DAXPY
    dot = pl.autotune_vec(True, n, -1, -1, pl.make_ctl(T=1 << 22, units=[0]))
    axpy = pl.autotune_vec(False, n, -1, -1, pl.make_ctl(T=1 << 22, units=[0]))
    assert dot.T == 1 << 22 and dot.pred_t < axpy.pred_t
    # device-resident: HBM-bound, about 24 B x 2^30 / 6.3 TB/s
    dev = pl.autotune_vec(False, n, 0, 0, pl.make_ctl(units=[0]))
    assert 0.003 < dev.pred_t < 0.006


def test_autotune_more_units_predicts_faster(pl):
    t = []
    for n in (1, 2, 4, 8):
        rep = pl.autotune_gemm(8, "N", "N", 32768, 32768, 32768, -1, -1, -1,
                               pl.make_ctl(units=list(range(n))))
        t.append(rep.pred_t)
    assert t[0] > t[1] > t[2] > t[3]


def test_invalid_arguments_report_status(pl):
    with pytest.raises(pl.ParaliaError) as e:
        pl.tile_slowdowns(0, 1, 1, 1, 1)
    assert e.value.code == pl.ERR_INVALID_ARG
    with pytest.raises(pl.ParaliaError) as e:
        pl.autotune_gemm(3, "N", "N", 8, 8, 8, -1, -1, -1, pl.make_ctl(units=[0]))
    assert e.value.code == pl.ERR_INVALID_ARG
    with pytest.raises(pl.ParaliaError) as e:
        pl.autotune_gemm(8, "X", "N", 8, 8, 8, -1, -1, -1, pl.make_ctl(units=[0]))
    assert e.value.code == pl.ERR_INVALID_ARG
    with pytest.raises(pl.ParaliaError) as e:
        pl.autotune_gemm(8, "N", "N", 8, 8, 8, -1, -1, -1, pl.make_ctl(units=[0, 0]))
    assert e.value.code == pl.ERR_INVALID_ARG


def test_missing_library_fails_loudly(pl, monkeypatch, tmp_path):
    monkeypatch.setattr(pl, "_lib", None)
    monkeypatch.setattr(pl, "LIB_PATH", tmp_path / "absent.so")
    with pytest.raises(pl.LibraryMissing):
        pl.lib()


def test_database_round_trip(pl, tmp_path):
    """Files in the reference's processed formats (GPUexec_lookup.cpp:79-81,
    CoModel.cpp:26-38) drive the model: exec time from the lookup table, link time from
    intercept + coefficient * bytes."""
    proc = tmp_path / "Processed"
    proc.mkdir()
    rate = 30e12
    rows = "".join(f"N,N,{T},{T},{T},{2.0 * T ** 3 / rate:e},0,0,0,10,1\n" for T in (1024, 2048, 4096))
    (proc / "Dgemm_lookup-table_dev-0.log").write_text(rows)
    for g in range(8):
        for (d, s) in ((g, -1), (-1, g)):
            (proc / f"Link-Stats_loc_dest-{d}_loc_src-{s}.log").write_text(
                "Intercept: 1.000000e-05\nCoefficient: 2.000000e-11\nSlowdown([0]->[1]): 1.000000e+00\n")
    # no aggregate cap in this database: the link files alone decide
    (proc / "Host-Link-Aggregate.log").write_text(
        "".join(f"{k} {n} 1.0e+06\n" for k in ("H2D", "D2H", "BIDIR") for n in (1, 8)))
    pl.load_database(str(tmp_path))
    try:
        auto = pl.autotune_gemm(8, "N", "N", 32768, 32768, 32768, -1, -1, -1,
                                pl.make_ctl(units=list(range(8))))
        # the same rate at every tile size: fill and drain favour small tiles, the host's cost
        # per enqueued launch and copy favours large ones; the arg-min lies in between
        assert 1024 < auto.T < 8192
        rep = pl.autotune_gemm(8, "N", "N", 32768, 32768, 32768, -1, -1, -1,
                               pl.make_ctl(T=1024, units=list(range(8))))
        assert rep.T == 1024 and (rep.grid_d1, rep.grid_d2) == (2, 4)
        assert auto.pred_t < rep.pred_t
        # host side of the call: a fixed part and 2.8 us per launch or tile copy. 32 x 32 C tiles
        # with 1 + 8 launches each; every A tile goes to the 4 GPUs of a grid row, every B tile
        # to the 2 GPUs of a grid column, every C tile in and out
        t_host = 0.5e-3 + 2.8e-6 * (1024 * 9 + 32 * 32 * 4 + 32 * 32 * 2 + 2 * 1024)
        tile = 1024 * 1024 * 8
        t_exec = (16384 / 1024) * (8192 / 1024) * 32 * (2.0 * 1024 ** 3 / rate)
        # per GPU: a quarter of its A row panel, half of its B column panel, its C block
        t_recv = 1e-5 + 2e-11 * 3 * 2 ** 30
        assert t_exec > t_recv
        # what overlap cannot hide: the first host tile in (A and B come over different host
        # links on a 2 x 4 grid) and its GPU -> GPU forward, the last band's two C tiles out
        t_fill = (1e-5 + 2e-11 * tile) + (10e-6 + tile / 700e9)
        t_drain = 1e-5 + 2e-11 * 2 * tile
        assert rep.pred_t == pytest.approx(t_fill + t_exec + t_drain + t_host, rel=1e-6)
        # a slow host link makes the same problem link-bound
        for g in range(8):
            (proc / f"Link-Stats_loc_dest-{g}_loc_src--1.log").write_text(
                "Intercept: 1.000000e-05\nCoefficient: 1.000000e-09\n")
        pl.load_database(str(tmp_path))
        rep2 = pl.autotune_gemm(8, "N", "N", 32768, 32768, 32768, -1, -1, -1,
                                pl.make_ctl(T=1024, units=list(range(8))))
        assert rep2.T == 1024
        t_recv2 = 1e-5 + 1e-9 * 3 * 2 ** 30
        t_fill2 = (1e-5 + 1e-9 * tile) + (10e-6 + tile / 700e9)
        assert rep2.pred_t == pytest.approx(t_recv2 + t_fill2 + t_host, rel=1e-6)
    finally:
        with pytest.raises(pl.ParaliaError):
            pl.load_database(str(tmp_path / "nowhere"))   # DB missing -> status, state kept


def test_runner_mask_parsing(pl):
    import importlib
    runner = importlib.import_module("paralia_framework_b200.runner")
    assert runner.parse_mask(2, "0101") == [0, 2]        # the reference's example
    assert runner.parse_mask(-1, "0") is None
    assert runner.parse_mask(8, "11111111") == list(range(8))
    with pytest.raises(SystemExit):
        runner.parse_mask(2, "0111")


def test_packaged_database_loads_and_fills_unmeasured_links(pl):
    # the database measured on one GPU serves every GPU of the box (identical links)
    pl.load_database(str(pl.DEFAULT_DB))
    t1 = pl.autotune_gemm(8, "N", "N", 32768, 32768, 32768, -1, -1, -1, pl.make_ctl(units=[0])).pred_t
    t8 = pl.autotune_gemm(8, "N", "N", 32768, 32768, 32768, -1, -1, -1,
                          pl.make_ctl(units=list(range(8)))).pred_t
    # measured: 2.0 s on one GPU, 0.25 s of compute on eight
    assert 1.8 < t1 < 2.3
    assert 0.22 < t8 < 0.33


def test_packaged_database_is_complete_for_an_eight_gpu_box(pl):
    """The shipped calibration database holds what the autotuner reads: tile tables of the four
    routines, both tensor peaks, the host aggregate table and a link file for every ordered
    pair of the nine locations (host and eight GPUs), each with its two model lines."""
    proc = pl.DEFAULT_DB / "Processed"
    for routine in ("Dgemm", "Sgemm", "Daxpy", "Ddot"):
        rows = (proc / f"{routine}_lookup-table_dev-0.log").read_text().strip().splitlines()
        assert len(rows) >= 20, routine
    fp64 = float((proc / "fp64_tensor_peak_dev-0.log").read_text())
    tf32 = float((proc / "tf32_tensor_peak_dev-0.log").read_text())
    assert 30.0 < fp64 < 45.0            # TFLOP/s, DMMA register loop
    assert 900.0 < tf32 < 1300.0         # TFLOP/s, tcgen05 kind::tf32 issue rate
    tf32_real = float((proc / "tf32_tensor_peak_random_dev-0.log").read_text())
    assert 600.0 < tf32_real <= tf32     # the same loop on random operands, under the power limit
    agg = (proc / "Host-Link-Aggregate.log").read_text().split()
    assert {"H2D", "D2H", "BIDIR"} <= set(agg)
    locs = [-1] + list(range(8))
    for dst in locs:
        for src in locs:
            if dst == src:
                continue
            text = (proc / f"Link-Stats_loc_dest-{dst}_loc_src-{src}.log").read_text()
            assert "Intercept" in text and "Coefficient" in text, (dst, src)


def test_sweep_matrix_is_the_reference_evaluation_matrix(pl):
    # Benchmarking/Full_performance_evaluation.in: 10 placement scenarios; squares
    # 2048..22528 step 1024; thin K = MN/{2,8,32} for MN 8192..32768 step 4096; fat K
    # 12288..36864 step 4096 with MN = K/{2,8,32}
    import importlib
    sweep = importlib.import_module("paralia_framework_b200.sweep")
    assert len(sweep.SCENARIOS) == 10
    assert sweep.SCENARIOS["Full_offload"] == (-1, -1, -1)
    assert sweep.SCENARIOS["Partial_offload_mixed"] == (-1, 0, 5)
    assert sweep.SCENARIOS["Device_only_offload_mixed4"] == (1, 6, 7)
    sq = sweep.shapes("square", False)
    assert len(sq) == 21 and sq[0] == (2048,) * 3 and sq[-1] == (22528,) * 3
    thin = sweep.shapes("thin", False)
    assert len(thin) == 21 and (8192, 8192, 4096) in thin and (32768, 32768, 1024) in thin
    fat = sweep.shapes("fat", False)
    assert len(fat) == 21 and (6144, 6144, 12288) in fat and (1152, 1152, 36864) in fat
    assert all(len(sweep.shapes(f, True)) <= 3 for f in ("square", "thin", "fat"))
    # ids of an 8-GPU box folded onto a smaller one; the host stays the host
    assert [sweep.fold(v, 2) for v in (-1, 0, 5, 6)] == [-1, 0, 1, 0]
    assert (sweep.ALPHA, sweep.BETA) == (1.2345, 1.1154)


def test_comparator_binds_the_vendor_symbols():
    # the yardstick module only loads the toolkit's cuBLAS; nothing is computed without a GPU
    import importlib
    comparators = importlib.import_module("paralia_framework_b200.comparators")
    lib = comparators.cublas()
    for name in ("cublasXtCreate", "cublasXtDeviceSelect", "cublasXtSetBlockDim", "cublasXtSetCpuRatio",
                 "cublasXtSetPinningMemMode", "cublasXtDgemm", "cublasXtSgemm", "cublasXtDestroy",
                 "cublasDgemm_v2", "cublasSgemm_v2"):
        assert hasattr(lib, name), name


def test_predictor_mode_needs_no_gpu_with_a_unit_list(pl, capsys):
    # the reference's dgemm_predictor: autotune only; with the units given the model runs on
    # the host alone (shipped B200 tables)
    import importlib
    runner = importlib.import_module("paralia_framework_b200.runner")
    out = runner.main(["dgemm_predict", "8", "11111111", "-1", "-1", "N", "N", "1", "1",
                       "32768", "32768", "32768", "-1", "-1", "-1", "-1"])
    capsys.readouterr()
    assert out["T"] in (2048, 4096) and out["grid"] == [2, 4] and out["units"] == list(range(8))
    assert out["subkernels"] == (32768 // out["T"]) ** 3
    # host-resident 32768^3 on 8 B200: the model says compute-bound, 0.25-0.30 s
    assert 0.25 < out["pred_t"] < 0.30
    one = runner.main(["dgemm_predict", "1", "1", "-1", "-1", "N", "N", "1", "1",
                       "32768", "32768", "32768", "-1", "-1", "-1", "-1"])
    capsys.readouterr()
    assert 4096 <= one["T"] <= 8192 and one["T"] % 256 == 0 and 1.9 < one["pred_t"] < 2.2


@pytest.mark.parametrize("dims,T,units", [((32768, 32768, 32768), 2048, 8), ((32768, 32768, 32768), 4096, 1),
                                          ((65536, 65536, 2048), 4096, 2), ((1156, 1412, 1228), 512, 3),
                                          ((300, 5000, 700), 256, 4), ((4096, 4096, 0), 1024, 2)])
@pytest.mark.parametrize("bounded", [False, True])
def test_launch_plan_is_complete_and_static(pl, dims, T, units, bounded):
    M, N, K = dims
    items, (d1, d2) = pl.plan_gemm(M, N, K, T, units, bounded)
    again, _ = pl.plan_gemm(M, N, K, T, units, bounded)
    assert items == again                                   # a function of its arguments alone
    Mt, Nt, Kt = -(-M // T), -(-N // T), -(-K // T)
    owner, g1, g2 = pl.distribute_2d(units, Mt, Nt, max(Kt, 1))
    assert (d1, d2) == (g1, g2)
    seen = {}
    per_tile = {}
    for (u, mi, ni, k0, k1) in items:
        assert 0 <= mi < Mt and 0 <= ni < Nt
        assert owner[(mi * Nt + ni) * max(Kt, 1)] == u      # the unit that owns the C tile runs it
        per_tile.setdefault((mi, ni), []).append((k0, k1))
        for k in range(k0, k1):
            assert (mi, ni, k) not in seen                  # every (mi, ni, ki) exactly once
            seen[(mi, ni, k)] = u
    assert len(per_tile) == Mt * Nt
    if Kt == 0:
        assert all(v == [(0, 0)] for v in per_tile.values())   # one beta-scaling launch per tile
        return
    assert len(seen) == Mt * Nt * Kt
    # the k split is the same for every C tile and depends on k alone: [0,1), then fours
    # (ones with a bounded cache), in increasing k
    want, k = [], 0
    while k < Kt:
        step = 1 if (bounded or k == 0) else 4
        want.append((k, min(Kt, k + step)))
        k = want[-1][1]
    assert all(v == want for v in per_tile.values())
    # round-robin over the units: among the first `active` launches no unit appears twice
    active = len({u for (u, *_rest) in items})
    first = [u for (u, *_rest) in items[:active]]
    assert sorted(first) == list(range(active))
    if bounded:   # tile-major: a C tile is finished before the unit starts its next one
        for u in range(active):
            mine = [(mi, ni) for (uu, mi, ni, _a, _b) in items if uu == u]
            order = [t for i, t in enumerate(mine) if i == 0 or mine[i - 1] != t]
            assert len(order) == len(set(order))


def _bands_of_unit(items, unit):
    """Band sizes of one unit read off its launch order: a band is a run of first-k launches."""
    bands, run = [], 0
    for (u, _mi, _ni, k0, _k1) in items:
        if u != unit:
            continue
        if k0 == 0:
            run += 1
        elif run:
            bands.append(run)
            run = 0
    if run:
        bands.append(run)
    return bands


@pytest.mark.parametrize("T,units", [(2048, 8), (4096, 8), (4096, 4), (4096, 1), (8192, 1)])
def test_band_sizes_first_band_feeds_itself_and_the_tail_shrinks(pl, T, units):
    pl.load_database(str(pl.DEFAULT_DB))
    n = 32768
    items, (d1, d2) = pl.plan_gemm(n, n, n, T, units)
    per_unit = (n // T) ** 2 // units
    for u in range(units):
        bands = _bands_of_unit(items, u)
        assert sum(bands) == per_unit
        # what is left to write back after the last launch is one or two tiles
        assert bands[-1] <= 2
        if len(bands) > 1:
            assert bands[-1] <= bands[-2]
        # whole tile rows of the unit's block in the first band
        row = (n // T) // d2
        assert bands[0] % row == 0 or bands[0] == per_unit
    if (T, units) == (2048, 8):
        # eight GPUs share 185 GB/s of host link: two tile rows (8 tiles) would be input-bound
        assert _bands_of_unit(items, 0)[0] >= 12


def test_model_reproduces_the_measured_eight_gpu_sweep(pl, golden_dir):
    """Calibration regression: the 70 problems of the placement matrix (ten placement scenarios x
    seven shapes, all eight GPUs forced) were timed on an 8 x B200 box and the measurements are
    kept in tests/golden/sweep_8gpu_measured.jsonl (written by sweep.py --summary). With the
    tile edge each problem was run with, the model must stay within 12 % of the measured time at
    the median and must not drift towards the 45 % it had before the host side of a call was
    modelled."""
    import math
    pl.load_database(str(pl.DEFAULT_DB))
    errs = []
    for line in (golden_dir / "sweep_8gpu_measured.jsonl").read_text().splitlines():
        r = json.loads(line)
        T, nu = (int(x) for x in r["control"].split(",")[:2])
        la, lb, lc = r["loc"]
        rep = pl.autotune_gemm(8, "N", "N", r["M"], r["N"], r["K"], la, lb, lc,
                               pl.make_ctl(T=T, units=list(range(nu))))
        errs.append(abs(rep.pred_t / r["t_avg"] - 1.0))
    errs.sort()
    assert len(errs) == 70
    assert errs[len(errs) // 2] <= 0.12
    assert sum(1 for e in errs if e <= 0.10) >= 30
    assert math.fsum(errs) / len(errs) <= 0.18
