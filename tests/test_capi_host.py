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
    want_T, want_sl = orc.optimize_tile(32768, 32768, 32768, 8, step=128)
    assert rep.T == want_T == 2048
    assert list(rep.T_slowdowns) == want_sl
    assert rep.active_unit_num == 8 and (rep.grid_d1, rep.grid_d2) == (2, 4)
    assert rep.subkernel_num == 16 * 16 * 16
    assert list(rep.subkernels_per_unit[:8]) == [512] * 8
    assert rep.pred_t > 0
    # a caller-fixed T is kept
    rep = pl.autotune_gemm(8, "N", "N", 32768, 32768, 32768, -1, -1, -1,
                           pl.make_ctl(T=4096, units=[0, 1]))
    assert rep.T == 4096 and rep.active_unit_num == 2


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
    pl.load_database(str(tmp_path))
    try:
        rep = pl.autotune_gemm(8, "N", "N", 32768, 32768, 32768, -1, -1, -1,
                               pl.make_ctl(units=list(range(8))))
        assert rep.T == 2048
        t_exec = (32768 / 2048) ** 3 * (2.0 * 2048 ** 3 / rate) / 8
        t_recv = 3 * (1e-5 + 2e-11 * 32768 * 32768 * 8 / 8)
        assert t_exec > t_recv
        # what overlap cannot hide: first A, B and C tiles in, last C tile out (4 tile copies)
        t_fill = 4 * (1e-5 + 2e-11 * 2048 * 2048 * 8)
        assert rep.pred_t == pytest.approx(t_exec * (1 + rep.T_slowdowns[0]) + t_fill, rel=1e-5)
        # a slow host link makes the same problem link-bound
        for g in range(8):
            (proc / f"Link-Stats_loc_dest-{g}_loc_src--1.log").write_text(
                "Intercept: 1.000000e-05\nCoefficient: 1.000000e-09\n")
        pl.load_database(str(tmp_path))
        rep2 = pl.autotune_gemm(8, "N", "N", 32768, 32768, 32768, -1, -1, -1,
                                pl.make_ctl(units=list(range(8))))
        t_recv2 = 3 * (1e-5 + 1e-9 * 32768 * 32768 * 8 / 8)
        tile = rep2.T * rep2.T * 8     # three tiles in over the slow direction, one out over the fast
        t_fill2 = 3 * (1e-5 + 1e-9 * tile) + (1e-5 + 2e-11 * tile)
        assert rep2.pred_t == pytest.approx(t_recv2 * (1 + rep2.T_slowdowns[0]) + t_fill2, rel=1e-5)
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
    assert out["T"] == 2048 and out["grid"] == [2, 4] and out["units"] == list(range(8))
    assert out["subkernels"] == 16 ** 3
    # host-resident 32768^3 on 8 B200: the model says compute-bound, 0.25-0.30 s
    assert 0.25 < out["pred_t"] < 0.30
    one = runner.main(["dgemm_predict", "1", "1", "-1", "-1", "N", "N", "1", "1",
                       "32768", "32768", "32768", "-1", "-1", "-1", "-1"])
    capsys.readouterr()
    assert one["T"] == 4096 and 1.9 < one["pred_t"] < 2.2


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
