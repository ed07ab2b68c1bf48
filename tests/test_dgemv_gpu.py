"""Parity of the CUDA DGEMV path against the CPU oracle, through the C ABI.
Tolerance: normwise relative error <= 8*K*eps64 with K the length of the sums."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
EPS64 = 2.0 ** -52


def _ngpu():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _case(orc, ta, M, N, pad=0, incx=1, incy=1):
    A = orc.matrix_f64(M, N, 42, M + pad)
    in_len, out_len = (M, N) if ta == "T" else (N, M)
    x = orc.uniform_f64(1 + (in_len - 1) * incx, 43)
    y = orc.uniform_f64(1 + (out_len - 1) * incy, 44)
    return A, x, y, in_len, out_len


@pytest.mark.parametrize("ta", ["N", "T"])
@pytest.mark.parametrize("dims,T,pad,incx,incy", [((1024, 768), 128, 0, 1, 1), ((289, 353), 64, 0, 1, 1),
                                                 ((2000, 3000), 0, 4, 1, 1), ((513, 1025), 256, 1, 2, 3),
                                                 ((1, 500), 64, 0, 1, 1), ((500, 1), 64, 0, 1, 1)])
def test_dgemv_host_resident_vs_oracle(pl, orc, ta, dims, T, pad, incx, incy):
    M, N = dims
    A, x, y, in_len, out_len = _case(orc, ta, M, N, pad, incx, incy)
    want = y.copy()
    orc.dgemv(ta, M, N, 1.23, A, M + pad, x, incx, 0.9876, want, incy)
    before = y.copy()
    rep = pl.dgemv(ta, M, N, 1.23, A, M + pad, x, incx, 0.9876, y, incy, ctl=pl.make_ctl(T=T, units=[0]))
    assert orc.normwise_rel_err(y[::incy], want[::incy]) <= 8 * in_len * EPS64
    if incy > 1:
        mask = np.ones(len(y), bool); mask[::incy] = False
        assert np.array_equal(y[mask], before[mask])
    assert rep.h2d_bytes == (M * N + in_len + out_len) * 8 and rep.d2h_bytes == out_len * 8
    # bit-reproducible
    y2 = before.copy()
    pl.dgemv(ta, M, N, 1.23, A, M + pad, x, incx, 0.9876, y2, incy, ctl=pl.make_ctl(T=T, units=[0]))
    assert np.array_equal(y, y2)


@pytest.mark.parametrize("ta", ["N", "T"])
def test_dgemv_device_resident(pl, orc, ta):
    import torch
    M, N = 3072, 2048
    A, x, y, in_len, out_len = _case(orc, ta, M, N)
    want = y.copy()
    orc.dgemv(ta, M, N, -0.5, A, M, x, 1, 0.0, want, 1)
    dA = torch.from_numpy(np.ascontiguousarray(A.T)).cuda()
    dx, dy = torch.from_numpy(x).cuda(), torch.full((out_len,), float("nan"), dtype=torch.float64, device="cuda")
    rep = pl.dgemv(ta, M, N, -0.5, dA, M, dx, 1, 0.0, dy, 1)
    torch.cuda.synchronize()
    assert orc.normwise_rel_err(dy.cpu().numpy(), want) <= 8 * in_len * EPS64   # beta = 0 ignores NaN in y
    assert rep.h2d_bytes == 0 and rep.d2h_bytes == 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("ta", ["N", "T"])
def test_dgemv_two_gpus(pl, orc, ta):
    M, N = 2050, 1538
    A, x, y, in_len, out_len = _case(orc, ta, M, N)
    want = y.copy()
    orc.dgemv(ta, M, N, 1.23, A, M, x, 1, 0.9876, want, 1)
    y1 = y.copy()
    pl.dgemv(ta, M, N, 1.23, A, M, x, 1, 0.9876, y1, 1, ctl=pl.make_ctl(T=256, units=[0]))
    rep = pl.dgemv(ta, M, N, 1.23, A, M, x, 1, 0.9876, y, 1, ctl=pl.make_ctl(T=256, units=[0, 1]))
    assert rep.active_unit_num == 2
    assert orc.normwise_rel_err(y, want) <= 8 * in_len * EPS64
    if ta == "T":
        assert np.array_equal(y, y1)     # each y[n] is one column's dot product on either split


def test_dgemv_invalid_arguments(pl, orc):
    A = orc.matrix_f64(8, 8, 1)
    x = orc.uniform_f64(8, 2)
    with pytest.raises(pl.ParaliaError) as e:
        pl.dgemv("N", 8, 8, 1.0, A, 4, x, 1, 0.0, x, 1)
    assert e.value.code == pl.ERR_INVALID_ARG
    with pytest.raises(pl.ParaliaError) as e:
        pl.dgemv("Q", 8, 8, 1.0, A, 8, x, 1, 0.0, x, 1)
    assert e.value.code == pl.ERR_INVALID_ARG


@pytest.mark.parametrize("ta", ["N", "T"])
@pytest.mark.parametrize("dims,pad,incx,incy", [((1024, 768), 0, 1, 1), ((289, 353), 1, 1, 1),
                                               ((513, 1025), 3, 2, 3), ((1, 300), 0, 1, 1),
                                               ((300, 1), 0, 3, 1)])
def test_tile_dgemv_vs_oracle(pl, orc, ta, dims, pad, incx, incy):
    # the per-tile entry on the caller's stream, strided x and y, odd leading dimension
    import torch
    M, N = dims
    A, x, y, in_len, out_len = _case(orc, ta, M, N, pad, incx, incy)
    want = y.copy()
    orc.dgemv(ta, M, N, -0.75, A, M + pad, x, incx, 1.5, want, incy)
    dA = torch.from_numpy(np.ascontiguousarray(A.T)).cuda()     # same bytes as column-major
    dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y.copy()).cuda()
    nbytes = pl.tile_dgemv_scratch_bytes(ta, M, N)
    assert (nbytes == 0) == (ta == "T")
    scratch = torch.empty(max(nbytes // 8, 1), dtype=torch.float64, device="cuda")
    stream = torch.cuda.current_stream()
    pl.tile_dgemv(0, ta, M, N, -0.75, dA, M + pad, dx, incx, 1.5, dy, incy,
                  scratch if nbytes else None, stream=stream.cuda_stream)
    stream.synchronize()
    got = dy.cpu().numpy()
    assert orc.normwise_rel_err(got[::incy], want[::incy]) <= 8 * in_len * EPS64
    if incy > 1:
        mask = np.ones(len(y), bool); mask[::incy] = False
        assert np.array_equal(got[mask], y[mask])


def test_tile_dgemv_invalid_arguments(pl):
    import torch
    d = torch.zeros(64, dtype=torch.float64, device="cuda")
    with pytest.raises(pl.ParaliaError):
        pl.tile_dgemv(0, "X", 4, 4, 1.0, d, 4, d, 1, 0.0, d, 1, d)
    with pytest.raises(pl.ParaliaError):
        pl.tile_dgemv(0, "N", 4, 4, 1.0, d, 2, d, 1, 0.0, d, 1, d)      # ldA < M
    with pytest.raises(pl.ParaliaError):
        pl.tile_dgemv(0, "N", 4, 4, 1.0, d, 4, d, 1, 0.0, d, 1, None)   # op = N without scratch
    with pytest.raises(pl.ParaliaError):
        pl.tile_dgemv(0, "T", 4, 4, 1.0, d, 4, d, 0, 0.0, d, 1, None)   # zero increment


def test_dgemv_host_vs_openblas_golden(pl, orc, golden_dir):
    import pathlib, sys
    sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent / "golden"))
    from gen_golden import DGEMV_CASES, dgemv_inputs
    gold = np.load(golden_dir / "blas_openblas_dgemv.npz")
    for i, case in enumerate(DGEMV_CASES):
        ta, M, N, alpha, beta, pad, incx, incy = case
        A, x, y = dgemv_inputs(case)
        pl.dgemv(ta, M, N, alpha, A, M + pad, x, incx, beta, y, incy, ctl=pl.make_ctl(T=64, units=[0]))
        in_len = M if ta == "T" else N
        assert orc.normwise_rel_err(y[::incy], gold[f"dgemv_{i}"]) <= 8 * in_len * EPS64, case


@pytest.mark.parametrize("ta", ["N", "T"])
@pytest.mark.parametrize("beta", [0.0, 1e-20, 0.5, 1.0])
def test_dgemv_empty_inner_dimension_scales_y(pl, ta, beta):
    """No columns (op = N) or no rows (op = T) to multiply: y <- beta*y in one rounding, and
    for beta == 0 y is set to zero without being read (a NaN in y must not survive), exactly
    as BLAS defines it."""
    n = 1001
    y = np.linspace(-3.0, 7.0, n)
    y[17] = np.nan if beta == 0.0 else 2.0 ** -600
    want = np.zeros(n) if beta == 0.0 else beta * y
    M, N = (n, 0) if ta == "N" else (0, n)
    A = np.zeros((max(M, 1), max(N, 1)), order="F")
    x = np.zeros(1)
    pl.dgemv(ta, M, N, 1.25, A, max(M, 1), x, 1, beta, y, 1, ctl=pl.make_ctl(units=[0]))
    assert np.array_equal(y, want)


@pytest.mark.gpu
@pytest.mark.parametrize("ta", ["N", "T"])
def test_tile_dgemv_microbenchmark_is_hbm_bound(pl, ta):
    """The calibration microbenchmark of the DGEMV tile (the reference's dgemv_microbench) moves
    8 bytes per element of A: on a B200 a 16384-wide tile must stream well above 3 TB/s."""
    T = 16384
    t = pl.bench_tile_dgemv(0, ta, T, 4)
    gbs = 8.0 * T * T / t / 1e9
    assert 3000.0 < gbs < 9000.0, gbs
    with pytest.raises(pl.ParaliaError):
        pl.bench_tile_dgemv(0, "C", T, 4)
