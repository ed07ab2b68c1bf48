"""Parity of the CUDA DAXPY / DDOT path against the CPU oracle, through the C ABI.

DAXPY is one fused multiply-add per element on both sides: bit-exact.
DDOT: |got - want| <= N * eps64 * sum|x_i y_i| (the standard bound for any summation order)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
EPS64 = 2.0 ** -52


@pytest.mark.parametrize("n,incx,incy,T", [(1 << 20, 1, 1, 1 << 16), (1000003, 1, 1, 1 << 17),
                                            (70001, 2, 3, 1 << 14), (1, 1, 1, 0), (5, 1, 1, 2),
                                            (1 << 18, 1, 1, 0)])
def test_daxpy_host_bit_exact(pl, orc, n, incx, incy, T):
    x = orc.uniform_f64(1 + (n - 1) * incx, 42)
    y = orc.uniform_f64(1 + (n - 1) * incy, 43)
    want = y.copy()
    orc.daxpy_tiled(n, -0.5, x, incx, want, incy, T if T else n)
    rep = pl.daxpy(n, -0.5, x, incx, y, incy, ctl=pl.make_ctl(T=T, units=[0]))
    assert np.array_equal(y, want)
    assert rep.kernel_launches >= 1 and rep.h2d_bytes == 2 * n * 8 and rep.d2h_bytes == n * 8


def test_daxpy_golden(pl, orc, golden_dir):
    import sys, pathlib
    sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent / "golden"))
    from gen_golden import L1_CASES
    gold = np.load(golden_dir / "blas_openblas.npz")
    for i, (n, incx, incy, alpha) in enumerate(L1_CASES):
        x = orc.uniform_f64(1 + (n - 1) * incx, 42)
        y = orc.uniform_f64(1 + (n - 1) * incy, 43)
        dot, _ = pl.ddot(n, x, incx, y, incy, 0.0, ctl=pl.make_ctl(units=[0]))
        mag = float(np.abs(x[::incx] * y[::incy]).sum())
        assert abs(dot - gold[f"ddot_{i}"][0]) <= n * EPS64 * mag
        pl.daxpy(n, alpha, x, incx, y, incy, ctl=pl.make_ctl(units=[0]))
        np.testing.assert_allclose(y[::incy], gold[f"daxpy_{i}"], rtol=0, atol=8 * EPS64)


@pytest.mark.parametrize("n", [1 << 20, 999999, 3])
def test_daxpy_device_resident(pl, orc, n):
    import torch
    x = orc.uniform_f64(n, 42)
    y = orc.uniform_f64(n, 43)
    want = y.copy()
    orc.daxpy_tiled(n, -0.5, x, 1, want, 1, n)
    dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
    rep = pl.daxpy(n, -0.5, dx, 1, dy, 1)
    torch.cuda.synchronize()
    assert np.array_equal(dy.cpu().numpy(), want)
    assert rep.h2d_bytes == 0 and rep.d2h_bytes == 0
    # the per-tile kernel entry point, odd offset -> unaligned start -> scalar path
    if n > 16:
        dy2 = torch.from_numpy(y).cuda()
        pl.tile_daxpy(0, n - 1, -0.5, dx[1:], 1, dy2[1:], 1)
        torch.cuda.synchronize()
        assert np.array_equal(dy2.cpu().numpy()[1:], want[1:])


@pytest.mark.parametrize("n,incx,incy,T", [(1 << 20, 1, 1, 1 << 16), (1000003, 1, 1, 1 << 17),
                                            (70001, 2, 3, 1 << 14), (1, 1, 1, 0), (1 << 18, 1, 1, 0)])
def test_ddot_host_vs_oracle(pl, orc, n, incx, incy, T):
    x = orc.uniform_f64(1 + (n - 1) * incx, 42)
    y = orc.uniform_f64(1 + (n - 1) * incy, 43)
    want, mag = orc.ddot_tiled(n, x, incx, y, incy, T if T else n, 0.0)
    got, rep = pl.ddot(n, x, incx, y, incy, 0.0, ctl=pl.make_ctl(T=T, units=[0]))
    assert abs(got - want) <= n * EPS64 * mag
    # accumulates into *result (ddot.cpp:431) and is bit-reproducible
    got2, _ = pl.ddot(n, x, incx, y, incy, 0.0, ctl=pl.make_ctl(T=T, units=[0]))
    assert got2 == got
    got3, _ = pl.ddot(n, x, incx, y, incy, 100.0, ctl=pl.make_ctl(T=T, units=[0]))
    assert abs(got3 - 100.0 - got) <= 64 * EPS64 * 100.0


def test_ddot_device_resident_and_tile_entry(pl, orc):
    import torch
    n = (1 << 21) + 1
    x = orc.uniform_f64(n, 42)
    y = orc.uniform_f64(n, 43)
    want, mag = orc.ddot_tiled(n, x, 1, y, 1, n, 0.0)
    dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
    got, rep = pl.ddot(n, dx, 1, dy, 1, 0.0)
    assert abs(got - want) <= n * EPS64 * mag and rep.h2d_bytes == 0
    scratch = torch.empty(pl.tile_ddot_scratch_bytes(n) // 8, dtype=torch.float64, device="cuda")
    res = torch.zeros(1, dtype=torch.float64, device="cuda")
    pl.tile_ddot(0, n, dx, 1, dy, 1, scratch, res)
    torch.cuda.synchronize()
    assert abs(res.item() - want) <= n * EPS64 * mag


def test_ddot_large_property(pl):
    # size-independent property: dot(x, x) of the uniform[-1,1) generator ~ N/3, and
    # dot(x, 2x) == 2*dot(x, x) exactly (scaling by 2 is exact, same summation order)
    import torch
    n = 1 << 27
    dx = torch.empty(n, dtype=torch.float64, device="cuda:0")
    pl.fill_f64(dx, n, 42, 0, 0)
    d1, _ = pl.ddot(n, dx, 1, dx, 1, 0.0)
    dx2 = dx * 2.0
    d2, _ = pl.ddot(n, dx, 1, dx2, 1, 0.0)
    assert d2 == 2.0 * d1
    assert abs(d1 / n - 1.0 / 3.0) < 1e-3


def test_level1_invalid_arguments(pl, orc):
    x = orc.uniform_f64(8, 1)
    with pytest.raises(pl.ParaliaError) as e:
        pl.daxpy(-1, 1.0, x, 1, x, 1)
    assert e.value.code == pl.ERR_INVALID_ARG
    with pytest.raises(pl.ParaliaError) as e:
        pl.daxpy(8, 1.0, x, 0, x, 1)
    assert e.value.code == pl.ERR_UNSUPPORTED
