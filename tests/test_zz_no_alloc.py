"""The allocation-free dot product (PARALiA_tile_ddot_noalloc).

Some users of the library cannot allocate device memory at the point where they need a
dot product -- they sit inside a loop where a cudaMalloc would stall the GPU, or their
host application gives them a fixed memory budget -- so they cannot hand
PARALiA_tile_ddot its scratch buffer. This entry point keeps the partial sums in a
fixed array inside the library instead. It runs the same kernels with the same grid as
the existing entry point, so its result must be identical bit for bit; the array is
shared by all calls and keeps the previous call's contents, hence two calls in a row
with different inputs. The results are also held to the CPU oracle's bound, the calls
must leave the amount of free device memory unchanged, and the per-GPU address lookup is
exercised on a second GPU when there is one."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run_both(pl, torch, n, seed_x, seed_y, dev=0, incx=1, incy=1):
    cuda = f"cuda:{dev}"
    nx, ny = 1 + (n - 1) * incx, 1 + (n - 1) * incy
    dx = torch.empty(nx, dtype=torch.float64, device=cuda)
    dy = torch.empty(ny, dtype=torch.float64, device=cuda)
    pl.fill_f64(dx, nx, seed_x, 0, dev)
    pl.fill_f64(dy, ny, seed_y, 0, dev)
    scratch = torch.empty(pl.tile_ddot_scratch_bytes(n) // 8, dtype=torch.float64, device=cuda)
    want = torch.zeros(1, dtype=torch.float64, device=cuda)
    got = torch.full((1,), float("nan"), dtype=torch.float64, device=cuda)
    pl.tile_ddot(dev, n, dx, incx, dy, incy, scratch, want)
    pl.tile_ddot_noalloc(dev, n, dx, incx, dy, incy, got)
    torch.cuda.synchronize(dev)
    return got.item(), want.item()


def _oracle_bound(orc, n, seed_x, seed_y, incx=1, incy=1):
    """Dot product and magnitude sum of the same seeded vectors on the CPU."""
    x = orc.uniform_f64(1 + (n - 1) * incx, seed_x)[::incx]
    y = orc.uniform_f64(1 + (n - 1) * incy, seed_y)[::incy]
    return float(np.dot(x, y)), float(np.dot(np.abs(x), np.abs(y)))


def test_noalloc_ddot_matches_existing_entry_twice(pl, orc):
    import torch
    # first call: a long vector that uses every partial-sum slot
    n1 = (1 << 23) + 3
    got, want = _run_both(pl, torch, n1, 42, 43)
    assert got == want
    ref, mag = _oracle_bound(orc, n1, 42, 43)
    assert abs(got - ref) <= n1 * 2.0 ** -52 * mag
    # second call right after it: shorter vector, different data; stale partials of the
    # first call are still in the array and must not leak into the result
    n2 = 100001
    got2, want2 = _run_both(pl, torch, n2, 7, 9)
    assert got2 == want2
    ref2, mag2 = _oracle_bound(orc, n2, 7, 9)
    assert abs(got2 - ref2) <= n2 * 2.0 ** -52 * mag2
    assert got2 != got


def test_noalloc_ddot_strided(pl, orc):
    import torch
    n = 300007
    got, want = _run_both(pl, torch, n, 11, 12, incx=2, incy=3)
    assert got == want
    ref, mag = _oracle_bound(orc, n, 11, 12, 2, 3)
    assert abs(got - ref) <= n * 2.0 ** -52 * mag


def test_noalloc_ddot_allocates_nothing(pl):
    import torch
    n = 1 << 22
    dx = torch.empty(n, dtype=torch.float64, device="cuda:0")
    dy = torch.empty(n, dtype=torch.float64, device="cuda:0")
    out = torch.zeros(1, dtype=torch.float64, device="cuda:0")
    pl.fill_f64(dx, n, 1, 0, 0)
    pl.fill_f64(dy, n, 2, 0, 0)
    pl.tile_ddot_noalloc(0, n, dx, 1, dy, 1, out)      # the first call looks the array up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(0)
    for _ in range(3):
        pl.tile_ddot_noalloc(0, n, dx, 1, dy, 1, out)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after == free_before


def test_noalloc_ddot_on_a_second_gpu(pl, orc):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    # each GPU has its own copy of the array at its own address
    n = (1 << 20) + 5
    got0, want0 = _run_both(pl, torch, n, 5, 6, dev=0)
    got1, want1 = _run_both(pl, torch, n, 5, 6, dev=1)
    assert got0 == want0 and got1 == want1 and got0 == got1
    ref, mag = _oracle_bound(orc, n, 5, 6)
    assert abs(got1 - ref) <= n * 2.0 ** -52 * mag


def test_noalloc_ddot_rejects_oversize(pl):
    import torch
    d = torch.zeros(8, dtype=torch.float64, device="cuda:0")
    with pytest.raises(pl.ParaliaError) as e:
        pl.tile_ddot_noalloc(0, pl.tile_ddot_noalloc_max_n() + 1, d, 1, d, 1, d)
    assert e.value.code == pl.ERR_INVALID_ARG
    assert "exceeds" in str(e.value)
