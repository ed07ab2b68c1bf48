"""The allocation-free dot product (PARALiA_tile_ddot_noalloc).

Some users of the library cannot allocate device memory at the point where they need a
dot product -- they sit inside a loop where a cudaMalloc would stall the GPU, or their
host application gives them a fixed memory budget -- so they cannot hand
PARALiA_tile_ddot its scratch buffer. This entry point keeps the partial sums in a
fixed array inside the library instead. It runs the same kernels with the same grid as
the existing entry point, so its result must be identical bit for bit; the array is
shared by all calls and keeps the previous call's contents, hence two calls in a row
with different inputs."""
import pytest

pytestmark = pytest.mark.gpu


def _run_both(pl, torch, n, seed_x, seed_y):
    dx = torch.empty(n, dtype=torch.float64, device="cuda:0")
    dy = torch.empty(n, dtype=torch.float64, device="cuda:0")
    pl.fill_f64(dx, n, seed_x, 0, 0)
    pl.fill_f64(dy, n, seed_y, 0, 0)
    scratch = torch.empty(pl.tile_ddot_scratch_bytes(n) // 8, dtype=torch.float64, device="cuda:0")
    want = torch.zeros(1, dtype=torch.float64, device="cuda:0")
    got = torch.full((1,), float("nan"), dtype=torch.float64, device="cuda:0")
    pl.tile_ddot(0, n, dx, 1, dy, 1, scratch, want)
    pl.tile_ddot_noalloc(0, n, dx, 1, dy, 1, got)
    torch.cuda.synchronize()
    return got.item(), want.item()


def test_noalloc_ddot_matches_existing_entry_twice(pl):
    import torch
    # first call: a long vector that uses every partial-sum slot
    got, want = _run_both(pl, torch, (1 << 23) + 3, 42, 43)
    assert got == want
    # second call right after it: shorter vector, different data; stale partials of the
    # first call are still in the array and must not leak into the result
    got2, want2 = _run_both(pl, torch, 100001, 7, 9)
    assert got2 == want2
    assert got2 != got


def test_noalloc_ddot_rejects_oversize(pl):
    import torch
    d = torch.zeros(8, dtype=torch.float64, device="cuda:0")
    with pytest.raises(pl.ParaliaError) as e:
        pl.tile_ddot_noalloc(0, pl.tile_ddot_noalloc_max_n() + 1, d, 1, d, 1, d)
    assert e.value.code == pl.ERR_INVALID_ARG
    assert "exceeds" in str(e.value)
