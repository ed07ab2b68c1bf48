"""The five benchmark configurations at their full sizes, checked through properties that do
not need an O(n^3) reference.

GEMM (configs 2, 3, 4): Freivalds' check. For random vectors x the identities
    C x   = alpha * op(A) (op(B) x)   + beta * C0 x
    C^T x = alpha * op(B)^T (op(A)^T x) + beta * C0^T x
cost O(n^2) each and a wrong tile, a tile added twice or a dropped k step breaks them with
probability 1. The matrix-vector products of the checker are torch FP64 ``mv`` (vendor
code, independent of the kernels under test). Tolerances: the stated normwise bounds,
8*K*eps64 for DGEMM and 4*K*eps32 for SGEMM, plus the rounding of the checker's own
matrix-vector products; the test also demands the far smaller error that a correct kernel
reaches in practice.
Level 1 (config 5, N = 2^30): DAXPY with alpha = -0.5 is exact in the product, so the result
must equal torch's bit for bit; DDOT is held to the standard bound N*eps*sum|x_i*y_i| and
must be reproduced bit for bit by a second call.
Every case also checks that a repeated call returns identical bits (fixed tile order)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
EPS64, EPS32 = 2.0 ** -52, 2.0 ** -23
GiB = 1 << 30


def _need(free_gib, gpus=1):
    import torch
    if torch.cuda.device_count() < gpus:
        pytest.skip(f"needs {gpus} GPUs")
    for d in range(gpus):
        free, _ = torch.cuda.mem_get_info(d)
        if free < free_gib * GiB:
            pytest.skip(f"needs {free_gib} GiB free on GPU {d}")


def _rel(a, b):
    return float((a - b).norm() / b.norm())


def _vectors(n, dev, dtype):
    import torch
    g = torch.Generator(device=f"cuda:{dev}").manual_seed(7)
    signs = (torch.randint(0, 2, (n,), generator=g, device=f"cuda:{dev}") * 2 - 1).to(dtype)
    unif = torch.rand(n, generator=g, device=f"cuda:{dev}", dtype=dtype) * 2 - 1
    return [signs, unif]


def _release(pl):
    import torch
    for d in range(torch.cuda.device_count()):
        pl.dev_cache_free(d)
    torch.cuda.empty_cache()


def test_config2_dgemm_32768_freivalds(pl):
    """DGEMM NN 32768^3, alpha = beta = 1, operands resident on the GPU."""
    import torch
    _need(60)
    n = 32768
    dev = "cuda:0"
    # a row-major (cols, rows) tensor holds the bytes of a column-major rows x cols matrix
    A = torch.empty((n, n), dtype=torch.float64, device=dev)
    B = torch.empty((n, n), dtype=torch.float64, device=dev)
    C = torch.empty((n, n), dtype=torch.float64, device=dev)
    for t, seed in ((A, 42), (B, 43), (C, 44)):
        pl.fill_f64(t, n * n, seed, 0, 0)
    C0 = C.clone()
    rep = pl.dgemm("N", "N", n, n, n, 1.0, A, n, B, n, 1.0, C, n, locA=0, locB=0, locC=0)
    assert rep.kernel_launches > 0
    tol = 8 * n * EPS64
    for x in _vectors(n, 0, torch.float64):
        # column-major M = t.T, so M x = mv(t.T, x) and M^T x = mv(t, x)
        want = torch.mv(A.T, torch.mv(B.T, x)) + torch.mv(C0.T, x)
        assert _rel(torch.mv(C.T, x), want) <= tol
        assert _rel(torch.mv(C.T, x), want) <= 1e-13
        want_t = torch.mv(B, torch.mv(A, x)) + torch.mv(C0, x)
        assert _rel(torch.mv(C, x), want_t) <= 1e-13
    # the library's own DGEMV at this size against the checker's
    y = torch.zeros(n, dtype=torch.float64, device=dev)
    x = _vectors(n, 0, torch.float64)[1]
    pl.dgemv("N", n, n, 1.0, C, n, x, 1, 0.0, y, 1, locA=0, locx=0, locy=0)
    assert _rel(y, torch.mv(C.T, x)) <= 8 * n * EPS64
    pl.dgemv("T", n, n, 1.0, C, n, x, 1, 0.0, y, 1, locA=0, locx=0, locy=0)
    assert _rel(y, torch.mv(C, x)) <= 8 * n * EPS64
    # fixed tile order: the same call gives the same bits
    first = C.clone()
    C.copy_(C0)
    pl.dgemm("N", "N", n, n, n, 1.0, A, n, B, n, 1.0, C, n, locA=0, locB=0, locC=0)
    assert torch.equal(C, first)
    del A, B, C, C0, first
    _release(pl)


def test_config3_dgemm_transposed_mixed_placement_freivalds(pl):
    """DGEMM TransA = T, M = N = 65536, K = 2048, beta = 0, A on GPU 0, B on GPU 1 (GPU 0 on a
    one-GPU box), C (32 GiB) in pinned host memory."""
    import torch
    _need(80)
    import psutil
    if psutil.virtual_memory().available < 80 * GiB:
        pytest.skip("needs 80 GiB of free host memory")
    M = N = 65536
    K = 2048
    devB = 1 if torch.cuda.device_count() > 1 else 0
    A = torch.empty((M, K), dtype=torch.float64, device="cuda:0")        # column-major K x M, ld K
    B = torch.empty((N, K), dtype=torch.float64, device=f"cuda:{devB}")  # column-major K x N, ld K
    pl.fill_f64(A, M * K, 42, 0, 0)
    pl.fill_f64(B, N * K, 43, 0, devB)
    C = torch.empty((N, M), dtype=torch.float64, pin_memory=True)
    C.fill_(float("nan"))                                                # beta = 0 must not read it
    rep = pl.dgemm("T", "N", M, N, K, 1.0, A, K, B, K, 0.0, C, M, locA=0, locB=devB, locC=-1)
    assert rep.d2h_bytes == M * N * 8 and rep.h2d_bytes == 0
    _release(pl)      # the tile cache held the C accumulators: make room for the checker's copy
    Cd = C.to("cuda:0")
    Bd = B.to("cuda:0")
    tol = 8 * K * EPS64
    for x in _vectors(N, 0, torch.float64):
        # op(A) = A, op(B) = Bd.T as (M x K) and (K x N) matrices
        want = torch.mv(A, torch.mv(Bd.T, x))
        assert _rel(torch.mv(Cd.T, x), want) <= tol
        want_t = torch.mv(Bd, torch.mv(A.T, x))
        assert _rel(torch.mv(Cd, x), want_t) <= tol
    assert not torch.isnan(Cd).any()
    del A, B, C, Cd, Bd
    _release(pl)


def test_config4_sgemm_40960_freivalds(pl):
    """SGEMM NN 40960^3, alpha = 1, beta = 0, normal(0,1) entries, operands on the GPU."""
    import torch
    _need(60)
    n = 40960
    dev = "cuda:0"
    A = torch.empty((n, n), dtype=torch.float32, device=dev)
    B = torch.empty((n, n), dtype=torch.float32, device=dev)
    C = torch.empty((n, n), dtype=torch.float32, device=dev)
    pl.fill_f32(A, n * n, 42, 1, 0)
    pl.fill_f32(B, n * n, 43, 1, 0)
    pl.fill_f32(C, n * n, 44, 1, 0)      # must be ignored: beta = 0
    rep = pl.sgemm("N", "N", n, n, n, 1.0, A, n, B, n, 0.0, C, n, locA=0, locB=0, locC=0)
    assert rep.kernel_launches > 0
    bound = 4 * n * EPS32
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        for x in _vectors(n, 0, torch.float32):
            # checker in FP32 matrix-vector products accumulated by the vendor's gemv: its own
            # rounding (about sqrt(n)*eps32 = 2.4e-5) sits far below the bound of 1.95e-2
            want = torch.mv(A.T, torch.mv(B.T, x))
            err = _rel(torch.mv(C.T, x), want)
            assert err <= bound
            assert err <= 1e-3
            want_t = torch.mv(B, torch.mv(A, x))
            assert _rel(torch.mv(C, x), want_t) <= 1e-3
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    first = C.clone()
    C.fill_(float("nan"))
    pl.sgemm("N", "N", n, n, n, 1.0, A, n, B, n, 0.0, C, n, locA=0, locB=0, locC=0)
    assert torch.equal(C, first)
    del A, B, C, first
    _release(pl)


def test_config5_daxpy_ddot_2_30(pl):
    """DAXPY (alpha = -0.5) and DDOT at N = 2^30 on GPU-resident vectors."""
    import torch
    _need(48)
    n = 1 << 30
    dev = "cuda:0"
    x = torch.empty(n, dtype=torch.float64, device=dev)
    y = torch.empty(n, dtype=torch.float64, device=dev)
    pl.fill_f64(x, n, 42, 0, 0)
    pl.fill_f64(y, n, 43, 0, 0)
    # the fill is the same counter-based stream on every device and on the host
    assert x[:5].tolist() != y[:5].tolist() and float(x.abs().max()) <= 1.0
    dot, rep = pl.ddot(n, x, 1, y, 1, result=0.0, locx=0, locy=0)
    ref = float(torch.dot(x, y))
    bound = n * EPS64 * float((x * y).abs().sum())
    assert abs(dot - ref) <= bound
    assert abs(dot - ref) <= 1e-7                                   # in practice far inside it
    dot2, _ = pl.ddot(n, x, 1, y, 1, result=0.0, locx=0, locy=0)
    assert dot2 == dot                                              # fixed summation order
    dot3, _ = pl.ddot(n, x, 1, y, 1, result=1.5, locx=0, locy=0)    # *result += x.y
    assert dot3 == pytest.approx(1.5 + dot, rel=1e-15, abs=1e-9)
    # alpha = -0.5: alpha*x is exact, so fused and unfused multiply-add round identically
    want = torch.add(y, x, alpha=-0.5)
    pl.daxpy(n, -0.5, x, 1, y, 1, locx=0, locy=0)
    assert torch.equal(y, want)
    del x, y, want
    _release(pl)


def _host_ok(gib):
    import psutil
    if psutil.virtual_memory().available < gib * GiB:
        pytest.skip(f"needs {gib} GiB of free host memory")


def _pinned_from_device(pl, dev_tensor, nbytes, dev):
    """A pinned host copy of a device buffer (raw pointer, freed by the caller)."""
    h = pl.malloc(nbytes, -1)
    pl.memcpy(h, -1, dev_tensor, dev, nbytes)
    return h


def test_config2_dgemm_32768_host_resident_all_gpus_freivalds(pl):
    """DGEMM NN 32768^3, alpha = beta = 1, A, B and C in pinned host memory as the
    configuration states, on every GPU of the box through the in-process scheduler."""
    import torch
    _need(60)
    _host_ok(40)
    n = 32768
    g = torch.cuda.device_count()
    dev = "cuda:0"
    A = torch.empty((n, n), dtype=torch.float64, device=dev)
    B = torch.empty((n, n), dtype=torch.float64, device=dev)
    C0 = torch.empty((n, n), dtype=torch.float64, device=dev)
    for t, seed in ((A, 42), (B, 43), (C0, 44)):
        pl.fill_f64(t, n * n, seed, 0, 0)
    nb = n * n * 8
    hA, hB, hC = (_pinned_from_device(pl, t, nb, 0) for t in (A, B, C0))
    try:
        ctl = pl.make_ctl(units=list(range(g)))
        rep = pl.dgemm("N", "N", n, n, n, 1.0, hA, n, hB, n, 1.0, hC, n, locA=-1, locB=-1, locC=-1, ctl=ctl)
        assert rep.active_unit_num == g
        # every host byte crosses the host link once: A, B, C in; C out
        assert rep.h2d_bytes == 3 * nb and rep.d2h_bytes == nb
        _release(pl)
        C = torch.empty((n, n), dtype=torch.float64, device=dev)
        pl.memcpy(C, 0, hC, -1, nb)
        for x in _vectors(n, 0, torch.float64):
            want = torch.mv(A.T, torch.mv(B.T, x)) + torch.mv(C0.T, x)
            assert _rel(torch.mv(C.T, x), want) <= 8 * n * EPS64
            assert _rel(torch.mv(C.T, x), want) <= 1e-13
            want_t = torch.mv(B, torch.mv(A, x)) + torch.mv(C0, x)
            assert _rel(torch.mv(C, x), want_t) <= 1e-13
        # fixed tile order: a second call from the same inputs gives the same bits
        pl.memcpy(hC, -1, C0, 0, nb)
        pl.dgemm("N", "N", n, n, n, 1.0, hA, n, hB, n, 1.0, hC, n, locA=-1, locB=-1, locC=-1, ctl=ctl)
        C2 = torch.empty((n, n), dtype=torch.float64, device=dev)
        _release(pl)
        pl.memcpy(C2, 0, hC, -1, nb)
        assert torch.equal(C, C2)
        del C, C2
    finally:
        for h in (hA, hB, hC):
            pl.free(h, -1)
        del A, B, C0
        _release(pl)


def test_config4_sgemm_40960_host_resident_all_gpus_freivalds(pl):
    """SGEMM NN 40960^3, alpha = 1, beta = 0, normal(0,1), operands in pinned host memory, on
    every GPU of the box."""
    import torch
    _need(60)
    _host_ok(30)
    n = 40960
    g = torch.cuda.device_count()
    dev = "cuda:0"
    A = torch.empty((n, n), dtype=torch.float32, device=dev)
    B = torch.empty((n, n), dtype=torch.float32, device=dev)
    pl.fill_f32(A, n * n, 42, 1, 0)
    pl.fill_f32(B, n * n, 43, 1, 0)
    nb = n * n * 4
    hA, hB = _pinned_from_device(pl, A, nb, 0), _pinned_from_device(pl, B, nb, 0)
    hC = pl.malloc(nb, -1)
    try:
        ctl = pl.make_ctl(units=list(range(g)))
        rep = pl.sgemm("N", "N", n, n, n, 1.0, hA, n, hB, n, 0.0, hC, n, locA=-1, locB=-1, locC=-1, ctl=ctl)
        assert rep.active_unit_num == g
        assert rep.h2d_bytes == 2 * nb and rep.d2h_bytes == nb      # beta = 0: C is not fetched
        _release(pl)
        C = torch.empty((n, n), dtype=torch.float32, device=dev)
        pl.memcpy(C, 0, hC, -1, nb)
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            for x in _vectors(n, 0, torch.float32):
                want = torch.mv(A.T, torch.mv(B.T, x))
                err = _rel(torch.mv(C.T, x), want)
                assert err <= 4 * n * EPS32 and err <= 1e-3
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
        del C
    finally:
        for h in (hA, hB, hC):
            pl.free(h, -1)
        del A, B
        _release(pl)
