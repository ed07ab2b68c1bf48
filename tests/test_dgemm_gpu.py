"""Parity of the CUDA DGEMM path against the CPU oracle, through the C ABI.

Tolerance (stated by the task): normwise relative error <= 8*K*eps64."""
import sys, pathlib
import numpy as np
import pytest

sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent / "golden"))
from gen_golden import DGEMM_CASES, stored_shape  # noqa: E402

pytestmark = pytest.mark.gpu
EPS64 = 2.0 ** -52


def tol(K):
    return 8 * max(K, 1) * EPS64


def _dev(t, dev=0):
    import torch
    return torch.from_numpy(np.ascontiguousarray(t.T)).to(f"cuda:{dev}")  # same bytes as F-order


def _host(t_dev, shape):
    out = np.asfortranarray(t_dev.cpu().numpy().T)
    assert out.shape == tuple(shape)
    return out


def _case(orc, ta, tb, M, N, K, pad=0):
    ar, ac = stored_shape(ta, M, K)
    br, bc = stored_shape(tb, K, N)
    A = orc.matrix_f64(ar, ac, 42, ar + pad)
    B = orc.matrix_f64(br, bc, 43, br + pad)
    C = orc.matrix_f64(M, N, 44, M + pad)
    return A, B, C, ar + pad, br + pad, M + pad


# ---------------------------------------------------------------- the tile kernel alone
@pytest.mark.parametrize("ta,tb", [("N", "N"), ("T", "N"), ("N", "T"), ("T", "T")])
@pytest.mark.parametrize("dims", [(128, 128, 16), (128, 128, 128), (256, 384, 160), (100, 36, 50),
                                  (290, 354, 308), (1, 1, 1), (130, 2, 2), (512, 512, 512)])
def test_tile_kernel_vs_oracle(pl, orc, ta, tb, dims):
    import torch
    M, N, K = dims
    A, B, C, lda, ldb, ldc = _case(orc, ta, tb, M, N, K)
    want = C.copy(order="F")
    orc.dgemm_tiled(ta, tb, M, N, K, 1.23, A, lda, B, ldb, 0.9876, want, ldc, 1 << 20)
    dA, dB, dC = _dev(A), _dev(B), _dev(C)
    pl.tile_dgemm(0, ta, tb, M, N, K, 1.23, dA, lda, dB, ldb, 0.9876, dC, ldc)
    torch.cuda.synchronize()
    got = _host(dC, C.shape)
    assert orc.normwise_rel_err(got, want) <= tol(K)


@pytest.mark.parametrize("dims", [(289, 353, 307), (33, 65, 17)])
@pytest.mark.parametrize("ta,tb", [("N", "N"), ("T", "T")])
def test_tile_kernel_odd_leading_dimension(pl, orc, ta, tb, dims):
    # leading dimensions TMA cannot address take the plain-load kernel
    import torch
    M, N, K = dims
    A, B, C, lda, ldb, ldc = _case(orc, ta, tb, M, N, K, pad=0)
    want = C.copy(order="F")
    orc.dgemm_tiled(ta, tb, M, N, K, -0.5, A, lda, B, ldb, 1.0, want, ldc, 1 << 20)
    dA, dB, dC = _dev(A), _dev(B), _dev(C)
    pl.tile_dgemm(0, ta, tb, M, N, K, -0.5, dA, lda, dB, ldb, 1.0, dC, ldc)
    torch.cuda.synchronize()
    assert orc.normwise_rel_err(_host(dC, C.shape), want) <= tol(K)


def test_tile_kernel_beta_zero_ignores_nan(pl, orc):
    import torch
    M = N = K = 256
    A, B, C, lda, ldb, ldc = _case(orc, "N", "N", M, N, K)
    want = np.zeros_like(C, order="F")
    orc.dgemm_tiled("N", "N", M, N, K, 1.0, A, lda, B, ldb, 0.0, want, ldc, 1 << 20)
    dC = torch.full((N, M), float("nan"), dtype=torch.float64, device="cuda:0")
    pl.tile_dgemm(0, "N", "N", M, N, K, 1.0, _dev(A), lda, _dev(B), ldb, 0.0, dC, ldc)
    torch.cuda.synchronize()
    assert orc.normwise_rel_err(_host(dC, C.shape), want) <= tol(K)


# ---------------------------------------------------------------- the whole path
@pytest.mark.parametrize("idx", range(len(DGEMM_CASES)))
def test_dgemm_host_vs_openblas_golden(pl, orc, golden_dir, idx):
    gold = np.load(golden_dir / "blas_openblas.npz")
    ta, tb, M, N, K, alpha, beta, pad = DGEMM_CASES[idx]
    A, B, C, lda, ldb, ldc = _case(orc, ta, tb, M, N, K, pad)
    before = C.copy(order="F")
    rep = pl.dgemm(ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc,
                   ctl=pl.make_ctl(T=16, units=[0]))
    assert orc.normwise_rel_err(C[:M, :], gold[f"dgemm_{idx}"]) <= tol(K)
    assert np.array_equal(C[M:, :], before[M:, :])
    assert rep.kernel_launches > 0 and rep.h2d_bytes > 0 and rep.d2h_bytes == M * N * 8


@pytest.mark.parametrize("ta,tb", [("N", "N"), ("T", "N"), ("N", "T"), ("T", "T")])
@pytest.mark.parametrize("dims,T", [((512, 512, 512), 256), ((289, 353, 307), 128),
                                    ((1024, 256, 768), 256), ((300, 300, 300), 304),
                                    ((1156, 1412, 1228), 512)])
def test_dgemm_host_resident_vs_oracle(pl, orc, ta, tb, dims, T):
    # host-resident operands (pageable numpy memory: pinned for the call), several tiles
    # per dimension, edge tiles; alpha/beta of the reference tester (dgemm_tester.cpp:74-75)
    M, N, K = dims
    A, B, C, lda, ldb, ldc = _case(orc, ta, tb, M, N, K)
    want = C.copy(order="F")
    orc.dgemm_tiled(ta, tb, M, N, K, 1.23, A, lda, B, ldb, 0.9876, want, ldc, T)
    rep = pl.dgemm(ta, tb, M, N, K, 1.23, A, lda, B, ldb, 0.9876, C, ldc,
                   ctl=pl.make_ctl(T=T, units=[0]))
    assert orc.normwise_rel_err(C, want) <= tol(K)
    Mt, Nt, Kt = -(-M // rep.T), -(-N // rep.T), -(-K // rep.T)
    assert rep.subkernel_num == Mt * Nt * Kt
    assert rep.h2d_bytes == (M * K + K * N + M * N) * 8   # every tile crosses once
    assert rep.d2h_bytes == M * N * 8


def test_dgemm_cfg1_shape(pl, orc):
    # BASELINE config 1: 4096^3, NN, alpha 1.25, beta 0.75, host-resident, seeds 42/43/44;
    # compared with OpenBLAS cblas_dgemm, the reference's CPU validation routine
    M = N = K = 4096
    A, B, C, lda, ldb, ldc = _case(orc, "N", "N", M, N, K)
    want = orc.openblas_dgemm("N", "N", 1.25, A, B, 0.75, C)
    rep = pl.dgemm("N", "N", M, N, K, 1.25, A, lda, B, ldb, 0.75, C, ldc,
                   ctl=pl.make_ctl(units=[0]))
    assert orc.normwise_rel_err(C, want) <= tol(K)
    # the tile is the model's choice: a streamed problem of this size wants tiles small enough
    # to overlap the host link with the kernels, large enough for the kernel to be efficient
    assert rep.T in (512, 768, 1024, 1280, 1536, 2048) and rep.pred_t > 0


@pytest.mark.parametrize("ta,tb", [("N", "N"), ("T", "N"), ("N", "T")])
def test_dgemm_device_resident_vs_oracle(pl, orc, ta, tb):
    # all operands on the GPU: tiles are read in place, C updated in place
    import torch
    M, N, K, T = 768, 640, 512, 256
    A, B, C, lda, ldb, ldc = _case(orc, ta, tb, M, N, K)
    want = C.copy(order="F")
    orc.dgemm_tiled(ta, tb, M, N, K, 1.23, A, lda, B, ldb, 0.9876, want, ldc, T)
    dA, dB, dC = _dev(A), _dev(B), _dev(C)
    rep = pl.dgemm(ta, tb, M, N, K, 1.23, dA, lda, dB, ldb, 0.9876, dC, ldc,
                   ctl=pl.make_ctl(T=T, units=[0]))
    torch.cuda.synchronize()
    assert orc.normwise_rel_err(_host(dC, C.shape), want) <= tol(K)
    assert rep.h2d_bytes == 0 and rep.d2h_bytes == 0


def test_dgemm_mixed_locations(pl, orc):
    # A on the GPU, B and C on the host, beta = 0 (the placement pattern of config 3)
    M, N, K, T = 512, 768, 256, 256
    A, B, C, lda, ldb, ldc = _case(orc, "T", "N", M, N, K)
    want = C.copy(order="F")
    orc.dgemm_tiled("T", "N", M, N, K, 1.0, A, lda, B, ldb, 0.0, want, ldc, T)
    dA = _dev(A)
    rep = pl.dgemm("T", "N", M, N, K, 1.0, dA, lda, B, ldb, 0.0, C, ldc,
                   ctl=pl.make_ctl(T=T, units=[0]))
    assert orc.normwise_rel_err(C, want) <= tol(K)
    assert rep.h2d_bytes == K * N * 8   # beta == 0: C is never read


def test_dgemm_bitwise_deterministic(pl, orc):
    M, N, K, T = 1024, 1024, 1024, 256
    A, B, C0, lda, ldb, ldc = _case(orc, "N", "N", M, N, K)
    outs = []
    for _ in range(3):
        C = C0.copy(order="F")
        pl.dgemm("N", "N", M, N, K, 1.23, A, lda, B, ldb, 0.9876, C, ldc,
                 ctl=pl.make_ctl(T=T, units=[0]))
        outs.append(C)
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])


def test_dgemm_bits_independent_of_placement(pl, orc):
    # same problem and T, A and B on the host vs on the GPU: identical bits (C is staged
    # through the tile cache in both runs; a C that lives on the executing GPU is updated
    # in place with beta applied first, which rounds differently)
    M, N, K, T = 768, 1024, 1280, 256
    A, B, C0, lda, ldb, ldc = _case(orc, "N", "N", M, N, K)
    Ch = C0.copy(order="F")
    pl.dgemm("N", "N", M, N, K, 1.23, A, lda, B, ldb, 0.9876, Ch, ldc, ctl=pl.make_ctl(T=T, units=[0]))
    dA, dB = _dev(A), _dev(B)
    Cd = C0.copy(order="F")
    pl.dgemm("N", "N", M, N, K, 1.23, dA, lda, dB, ldb, 0.9876, Cd, ldc, ctl=pl.make_ctl(T=T, units=[0]))
    assert np.array_equal(Cd, Ch)


def test_dgemm_linearity_large(pl, orc):
    # size-independent property at a size the oracle does not finish quickly:
    # with beta = 0, (2*alpha) * A*B == 2 * (alpha * A*B) exactly in binary floating point
    import torch
    n = 8192
    pl.init()
    g = torch.Generator(device="cuda:0")
    dA = torch.empty(n * n, dtype=torch.float64, device="cuda:0")
    dB = torch.empty(n * n, dtype=torch.float64, device="cuda:0")
    pl.fill_f64(dA, n * n, 42, 0, 0)
    pl.fill_f64(dB, n * n, 43, 0, 0)
    dC1 = torch.zeros(n * n, dtype=torch.float64, device="cuda:0")
    dC2 = torch.zeros(n * n, dtype=torch.float64, device="cuda:0")
    pl.dgemm("N", "N", n, n, n, 0.75, dA, n, dB, n, 0.0, dC1, n, ctl=pl.make_ctl(units=[0]))
    pl.dgemm("N", "N", n, n, n, 1.5, dA, n, dB, n, 0.0, dC2, n, ctl=pl.make_ctl(units=[0]))
    torch.cuda.synchronize()
    assert torch.equal(dC1 * 2.0, dC2)
    # spot-check 64 entries against float64 dot products of the same rows and columns
    A = dA.view(n, n).T   # A[i, k]
    B = dB.view(n, n).T
    idx = torch.randint(0, n, (64, 2), generator=torch.Generator().manual_seed(0))
    for i, j in idx.tolist():
        ref = torch.dot(A[i, :], B[:, j]).item() * 0.75
        assert abs(dC1.view(n, n).T[i, j].item() - ref) <= tol(n) * n ** 0.5


def test_dgemm_metadata_reuse(pl, orc):
    # second call with the same signature skips the autotuner (reference: PMD_cache,
    # dgemm.cpp:342-380) and gives the same bits
    M, N, K = 640, 512, 384
    A, B, C0, lda, ldb, ldc = _case(orc, "N", "T", M, N, K)
    C1, C2, C3 = (C0.copy(order="F") for _ in range(3))
    ctl = pl.make_ctl(T=128, units=[0])
    pl.dgemm("N", "T", M, N, K, 1.5, A, lda, B, ldb, 0.25, C1, ldc, ctl=ctl)
    r2 = pl.dgemm("N", "T", M, N, K, 1.5, A, lda, B, ldb, 0.25, C2, ldc, ctl=ctl)
    r3 = pl.dgemm("N", "T", M, N, K, 1.5, A, lda, B, ldb, 0.25, C3, ldc,
                  ctl=pl.make_ctl(T=128, units=[0], flags=pl.FLAG_NO_METADATA_REUSE))
    assert r2.metadata_reused == 1 and r3.metadata_reused == 0
    assert np.array_equal(C1, C2) and np.array_equal(C1, C3)


def test_dgemm_k_zero_and_empty(pl, orc):
    M, N = 64, 48
    C = orc.matrix_f64(M, N, 44)
    want = C * 0.5
    A = np.zeros((M, 1), order="F")
    B = np.zeros((1, N), order="F")
    pl.dgemm("N", "N", M, N, 0, 1.0, A, M, B, 1, 0.5, C, M, ctl=pl.make_ctl(units=[0]))
    np.testing.assert_allclose(C, want, rtol=1e-15)
    pl.dgemm("N", "N", 0, N, 8, 1.0, A, 1, B, 8, 0.5, C, 1, ctl=pl.make_ctl(units=[0]))  # no-op


def test_dgemm_invalid_arguments(pl, orc):
    A = orc.matrix_f64(8, 8, 1)
    with pytest.raises(pl.ParaliaError) as e:
        pl.dgemm("N", "N", 8, 8, 8, 1.0, A, 4, A, 8, 0.0, A, 8)      # ldA < M
    assert e.value.code == pl.ERR_INVALID_ARG
    with pytest.raises(pl.ParaliaError) as e:
        pl.dgemm("Q", "N", 8, 8, 8, 1.0, A, 8, A, 8, 0.0, A, 8)
    assert e.value.code == pl.ERR_INVALID_ARG
    with pytest.raises(pl.ParaliaError) as e:
        pl.dgemm("N", "N", 8, 8, 8, 1.0, A, 8, A, 8, 0.0, A, 8, locA=0)  # host pointer, GPU id
    assert e.value.code == pl.ERR_INVALID_ARG


def test_dgemm_cache_limit_too_small(pl, orc):
    M = N = K = 512
    A, B, C, lda, ldb, ldc = _case(orc, "N", "N", M, N, K)
    with pytest.raises(pl.ParaliaError) as e:
        pl.dgemm("N", "N", M, N, K, 1.0, A, lda, B, ldb, 0.5, C, ldc,
                 ctl=pl.make_ctl(T=128, units=[0], cache_limit=3 * 128 * 128 * 8))
    assert e.value.code == pl.ERR_OUT_OF_MEMORY       # beta != 0 needs A, B, accumulator, original C


@pytest.mark.parametrize("ta,tb", [("N", "N"), ("T", "N"), ("N", "T")])
@pytest.mark.parametrize("blocks", [4, 7, 20])
def test_dgemm_bounded_cache_recycles_blocks(pl, orc, ta, tb, blocks):
    # the reference's "run_large" cases (dgemm_tester.cpp:284-403): a cache far smaller than
    # the working set (64 blocks here) still gives the right answer, at the price of
    # fetching tiles more than once
    M, N, K, T = 1024, 1024, 1024, 256
    A, B, C, lda, ldb, ldc = _case(orc, ta, tb, M, N, K)
    want = C.copy(order="F")
    orc.dgemm_tiled(ta, tb, M, N, K, 1.23, A, lda, B, ldb, 0.9876, want, ldc, T)
    rep = pl.dgemm(ta, tb, M, N, K, 1.23, A, lda, B, ldb, 0.9876, C, ldc,
                   ctl=pl.make_ctl(T=T, units=[0], cache_limit=blocks * T * T * 8))
    assert orc.normwise_rel_err(C, want) <= tol(K)
    minimal = (M * K + K * N + M * N) * 8
    assert rep.h2d_bytes > minimal
    assert rep.d2h_bytes == M * N * 8
    # a larger cache re-fetches less
    if blocks == 4:
        rep2 = pl.dgemm(ta, tb, M, N, K, 1.23, A, lda, B, ldb, 0.0, C, ldc,
                        ctl=pl.make_ctl(T=T, units=[0], cache_limit=24 * T * T * 8))
        rep3 = pl.dgemm(ta, tb, M, N, K, 1.23, A, lda, B, ldb, 0.0, C, ldc,
                        ctl=pl.make_ctl(T=T, units=[0], cache_limit=4 * T * T * 8))
        assert rep2.h2d_bytes < rep3.h2d_bytes


def test_dgemm_bounded_cache_is_deterministic(pl, orc):
    M, N, K, T = 768, 768, 1024, 256
    A, B, C0, lda, ldb, ldc = _case(orc, "N", "N", M, N, K)
    outs = []
    for _ in range(2):
        C = C0.copy(order="F")
        pl.dgemm("N", "N", M, N, K, 1.23, A, lda, B, ldb, 0.9876, C, ldc,
                 ctl=pl.make_ctl(T=T, units=[0], cache_limit=6 * T * T * 8))
        outs.append(C)
    assert np.array_equal(outs[0], outs[1])


def test_fill_same_bits_on_host_and_device(pl, orc):
    import torch
    n = 100003
    d = torch.empty(n, dtype=torch.float64, device="cuda:0")
    pl.fill_f64(d, n, 42, 0, 0)
    h = np.empty(n)
    pl.fill_f64(h, n, 42, 0, -1)
    assert np.array_equal(d.cpu().numpy(), h)
    assert np.array_equal(h, orc.uniform_f64(n, 42))
    d32 = torch.empty(n, dtype=torch.float32, device="cuda:0")
    pl.fill_f32(d32, n, 43, 0, 0)
    assert np.array_equal(d32.cpu().numpy(), orc.uniform_f32(n, 43))


def test_call_waits_for_default_stream_work(pl, orc):
    # operands produced by still-running work on the default stream (torch's stream): the
    # call has to order itself after it although its own streams are non-blocking
    import torch
    M = N = K = 1024
    A, B, C, lda, ldb, ldc = _case(orc, "N", "N", M, N, K)
    want = C.copy(order="F")
    orc.dgemm_tiled("N", "N", M, N, K, 1.0, A, lda, B, ldb, 1.0, want, ldc, 512)
    dA, dB, dC0 = _dev(A), _dev(B), _dev(C)
    big = torch.empty(1 << 28, dtype=torch.float64, device="cuda:0")   # 2 GiB of queued work
    dC = torch.empty_like(dC0)
    torch.cuda.synchronize()
    for _ in range(8):
        big.add_(1.0)
    dC.copy_(dC0)                       # C becomes valid only after the queue above drains
    pl.dgemm("N", "N", M, N, K, 1.0, dA, lda, dB, ldb, 1.0, dC, ldc, locA=0, locB=0, locC=0,
             ctl=pl.make_ctl(T=512, units=[0]))
    assert orc.normwise_rel_err(_host(dC, C.shape), want) <= tol(K)


@pytest.mark.parametrize("dims,T", [((1156, 1412, 1228), 256), ((512, 512, 2304), 256)])
def test_executor_launches_what_the_plan_says(pl, orc, dims, T):
    # host-resident operands, whole working set cached: one kernel launch per plan item
    M, N, K = dims
    A, B, C, lda, ldb, ldc = _case(orc, "N", "N", M, N, K)
    rep = pl.dgemm("N", "N", M, N, K, 1.0, A, lda, B, ldb, 1.0, C, ldc, ctl=pl.make_ctl(T=T, units=[0]))
    items, grid = pl.plan_gemm(M, N, K, T, 1)
    assert rep.kernel_launches == len(items)
    assert (rep.grid_d1, rep.grid_d2) == grid


def test_dgemm_operands_are_interleaved_views_of_one_parent(pl, orc):
    """A and C are row ranges of ONE pageable parent matrix: their address ranges interleave
    column by column, so page-locking the first makes the second start inside a registered
    range that does not cover its end. The call must still succeed and be right."""
    M, N, K = 300, 256, 256          # A is M x K, C is M x N, both cut out of a (2M) x 256 parent
    parent = orc.matrix_f64(2 * M, 256, 77)
    A = parent[:M, :]
    C = parent[M:, :]
    B = orc.matrix_f64(K, N, 43)
    want = np.asfortranarray(C.copy())
    orc.dgemm_tiled("N", "N", M, N, K, 1.0, np.asfortranarray(A), M, B, K, 0.5, want, M, 128)
    pl.dgemm("N", "N", M, N, K, 1.0, A.ctypes.data, 2 * M, B, K, 0.5, C.ctypes.data, 2 * M,
             locA=-1, locB=-1, locC=-1, ctl=pl.make_ctl(T=128, units=[0]))
    assert orc.normwise_rel_err(C, want) <= tol(K)
    # the rows of the parent that belong to A are untouched
    assert np.array_equal(parent[:M, :], orc.matrix_f64(2 * M, 256, 77)[:M, :])
