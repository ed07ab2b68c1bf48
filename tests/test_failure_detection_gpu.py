"""Failure detection without faulting a GPU: a device-side wait that can never be
satisfied gives up after its budget and reports through the status word; a rank that
never joins a group is reported by a bounded barrier. The CUDA context stays usable."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_bounded_wait_gives_up_and_context_survives(pl, orc):
    import torch
    pl.init()
    with pytest.raises(pl.ParaliaError) as e:
        pl.selftest_bounded_wait(0, 2.0)
    assert e.value.code == pl.ERR_TIMEOUT
    assert "bounded wait" in str(e.value)
    # the status word was cleared and the GPU still computes correctly
    M = N = K = 256
    A = orc.matrix_f64(M, K, 42)
    B = orc.matrix_f64(K, N, 43)
    C = orc.matrix_f64(M, N, 44)
    want = C.copy(order="F")
    orc.dgemm_tiled("N", "N", M, N, K, 1.0, A, M, B, K, 1.0, want, M, 128)
    pl.dgemm("N", "N", M, N, K, 1.0, A, M, B, K, 1.0, C, M, ctl=pl.make_ctl(T=128, units=[0]))
    assert orc.normwise_rel_err(C, want) <= 8 * K * 2.0 ** -52
    assert torch.cuda.is_available()


def _lonely_rank(out_path):
    sys.path.insert(0, str(ROOT))
    os.environ["PARALIA_GROUP_TIMEOUT_MS"] = "1500"
    import time
    import __graft_entry__ as entry
    pl = entry.load_package()
    t0 = time.perf_counter()
    try:
        pl.group_init(f"lonely_{os.getpid()}", 0, 2, 0)   # rank 1 never shows up
        res = "joined"
    except pl.ParaliaError as e:
        res = f"{e.code}:{time.perf_counter() - t0:.2f}"
    # after the failed hand-shake the process can still use the library on its own
    import numpy as np
    x = np.ones(1024)
    d, _ = pl.ddot(1024, x, 1, x, 1, 0.0, ctl=pl.make_ctl(units=[0]))
    open(out_path, "w").write(f"{res}:{d}")


def test_missing_rank_is_reported_by_a_bounded_barrier(pl, tmp_path):
    import torch.multiprocessing as mp
    out = tmp_path / "res.txt"
    ctx = mp.get_context("spawn")
    p = ctx.Process(target=_lonely_rank, args=(str(out),))
    p.start()
    p.join(120)
    assert p.exitcode == 0
    code, secs, dot = out.read_text().split(":")
    assert int(code) == pl.ERR_TIMEOUT
    assert 1.0 < float(secs) < 30.0
    assert float(dot) == 1024.0


def test_host_join_has_a_deadline(pl):
    """The whole-problem routines join their GPUs by waiting for an end event with a deadline.
    A kernel that ends by itself after 300 ms is queued; a join with a 50 ms deadline must come
    back with a time-out (instead of blocking) and the context must stay usable."""
    import time
    pl.init()
    t0 = time.perf_counter()
    with pytest.raises(pl.ParaliaError) as e:
        pl.selftest_join_deadline(0, 300.0, 50.0)
    dt = time.perf_counter() - t0
    assert e.value.code == pl.ERR_TIMEOUT and "deadline" in str(e.value)
    assert dt < 5.0
    # a deadline longer than the kernel: the join succeeds
    pl.selftest_join_deadline(0, 20.0, 5000.0)
    x = np.ones(4096)
    d, _ = pl.ddot(4096, x, 1, x, 1, 0.0, ctl=pl.make_ctl(units=[0]))
    assert d == 4096.0
