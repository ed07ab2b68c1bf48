"""The hand-shake layer of process groups, exercised on the CPU with real processes.

A rank that fails inside a collective (bad argument, failed allocation) or that never
arrives must not cost its peers the full time-out, and must not leave the arrival counter
off by one for later hand-shakes: the group is abandoned, and every later hand-shake of
every rank fails at once with the reason. No GPU is involved (the rendezvous is a POSIX
shared-memory segment), so nothing here can fault or hang a device."""
import multiprocessing as mp
import os
import sys
import time
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _rank(rank, world, name, rounds, fail_rank, fail_round, fail_mode, timeout_ms, q):
    os.environ["PARALIA_GROUP_TIMEOUT_MS"] = str(timeout_ms)
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    pl = entry.load_package()
    t0 = time.perf_counter()
    rc, waited = pl.selftest_group_rendezvous(name, rank, world, rounds, fail_rank, fail_round, fail_mode)
    msg = pl.lib().PARALiA_last_error().decode() if rc else ""
    q.put((rank, rc, waited, time.perf_counter() - t0, msg))


def _run(world, rounds, fail_rank=-1, fail_round=0, fail_mode=0, timeout_ms=20000):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    name = f"rv{os.getpid()}_{world}_{fail_mode}_{fail_round}_{int(time.time() * 1e3) % 100000}"
    procs = [ctx.Process(target=_rank, args=(r, world, name, rounds, fail_rank, fail_round, fail_mode,
                                             timeout_ms, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    return out


def test_all_ranks_pass_every_barrier(pl):
    for (_rank_id, rc, _w, _t, _m) in _run(3, 50):
        assert rc == pl.OK


def test_a_rank_that_reports_an_error_releases_its_peers_at_once(pl):
    # rank 1 fails at round 2 the way a collective call with a bad argument does; the time-out
    # is 20 s, the peers must be back within a small fraction of it
    res = _run(3, 6, fail_rank=1, fail_round=2, fail_mode=1, timeout_ms=20000)
    for (rank, rc, waited, total, msg) in res:
        if rank == 1:
            assert rc == pl.ERR_INVALID_ARG
        else:
            assert rc == pl.ERR_GROUP_FAILED, msg
            assert "abandoned by rank 1" in msg and "injected failure" in msg
            assert waited < 2000.0 and total < 10.0


def test_a_missing_rank_times_out_once_and_abandons_the_group(pl):
    # rank 2 silently stops arriving at round 1: the first peer to time out abandons the group,
    # the other follows without waiting out its own time-out on a later hand-shake
    res = _run(3, 4, fail_rank=2, fail_round=1, fail_mode=2, timeout_ms=1500)
    codes = {rank: rc for (rank, rc, _w, _t, _m) in res}
    assert codes[2] == pl.ERR_UNSUPPORTED            # the injected "stops arriving"
    assert set(codes[r] for r in (0, 1)) <= {pl.ERR_TIMEOUT, pl.ERR_GROUP_FAILED}
    assert pl.ERR_TIMEOUT in (codes[0], codes[1])
    for (rank, rc, waited, total, msg) in res:
        if rank != 2:
            assert 1000.0 < waited < 6000.0 and total < 15.0
