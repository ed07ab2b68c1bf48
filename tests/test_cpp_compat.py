"""A C++ program written against ``include/PARALiA.hpp`` the way the reference's runners
call the library (Benchmarking/CuCuBLAS/src/PARALia/dgemm_runner.cpp:80-151): it must
compile and link unchanged against ``libparalia.so`` (checked without a GPU) and, on a GPU,
every routine must agree with naive loops (tests/cpp/compat_caller.cpp)."""
import os
import pathlib
import subprocess

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
SRC = ROOT / "tests" / "cpp" / "compat_caller.cpp"


def _build(pl, out_dir) -> pathlib.Path:
    exe = pathlib.Path(out_dir) / "compat_caller"
    lib_dir = pl.LIB_PATH.parent
    cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-I", str(ROOT / "include"), str(SRC),
           "-L", str(lib_dir), "-lparalia", f"-Wl,-rpath,{lib_dir}",
           "-Wl,-rpath-link,/usr/local/cuda/lib64", "-o", str(exe)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def test_reference_style_caller_compiles_and_links(pl, tmp_path):
    exe = _build(pl, tmp_path)
    assert exe.exists()
    undefined = subprocess.run(["nm", "-u", "-C", str(exe)], check=True, capture_output=True,
                               text=True).stdout
    for name in ("PARALiADgemm(", "PARALiADgemmControled(", "PARALiASgemm(", "PARALiADgemv(",
                 "PARALiADaxpy(", "PARALiADdot(", "PARALiADevCacheFree(short)"):
        assert name in undefined, name      # resolved by libparalia.so at load time


@pytest.mark.gpu
def test_reference_style_caller_runs(pl, tmp_path):
    exe = _build(pl, tmp_path)
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = "/usr/local/cuda/lib64:" + env.get("LD_LIBRARY_PATH", "")
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "ALL OK" in res.stdout and "FAILED" not in res.stdout
    assert res.stdout.count(" ok\n") == 7     # seven report lines
