"""Host-side rules of the vendor comparators and of the package's imports.

cuBLASXt (the reference's comparator, Benchmarking/CuCuBLAS/src/cuBLASXt/cuBLASXtWrappers.cpp:30-75)
runs vendor GEMM kernels on each GPU of its device list. Such a kernel must never be handed an
operand that lives on another GPU, so the binding refuses those placements before any CUDA
call; and nothing under the package directory may import the CPU oracle.
"""
import importlib
import pathlib
import re

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
PKG = ROOT / "paralia-framework_b200"


@pytest.fixture(scope="module")
def xt(pl):
    return importlib.import_module("paralia_framework_b200.comparators")


@pytest.mark.parametrize("devs,locs", [
    ((0, 1), (0, -1, -1)),        # two GPUs, A on GPU 0
    ((0, 1), (-1, 1, -1)),
    ((0, 1, 2, 3), (0, 0, 0)),
    ((0,), (1, -1, -1)),          # one GPU, operand on a different one
    ((1,), (1, 0, -1)),
    ((), (-1, -1, -1)),
])
def test_placements_that_are_refused(xt, devs, locs):
    with pytest.raises(xt.ComparatorRefused):
        xt.check_xt_placement(devs, locs)
    # the GEMM binding refuses before it touches CUDA (there is no GPU in a CPU run)
    with pytest.raises(xt.ComparatorRefused):
        xt.cublasxt_gemm(8, "N", "N", 4, 4, 4, 1.0, 0, 4, 0, 4, 0.0, 0, 4, dev_ids=devs, locs=locs)


@pytest.mark.parametrize("devs,locs", [
    ((0, 1, 2, 3), (-1, -1, -1)),  # any number of GPUs on host operands
    ((0,), (-1, -1, -1)),
    ((0,), (0, 0, 0)),            # one GPU that holds its own operands
    ((2,), (2, -1, 2)),
])
def test_placements_that_are_allowed(xt, devs, locs):
    xt.check_xt_placement(devs, locs)


def test_package_files_do_not_import_the_oracle():
    pat = re.compile(r"^\s*(import\s+oracle\b|from\s+oracle\b)", re.M)
    bad = [p.name for p in PKG.glob("*.py") if pat.search(p.read_text())]
    assert bad == []
