"""Build libparalia.so (sm_100a only) with nvcc, in-tree.

Each translation unit under csrc/ is compiled to an object file (in parallel) and the
objects are linked into ``paralia-framework_b200/lib/libparalia.so``. A source is
recompiled only when it, or any header next to it, is newer than its object.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "_build"
LIB_PATH = PKG_DIR / "lib" / "libparalia.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
          "-Xptxas", "-v"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; libparalia.so cannot be built")
    return cand


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _headers_mtime() -> float:
    hdrs = list(CSRC.glob("*.h")) + list(CSRC.glob("*.hpp")) + list(CSRC.glob("*.cuh"))
    hdrs += list((PKG_DIR.parent / "include").glob("*.h*"))
    return max((h.stat().st_mtime for h in hdrs), default=0.0)


def _compile_one(src: Path, hdr_mtime: float, force: bool, verbose: bool) -> Path:
    obj = OBJ_DIR / (src.name + ".o")
    if (not force and obj.exists() and obj.stat().st_mtime > src.stat().st_mtime
            and obj.stat().st_mtime > hdr_mtime):
        return obj
    cmd = [_nvcc(), *ARCH_FLAGS, *COMMON, "-x", "cu", "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        (OBJ_DIR / (src.name + ".ptxas.txt")).write_text(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = True) -> Path:
    """Compile and link; returns the path of the shared library."""
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_PATH.parent.mkdir(exist_ok=True)
    srcs = _sources()
    hdr_mtime = _headers_mtime()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, hdr_mtime, force, verbose), srcs))
    newest = max(o.stat().st_mtime for o in objs)
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest:
        cmd = [_nvcc(), *ARCH_FLAGS, "-shared", "-o", str(LIB_PATH), *map(str, objs),
               "-cudart", "static", "-lpthread", "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    p = build(force="--force" in sys.argv)
    print(p)
