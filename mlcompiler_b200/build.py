"""Compile the CUDA sources of this package into mlcompiler_b200/libmlc_b200.so.

Everything is built for sm_100a only (`-gencode arch=compute_100a,code=sm_100a`),
in-tree, with the CUDA runtime linked statically so that the library loads - and
the host-side objects in it work - on a machine without a GPU or a driver.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "_build"
LIB = PKG / "libmlc_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "--expt-relaxed-constexpr",
    "-cudart", "static",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built")
    return exe


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _newest_header() -> float:
    hdrs = list(CSRC.glob("*.hpp")) + list(CSRC.glob("*.h")) + list((PKG.parent / "include").glob("*.h"))
    return max((h.stat().st_mtime for h in hdrs), default=0.0)


def _compile(src: Path, hdr_time: float, verbose: bool, extra: list[str]) -> Path:
    obj = OBJ / (src.name + ".o")
    if obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, hdr_time,
                                                   Path(__file__).stat().st_mtime):
        return obj
    cmd = [nvcc(), *NVCC_FLAGS, *extra, "-x", "cu", "-c", str(src), "-o", str(obj)]
    if verbose:
        print("[build]", " ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True)
    return obj


def build(verbose: bool = False, ptxas_info: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    hdr_time = _newest_header()
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as ex:
        objs = list(ex.map(lambda s: _compile(s, hdr_time, verbose, extra), srcs))
    if LIB.exists() and all(LIB.stat().st_mtime >= o.stat().st_mtime for o in objs):
        return LIB
    cmd = [nvcc(), "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
           "-o", str(LIB), *map(str, objs), "-lpthread", "-ldl"]
    if verbose:
        print("[build]", " ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    build(verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(LIB)
