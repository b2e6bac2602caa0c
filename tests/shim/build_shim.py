#!/usr/bin/env python3
"""Compiles include/mlc_b200_shim.cpp and tests/shim/shim_driver.cpp against the reference's own
header (compiler/runtime/metal_runtime.hpp in the MLcompiler checkout, MLC_REFERENCE_ROOT) and links
them with mlcompiler_b200/libmlc_b200.so into tests/shim/_built/shim_driver.

That the two files compile against the unmodified header is the proof that callers written for
mlc::runtime::MetalExecutor keep compiling; the binary it leaves behind (git-ignored, found through
an rpath relative to itself) is what the GPU test runs, also on a machine without the checkout.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parents[1]
OUT = HERE / "_built"
BINARY = OUT / "shim_driver"
SOURCES = [REPO / "include" / "mlc_b200_shim.cpp", HERE / "shim_driver.cpp"]
CXX = os.environ.get("CXX", "g++")


def reference_root() -> Path | None:
    root = Path(os.environ.get("MLC_REFERENCE_ROOT", str(REPO.parent / "reference")))
    return root if (root / "compiler" / "runtime" / "metal_runtime.hpp").exists() else None


def build(verbose: bool = False) -> Path | None:
    """Returns the binary, rebuilt when the checkout is present and a source is newer; a binary
    built earlier is returned as it is when the checkout is absent; None when there is neither."""
    root = reference_root()
    lib = REPO / "mlcompiler_b200" / "libmlc_b200.so"
    if root is None:
        return BINARY if BINARY.exists() else None
    if not lib.exists():
        raise RuntimeError(f"{lib} is missing: build the CUDA library first")
    newest = max(p.stat().st_mtime for p in [*SOURCES, REPO / "include" / "mlc_b200.h", Path(__file__)])
    if BINARY.exists() and BINARY.stat().st_mtime >= newest:
        return BINARY
    OUT.mkdir(exist_ok=True)
    cmd = [CXX, "-std=c++17", "-O2", "-Wall", "-Wextra", "-Werror", f"-I{root}", f"-I{root}/compiler",
           f"-I{REPO}/include", *map(str, SOURCES), "-o", str(BINARY), f"-L{lib.parent}", "-lmlc_b200",
           "-Wl,-rpath,$ORIGIN/../../../mlcompiler_b200"]
    if verbose:
        print("[shim]", " ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True)
    return BINARY


if __name__ == "__main__":
    b = build(verbose=True)
    print(b if b else "reference checkout absent and no binary built earlier")
    sys.exit(0 if b else 1)
