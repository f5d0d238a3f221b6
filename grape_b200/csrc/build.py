"""Builds the CUDA shared library of the package in-tree with nvcc for sm_100a.

    python grape_b200/csrc/build.py [--force] [-v]

The library is ``grape_b200/libgrape_b200.so``; it is rebuilt when any source under
``grape_b200/csrc`` or ``include`` is newer than it.  This file is a plain script (it does not
import the package, whose import needs the library to exist already).
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parents[1]
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "libgrape_b200.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def sources():
    return sorted(CSRC.glob("*.cu"))


def _deps():
    return [p for p in CSRC.glob("*") if p.suffix in (".cu", ".cuh", ".hpp", ".h")] + list((ROOT / "include").glob("*.h"))


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    return any(p.stat().st_mtime > t for p in _deps())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    objs = []
    procs = []
    build_dir = PKG / "build"
    build_dir.mkdir(exist_ok=True)
    for src in sources():
        obj = build_dir / (src.stem + ".o")
        objs.append(obj)
        cmd = [NVCC, *ARCH, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-O2,-fopenmp",
               "-I", str(ROOT / "include"), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {src.name}:\n{out}\n")
        elif verbose or out.strip():
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("grape_b200: CUDA build failed")
    link = [NVCC, *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-Xcompiler", "-fopenmp", "-lcudart"]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
