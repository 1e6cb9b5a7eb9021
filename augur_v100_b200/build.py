"""Builds the sm_100a NVFP4 shared library in-tree with nvcc.

``python -m augur_v100_b200.build`` compiles every ``csrc/*.cu`` for
``sm_100a`` only and writes ``libaugur_nvfp4_sm100.so`` next to this file.
nvcc cross-compiles, so this works on a machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
LIB = HERE / "libaugur_nvfp4_sm100.so"
SOURCES = sorted((HERE / "csrc").glob("*.cu"))
HEADERS = sorted((HERE / "csrc").glob("*.h")) + sorted((HERE / "csrc").glob("*.cuh")) + [
    ROOT / "include" / "augur_cuda_nvfp4_sm100.h"]


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the sm_100a library cannot be built")
    return found


def is_stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in SOURCES + HEADERS)
    return LIB.stat().st_mtime < newest


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return LIB
    objects = []
    build_dir = HERE / "build"
    build_dir.mkdir(exist_ok=True)
    common = [
        nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC", "-DAUGUR_SM100A_BUILD", "-I", str(ROOT / "include"), "-I", str(HERE / "csrc"),
        "-ccbin", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++",
    ]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    for source in SOURCES:
        obj = build_dir / (source.stem + ".o")
        objects.append(obj)
        procs.append((source, subprocess.Popen(common + ["-c", str(source), "-o", str(obj)],
                                               stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for source, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0 or verbose:
            sys.stderr.write(f"--- {source.name} ---\n{out}\n")
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.run(common[:1] + ["-shared", "-o", str(LIB)] + [str(o) for o in objects] +
                   ["-ccbin", common[common.index("-ccbin") + 1], "-cudart", "static"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
