"""Build libbibo_moe.so in-tree with nvcc for sm_100a.

    python -m bibo_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU, so this also runs on a CPU-only machine.
"""
from __future__ import annotations

import os
import pathlib
import subprocess
import sys

CSRC = pathlib.Path(__file__).resolve().parent / "csrc"
LIB = CSRC / "libbibo_moe.so"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def sources():
    return sorted(CSRC.glob("*.cu"))


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [CSRC.parents[1] / "include" / "bibo_moe.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    objs = []
    procs = []
    for src in sources():
        obj = src.with_suffix(".o")
        cmd = [nvcc, *ARCH, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            print(f"--- {src.name}\n{out}", file=sys.stderr)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [nvcc, *ARCH, "-shared", "-o", str(LIB), *objs, "-lcudart"]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
