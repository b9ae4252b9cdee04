"""Builds the CUDA backend in-tree: dooms_b200/csrc/**/*.{cu,cpp} -> dooms_b200/lib/libdooms_cuda.so, for sm_100a only.

    python -m dooms_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. Objects are rebuilt when a source or any header is newer than them.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "lib" / "obj"
LIB = ROOT / "lib" / "libdooms_cuda.so"
INCLUDE = ROOT.parent / "include"

NVCC_FLAGS = [
    "-std=c++20", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unknown-pragmas", f"-I{INCLUDE}", f"-I{CSRC}",
]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def sources() -> list[Path]:
    return sorted(list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cpp")))


def headers_mtime() -> float:
    hs = list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + list(INCLUDE.rglob("*.h")) + [Path(__file__)]
    return max(h.stat().st_mtime for h in hs)


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    hm = headers_mtime()
    jobs = []
    objs = []
    for src in sources():
        obj = OBJ / (str(src.relative_to(CSRC)).replace("/", "_") + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hm):
            extra = ["-Xptxas", "-v"] if verbose else []
            jobs.append([nvcc(), *NVCC_FLAGS, *extra, "-x", "cu", "-c", str(src), "-o", str(obj)])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    failed = False
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            failed |= r.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if jobs or not LIB.exists():
        cmd = [nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-ldl", "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
