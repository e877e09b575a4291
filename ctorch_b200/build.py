"""Builds ctorch_b200/libctorch_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m ctorch_b200.build [--force] [--verbose]

Every .cu / .cpp under ctorch_b200/csrc is compiled to an object under ctorch_b200/build/ (rebuilt only when the
source or a header is newer) and linked into one shared library with a static CUDA runtime, so that the library
loads on machines without a GPU or driver.

The library's SONAME is libctorch_b200.so.  Beside it the build leaves the reference package's names as symbolic
links (libctorch.so and libctorch.so.0: target `ctorch`, SOVERSION 0), so that a program built for the reference
with `-lctorch` and the headers under include/dl/ links against this directory unchanged.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libctorch_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++20",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wextra,-Wno-unused-parameter",
    "--expt-relaxed-constexpr", "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-I", os.path.join(CSRC, "kernels"),
]


def sources() -> list[str]:
    found = []
    for base, _, files in os.walk(CSRC):
        for name in sorted(files):
            if name.endswith((".cu", ".cpp")):
                found.append(os.path.join(base, name))
    return sorted(found)


def headers_mtime() -> float:
    newest = 0.0
    for top in (CSRC, os.path.join(ROOT, "include")):
        for base, _, files in os.walk(top):
            for name in files:
                if name.endswith((".h", ".cuh", ".hpp")):
                    newest = max(newest, os.path.getmtime(os.path.join(base, name)))
    return newest


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    newest_header = headers_mtime()
    jobs, objects = [], []
    for src in sources():
        obj = os.path.join(OBJ, os.path.relpath(src, CSRC).replace(os.sep, "__") + ".o")
        objects.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), newest_header)
        if stale:
            cmd = [NVCC, *FLAGS, "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            if src.endswith(".cpp"):
                cmd[1:1] = ["-x", "cu"]
            jobs.append(cmd)

    def run(cmd):
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0 or verbose:
            sys.stderr.write(" ".join(cmd[-3:]) + "\n" + result.stdout + result.stderr)
        if result.returncode != 0:
            raise RuntimeError("nvcc failed on " + cmd[-3])

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(run, jobs))
    if jobs or not os.path.exists(LIB):
        link = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
                "-Xcompiler", "-fPIC", "-Xlinker", "-soname=libctorch_b200.so", "-o", LIB, *objects, "-lpthread", "-ldl"]
        result = subprocess.run(link, capture_output=True, text=True)
        if result.returncode != 0:
            sys.stderr.write(result.stdout + result.stderr)
            raise RuntimeError("link failed")
    for alias in ("libctorch.so", "libctorch.so.0"):   # the reference package's library names
        path = os.path.join(HERE, alias)
        if not os.path.islink(path):
            if os.path.exists(path):
                os.remove(path)
            os.symlink("libctorch_b200.so", path)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
