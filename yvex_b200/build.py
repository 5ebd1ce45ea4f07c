"""Builds yvex_b200/libyvex_b200.so in-tree: every .cu under csrc/ for sm_100a with nvcc, every
C11 host file under host/ with the C compiler, linked into one shared library.

    python -m yvex_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
HOST = os.path.join(HERE, "host")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libyvex_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-I", INCLUDE]
CC_FLAGS = ["-O2", "-std=c11", "-fPIC", "-Wall", "-Wextra", "-I", INCLUDE, "-I", "/usr/local/cuda/include"]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _sources():
    cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    c = sorted(f for f in os.listdir(HOST) if f.endswith(".c")) if os.path.isdir(HOST) else []
    return cu, c


def _newest_dep():
    newest = 0.0
    for d in (CSRC, HOST, INCLUDE):
        if os.path.isdir(d):
            for f in os.listdir(d):
                newest = max(newest, os.path.getmtime(os.path.join(d, f)))
    return newest


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_dep():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    cu, c = _sources()
    jobs = []
    for f in cu:
        obj = os.path.join(OBJ, f + ".o")
        jobs.append(([_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c",
                      os.path.join(CSRC, f), "-o", obj], obj))
    for f in c:
        obj = os.path.join(OBJ, f + ".o")
        jobs.append(([os.environ.get("CC", "gcc"), *CC_FLAGS, "-c", os.path.join(HOST, f), "-o", obj], obj))

    def run(job):
        cmd, _ = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("build failed: %s\n%s%s" % (" ".join(cmd), r.stdout, r.stderr))
        return r.stderr if verbose else ""

    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
        for log in pool.map(run, jobs):
            if log:
                sys.stderr.write(log)
    link = [_nvcc(), "-shared", "-o", LIB, *[o for _, o in jobs], "-lpthread", "-ldl"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
