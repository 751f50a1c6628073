"""Builds ``libmggb200.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

Run as ``python mgg_osdi23_b200/build.py`` (by path: importing the package itself needs the library
to exist already) or load this file by path and call :func:`build_library`.  The command-line drivers
are built by :func:`build_cli`.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libmggb200.so")
BIN_DIR = os.path.join(PKG_DIR, "bin")
OBJ_DIR = os.path.join(PKG_DIR, "_obj")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC,-fopenmp",
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compiles every source to an object file under ``_obj/`` (only the stale ones, in parallel) and
    links them into the shared library."""
    from concurrent.futures import ThreadPoolExecutor
    srcs = _sources()
    headers = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(PKG_DIR, "..", "include", "*.h"))
    os.makedirs(OBJ_DIR, exist_ok=True)
    objs = [os.path.join(OBJ_DIR, os.path.basename(src) + ".o") for src in srcs]

    def compile_one(pair):
        src, obj = pair
        if not force and not _stale(obj, [src] + headers):
            return None
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        return src, subprocess.run(cmd, capture_output=True, text=True)

    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
        results = [r for r in pool.map(compile_one, zip(srcs, objs)) if r is not None]
    for src, r in results:
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed compiling {src}")
    if not results and not _stale(LIB_PATH, objs):
        return LIB_PATH
    r = subprocess.run([_nvcc(), "-shared"] + objs + ["-o", LIB_PATH, "-lgomp"], capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed linking libmggb200.so")
    return LIB_PATH


def build_cli(force: bool = False, verbose: bool = False):
    """Builds the three command-line drivers (same names and argument order as the reference's)."""
    build_library(force=force, verbose=verbose)
    os.makedirs(BIN_DIR, exist_ok=True)
    out = []
    inc = os.path.join(PKG_DIR, "..", "include")
    for src in sorted(glob.glob(os.path.join(CSRC, "cli", "*.cu"))):
        exe = os.path.join(BIN_DIR, "MGG_" + os.path.splitext(os.path.basename(src))[0][len("mgg_"):])
        deps = [src, LIB_PATH] + glob.glob(os.path.join(inc, "*.h*")) + glob.glob(os.path.join(CSRC, "cli", "*.h*"))
        if force or _stale(exe, deps):
            cmd = [_nvcc(), "-std=c++17", "-O2", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
                   "-Xcompiler", "-fopenmp", "-I", inc, src, "-o", exe,
                   "-L", PKG_DIR, "-lmggb200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/..", "-lgomp"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed building {exe}")
        out.append(exe)
    return out


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    for e in build_cli(force="--force" in sys.argv, verbose="-v" in sys.argv):
        print(e)
