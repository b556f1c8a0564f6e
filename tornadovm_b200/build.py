"""In-tree build of libtornado_b200.so with nvcc for sm_100a (no GPU needed).

Every .cu file under csrc/ is one translation unit; they are compiled side by
side and linked into one shared library.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_DIR = os.path.join(PKG_DIR, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libtornado_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-diag-suppress", "1886", "-diag-suppress", "177",
]


def _units():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    return [os.path.join(INCLUDE, "tornado_b200.h")] + [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cuh", ".h"))]


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(s) > t for s in _headers() + [os.path.join(CSRC, u) for u in _units()])


def _compile(nvcc: str, unit: str, verbose: bool):
    obj = os.path.join(OBJ_DIR, unit[:-3] + ".o")
    cmd = [nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-I", CSRC]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-c", "-o", obj, os.path.join(CSRC, unit)]
    return unit, obj, subprocess.run(cmd, capture_output=True, text=True)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/*.cu (one object each, in parallel) and link lib/libtornado_b200.so.
    Objects newer than their source and every header are reused unless ``force``."""
    if not force and not needs_build():
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    newest_header = max(os.path.getmtime(h) for h in _headers())
    todo, objs = [], []
    for unit in _units():
        obj = os.path.join(OBJ_DIR, unit[:-3] + ".o")
        objs.append(obj)
        src_time = max(os.path.getmtime(os.path.join(CSRC, unit)), newest_header)
        if force or verbose or not os.path.exists(obj) or os.path.getmtime(obj) < src_time:
            todo.append(unit)
    with ThreadPoolExecutor(max_workers=max(1, min(len(todo), os.cpu_count() or 1))) as pool:
        results = list(pool.map(lambda u: _compile(nvcc, u, verbose), todo))
    for unit, _, res in results:
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError(f"nvcc failed on {unit}")
        if verbose:
            sys.stderr.write(res.stderr)
    res = subprocess.run([nvcc, "-shared", "-o", LIB_PATH, *objs, "-lcudart"], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("linking libtornado_b200.so failed")
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
