"""Ahead-of-time build of the CUDA library (sm_100a only).

The reference JIT-compiles one kernel per call site with nvcc
(tilelang/cuda/backend.py:59-120, ``-arch=sm_100a`` chosen in
tilelang/contrib/nvcc.py:523-531). This library has a fixed kernel set, so it is
compiled once into ``libb200dq.so`` next to this file.
"""
from __future__ import annotations

import os
import re
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(_HERE, "libb200dq.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _sources():
    return [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".cu")]


def _inputs():
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    paths.append(os.path.join(os.path.dirname(_HERE), "include", "b200dq.h"))
    return [p for p in paths if os.path.isfile(p)]


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(p) > t for p in _inputs())


_INCLUDE_RE = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)


def _deps(path, seen=None):
    """The file and every quoted include it reaches (so one object is rebuilt only when a
    header it really uses changed)."""
    seen = set() if seen is None else seen
    path = os.path.normpath(path)
    if path in seen or not os.path.isfile(path):
        return seen
    seen.add(path)
    with open(path, "r", encoding="utf-8") as f:
        text = f.read()
    for inc in _INCLUDE_RE.findall(text):
        _deps(os.path.join(os.path.dirname(path), inc), seen)
    return seen


def _object_is_stale(src, obj):
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(d) > t for d in _deps(src))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every ``csrc/*.cu`` (only the objects whose sources changed, unless ``force``)
    and link them into ``libb200dq.so``; returns its path."""
    nvcc = os.environ.get("NVCC", "nvcc")
    objs = []
    procs = []
    for src in _sources():
        obj = os.path.splitext(src)[0] + ".o"
        objs.append(obj)
        if not force and not _object_is_stale(src, obj):
            continue
        cmd = [nvcc, *[f for f in NVCC_FLAGS if f != "-shared"], "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), file=sys.stderr)
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose and out:
            print(out, file=sys.stderr)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed ({' '.join(cmd)}):\n{out}")
    if not procs and os.path.exists(LIB_PATH) and all(os.path.getmtime(o) <= os.path.getmtime(LIB_PATH) for o in objs):
        return LIB_PATH
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH, *objs]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
