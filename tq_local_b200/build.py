"""Builds the CUDA library in-tree with nvcc for sm_100a.

``python -m tq_local_b200.build`` (or ``build_library()``) compiles every ``.cu``
under ``csrc/`` into ``tq_local_b200/libtq_b200.so``.  Nothing is JIT-compiled at
import time; the package fails loudly when the library is missing.

``--checked`` (``build_library(checked=True)``) builds ``libtq_b200_checked.so`` from the same
sources with ``-DTQ_DEBUG_BOUNDS``: the decode kernel then checks every bulk-copy request and
every partial it stores against the cache's and the workspace's extents, records a violation in
the device status word (6) and drops the access instead of making it.  Point the environment
variable ``TQ_B200_LIBRARY`` at it to run anything (the test suite included) on the checked build;
``compute-sanitizer`` is not available where this library is developed, this build stands in.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtq_b200.so")
LIB_CHECKED = os.path.join(HERE, "libtq_b200_checked.so")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--shared",
]


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps() -> list[str]:
    inc = os.path.join(os.path.dirname(HERE), "include", "tq_b200.h")
    return sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")] + [inc]


def is_stale(lib: str = LIB) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    return any(os.path.getmtime(p) > t for p in _deps())


def build_library(force: bool = False, verbose: bool = False, extra: list[str] | None = None,
                  checked: bool = False) -> str:
    lib = LIB_CHECKED if checked else LIB
    if not force and not is_stale(lib):
        return lib
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    objs = []
    procs = []
    obj_dir = os.path.join(HERE, "build_checked" if checked else "build")
    os.makedirs(obj_dir, exist_ok=True)
    flags = [f for f in NVCC_FLAGS if f != "--shared"] + (["-Xptxas", "-v"] if verbose else []) + (extra or []) \
        + (["-DTQ_DEBUG_BOUNDS"] if checked else [])
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if not force and os.path.exists(obj) and all(
                os.path.getmtime(obj) > os.path.getmtime(p)
                for p in [src] + [d for d in _deps() if d.endswith((".cuh", ".h"))]):
            continue
        procs.append((src, subprocess.Popen([nvcc, *flags, "-c", src, "-o", obj],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    # cudart is linked statically (nvcc default) so the library does not depend on which
    # libcudart.so the host process happens to have loaded.
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "--shared", "-o", lib, *objs], check=True)
    return lib


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv, checked="--checked" in sys.argv))
