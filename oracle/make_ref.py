"""Installs the UNMODIFIED reference package into ``oracle/_ref`` (test and benchmark
infrastructure only; the directory is git-ignored and never imported by the product).

    python oracle/make_ref.py [--reference /path/to/reference/checkout]

The reference is a pure-Python project (setuptools, ``src/turboquant``).  It is installed with
pip, offline and without its dependencies (torch / transformers / numpy are already here):

    python -m pip install --no-index --no-build-isolation --no-deps \
        --find-links /opt/wheelhouse --target oracle/_ref <copy of the checkout>

The checkout is copied to a temporary directory first because the build writes an ``egg-info``
folder into the source tree and the checkout may be read-only.  With the package in place,
``bench.py --impl reference`` and ``bench.py``'s ``cpu_baseline`` time the reference's own CPU
code (``kind: "reference"``) instead of this repository's restatement of it, and
``bench.py --gpu-comparator`` can time the reference's GPU path next to this library's.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")


def installed() -> bool:
    return os.path.isfile(os.path.join(TARGET, "turboquant", "runtime", "packed_qmse_cache.py"))


def install(reference: str, force: bool = False) -> str:
    """Install the checkout at ``reference`` into ``oracle/_ref``; returns the target path."""
    if installed() and not force:
        return TARGET
    if not os.path.isfile(os.path.join(reference, "pyproject.toml")):
        raise FileNotFoundError(f"{reference} does not look like the reference checkout (no pyproject.toml)")
    shutil.rmtree(TARGET, ignore_errors=True)
    with tempfile.TemporaryDirectory(prefix="tq_ref_src_") as tmp:
        src = os.path.join(tmp, "reference")
        shutil.copytree(reference, src)
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--quiet",
               "--find-links", "/opt/wheelhouse", "--target", TARGET, src]
        subprocess.run(cmd, check=True)
    if not installed():
        raise RuntimeError("pip reported success but oracle/_ref/turboquant is incomplete")
    return TARGET


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("TQ_REFERENCE_SRC"), required="TQ_REFERENCE_SRC" not in os.environ,
                    help="root of the unmodified reference checkout")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(install(a.reference, a.force))
