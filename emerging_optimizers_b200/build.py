"""Build ``libeo_b200.so`` in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Usage: ``python -m emerging_optimizers_b200.build [--force] [--verbose]``
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys


PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
OUT = os.path.join(PKG_DIR, "libeo_b200.so")
SOURCES = ["eo_b200.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-shared", "-Xcompiler", "-fPIC",
]  # fmt: skip


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libeo_b200.so cannot be built")
    return exe


def _inputs() -> list[str]:
    files = []
    for root in (CSRC, os.path.join(os.path.dirname(PKG_DIR), "include")):
        for name in sorted(os.listdir(root)):
            if name.endswith((".cu", ".cuh", ".h")):
                files.append(os.path.join(root, name))
    return files


def needs_build() -> bool:
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    return any(os.path.getmtime(f) > built for f in _inputs())


def build(force: bool = False, verbose: bool = False, extra_flags: list[str] | None = None) -> str:
    """Compile the library if any source is newer than it; return the path of the shared object."""
    if not force and not needs_build():
        return OUT
    cmd = [_nvcc(), *NVCC_FLAGS, *(extra_flags or [])]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    tmp = f"{OUT}.{os.getpid()}.tmp"  # a reader never sees a half-written library
    cmd += ["-o", tmp, *[os.path.join(CSRC, s) for s in SOURCES]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, OUT)
    if verbose:
        print(res.stderr, file=sys.stderr)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--define", action="append", default=[])
    args = ap.parse_args()
    print(build(args.force, args.verbose, [f"-D{d}" for d in args.define]))
