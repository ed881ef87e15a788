"""Builds ``libcrystalformer_b200.so`` in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m crystalformer_b200.build [--verbose]

The library is rebuilt only when a source is newer than the existing binary.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
LIB_PATH = os.path.join(PKG, "libcrystalformer_b200.so")
SOURCES = sorted(glob.glob(os.path.join(PKG, "csrc", "*.cu")))
HEADERS = sorted(glob.glob(os.path.join(PKG, "csrc", "*.cuh"))) + [os.path.join(ROOT, "include", "crystalformer_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "--std=c++17",
    "-Xcompiler", "-fPIC", "-shared", "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(PKG, "csrc"),
]


def up_to_date() -> bool:
    if not os.path.exists(LIB_PATH):
        return False
    built = os.path.getmtime(LIB_PATH)
    return all(os.path.getmtime(f) <= built for f in SOURCES + HEADERS + [os.path.abspath(__file__)])


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + SOURCES + ["-o", LIB_PATH]
    env = dict(os.environ)
    # the host compiler must be the system gcc
    env["PATH"] = "/usr/bin:" + env.get("PATH", "")
    proc = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if verbose:
        sys.stderr.write(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose="--verbose" in sys.argv))
