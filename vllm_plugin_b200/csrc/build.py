"""Build ``libmmoe_b200.so`` (the C-ABI library of the MegaMoE expert backend) in-tree with nvcc for sm_100a.

    python vllm_plugin_b200/csrc/build.py [--verbose]

The library is written next to the package (``vllm_plugin_b200/_lib/``) so that it ships with the source tree.
"""

from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(os.path.dirname(HERE), "_lib")
SOURCES = ("mmoe_abi.cu", "mmoe_support.cu", "mmoe_umma.cu", "mmoe_umma_tm.cu", "mmoe_ep.cu", "mmoe_weights.cu")
LIB_NAME = "libmmoe_b200.so"


def lib_path() -> str:
    return os.path.join(OUT_DIR, LIB_NAME)


def needs_build() -> bool:
    out = lib_path()
    if not os.path.exists(out):
        return True
    newest = max(os.path.getmtime(os.path.join(HERE, f)) for f in os.listdir(HERE) if f.endswith((".cu", ".cuh")))
    header = os.path.join(os.path.dirname(os.path.dirname(HERE)), "include", "mmoe.h")
    return max(newest, os.path.getmtime(header)) > os.path.getmtime(out)


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and not needs_build():
        return lib_path()
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
           "-shared", "-o", lib_path()] + [os.path.join(HERE, s) for s in SOURCES]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building " + LIB_NAME)
    if verbose:
        sys.stderr.write(res.stderr)
    return lib_path()


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force=True))
