"""Build recipe of libbonsai_cuda.so (hand-written sm_100a kernels + the C ABI) and of the host
tools. Everything is compiled in-tree with nvcc / g++; nothing is installed."""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libbonsai_cuda.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    # no silent fused multiply-add: the kernels spell fmaf() where the arithmetic contract has one
    "-fmad=false",
    "-Xcompiler", "-fPIC", "-shared",
]


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_lib(verbose: bool = False, force: bool = False) -> str:
    srcs = sorted(glob.glob(os.path.join(HERE, "csrc", "*.cu")))
    deps = srcs + glob.glob(os.path.join(HERE, "csrc", "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    if not force and not _stale(LIB, deps):
        return LIB
    cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + srcs
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed building libbonsai_cuda.so")
    return LIB


HOST_BIN = os.path.join(HERE, "host", "bonsai_run")


def build_host(force: bool = False) -> str:
    """The C++ command-line host (GGUF reader, contract checks, loader, run mode). Links the library by
    path and finds it next to the package at run time ($ORIGIN/..)."""
    srcs = [os.path.join(HERE, "host", "bonsai_run.cpp")]
    deps = srcs + [os.path.join(HERE, "host", "bonsai_host.h"), LIB] + glob.glob(os.path.join(ROOT, "include", "*.h"))
    if not force and not _stale(HOST_BIN, deps):
        return HOST_BIN
    cmd = ["g++", "-O2", "-std=c++17", "-Wall", "-o", HOST_BIN] + srcs + ["-L" + HERE, "-lbonsai_cuda", "-Wl,-rpath,$ORIGIN/.."]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("g++ failed building bonsai_run")
    return HOST_BIN


def build_oracle() -> None:
    """Compile the CPU checker under oracle/ (and the reference shim when the reference tree is
    present). Building the checker is not using it: only tests and the benchmark baselines load it."""
    # the reference tree: $BONSAI_REF, else a directory named "reference" beside this repository
    ref = os.environ.get("BONSAI_REF") or os.path.join(os.path.dirname(ROOT), "reference")
    cmd = ["make", "-C", os.path.join(ROOT, "oracle")] + ([f"REF={ref}"] if os.path.isdir(os.path.join(ref, "runtime_vk")) else [])
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("oracle build failed")


if __name__ == "__main__":
    build_lib(verbose="-v" in sys.argv, force=True)
    build_host(force=True)
    build_oracle()
    print("built", LIB)
