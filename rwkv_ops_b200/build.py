"""Build librwkv_ops_b200.so (sm_100a only) in-tree with nvcc.

    python -m rwkv_ops_b200.build [--force] [--verbose]

The library is a plain C-ABI shared object (no torch, no pybind): one nvcc
invocation per ``csrc/*.cu`` into ``csrc/_build/*.o`` and a link step.  A source is
recompiled only when it or a header is newer than its object.

A second library, ``librwkv_ops_b200_dev.so``, is the same sources with ``-DRWKVB200_DEVTOOLS``: it adds the
building-block self-test and the phase-stamp instrumentation that the unit tests of the tensor-core
primitives use (``include/rwkv_ops_b200_devtools.h``).  The product never loads it.
"""
from __future__ import annotations

import argparse
import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
BUILD = os.path.join(CSRC, "_build")
LIB = os.path.join(PKG, "librwkv_ops_b200.so")
DEV_LIB = os.path.join(PKG, "librwkv_ops_b200_dev.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return nvcc


def _newest_header() -> float:
    hs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    return max(os.path.getmtime(h) for h in hs)


def build(force: bool = False, verbose: bool = False, dev: bool = False) -> str:
    """Build the product library, or with ``dev`` the developer build."""
    build_dir = os.path.join(BUILD, "dev") if dev else BUILD
    lib = DEV_LIB if dev else LIB
    flags = NVCC_FLAGS + (["-DRWKVB200_DEVTOOLS"] if dev else [])
    os.makedirs(build_dir, exist_ok=True)
    nvcc = _nvcc()
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdr_m = _newest_header()
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(build_dir, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_m):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        cmd = [nvcc, *flags, "-I", INCLUDE, "-c", s, "-o", o]
        p = subprocess.run(cmd, capture_output=True, text=True)
        log = p.stdout + p.stderr
        with open(o[:-2] + ".ptxas.log", "w") as f:
            f.write(log)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}:\n{log}")
        if verbose:
            print(log)
        return o

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    if jobs or force or not os.path.exists(lib):
        cmd = [nvcc, "-shared", "-o", lib, *objs, "-lcudart"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError("link failed:\n" + p.stdout + p.stderr)
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--dev", action="store_true", help="build the developer library instead")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.dev))
    sys.exit(0)
