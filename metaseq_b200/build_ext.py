"""Builds the native libraries of the package in-tree.

* ``metaseq_b200/_C/libmsq_kernels.so`` -- every sm_100a CUDA kernel
  (``csrc/*.cu``), compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``.
  The kernels export a plain C ABI and are called through ``ctypes`` with raw
  device pointers and the current CUDA stream, so no torch headers are needed
  and a full rebuild takes seconds.
* ``metaseq_b200/_C/libmsq_host.so`` -- host-side C++ helpers (data batching,
  token-block slicing, flat-parameter packing), ``csrc/host/*.cpp``.

nvcc cross-compiles without a GPU.  Objects are rebuilt only when their source
(or a shared header) is newer than the object.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT = ROOT / "_C"
OBJ = OUT / "obj"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=default",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-shared", "-Wall"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put the CUDA toolkit on PATH")
    return cand


def _newest(paths) -> float:
    return max((p.stat().st_mtime for p in paths), default=0.0)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"command failed: {' '.join(str(c) for c in cmd)}")
    return res.stdout + res.stderr


def kernel_sources():
    return sorted(CSRC.glob("*.cu"))


def host_sources():
    return sorted((CSRC / "host").glob("*.cpp"))


def build(force: bool = False, verbose: bool = False) -> dict:
    """Compile everything that is stale.  Returns the paths of the two libraries."""
    OBJ.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    hdr_time = _newest(headers)

    jobs = []
    objs = []
    for src in kernel_sources():
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time)
        if stale:
            jobs.append([nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj])
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))

    lib = OUT / "libmsq_kernels.so"
    if objs and (force or jobs or not lib.exists() or lib.stat().st_mtime < _newest(objs)):
        _run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib, *objs], verbose)

    host_lib = OUT / "libmsq_host.so"
    hsrcs = host_sources()
    if hsrcs and (force or not host_lib.exists() or host_lib.stat().st_mtime < _newest(hsrcs)):
        cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
        _run([cxx, *CXX_FLAGS, "-o", host_lib, *hsrcs], verbose)
    return {"kernels": lib, "host": host_lib}


if __name__ == "__main__":
    out = build(force="--force" in sys.argv, verbose=True)
    for k, v in out.items():
        print(k, v, "OK" if Path(v).exists() else "missing")
