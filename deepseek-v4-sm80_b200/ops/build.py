"""In-tree build of the native libraries.

Two shared objects are produced next to this file:

* ``libdsv4_b200.so``  -- every sm_100a CUDA kernel (``csrc/*.cu``), compiled with
  ``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` as relocatable device
  code and linked once.  Exported functions are plain ``extern "C"`` launchers that
  take raw pointers and a stream; Python calls them through ctypes.
* ``libdsv4_host.so``  -- host-only C++ (``csrc/host/*.cpp``): radix key compare,
  page-table builders and tensor checks.  It needs no CUDA at run time, so CPU-only
  tests can load it.

The reference builds its native code lazily on first use through TVM-FFI
(python/minisgl/kernel/utils.py:53-129); here the build is an explicit step so the
objects travel with the source tree.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "build"
CUDA_LIB = HERE / "libdsv4_b200.so"
HOST_LIB = HERE / "libdsv4_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-rdc=true",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    return exe


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    r = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout, r.stderr))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr, flush=True)


def build_cuda(force: bool = False, verbose: bool = False, ptxas_v: bool = False) -> Path:
    srcs = sorted(CSRC.glob("*.cu"))
    hdrs = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    stamp = BUILD / "cuda.stamp"
    dig = _digest(srcs + hdrs)
    if not force and CUDA_LIB.exists() and stamp.exists() and stamp.read_text() == dig:
        return CUDA_LIB
    BUILD.mkdir(exist_ok=True)
    nvcc = _nvcc()
    hdr_dig = _digest(hdrs)
    extra = ["-Xptxas", "-v"] if ptxas_v else []

    def one(src: Path):
        obj = BUILD / (src.stem + ".o")
        ostamp = BUILD / (src.stem + ".stamp")
        d = hashlib.sha256(src.read_bytes() + hdr_dig.encode()).hexdigest()
        if not force and not ptxas_v and obj.exists() and ostamp.exists() and ostamp.read_text() == d:
            return obj
        _run([nvcc, *NVCC_FLAGS, *extra, "-I", CSRC, "-dc", src, "-o", obj], verbose or ptxas_v)
        ostamp.write_text(d)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(one, srcs))
    _run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", *objs,
          "-o", CUDA_LIB, "-lcudart_static", "-lpthread", "-ldl", "-lrt"], verbose)
    stamp.write_text(dig)
    return CUDA_LIB


def build_host(force: bool = False, verbose: bool = False) -> Path:
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    hdrs = sorted((CSRC / "host").glob("*.h"))
    stamp = BUILD / "host.stamp"
    dig = _digest(srcs + hdrs)
    if not force and HOST_LIB.exists() and stamp.exists() and stamp.read_text() == dig:
        return HOST_LIB
    BUILD.mkdir(exist_ok=True)
    cxx = shutil.which("g++") or "g++"
    _run([cxx, "-O3", "-std=c++20", "-fPIC", "-shared", "-fvisibility=hidden", "-I", CSRC / "host", *srcs,
          "-o", HOST_LIB], verbose)
    stamp.write_text(dig)
    return HOST_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_host(force, verbose)
    build_cuda(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    if "--ptxas" in sys.argv:
        build_cuda(force=True, verbose=True, ptxas_v=True)
