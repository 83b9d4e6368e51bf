"""In-tree build of the native libraries.

* ``lib/libneox_b200.so``  – every CUDA kernel, compiled by nvcc for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``), exposing a plain C ABI that
  ``gpt_neox_b200.ops`` binds with ctypes.
* ``lib/libneox_data.so`` – the CPU dataset-index builders (g++), the counterpart of the
  reference's ``megatron/data/helpers.cpp`` built by ``megatron/data/Makefile``.
* ``lib/libneox_host.so`` – host AdamW for optimizer-state offload (g++, csrc/cpu_adam.cpp).

Objects are cached under ``build/`` and rebuilt when a source or any header is newer.
Run ``python -m gpt_neox_b200.build`` (``--force`` to rebuild everything).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
OBJ = PKG.parent / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--use_fast_math",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-shared", "-Wall", "-pthread"]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


#: sources without 16-bit tensor code: compiled once.  Every other .cu file is compiled twice, for bf16 and
#: (``-DNX_HALF``: namespace nxh, exported symbols ``nx_*_f16``) for fp16.
SINGLE_BUILD = {"common.cu", "colsum_noalloc.cu"}


def _compile_one(src: Path, headers, force: bool, verbose: bool, half: bool = False, debug_bounds: bool = False):
    stem = src.stem + ("_f16" if half else "") + ("_dbg" if debug_bounds else "")
    obj = OBJ / (stem + ".o")
    if not force and not _stale(obj, [src, *headers]):
        return obj, ""
    cmd = [_nvcc(), *NVCC_FLAGS, *(["-DNX_HALF"] if half else []), *(["-DNEOX_DEBUG_BOUNDS"] if debug_bounds else []),
           "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    log = r.stderr
    (OBJ / (stem + ".ptxas.log")).write_text(log)
    if verbose:
        print(log)
    return obj, log


def build_cuda(force: bool = False, verbose: bool = False, debug_bounds: bool = False) -> Path:
    """``debug_bounds``: a second library, ``lib/libneox_b200_dbg.so``, whose communication kernels range-check every
    access into a symmetric workspace (``-DNEOX_DEBUG_BOUNDS``); ``NEOX_KERNEL_LIB=debug`` makes the ops load it."""
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB.mkdir(parents=True, exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu"))
    headers = sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))
    jobs = [(s, False) for s in srcs] + [(s, True) for s in srcs if s.name not in SINGLE_BUILD]
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = [o for o, _ in ex.map(lambda j: _compile_one(j[0], headers, force, verbose, j[1], debug_bounds), jobs)]
    out = LIB / ("libneox_b200_dbg.so" if debug_bounds else "libneox_b200.so")
    if force or _stale(out, objs):
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-o", str(out), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return out


def build_data_helpers(force: bool = False) -> Path:
    LIB.mkdir(parents=True, exist_ok=True)
    src = CSRC / "data_helpers.cpp"
    out = LIB / "libneox_data.so"
    if src.exists() and (force or _stale(out, [src])):
        cmd = [os.environ.get("CXX", "g++"), *CXX_FLAGS, str(src), "-o", str(out)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"g++ failed:\n{r.stdout}\n{r.stderr}")
    return out


def build_host_ops(force: bool = False) -> Path:
    """``lib/libneox_host.so``: host-side compute used by optimizer-state offload (csrc/cpu_adam.cpp)."""
    LIB.mkdir(parents=True, exist_ok=True)
    src = CSRC / "cpu_adam.cpp"
    out = LIB / "libneox_host.so"
    if src.exists() and (force or _stale(out, [src])):
        cmd = [os.environ.get("CXX", "g++"), *CXX_FLAGS, "-fopenmp-simd", "-fvisibility=hidden", str(src), "-o", str(out)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"g++ failed:\n{r.stdout}\n{r.stderr}")
    return out


def build_data_helpers_sanitized(out_dir, cxx=None) -> Path:
    """The dataset-index builders compiled with AddressSanitizer + UBSan (host code only; the GPU pool offers
    no compute-sanitizer).  The library must be loaded into a process that preloads the ASan runtime:
    ``LD_PRELOAD=$(g++ -print-file-name=libasan.so)``."""
    out = Path(out_dir) / "libneox_data_asan.so"
    flags = [f for f in CXX_FLAGS if f not in ("-O3",)] + ["-O1", "-g", "-fsanitize=address,undefined",
                                                         "-fno-omit-frame-pointer"]
    cmd = [cxx or os.environ.get("CXX", "g++"), *flags, str(CSRC / "data_helpers.cpp"), "-o", str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ (sanitized) failed:\n{r.stdout}\n{r.stderr}")
    return out


def build_all(force: bool = False, verbose: bool = False):
    a = build_data_helpers(force)
    build_host_ops(force)
    b = build_cuda(force, verbose)
    return a, b


def ptxas_report() -> str:
    """Registers / spills / shared memory of every kernel, from the cached ptxas logs."""
    out = []
    for f in sorted(OBJ.glob("*.ptxas.log")):
        out.append(f"== {f.stem}")
        out.append(f.read_text())
    return "\n".join(out)


if __name__ == "__main__":
    force = "--force" in sys.argv
    verbose = "--verbose" in sys.argv
    a, b = build_all(force, verbose)
    print("built", a)
    print("built", b)
    if "--debug-bounds" in sys.argv:
        print("built", build_cuda(force, verbose, debug_bounds=True))
