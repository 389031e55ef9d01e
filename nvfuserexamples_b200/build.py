"""Builds the native code in-tree with nvcc, for sm_100a only.

Two artefacts:
  nvfuserexamples_b200/lib/libfmha_sm100.so   the C-ABI kernel library (no torch, no Python)
  mha_manual.cpython-*.so (repository root)   the torch operator extension; links the above

Run as ``python -m nvfuserexamples_b200.build`` (add ``--force`` to rebuild, ``-v`` for
``-Xptxas -v`` resource usage).  Needs no GPU: nvcc cross-compiles.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
LIB = LIBDIR / "libfmha_sm100.so"

KERNEL_SOURCES = ["fmha_capi.cu", "fmha_fwd_sm100.cu", "fmha_fwd_dense_sm100.cu", "fmha_fwd_fast_sm100.cu", "fmha_bwd_sm100.cu"]
KERNEL_HEADERS = ["sm100_ptx.cuh", "philox.cuh", "fmha_device_utils.cuh", "fmha_kernel_args.h", "../../include/fmha_sm100.h"]
GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def ext_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return ROOT / f"mha_manual{suffix}"


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.exists() and d.stat().st_mtime > t for d in deps)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0 or verbose:
        sys.stdout.write(proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed ({proc.returncode}): {' '.join(cmd)}")


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the CUDA kernels and the C ABI into libfmha_sm100.so."""
    LIBDIR.mkdir(exist_ok=True)
    objs = []
    headers = [CSRC / h for h in KERNEL_HEADERS]
    procs = []
    for src in KERNEL_SOURCES:
        s = CSRC / src
        o = LIBDIR / (Path(src).stem + ".o")
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [_nvcc(), "-std=c++17", "-O3", "-lineinfo", *GENCODE, "-Xcompiler", "-fPIC",
                   "-c", str(s), "-o", str(o)]
            if verbose:
                cmd += ["-Xptxas", "-v"]
                print(" ".join(cmd), flush=True)
            procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stdout.write(out)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _stale(LIB, objs):
        _run([_nvcc(), "-shared", *GENCODE, "-o", str(LIB), *map(str, objs), "-cudart", "static"], verbose)
    return LIB


def build_extension(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the torch operator layer (`import mha_manual`) against libfmha_sm100.so."""
    from torch.utils import cpp_extension as ce

    target = ext_path()
    src = CSRC / "mha_manual_ext.cpp"
    if not (force or _stale(target, [src, CSRC / "../../include/fmha_sm100.h", LIB])):
        return target
    import torch

    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}", f"-I{ROOT / 'include'}",
                                                      "-I/usr/local/cuda/include"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    libs = [f"-L{p}" for p in ce.library_paths()] + ["-L/usr/local/cuda/lib64", f"-L{LIBDIR}"]
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=mha_manual",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *inc, str(src), "-o", str(target),
           *libs, "-lfmha_sm100", "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
           "-lcudart", "-Wl,-rpath,$ORIGIN/nvfuserexamples_b200/lib",
           *[f"-Wl,-rpath,{p}" for p in ce.library_paths()]]
    _run(cmd, verbose)
    return target


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force, verbose)
    build_extension(force, verbose)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("--kernels-only", action="store_true")
    ns = ap.parse_args()
    build_kernels(ns.force, ns.verbose)
    if not ns.kernels_only:
        build_extension(ns.force, ns.verbose)
    print("built:", LIB, "" if ns.kernels_only else ext_path())
