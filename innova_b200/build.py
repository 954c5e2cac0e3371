"""In-tree build of the native libraries.

``libinnova_cuda.so``  — every ``csrc/*.cu`` compiled for sm_100a (tcgen05 / TMA need the ``a`` target).
``libinnova_host.so``  — the C++ host runtime in ``csrc/host`` (.oil container, block codecs, format
registry and planner, codebooks, paged-KV page tables, CPU sampler).

Both expose a C ABI and are loaded with ctypes (see ``_native.py``), so a build takes seconds and
needs no Python headers. ``python -m innova_b200.build`` rebuilds what is out of date.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = LIB / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-O3",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread"]


def _nvcc() -> str | None:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def _newer(src_list, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in src_list)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout, r.stderr))
    return r.stdout + r.stderr


def cuda_sources():
    return sorted(CSRC.glob("*.cu"))


def host_sources():
    return sorted((CSRC / "host").glob("*.cpp"))


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    out = LIB / "libinnova_cuda.so"
    srcs = cuda_sources()
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    nvcc = _nvcc()
    if nvcc is None:
        if out.exists():
            return out
        raise RuntimeError("nvcc not found and %s is not built" % out)
    OBJ.mkdir(parents=True, exist_ok=True)
    jobs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        if force or _newer([s] + headers, o):
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(s), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            logs = list(ex.map(_run, jobs))
        if verbose:
            print("\n".join(logs))
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    if force or jobs or _newer(objs, out):
        _run([nvcc, "-shared", "-o", str(out), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"])
    return out


def build_host(force: bool = False) -> Path:
    out = LIB / "libinnova_host.so"
    srcs = host_sources()
    if not srcs:
        return out
    headers = list((CSRC / "host").glob("*.h"))
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        if out.exists():
            return out
        raise RuntimeError("no C++ compiler found and %s is not built" % out)
    OBJ.mkdir(parents=True, exist_ok=True)
    jobs = []
    for s in srcs:
        o = OBJ / ("host_" + s.stem + ".o")
        if force or _newer([s] + headers, o):
            jobs.append([cxx, *CXX_FLAGS, "-I", str(CSRC / "host"), "-c", str(s), "-o", str(o)])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    objs = [OBJ / ("host_" + s.stem + ".o") for s in srcs]
    if force or jobs or _newer(objs, out):
        _run([cxx, "-shared", "-pthread", "-o", str(out), *map(str, objs)])
    return out


def build_host_sanitized() -> Path:
    """``libinnova_host_asan.so``: the host runtime with AddressSanitizer and UndefinedBehaviorSanitizer (the reference's
    ``OIL_SANITIZE`` build, cmake/compiler.cmake:11-14). Load it in a process started with ``LD_PRELOAD=$(gcc
    -print-file-name=libasan.so)`` and ``INNOVA_HOST_LIB`` pointing at it; any heap error or undefined operation in the
    codecs, the container, the page tables or the arena aborts that process with a report."""
    out = LIB / "libinnova_host_asan.so"
    srcs = host_sources()
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("no C++ compiler found")
    LIB.mkdir(exist_ok=True)
    if _newer(srcs + list((CSRC / "host").glob("*.h")), out):
        _run([cxx, "-O1", "-g", "-std=c++17", "-fPIC", "-pthread", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
              "-fno-sanitize-recover=undefined", "-I", str(CSRC / "host"), "-shared", "-o", str(out), *map(str, srcs)])
    return out


def asan_runtime() -> str:
    cc = shutil.which("gcc") or shutil.which("cc")
    return subprocess.run([cc, "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip() if cc else ""


def build_capi(force: bool = False) -> Path | None:
    """``liboil_capi.so``: the C entry points ``oil_model_load`` ... ``oil_last_error`` (csrc/capi/oil_capi.h) over the
    Python engine. Needs the Python development headers and shared library; returns None when they are missing."""
    import sysconfig
    out = LIB / "liboil_capi.so"
    src = CSRC / "capi" / "oil_capi.cpp"
    inc = sysconfig.get_config_var("INCLUDEPY")
    libdir = sysconfig.get_config_var("LIBDIR")
    ver = sysconfig.get_config_var("LDVERSION")
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None or not inc or not os.path.exists(os.path.join(inc, "Python.h")) or not sysconfig.get_config_var("Py_ENABLE_SHARED"):
        return out if out.exists() else None
    if force or _newer([src, CSRC / "capi" / "oil_capi.h"], out):
        LIB.mkdir(exist_ok=True)
        _run([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-I", inc, "-I", str(CSRC / "capi"), str(src), "-o", str(out),
              "-L", str(libdir), f"-lpython{ver}", "-ldl", f"-Wl,-rpath,{libdir}"])
    return out


def build_all(force: bool = False, verbose: bool = False):
    LIB.mkdir(exist_ok=True)
    paths = [build_cuda(force, verbose), build_host(force)]
    capi = build_capi(force)
    if capi is not None:
        paths.append(capi)
    return tuple(paths)


if __name__ == "__main__":
    paths = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    for p in paths:
        print(p)
