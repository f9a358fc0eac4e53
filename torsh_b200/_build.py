"""In-tree native build: nvcc for the sm_100a kernels, g++ for the host runtime.

Two shared libraries are produced under ``torsh_b200/lib``:

* ``libtorsh_b200_cuda.so``  - every ``csrc/kernels/*.cu`` (kernels + ``extern "C"`` launchers)
* ``libtorsh_b200_host.so``  - every ``csrc/host/*.cpp`` (TCP store, TRSH codec, bucket planner,
  pipeline scheduler, caching-allocator model, C ABI, ...)

Both are loaded with ``ctypes`` by :mod:`torsh_b200._native`. Objects are rebuilt only when a
source or header is newer. The reference detects CUDA in ``crates/torsh-backend/build.rs:21-101``
and lists ``sm_70..sm_89`` arch flags in ``crates/torsh-utils/src/cpp_extension.rs``; here there is
exactly one target, ``sm_100a``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIBDIR = Path(__file__).resolve().parent / "lib"
OBJDIR = ROOT / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr", "--extended-lambda",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or install CUDA >= 12.8)")


def _newer(src: Path, dst: Path, deps: list[Path]) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *deps])


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"native build failed: {' '.join(cmd[:4])} ...")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr, flush=True)


def build_cuda(verbose: bool = False, ptxas_info: bool = False) -> Path:
    nvcc = _nvcc()
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    hdrs = sorted((CSRC / "kernels").glob("*.cuh")) + sorted((CSRC / "kernels").glob("*.h")) + sorted(
        (CSRC / "include").glob("*.h"))
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    objs, jobs = [], []
    for s in srcs:
        o = OBJDIR / (s.stem + ".cu.o")
        objs.append(o)
        if _newer(s, o, hdrs):
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC / "include"), "-I", str(CSRC / "kernels"), "-c", str(s), "-o", str(o)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(lambda c: _run(c, verbose or ptxas_info), jobs))
    out = LIBDIR / "libtorsh_b200_cuda.so"
    if jobs or not out.exists():
        _run([nvcc, "-shared", "-o", str(out), *map(str, objs), "-cudart", "static", "-Xcompiler", "-fPIC"], verbose)
    return out


def build_host(verbose: bool = False) -> Path:
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    hdrs = sorted((CSRC / "host").glob("*.h")) + sorted((CSRC / "include").glob("*.h"))
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    objs, jobs = [], []
    for s in srcs:
        o = OBJDIR / (s.stem + ".cpp.o")
        objs.append(o)
        if _newer(s, o, hdrs):
            jobs.append([cxx, *CXX_FLAGS, "-I", str(CSRC / "include"), "-I", str(CSRC / "host"), "-c", str(s), "-o", str(o)])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    out = LIBDIR / "libtorsh_b200_host.so"
    if srcs and (jobs or not out.exists()):
        _run([cxx, "-shared", "-o", str(out), *map(str, objs), "-pthread", "-lz", "-ldl", "-Wl,-Bsymbolic", "-Wl,--exclude-libs,ALL"], verbose)
    return out


def build_all(verbose: bool = False) -> None:
    build_cuda(verbose)
    build_host(verbose)


if __name__ == "__main__":
    build_cuda(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    build_host(verbose="-v" in sys.argv)
    print("built:", *[p.name for p in LIBDIR.glob("*.so")])
