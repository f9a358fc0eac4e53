"""Build user CUDA / C++ extensions (``crates/torsh-utils/src/cpp_extension.rs``).  The reference emits
``-gencode`` flags for sm_70 .. sm_89; this build targets one architecture, ``sm_100a``, and produces a shared library
with ``extern "C"`` entry points that is loaded with ``ctypes`` (the same mechanism as the framework's own kernels), so
no Python headers and no JIT cache are involved: the ``.so`` lands next to the sources (or in ``build_directory``)."""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
from dataclasses import dataclass, field
from pathlib import Path

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


@dataclass
class CppExtensionConfig:
    name: str
    sources: list[str]
    include_dirs: list[str] = field(default_factory=list)
    extra_cflags: list[str] = field(default_factory=lambda: ["-O3"])
    extra_cuda_cflags: list[str] = field(default_factory=lambda: ["-O3", "-lineinfo"])
    extra_ldflags: list[str] = field(default_factory=list)
    build_directory: str | None = None
    verbose: bool = False

    @property
    def with_cuda(self) -> bool:
        return any(s.endswith((".cu", ".cuh")) for s in self.sources)


def find_nvcc() -> str | None:
    cand = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH") or "/usr/local/cuda"
    p = Path(cand) / "bin" / "nvcc"
    return str(p) if p.exists() else shutil.which("nvcc")


def kernel_include_dir() -> str:
    """Directory of the framework's device headers (``sm100.cuh``: mbarrier / TMA / tcgen05 wrappers)."""
    return str(Path(__file__).resolve().parents[2] / "csrc" / "kernels")


def build_command(cfg: CppExtensionConfig, output: Path) -> list[str]:
    inc = [f"-I{d}" for d in cfg.include_dirs + [kernel_include_dir()]]
    if cfg.with_cuda:
        nvcc = find_nvcc()
        if nvcc is None:
            raise RuntimeError("nvcc not found (set CUDA_HOME)")
        return [nvcc, "-shared", "-std=c++17", "-Xcompiler", "-fPIC", *ARCH_FLAGS, *cfg.extra_cuda_cflags, *inc,
                "--cudart", "static", *cfg.sources, "-o", str(output), *cfg.extra_ldflags, "-lcuda"]
    return [os.environ.get("CXX", "g++"), "-shared", "-fPIC", "-std=c++17", *cfg.extra_cflags, *inc, *cfg.sources,
            "-o", str(output), *cfg.extra_ldflags]


def build(cfg: CppExtensionConfig) -> Path:
    out_dir = Path(cfg.build_directory or Path(cfg.sources[0]).resolve().parent)
    out_dir.mkdir(parents=True, exist_ok=True)
    out = out_dir / f"lib{cfg.name}.so"
    h = hashlib.sha256()
    for s in cfg.sources:
        h.update(Path(s).read_bytes())
    h.update(" ".join(cfg.extra_cflags + cfg.extra_cuda_cflags + cfg.extra_ldflags).encode())
    stamp = out_dir / f".{cfg.name}.sha256"
    if out.exists() and stamp.exists() and stamp.read_text() == h.hexdigest():
        return out
    cmd = build_command(cfg, out)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if cfg.verbose or r.returncode:
        print(" ".join(cmd)); print(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError(f"building {cfg.name} failed:\n{r.stderr[-4000:]}")
    stamp.write_text(h.hexdigest())
    return out


def load(name: str, sources: list[str], **kw) -> ctypes.CDLL:
    """Compile (if stale) and load; call exported ``extern "C"`` functions through the returned handle."""
    return ctypes.CDLL(str(build(CppExtensionConfig(name, sources, **kw))), mode=ctypes.RTLD_LOCAL)
