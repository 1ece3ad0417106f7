"""Builds ``libfpt_b200.so`` (the CUDA library behind the C ABI) in-tree with nvcc for sm_100a.

    python -m fast_polynomial_transcendentals_b200.build [--force] [--verbose]

Objects go to ``fast_polynomial_transcendentals_b200/_build/`` and the shared library is written
next to this file, so the package finds it without an install step.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "_build"
LIB = PKG / "libfpt_b200.so"
COMPAT_LIB = PKG / "libfpt_b200_compat.so"          # the reference's launch_* names over the fpt_* C ABI
COMPAT_SRC = CSRC / "fpt_compat_launch.cpp"
TORCH_BINDING_SRC = CSRC / "fpt_torch_binding.cpp"   # compiled PyTorch binding of the hot element-wise operators
TORCH_BINDING_NAME = "_fpt_torch"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
              "--expt-relaxed-constexpr", "-I", str(PKG.parent / "include")]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(src: Path, force: bool, verbose: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.inc")) + \
        list((PKG.parent / "include").glob("*.h"))
    if force or _stale(obj, [src, *headers]):
        cmd = [nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        (OBJ / (src.stem + ".log")).write_text(proc.stdout + proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stderr[-4000:]}")
        if verbose:
            print(f"compiled {src.name}")
    return obj


def build_variant(out: Path, defines: list[str], only: list[str]) -> Path:
    """Build a tuning variant (extra -D flags, a subset of the sources) into ``out``; used by sweeps."""
    objdir = out.parent / (out.stem + "_obj")
    objdir.mkdir(parents=True, exist_ok=True)
    objs = []
    for src in sources():
        if src.stem not in only:
            continue
        obj = objdir / (src.stem + ".o")
        cmd = [nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-c", str(src), "-o", str(obj)]
        subprocess.run(cmd, check=True, capture_output=True)
        objs.append(obj)
    subprocess.run([nvcc(), *ARCH_FLAGS, "-shared", "-o", str(out), *map(str, objs), "-lcudart"], check=True,
                   capture_output=True)
    return out


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
        objs = list(pool.map(lambda s: _compile(s, force, verbose), srcs))
    if force or _stale(LIB, objs):
        cmd = [nvcc(), *ARCH_FLAGS, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stderr[-4000:]}")
        if verbose:
            print(f"linked {LIB}")
    _build_compat(force, verbose)
    _build_torch_binding(force, verbose)
    return LIB


def torch_binding_path() -> Path:
    import sysconfig
    return PKG / (TORCH_BINDING_NAME + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def _build_torch_binding(force: bool, verbose: bool) -> Path:
    """Host-only C++ against the PyTorch headers; resolves fpt_* from libfpt_b200.so beside it (rpath $ORIGIN)."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension
    out = torch_binding_path()
    deps = [TORCH_BINDING_SRC, LIB, PKG.parent / "include" / "fpt_b200.h"]
    if force or _stale(out, deps):
        cuda_home = Path(shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc").resolve().parents[1]
        includes = [*cpp_extension.include_paths(), sysconfig.get_paths()["include"], str(cuda_home / "include")]
        libdirs = cpp_extension.library_paths()
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-w", f"-DTORCH_EXTENSION_NAME={TORCH_BINDING_NAME}",
               "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
               *[f"-I{i}" for i in includes], str(TORCH_BINDING_SRC), "-o", str(out),
               *[f"-L{d}" for d in libdirs], "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
               f"-L{PKG}", "-lfpt_b200", "-Wl,-rpath,$ORIGIN", *[f"-Wl,-rpath,{d}" for d in libdirs]]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"torch binding build failed:\n{proc.stderr[-4000:]}")
        if verbose:
            print(f"built {out}")
    return out


def _build_compat(force: bool, verbose: bool) -> Path:
    """Host-only shim library; resolves fpt_* from libfpt_b200.so beside it (rpath $ORIGIN)."""
    deps = [COMPAT_SRC, LIB, PKG.parent / "include" / "fpt_b200.h", PKG.parent / "include" / "fpt_b200_compat.h"]
    if force or _stale(COMPAT_LIB, deps):
        cmd = [nvcc(), "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-o", str(COMPAT_LIB), str(COMPAT_SRC),
               "-L", str(PKG), "-lfpt_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN", "-lcudart"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"compat link failed:\n{proc.stderr[-4000:]}")
        if verbose:
            print(f"linked {COMPAT_LIB}")
    return COMPAT_LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
