"""In-tree build of the native parts.

* ``lib/libpla_b200.so``  — the CUDA kernels behind the C ABI of ``include/pla_b200.h``
  (nvcc, sm_100a only, no torch).
* ``lib/pla_b200_ops.so`` — the C++ host layer registered as PyTorch custom ops
  (``TORCH_LIBRARY(pla_b200, ...)``); it validates tensors, fills the POD
  argument structs and calls the C ABI on the current CUDA stream.

Run ``python -m pla_b200.build`` (add ``--force`` to rebuild everything).
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
OBJ = PKG / "_obj"
NATIVE_LIB = LIB / "libpla_b200.so"
OPS_LIB = LIB / "pla_b200_ops.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else "nvcc"


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _headers():
    return list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [ROOT / "include" / "pla_b200.h"]


def build_native(force: bool = False, verbose: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = _headers()

    def compile_one(src: Path) -> Path:
        obj = OBJ / (src.stem + ".o")
        if not force and _newer(obj, [src] + headers):
            return obj
        cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(ROOT / "include"), "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        (OBJ / (src.stem + ".ptxas.log")).write_text(res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(f"[pla_b200.build] compiled {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(compile_one, sources))
    if force or not _newer(NATIVE_LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", str(NATIVE_LIB), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return NATIVE_LIB


def build_ops(force: bool = False, verbose: bool = False) -> Path:
    """Compile the torch-facing C++ host layer (g++ only; links libpla_b200.so)."""
    import torch
    from torch.utils import cpp_extension as ce

    build_native(force=force, verbose=verbose)
    sources = sorted((CSRC / "torch").glob("*.cpp"))
    headers = _headers() + list((CSRC / "torch").glob("*.h"))
    if not force and _newer(OPS_LIB, sources + headers + [NATIVE_LIB]):
        return OPS_LIB
    OBJ.mkdir(exist_ok=True)
    inc = ce.include_paths() + [str(ROOT / "include"), "/usr/local/cuda/include"]
    import sysconfig
    inc.append(sysconfig.get_paths()["include"])
    cxx = os.environ.get("CXX", "g++")
    flags = ["-O2", "-std=c++17", "-fPIC", "-DTORCH_API_INCLUDE_EXTENSION_H",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]

    def compile_one(src: Path) -> Path:
        obj = OBJ / ("torch_" + src.stem + ".o")
        if not force and _newer(obj, [src] + headers):
            return obj
        cmd = [cxx, *flags, *[f"-I{p}" for p in inc], "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"{cxx} failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(f"[pla_b200.build] compiled torch/{src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(sources)))) as pool:
        objs = list(pool.map(compile_one, sources))
    torch_lib = Path(torch.__file__).parent / "lib"
    cmd = [cxx, "-shared", "-o", str(OPS_LIB), *map(str, objs),
           f"-L{LIB}", "-lpla_b200", f"-L{torch_lib}", "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return OPS_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_native(force=force, verbose=verbose)
    build_ops(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print(NATIVE_LIB)
    print(OPS_LIB)
