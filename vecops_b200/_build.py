"""In-tree build of libvecops_b200.so: hand-written CUDA for sm_100a plus the C++ host runtime.

nvcc cross-compiles without a GPU.  Only sm_100a machine code is embedded
(``code=sm_100a``, no PTX), so nothing is JIT-compiled when the library loads.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
ROOT = PACKAGE.parent
CSRC = PACKAGE / "csrc"
INCLUDE = ROOT / "include"
BUILD = ROOT / "build"
LIB_DIR = PACKAGE / "lib"
LIBRARY = LIB_DIR / "libvecops_b200.so"

NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]
CXX_FLAGS = ["-std=c++20", "-O2", "-fPIC", "-Wall", "-Wextra"]  # default visibility: the C++ runtime classes are part of the library's API


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build vecops_b200")
    return found


def _sources() -> tuple[list[Path], list[Path], list[Path]]:
    cuda = sorted((CSRC / "cuda").glob("*.cu"))
    # runtime/: the matmul operator, recipes, dispatch policy, provider and C bridge of this library;
    # runtime_mirror/: vecops' runtime classes restated so that the library stands alone (unused inside a vecops build)
    host = sorted((CSRC / "runtime").glob("*.cpp")) + sorted((CSRC / "runtime_mirror").glob("*.cpp"))
    # this file counts as an input: a change of flags rebuilds everything
    headers = sorted(CSRC.rglob("*.h")) + sorted(CSRC.rglob("*.cuh")) + sorted(INCLUDE.rglob("*.h")) + [Path(__file__)]
    return cuda, host, headers


def _stale(target: Path, inputs: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(p.stat().st_mtime > stamp for p in inputs)


def build(force: bool = False, verbose: bool = False) -> Path:
    cuda, host, headers = _sources()
    BUILD.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    objects: list[Path] = []
    run = lambda cmd: subprocess.run(cmd, check=True, stdout=None if verbose else subprocess.DEVNULL)
    for source in cuda:
        obj = BUILD / (source.stem + ".cu.o")
        if force or _stale(obj, [source, *headers]):
            extra = ["-Xptxas", "-v"] if verbose else []
            run([_nvcc(), *NVCC_FLAGS, *extra, f"-I{INCLUDE}", f"-I{CSRC / 'cuda'}", "-c", str(source), "-o", str(obj)])
        objects.append(obj)
    for source in host:
        obj = BUILD / (source.stem + ".cpp.o")
        if force or _stale(obj, [source, *headers]):
            run([os.environ.get("CXX", "g++"), *CXX_FLAGS, f"-I{INCLUDE}", f"-I{CSRC / 'runtime'}", f"-I{CSRC / 'cuda'}",
                 "-c", str(source), "-o", str(obj)])
        objects.append(obj)
    if force or _stale(LIBRARY, objects):
        # cudart is linked statically (nvcc's default), so the library loads on a host without a driver.
        run([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIBRARY), *map(str, objects), "-Xlinker", "--no-undefined", "-lpthread", "-ldl"])
    return LIBRARY


TORCH_BRIDGE = LIB_DIR / "libvecops_b200_torch.so"


def build_torch_bridge(force: bool = False, verbose: bool = False) -> Path:
    """The Torch operator library (torch.ops.vecops_b200.*): csrc/torch/torch_bridge.cpp against the installed torch's
    headers, linked to libvecops_b200.so beside it.  Host code only - no device code lives in it."""
    import torch
    from torch.utils import cpp_extension
    library = build(force=False, verbose=verbose)
    source = CSRC / "torch" / "torch_bridge.cpp"
    if not force and not _stale(TORCH_BRIDGE, [source, library, *sorted(INCLUDE.rglob("*.h")), Path(__file__)]):
        return TORCH_BRIDGE
    includes = [f"-I{path}" for path in cpp_extension.include_paths()] + [f"-I{INCLUDE}", "-I/usr/local/cuda/include"]
    library_dirs = cpp_extension.library_paths()
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    command = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *includes, str(source),
               "-o", str(TORCH_BRIDGE), f"-L{LIB_DIR}", "-lvecops_b200", "-Wl,-rpath,$ORIGIN",
               *[f"-L{d}" for d in library_dirs], *[f"-Wl,-rpath,{d}" for d in library_dirs], "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda",
               "-lc10_cuda"]
    subprocess.run(command, check=True, stdout=None if verbose else subprocess.DEVNULL)
    return TORCH_BRIDGE


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--torch" in sys.argv:
        print(build_torch_bridge(force="--force" in sys.argv, verbose="-v" in sys.argv))
