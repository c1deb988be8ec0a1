"""In-tree build of the sm_100a kernel library (``viola_b200/_C.so``).

The ``.cu`` sources are compiled by nvcc without any torch header (seconds per file,
``-gencode arch=compute_100a,code=sm_100a``); only ``bindings.cpp`` sees torch.  The
resulting shared object exports both the ``extern "C"`` kernel ABI (``csrc/api.h``) and the
``torch.ops.viola_b200`` operators.  Objects are rebuilt only when a source or header is
newer, so repeated ``build()`` calls are cheap.  nvcc cross-compiles without a GPU.
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
OBJ = ROOT / "build"
TARGET = ROOT / "_C.so"

CUDA_SOURCES = ["quant.cu", "gemm_sm100.cu", "mxfp8_gemm_sm100.cu", "attention_sm100.cu", "optim.cu", "codec.cu", "comm.cu", "fused.cu", "multi.cu", "noalloc.cu"]
CPP_SOURCES = ["bindings.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = Path(cuda_home) / "bin" / "nvcc"
    return str(candidate) if candidate.exists() else (shutil.which("nvcc") or "nvcc")


def _newest(paths) -> float:
    return max((p.stat().st_mtime for p in paths if p.exists()), default=0.0)


def _headers():
    return [*CSRC.glob("*.h"), *CSRC.glob("common/*.cuh"), *CSRC.glob("*.cuh")]


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(map(str, cmd))}\n{result.stdout}\n{result.stderr}")
    return result.stdout + result.stderr


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every CUDA extension for sm_100a and link ``_C.so``; returns its path."""
    import torch
    from torch.utils import cpp_extension

    OBJ.mkdir(exist_ok=True)
    header_time = _newest(_headers())
    cuda_sources = [CSRC / name for name in CUDA_SOURCES if (CSRC / name).exists()]
    cpp_sources = [CSRC / name for name in CPP_SOURCES if (CSRC / name).exists()]
    jobs, objects = [], []
    for src in cuda_sources:
        obj = OBJ / (src.stem + ".o")
        objects.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_time):
            flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])
            jobs.append([_nvcc(), *flags, f"-I{CSRC}", "-c", str(src), "-o", str(obj)])
    include = [f"-I{path}" for path in cpp_extension.include_paths("cuda")]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for src in cpp_sources:
        obj = OBJ / (src.stem + ".o")
        objects.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_time):
            jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                         "-DTORCH_EXTENSION_NAME=_C", *include, f"-I{CSRC}", "-c", str(src), "-o", str(obj)])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            for output in pool.map(lambda cmd: _run(cmd, verbose), jobs):
                if ptxas_info and output.strip():
                    print(output)
    if force or jobs or not TARGET.exists() or TARGET.stat().st_mtime < _newest(objects):
        torch_lib = Path(torch.__file__).parent / "lib"
        cuda_lib = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "lib64"
        link = ["g++", "-shared", "-o", str(TARGET), *map(str, objects), f"-L{torch_lib}", f"-L{cuda_lib}",
                "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart",
                f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath,{cuda_lib}"]
        _run(link, verbose)
    return TARGET


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
