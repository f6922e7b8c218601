"""Builds the in-tree native libraries with nvcc for sm_100a.

    python -m pth_flash_attn_b200.build            # libpthb200_attn.so + _C.abi3.so
    python -m pth_flash_attn_b200.build --verbose  # with -Xptxas -v

`libpthb200_attn.so` is the C ABI library (CUDA kernels + launcher, no torch).
`_C.abi3.so` registers the torch op through the libtorch stable ABI and links
against the former.  Both land next to this file so they travel with the tree.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libpthb200_attn.so"
OP_LIB = HERE / "_C.abi3.so"

CUDA_SOURCES = ["launcher.cu", "scalar_kernel.cu", "combine_kernel.cu", "umma_kernel.cu", "umma_i8_kernel.cu",
                "umma_rows_kernel.cu", "umma_rows256_kernel.cu", "umma_rows2_kernel.cu", "writer_kernel.cu", "copy_ceiling_kernel.cu"]
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fno-gnu-unique", "-rdc=false",
]


def _nvcc() -> str:
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    return str(Path(home) / "bin" / "nvcc")


def _newer(target: Path, sources: list[Path]) -> bool:
    if not target.is_file():
        return False
    t = target.stat().st_mtime
    return all(s.stat().st_mtime <= t for s in sources)


def build_library(verbose: bool = False, force: bool = False) -> Path:
    sources = [CSRC / s for s in CUDA_SOURCES]
    deps = sources + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "pthb200_attn.h"]
    if not force and _newer(LIB, deps):
        return LIB
    objs = []
    for src in sources:
        obj = CSRC / (src.stem + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        subprocess.run(cmd, check=True)
        objs.append(str(obj))
    subprocess.run([_nvcc(), "-shared", "-o", str(LIB), *objs, "-lcudart"], check=True)
    return LIB


def build_op_library(force: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    src = CSRC / "torch_op.cpp"
    if not force and _newer(OP_LIB, [src, LIB]):
        return OP_LIB
    includes = [f"-I{p}" for p in cpp_extension.include_paths()]
    cuda_inc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
    torch_lib = Path(torch.__file__).parent / "lib"
    cmd = [
        "g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fno-gnu-unique", str(src), "-o", str(OP_LIB),
        *includes, f"-I{cuda_inc}", f"-L{HERE}", "-lpthb200_attn", "-Wl,-rpath,$ORIGIN",
        f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", f"-Wl,-rpath,{torch_lib}",
    ]
    subprocess.run(cmd, check=True)
    return OP_LIB


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_library(verbose=verbose, force=force)
    if (CSRC / "torch_op.cpp").is_file():
        build_op_library(force=force)


if __name__ == "__main__":
    build_all(verbose="--verbose" in sys.argv, force="--force" in sys.argv)
    print(f"built {LIB}")
