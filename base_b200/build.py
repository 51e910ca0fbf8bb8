"""Build the native library in-tree.

Two steps, both cross-compilable on a host without a GPU:
  1. nvcc compiles csrc/kernels/all.cu to ONE sm_100a cubin;
  2. g++ links the C-ABI layer, the runtime and the stage programs into
     base_b200/libb200base.so with that cubin embedded (.incbin), so the
     library is self-contained and loads its kernels with cuModuleLoadData.

`python -m base_b200.build` rebuilds when a source is newer than the library.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
BUILD = PKG / "_build"
LIB = PKG / "libb200base.so"
CUBIN = BUILD / "kernels.cubin"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")
CUDA_INC = os.environ.get("CUDA_INC", "/usr/local/cuda/include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-cubin", "-O3", "-lineinfo",
    "-std=c++17", "--use_fast_math=false",
]


def _sources():
    cpp = sorted(p for d in ("abi", "runtime", "stages") for p in (CSRC / d).glob("*.cpp"))
    hdr = sorted(CSRC.rglob("*.h")) + sorted(CSRC.rglob("*.cuh")) + sorted(CSRC.rglob("*.inc")) + sorted((ROOT / "include").glob("*.h"))
    cu = sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "noalloc").glob("*.cu"))
    return cpp, hdr, cu


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd, **kw):
    r = subprocess.run(cmd, capture_output=True, text=True, **kw)
    if r.returncode != 0:
        sys.stderr.write(" ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]}")
    return r.stdout + r.stderr


def build_cubin(verbose: bool = False) -> str:
    BUILD.mkdir(exist_ok=True)
    cmd = [NVCC, *[f for f in NVCC_FLAGS if f != "--use_fast_math=false"], "-I", str(CSRC / "kernels"),
           "-o", str(CUBIN), str(CSRC / "kernels" / "all.cu")]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    return _run(cmd)


def build(force: bool = False, verbose: bool = False) -> Path:
    cpp, hdr, cu = _sources()
    kernel_deps = cu + [h for h in hdr if h.suffix == ".cuh"]
    log = ""
    if force or _newer(CUBIN, kernel_deps):
        log += build_cubin(verbose)
    if force or _newer(LIB, cpp + hdr + cu + [CUBIN, Path(__file__)]):
        BUILD.mkdir(exist_ok=True)
        asm = BUILD / "kernels_image.S"
        asm.write_text(
            '.section .rodata\n'
            '.global b200_kernels_image_start\n'
            '.global b200_kernels_image_end\n'
            '.balign 64\n'
            'b200_kernels_image_start:\n'
            f'.incbin "{CUBIN}"\n'
            'b200_kernels_image_end:\n'
            '.byte 0\n'
            '.section .note.GNU-stack,"",@progbits\n')
        # The one runtime-API translation unit (static scratch + cudaGetSymbolAddress).
        na_src = CSRC / "noalloc" / "argmax_noalloc.cu"
        na_obj = BUILD / "argmax_noalloc.o"
        log += _run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
                     "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-c", str(na_src), "-o", str(na_obj)])
        cuda_lib = str(Path(NVCC).resolve().parent.parent / "lib64")
        cmd = [CXX, "-shared", "-fPIC", "-O2", "-std=c++17", "-Wall", "-Wno-unused-function",
               "-fvisibility=hidden", "-I", str(ROOT / "include"), "-I", str(CSRC / "abi"),
               "-I", str(CSRC / "runtime"), "-I", str(CSRC / "stages"), "-I", CUDA_INC, *map(str, cpp), str(asm),
               str(na_obj), "-o", str(LIB),
               "-L", cuda_lib, "-lcudart_static", "-lrt", "-ldl", "-lpthread"]
        log += _run(cmd)
    if verbose and log:
        print(log)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
    print(LIB)
