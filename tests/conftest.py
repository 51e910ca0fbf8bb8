import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _has_gpu() -> bool:
    if os.environ.get("B200_FORCE_NO_GPU"):
        return False
    import ctypes
    try:
        cu = ctypes.CDLL("libcuda.so.1")
    except OSError:
        return False
    if cu.cuInit(0) != 0:
        return False
    n = ctypes.c_int(0)
    return cu.cuDeviceGetCount(ctypes.byref(n)) == 0 and n.value > 0


HAS_GPU = _has_gpu()


def pytest_collection_modifyitems(config, items):
    if HAS_GPU:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    return GOLDEN


def build_probe_kernels() -> Path:
    """Compile tests/kernels/probe_kernels.cu (test and probe kernels, not part of the library's image) to a cubin
    next to it; nvcc cross-compiles, so this also runs on a host without a GPU."""
    import subprocess
    src = Path(__file__).resolve().parent / "kernels" / "probe_kernels.cu"
    out = src.parent / "_build" / "probe_kernels.cubin"
    inc = ROOT / "base_b200" / "csrc" / "kernels"
    deps = [src] + list(inc.glob("*.cuh"))
    if not out.exists() or any(d.stat().st_mtime > out.stat().st_mtime for d in deps):
        out.parent.mkdir(exist_ok=True)
        nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
        subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-cubin", "-O3", "-lineinfo", "-std=c++17",
                        "-I", str(inc), "-o", str(out), str(src)], check=True)
    return out

