"""A plain C host over include/b200abi.h and include/b200base.h: the headers must be valid C99, every entry point the
host names must link against libb200base.so, and the upper face (Artifact / Base) must work without a GPU."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_c_host_compiles_links_and_runs(tmp_path):
    from base_b200 import lib
    lib()                                                   # builds the library if it is not there yet
    exe = tmp_path / "host_check"
    libdir = ROOT / "base_b200"
    cmd = ["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", f"-I{ROOT / 'include'}", str(ROOT / "tests" / "c_host" / "host_check.c"),
           "-o", str(exe), f"-L{libdir}", "-lb200base", f"-Wl,-rpath,{libdir}"]
    built = subprocess.run(cmd, capture_output=True, text=True)
    assert built.returncode == 0, built.stderr
    ran = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert ran.returncode == 0, ran.stderr
    assert ran.stdout.startswith("host_check ok")
