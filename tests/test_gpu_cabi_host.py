"""The C ABI from a host that is neither Python nor C++: tests/cabi_host.c (plain C99, cudaMalloc'd
buffers, default stream) routes a mask, runs MaskedLinear forward, the one-call MaskedFFN forward and
the training forward, and checks them against its own float loop.  The program is test code: it is
compiled here, next to the test, and is not part of the library build."""
import os
import shutil
import subprocess

import pytest

from conftest import ROOT
from ffn_kernel_b200 import _lib
from ffn_kernel_b200.build import _nvcc

pytestmark = pytest.mark.gpu

SRC = os.path.join(ROOT, "tests", "cabi_host.c")
OUT_DIR = os.path.join(ROOT, "tests", "_build")
EXE = os.path.join(OUT_DIR, "cabi_host")


def build_c_host() -> str:
    """gcc -std=c99 against include/ffnk.h, linked with libffnk.so and the CUDA runtime."""
    gcc = shutil.which("gcc")
    assert gcc, "gcc is needed to build tests/cabi_host.c"
    header_dir = os.path.join(ROOT, "include")
    libdir = os.path.dirname(_lib.LIB_PATH)
    deps = [SRC, os.path.join(header_dir, "ffnk.h"), _lib.LIB_PATH]
    if os.path.exists(EXE) and all(os.path.getmtime(EXE) >= os.path.getmtime(d) for d in deps):
        return EXE
    os.makedirs(OUT_DIR, exist_ok=True)
    cuda = os.path.dirname(os.path.dirname(_nvcc()))
    cmd = [gcc, "-std=c99", "-O1", "-Wall", "-Werror", SRC, "-I", header_dir, "-I", os.path.join(cuda, "include"),
           "-L", libdir, "-lffnk", "-L", os.path.join(cuda, "lib64"), "-lcudart", "-lm",
           "-Wl,-rpath," + libdir, "-Wl,-rpath," + os.path.join(cuda, "lib64"), "-o", EXE]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, " ".join(cmd) + "\n" + r.stdout + r.stderr
    return EXE


def test_plain_c_host_gets_the_same_answers(libffnk):
    exe = build_c_host()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "cabi_host: OK" in res.stdout
