"""The C++ launcher shims (include/fnb200_fn.hpp): a host program in the reference's test style is compiled against
the header, the CUDA library and the oracle; its rejection cases run here without a GPU, its parity cases on the GPU."""
import os
import subprocess

import pytest

from fnfl_v100_b200 import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "shim_test.cpp")
EXE = os.path.join(ROOT, "tests", "cpp", "shim_test.bin")


@pytest.fixture(scope="module")
def exe(oracle):
    build.build()
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    pkg, orc = os.path.join(ROOT, "fnfl_v100_b200"), os.path.join(ROOT, "oracle")
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I" + os.path.join(ROOT, "include"), "-I" + orc,
           "-I" + os.path.join(cuda, "include"), SRC, "-o", EXE, "-L" + pkg, "-l:libfnb200.so", "-L" + orc, "-l:liboracle.so",
           "-L" + os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath," + pkg, "-Wl,-rpath," + orc,
           "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return EXE


def test_shims_compile_and_reject_bad_arguments(exe):
    r = subprocess.run([exe, "--reject"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr


@pytest.mark.gpu
def test_shims_parity_on_gpu(exe):
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
