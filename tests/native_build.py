"""Builds the test-only CUDA libraries (never shipped, never loaded by the product):

  tests/native/libfnbt_selftest.so   exhaustive / randomised self-checks of the device arithmetic (selftest.cu)
  tests/native/libfnb200_shortwait.so  the three bulk-copy pipeline kernels of the product compiled with
                                     FNB_PRIMARY_SPIN_LIMIT = 2: every data-path barrier wait gives up after two
                                     polls while the unwinding waits keep the full limit, so a launch ends by
                                     itself with FNB_ERR_TIMEOUT in the error word and no copy in flight.

Both need nvcc; they are built on demand (and by the repository's build entry point, so that the files travel
with the tree to a machine that only runs the tests).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)

from fnfl_v100_b200 import build as B  # noqa: E402

NATIVE = os.path.join(HERE, "native")
SELFTEST_SO = os.path.join(NATIVE, "libfnbt_selftest.so")
SHORTWAIT_SO = os.path.join(NATIVE, "libfnb200_shortwait.so")
SHORTWAIT_SOURCES = ["swiglu_quant.cu", "rms_norm_quant.cu", "rope_kv_pipe.cu", "rope_kv.cu"]


def _deps() -> list[str]:
    return B.sources() + B._headers()


def build_selftest(force: bool = False) -> str:
    src = os.path.join(NATIVE, "selftest.cu")
    if force or B._newer(SELFTEST_SO, [src] + B._headers()):
        nvcc = os.environ.get("NVCC", "nvcc")
        r = subprocess.run([nvcc] + B.NVCC_FLAGS + ["-shared", src, "-o", SELFTEST_SO], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed on selftest.cu:\n" + r.stdout + r.stderr)
    return SELFTEST_SO


def build_shortwait(force: bool = False) -> str:
    srcs = [os.path.join(B.CSRC, n) for n in SHORTWAIT_SOURCES]
    if force or B._newer(SHORTWAIT_SO, srcs + B._headers()):
        objs = B.compile_objects(srcs, os.path.join(NATIVE, "build_shortwait"), ["-DFNB_PRIMARY_SPIN_LIMIT=2"],
                                 force, False)
        B.link(objs, SHORTWAIT_SO)
    return SHORTWAIT_SO


def build_all(force: bool = False) -> None:
    build_selftest(force)
    build_shortwait(force)


if __name__ == "__main__":
    build_all("--force" in sys.argv)
    print(SELFTEST_SO)
    print(SHORTWAIT_SO)
