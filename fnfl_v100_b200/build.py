"""Compile the CUDA library in-tree for sm_100a: fnfl_v100_b200/libfnb200.so.

The library is plain `nvcc -shared`: a C ABI (include/fnb200.h), no Python or torch types in it.
--fmad=false because parity with the CPU definition depends on products and sums rounding separately.
Each translation unit is compiled to its own object (in parallel, only when it or a header changed) and the
objects are linked into the one shared library.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libfnb200.so")
OBJ_DIR = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "--fmad=false", "--ftz=false", "--prec-div=true", "--prec-sqrt=true",
    "-Xcompiler", "-fPIC",
]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers() -> list[str]:
    return (glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.inc"))
            + glob.glob(os.path.join(HERE, "..", "include", "*")))


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(p) > t for p in deps)


def stale() -> bool:
    return _newer(LIB, sources() + _headers())


def compile_objects(srcs: list[str], obj_dir: str, extra: list[str], force: bool, verbose: bool) -> list[str]:
    """Compile every source in `srcs` into `obj_dir` (skipping up-to-date objects); returns the object paths."""
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    hdrs = _headers()

    def one(src: str) -> tuple[str, str]:
        obj = os.path.join(obj_dir, os.path.splitext(os.path.basename(src))[0] + ".o")
        if not force and not _newer(obj, [src] + hdrs):
            return obj, ""
        cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s%s" % (src, r.stdout, r.stderr))
        return obj, r.stderr

    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 1)) as pool:
        done = list(pool.map(one, srcs))
    if verbose:
        for _, log in done:
            if log:
                print(log)
    return [o for o, _ in done]


def link(objs: list[str], out: str) -> str:
    nvcc = os.environ.get("NVCC", "nvcc")
    r = subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a"] + objs + ["-o", out],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return out


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not stale():
        return LIB
    return link(compile_objects(sources(), OBJ_DIR, [], force, verbose), LIB)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
