import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def dev():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(scope="session")
def selftest_lib():
    """The test-only library of device self-checks (tests/native/selftest.cu), built on demand."""
    import ctypes as C
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import native_build
    lib = C.CDLL(native_build.build_selftest())
    P, U64 = C.c_void_p, C.c_uint64
    lib.fnbt_selftest_glu_math.argtypes, lib.fnbt_selftest_glu_math.restype = [U64, U64, P, P], C.c_int32
    lib.fnbt_selftest_q8_rule.argtypes, lib.fnbt_selftest_q8_rule.restype = [P, P], C.c_int32
    lib.fnbt_selftest_kv8_math.argtypes, lib.fnbt_selftest_kv8_math.restype = [U64, U64, P, P], C.c_int32
    lib.fnbt_selftest_expf.argtypes, lib.fnbt_selftest_expf.restype = [P, P], C.c_int32
    return lib


@pytest.fixture(scope="session")
def shortwait_lib():
    """The product's pipeline kernels rebuilt with a data-path wait limit of two polls (see tests/native_build.py)."""
    import ctypes as C
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import native_build
    from fnfl_v100_b200 import _lib
    lib = C.CDLL(native_build.build_shortwait())
    for name in ("fnb_swiglu_q8_1", "fnb_quantize_q8_1", "fnb_rms_norm_q8_1", "fnb_rope_neox_q8_0_append"):
        res, args = _lib.SIGNATURES[name]
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib
