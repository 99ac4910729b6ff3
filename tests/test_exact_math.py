"""The restated expf / sinf / cosf (oracle/fnb_exact_math.h) against this host's C library.

glibc 2.39's generic (non-FMA) build is bit-identical to the restatement; on x86-64 the dynamic loader may pick
an FMA-contracted build of the same algorithm, which differs in about one input per 10^8.  The first test runs
the comparison in a child with that selection disabled and demands zero mismatches; the second accepts the
in-process libm up to that rate."""
import os
import subprocess
import sys
import textwrap

import numpy as np

CHILD = textwrap.dedent("""
    import ctypes, sys, numpy as np
    sys.path.insert(0, %r)
    from oracle import oracle as O
    l = O.lib(); m = ctypes.CDLL("libm.so.6")
    for f in (m.expf, m.sinf, m.cosf): f.restype = ctypes.c_float; f.argtypes = [ctypes.c_float]
    g = np.random.default_rng(7)
    xs = np.concatenate([g.uniform(-20, 20, 30000), g.uniform(-104, 89, 10000)]).astype(np.float32)
    th = np.concatenate([g.uniform(0, 262144, 30000), g.uniform(0, 130, 10000), 10.0 ** g.uniform(-6, 0, 5000),
                         -g.uniform(0, 262144, 5000)]).astype(np.float32)
    bad = 0
    for x in xs:
        bad += np.float32(m.expf(float(x))).view(np.uint32) != np.float32(l.fnbo_expf_exact(float(x))).view(np.uint32)
    for t in th:
        bad += np.float32(m.sinf(float(t))).view(np.uint32) != np.float32(l.fnbo_sinf_exact(float(t))).view(np.uint32)
        bad += np.float32(m.cosf(float(t))).view(np.uint32) != np.float32(l.fnbo_cosf_exact(float(t))).view(np.uint32)
    print("MISMATCH", int(bad))
""")


def _run(env_extra):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, **env_extra)
    r = subprocess.run([sys.executable, "-c", CHILD % root], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    return int(r.stdout.strip().split()[-1])


def test_restatement_is_bit_identical_to_generic_glibc():
    assert _run({"GLIBC_TUNABLES": "glibc.cpu.hwcaps=-FMA,-AVX2,-FMA4"}) == 0


def test_restatement_against_default_libm(oracle):
    assert _run({}) <= 2     # 120k evaluations; the FMA build differs in ~1e-8 of inputs


def test_special_values(oracle):
    l = oracle.lib()
    assert l.fnbo_expf_exact(0.0) == 1.0
    assert l.fnbo_expf_exact(float("-inf")) == 0.0 and l.fnbo_expf_exact(100.0) == float("inf")
    assert np.isnan(l.fnbo_expf_exact(float("nan"))) and l.fnbo_expf_exact(-200.0) == 0.0
    assert l.fnbo_sinf_exact(0.0) == 0.0 and l.fnbo_cosf_exact(0.0) == 1.0
    assert np.isnan(l.fnbo_sinf_exact(float("inf")))
    assert l.fnbo_sinf_exact(1e-5) == np.float32(1e-5)


def test_fused_horner_expf_is_the_same_function_for_every_float(tmp_path):
    """Enumerates all floats |x| < 88: the CUDA fast path's evaluation order (fused Horner cubic) gives the float the
    definition gives, and fusing the reduction as well does not (so the kernels must not do that)."""
    if "fma" not in open("/proc/cpuinfo").read().split("flags", 1)[-1].split("\n", 1)[0].split():
        import pytest
        pytest.skip("host has no hardware fused multiply-add; the enumeration would take hours in software")
    here = os.path.dirname(os.path.abspath(__file__))
    exe = str(tmp_path / "expf_fma_exhaustive.bin")
    subprocess.run(["gcc", "-O2", "-mfma", "-ffp-contract=off", "-o", exe,
                    os.path.join(here, "cpp", "expf_fma_exhaustive.c"), "-lm", "-lpthread"], check=True)
    out = subprocess.run([exe, str(os.cpu_count() or 8)], check=True, capture_output=True, text=True).stdout.split()
    rec = dict(zip(out[0::2], map(int, out[1::2])))
    assert rec["inputs"] == 2 * 0x42b00000 and rec["float_differ"] == 0 and rec["max_double_ulp"] <= 2
    assert rec["float_differ_fused_reduction"] > 0
