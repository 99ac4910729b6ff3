"""The C-ABI library on a machine without a GPU: it loads, exports every symbol include/fnb200.h declares, and
rejects arguments outside the contract before touching CUDA (nothing enqueued)."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

from fnfl_v100_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fnb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fnb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_the_binding_binds():
    assert declared_symbols() == sorted(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol(lib):
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = set(re.findall(r"\bT (fnb_[a-z0-9_]+)$", out, flags=re.M))
    missing = [s for s in declared_symbols() if s not in exported]
    assert not missing, missing


def test_version_and_status_names(lib):
    assert lib.fnb_version() >= 100
    assert _lib.status_name(0) == "ok" and "rejected" in _lib.status_name(1) and "launch" in _lib.status_name(2)


def test_theta_scale_is_powf(lib, oracle):
    assert lib.fnb_rope_theta_scale(1e7, 64) == pytest.approx(oracle.theta_scale(1e7, 64), abs=0)


def test_check_tokens(lib):
    ids = np.array([0, 5, 151935, 151936, -1], np.int32)
    p = C.c_void_p(ids.ctypes.data)
    assert lib.fnb_check_tokens(p, 3, 151936) == 0
    assert lib.fnb_check_tokens(p, 5, 151936) == 4      # 1 + index of the first bad id
    assert lib.fnb_check_tokens(None, 5, 151936) == -1


A16 = 0x7F0000001000   # a 16-byte aligned, never dereferenced address: rejection happens before any launch
ODD = A16 + 4


def test_rejections_enqueue_nothing(lib):
    R = _lib.REJECTED
    # rms_norm: null, misaligned, bad shapes
    assert lib.fnb_rms_norm_f32(None, A16, 1e-6, A16, 4, 2048, None) == R
    assert lib.fnb_rms_norm_f32(ODD, A16, 1e-6, A16, 4, 2048, None) == R
    assert lib.fnb_rms_norm_f32(A16, A16, 1e-6, A16, 0, 2048, None) == R
    assert lib.fnb_rms_norm_f32(A16, A16, 1e-6, A16, 4, 2050, None) == R
    assert lib.fnb_rms_norm_f32(A16, A16, -1.0, A16, 4, 2048, None) == R
    assert lib.fnb_rms_norm_heads_f32(A16, A16, 1e-6, A16, 4, 0, 256, None) == R
    # swiglu / requantisers: cols must be a multiple of 32, pointers 16-byte aligned
    assert lib.fnb_swiglu_q8_1(A16, A16, A16, None, 8, 48, None, None) == R
    assert lib.fnb_swiglu_q8_1(A16, None, A16, None, 8, 512, None, None) == R
    assert lib.fnb_swiglu_q8_1(A16, A16, ODD, None, 8, 512, None, None) == R
    assert lib.fnb_swiglu_q8_1(A16, A16, A16, None, 8, 512, A16 + 2, None) == R   # the error word needs 4-byte alignment
    assert lib.fnb_swiglu_act(A16, A16, A16, None, None, 8, 512, None, None) == R
    assert lib.fnb_quantize_q8_1(A16, A16, -3, 512, None, None) == R
    assert lib.fnb_quantize_q8_0(None, A16, 3, 512, None, None) == R
    assert lib.fnb_quantize_q8_k(A16, A16, 4, 300, None) == R      # cols not a multiple of 256
    assert lib.fnb_quantize_q8_k(ODD, A16, 4, 512, None) == R
    assert lib.fnb_quantize_q8_k(A16, None, 4, 512, None) == R
    # experts' gate / up rows: n not a multiple of 256, rows not back to back, a window whose activations exceed shared
    # memory, the debug planes with a window of more than one pass
    okg = (A16, A16, 1440, 2560, A16, 2920, 3, A16, 640, None, 0, 640, None)
    for i, bad in ((3, 2500), (2, 1444), (6, 0), (6, 65), (11, 0), (8, 100), (0, ODD), (4, None)):
        a = list(okg)
        a[i] = bad
        assert lib.fnb_expert_gate_up_rows_q4_k(*a) == R, (i, bad)
    big = list(okg)
    big[2], big[3], big[5] = 144 * 64, 16384, 292 * 64
    assert lib.fnb_expert_gate_up_rows_q4_k(*big) == R
    dbg = list(okg)
    dbg[6], dbg[9] = 9, A16
    assert lib.fnb_expert_gate_up_rows_q4_k(*dbg) == R
    ok5 = (A16, A16, 1760, 2560, A16, 2920, 3, A16, 640, None, 0, 640, None)
    for i, bad in ((3, 2500), (2, 1440), (6, 0), (6, 65), (11, 0), (8, 100), (0, ODD), (4, None)):
        a = list(ok5)
        a[i] = bad
        assert lib.fnb_expert_gate_up_rows_q5_k(*a) == R, (i, bad)
    # IQ4_NL down rows: an odd number of blocks a row, rows not back to back, a window of 0 rows, short out rows
    ok4 = (A16, 360, 640, A16, 680, 3, A16, 2560, 0, 2560, None)
    for i, bad in ((2, 672), (1, 364), (5, 0), (5, 65), (9, 0), (7, 100), (0, None), (4, 678), (4, 681)):
        a = list(ok4)
        a[i] = bad
        assert lib.fnb_expert_down_rows_iq4_nl(*a) == R, (i, bad)
    # Q2_0 down rows: n not whole pairs of 64-weight blocks, rows not back to back, codes rows off 16 bytes, no scales
    okq = (A16, 180, 640, A16, 640, A16, 20, 3, A16, 2560, 0, 2560, None)
    for i, bad in ((2, 576), (1, 184), (4, 648), (4, 624), (6, 19), (5, None), (7, 0), (11, 0), (9, 100)):
        a = list(okq)
        a[i] = bad
        assert lib.fnb_expert_down_rows_q2_0(*a) == R, (i, bad)
    assert lib.fnb_quantize_act_q(A16, A16, A16, 4, 48, None) == R
    assert lib.fnb_quantize_act_q(A16, ODD, A16, 4, 64, None) == R
    # the IQ3_XXS form: an odd number of super-blocks a row (rows off 4-byte boundaries), rows not back to back
    ok3 = (A16, A16, 980, 2560, A16, 2920, 3, A16, 640, None, 0, 640, None)
    for i, bad in ((3, 2304), (2, 984), (6, 0), (6, 65), (11, 0), (8, 100), (0, ODD), (4, None), (5, 2916)):
        a = list(ok3)
        a[i] = bad
        assert lib.fnb_expert_gate_up_rows_iq3_xxs(*a) == R, (i, bad)
    ok3s = (A16, A16, 1100, 2560, A16, 2920, 3, A16, 640, None, 0, 640, None)
    for i, bad in ((3, 2304), (2, 980), (6, 0), (11, 0), (0, ODD)):
        a = list(ok3s)
        a[i] = bad
        assert lib.fnb_expert_gate_up_rows_iq3_s(*a) == R, (i, bad)
    dbg3 = list(ok3)
    dbg3[6], dbg3[9] = 9, A16
    assert lib.fnb_expert_gate_up_rows_iq3_xxs(*dbg3) == R
    # experts' down rows: n not a multiple of 32, rows not back to back, window of 0 or 65 rows, r1 <= r0, short out rows
    ok = (A16, 480, 640, A16, 720, 3, A16, 2560, 0, 2560, None)
    for i, bad in ((2, 650), (1, 484), (5, 0), (5, 65), (9, 0), (7, 100), (0, None), (3, ODD + 1), (4, 718)):
        a = list(ok)
        a[i] = bad
        assert lib.fnb_expert_down_rows_q5_1(*a) == R, (i, bad)
    # cache read-back: head_dim outside {64, 128, 256}, a span past the cache, missing pointers
    ka = _lib.KvReadArgs(A16, None, None, A16, None, 8, 64, 0, 2, 256)
    for field, bad in (("head_dim", 96), ("cell0", 60), ("rows", 0), ("out", None), ("cache", ODD), ("n_kv_heads", 0)):
        kb = _lib.KvReadArgs.from_buffer_copy(ka)
        setattr(kb, field, bad)
        assert lib.fnb_kv_read_f32(C.byref(kb), None) == R, field
    assert lib.fnb_kv_read_f32(None, None) == R
    assert lib.fnb_act_quantize(A16, A16, ODD + 2, 3, 512, None, None) == R       # scales need 8-byte alignment
    # get_rows
    assert lib.fnb_get_rows_q4_k(A16, 100, A16, A16, None, 8, 2000, None) == R
    assert lib.fnb_get_rows_q4_k(A16, 0, A16, A16, None, 8, 2048, None) == R
    assert lib.fnb_get_rows_iq3_xxs(A16, 100, None, A16, None, 8, 2048, None) == R
    assert lib.fnb_get_rows_q8_0(A16, 100, A16, ODD, None, 8, 2048, None) == R
    # rope: head_dim, n_rot, null struct
    assert lib.fnb_rope_neox_q8_0_append(None, None) == R
    a = _lib.RopeKvArgs(A16, A16, A16, A16, None, None, None, A16, A16, A16, None, None, 4, 64, 16, 2, 256, 64,
                        0.5, 1e-6)
    for field, bad in (("head_dim", 96), ("n_rot", 66), ("n_rot", 512), ("rows", 0), ("cache_slots", 0),
                       ("q", ODD), ("k_cache", None), ("theta_scale", 0.0)):
        b = _lib.RopeKvArgs.from_buffer_copy(a)
        setattr(b, field, bad)
        assert lib.fnb_rope_neox_q8_0_append(C.byref(b), None) == R, field
    k8 = _lib.RopeKv8Args(a, None, A16)
    assert lib.fnb_rope_neox_kv8_append(C.byref(k8), None) == R


def test_embed_layout_rejections(lib):
    R = _lib.REJECTED
    ok = dict(table=A16, tok=A16, own=A16, full=A16, streams=A16, err=None, n_vocab=100, rows=8, fmt=_lib.TABLE_IQ3_S,
              n_own=1280, n_full=2560, col0=1280, n_streams=4)
    for field, bad in (("n_own", 1000), ("col0", 1284), ("col0", 2), ("n_full", 1000), ("rows", 0), ("fmt", 0),
                       ("tok", None), ("own", ODD), ("n_streams", 0), ("n_vocab", 0)):
        a = _lib.EmbedArgs(**{**ok, field: bad})
        assert lib.fnb_embed_rows(C.byref(a), None) == R, field
    a = _lib.EmbedArgs(**ok)
    assert lib.fnb_embed_join(C.byref(a), None, 0, None) == R
    assert lib.fnb_embed_join(C.byref(a), A16, 1284, None) == R
    assert lib.fnb_embed_supply(C.byref(a), A16, 6, 3, None) == R          # rows 6..8 of 8
    assert lib.fnb_embed_supply(C.byref(a), ODD, 0, 1, None) == R
    none = _lib.EmbedArgs(**{**ok, "own": None, "full": None, "streams": None})
    assert lib.fnb_embed_rows(C.byref(none), None) == R
    # fused norm + requant
    assert lib.fnb_rms_norm_q8_1(A16, A16, 1e-6, A16, None, 4, 2040, None, None) == R
    assert lib.fnb_rms_norm_q8_0(A16, A16, 1e-6, None, None, 4, 2048, None, None) == R
    assert lib.fnb_rms_norm_act(A16, A16, 1e-6, A16, None, None, 4, 2048, None, None) == R
    assert lib.fnb_rms_norm_q8_1(A16, A16, 1e-6, A16, None, 4, 8192, None, None) == R
    assert lib.fnb_rms_norm_q8_1(A16, A16, 1e-6, A16, None, 4, 2048, A16 + 2, None) == R
