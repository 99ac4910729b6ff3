"""TEST INFRASTRUCTURE: ctypes access to the CPU oracle (liboracle.so) and, when it was built, to the
reference's own CPU sources (oracle/_ref/libfnb_ref.so).

Only tests, the smoke check and the bench's CPU-baseline leg import this module.  Nothing under the product
package does, and the product never falls back to it.

All functions take and return numpy arrays; layouts are ggml's block layouts
(ggml/src/ggml-common.h:258-276, :334-345, :414-418 in the reference tree).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "liboracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libfnb_ref.so")

ERR_TOKEN = 1
ERR_SLOT = 2

Q8_0_BYTES, Q8_1_BYTES, Q4_K_BYTES, IQ3_XXS_BYTES = 34, 36, 144, 98


def reference_root(reference: str | None = None) -> str | None:
    """Where the reference tree is: the argument, else the FNB_REFERENCE environment variable, else a directory named
    `reference` beside this repository; None when there is none (then only the oracle itself is built)."""
    for cand in (reference, os.environ.get("FNB_REFERENCE"),
                 os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "ggml", "src")):
            return cand
    return None


def build(with_ref: bool | None = None, reference: str | None = None) -> None:
    """Compile the oracle, and the reference's own sources where they lie when a reference tree is found."""
    ref_root = reference_root(reference)
    if with_ref is None:
        with_ref = ref_root is not None
    if with_ref and ref_root is None:
        raise FileNotFoundError("no reference tree: pass reference=... or set FNB_REFERENCE")
    cmd = ["make", "-C", _HERE, "all"] + (["ref", "ref-gguf", "REFERENCE=" + ref_root] if with_ref else [])
    subprocess.run(cmd, check=True, capture_output=True)
    if with_ref:
        # the reference's own GPU launchers for three operations (needs nvcc); a tree whose translation units do not
        # build for this GPU architecture leaves the library out and the tests that use it skip
        subprocess.run(["make", "-C", _HERE, "ref-gpu", "REFERENCE=" + ref_root], check=False, capture_output=True)


class _RopeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("pos", C.c_void_p), ("slots", C.c_void_p),
        ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p), ("q_out", C.c_void_p), ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p), ("k_f32", C.c_void_p), ("err", C.c_void_p), ("rows", C.c_int64),
        ("cache_slots", C.c_int64), ("n_q_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("n_rot", C.c_int32), ("theta_scale", C.c_float), ("eps", C.c_float), ("planes", C.c_void_p),
    ]


_lib = None
_ref = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build()
        _lib = C.CDLL(ORACLE_SO)
        _lib.fnbo_f32_to_f16.restype = C.c_uint16
        _lib.fnbo_f32_to_f16.argtypes = [C.c_float]
        _lib.fnbo_f16_to_f32.restype = C.c_float
        _lib.fnbo_f16_to_f32.argtypes = [C.c_uint16]
        for name in ("fnbo_expf_exact", "fnbo_sinf_exact", "fnbo_cosf_exact"):
            getattr(_lib, name).restype = C.c_float
            getattr(_lib, name).argtypes = [C.c_float]
    return _lib


def have_ref() -> bool:
    return os.path.exists(REF_SO)


REF_GPU_SO = os.path.join(_HERE, "_ref", "libfnb_ref_gpu.so")


def ref_gpu():
    """The reference's own GPU launchers (oracle/ref_gpu_shim.cu), or None when the library was not built."""
    if not os.path.exists(REF_GPU_SO):
        return None
    l = C.CDLL(REF_GPU_SO)
    P, I = C.c_void_p, C.c_int32
    l.fnbr_dcp_norm.argtypes, l.fnbr_dcp_norm.restype = [I, P, P, P, P, P, P, P, P, P], I
    l.fnbr_glu_finish.argtypes, l.fnbr_glu_finish.restype = [P, P, I, P, P, P], I
    l.fnbr_qsp_kv8.argtypes, l.fnbr_qsp_kv8.restype = [P, P, P, I, I, I, P, P, P, P, I, P, P], I
    l.fnbr_rope_theta_scale.argtypes, l.fnbr_rope_theta_scale.restype = [], C.c_float
    return l


REF_GGUF_SO = os.path.join(_HERE, "_ref", "libfnb_ref_gguf.so")
_ref_gguf = None


def build_ref_gguf() -> None:
    """Compile the reference's GGUF writer / reader (ggml/src/gguf.cpp with the ggml core) where it lies."""
    ref_root = reference_root()
    if ref_root is None:
        raise FileNotFoundError("no reference tree: set FNB_REFERENCE")
    subprocess.run(["make", "-C", _HERE, "REFERENCE=" + ref_root, "ref-gguf"], check=True, capture_output=True)


def have_ref_gguf() -> bool:
    return os.path.exists(REF_GGUF_SO)


def ref_gguf() -> C.CDLL:
    global _ref_gguf
    if _ref_gguf is None:
        _ref_gguf = C.CDLL(REF_GGUF_SO)
    return _ref_gguf


def ref_gguf_write(path: str, tensors, alignment: int = 32) -> None:
    """tensors: (name, ggml type, dims (ne0, ne1, ...), raw uint8 array); written by the reference's own gguf writer."""
    n = len(tensors)
    names = (C.c_char_p * n)(*[t[0].encode() for t in tensors])
    types = (C.c_int32 * n)(*[t[1] for t in tensors])
    nd = (C.c_int32 * n)(*[len(t[2]) for t in tensors])
    ne = (C.c_int64 * (4 * n))(*[d for t in tensors for d in (list(t[2]) + [1, 1, 1, 1])[:4]])
    bufs = [np.ascontiguousarray(t[3], np.uint8) for t in tensors]
    data = (C.c_void_p * n)(*[b.ctypes.data for b in bufs])
    rc = ref_gguf().ref_gguf_write(path.encode(), n, names, types, nd, ne, data, C.c_uint32(alignment))
    if rc != 0:
        raise RuntimeError(f"reference gguf writer failed ({rc})")


def ref_gguf_find(path: str, name: str):
    """(absolute file offset, ggml type, bytes, tensor count) as the reference's own reader reports them."""
    off, typ, nb, cnt = C.c_int64(), C.c_int32(), C.c_int64(), C.c_int64()
    rc = ref_gguf().ref_gguf_find(path.encode(), name.encode(), C.byref(off), C.byref(typ), C.byref(nb), C.byref(cnt))
    if rc != 0:
        raise KeyError(name)
    return off.value, typ.value, nb.value, cnt.value


def ref() -> C.CDLL:
    """The reference's own CPU sources (only exists where the reference tree was present at build time)."""
    global _ref
    if _ref is None:
        _ref = C.CDLL(REF_SO)
        _ref.ref_f32_to_f16.restype = C.c_uint16
        _ref.ref_f32_to_f16.argtypes = [C.c_float]
        _ref.ref_f16_to_f32.restype = C.c_float
        _ref.ref_f16_to_f32.argtypes = [C.c_uint16]
        _ref.ref_kv_q8_stress_rows.restype = C.c_int64
    return _ref


def _p(a: np.ndarray | None) -> C.c_void_p:
    if a is None:
        return C.c_void_p(0)
    assert a.flags["C_CONTIGUOUS"]
    return C.c_void_p(a.ctypes.data)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def use_libm(on: bool) -> None:
    lib().fnbo_use_libm(C.c_int(1 if on else 0))


# ---- scalar helpers -------------------------------------------------------------------------------------

def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    l = lib()
    return np.array([l.fnbo_f32_to_f16(float(v)) for v in np.asarray(x, np.float32).ravel()], np.uint16)


def f16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    l = lib()
    return np.array([l.fnbo_f16_to_f32(int(v)) for v in np.asarray(h, np.uint16).ravel()], np.float32)


# ---- quantisers / decoders ------------------------------------------------------------------------------

def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.size // 32 * Q8_0_BYTES, np.uint8)
    lib().fnbo_quantize_row_q8_0(_p(x), _p(out), C.c_int64(x.size))
    return out


def quantize_q8_1(x: np.ndarray) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.size // 32 * Q8_1_BYTES, np.uint8)
    lib().fnbo_quantize_row_q8_1(_p(x), _p(out), C.c_int64(x.size))
    return out


def dequantize_q8_0(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, np.uint8)
    out = np.empty(b.size // Q8_0_BYTES * 32, np.float32)
    lib().fnbo_dequantize_row_q8_0(_p(b), _p(out), C.c_int64(out.size))
    return out


def dequantize_q4_k(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, np.uint8)
    out = np.empty(b.size // Q4_K_BYTES * 256, np.float32)
    lib().fnbo_dequantize_row_q4_k(_p(b), _p(out), C.c_int64(out.size))
    return out


def dequantize_iq3_xxs(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, np.uint8)
    out = np.empty(b.size // IQ3_XXS_BYTES * 256, np.float32)
    lib().fnbo_dequantize_row_iq3_xxs(_p(b), _p(out), C.c_int64(out.size))
    return out


def dequantize_iq3_s(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, np.uint8)
    out = np.empty(b.size // 110 * 256, np.float32)
    lib().fnbo_dequantize_row_iq3_s(_p(b), _p(out), C.c_int64(out.size))
    return out


def get_rows(fmt: str, table: np.ndarray, n_vocab: int, ids: np.ndarray, cols: int, out: np.ndarray | None = None):
    """Returns (out [rows][cols] F32, err word).  Rows with a bad id keep `out`'s previous contents."""
    table = np.ascontiguousarray(table, np.uint8)
    ids = np.ascontiguousarray(ids, np.int32)
    if out is None:
        out = np.zeros((ids.size, cols), np.float32)
    err = np.zeros(1, np.uint32)
    fn = {"q4_k": lib().fnbo_get_rows_q4_k, "iq3_xxs": lib().fnbo_get_rows_iq3_xxs}[fmt]
    fn(_p(table), C.c_int64(n_vocab), _p(ids), _p(out), _p(err), C.c_int64(ids.size), C.c_int32(cols))
    return out, int(err[0])


def rms_norm(x: np.ndarray, w: np.ndarray | None, eps: float) -> np.ndarray:
    x = _f32(x)
    cols = x.shape[-1]
    w = None if w is None else _f32(w)
    y = np.empty_like(x)
    lib().fnbo_rms_norm_f32(_p(x), _p(w), C.c_float(eps), _p(y), C.c_int64(x.size // cols), C.c_int32(cols))
    return y


def swiglu_q8_1(gate: np.ndarray, up: np.ndarray, want_f32: bool = False):
    gate, up = _f32(gate), _f32(up)
    cols = gate.shape[-1]
    rows = gate.size // cols
    out = np.empty((rows, cols // 32 * Q8_1_BYTES), np.uint8)
    f32 = np.empty_like(gate) if want_f32 else None
    lib().fnbo_swiglu_q8_1(_p(gate), _p(up), _p(out), _p(f32), C.c_int64(rows), C.c_int32(cols))
    return (out, f32) if want_f32 else out


def swiglu_act(gate: np.ndarray, up: np.ndarray):
    gate, up = _f32(gate), _f32(up)
    cols = gate.shape[-1]
    rows = gate.size // cols
    codes = np.empty((rows, cols), np.int8)
    scales = np.empty((rows, cols // 32, 2), np.float32)
    f32 = np.empty_like(gate)
    lib().fnbo_swiglu_act(_p(gate), _p(up), _p(codes), _p(scales), _p(f32), C.c_int64(rows), C.c_int32(cols))
    return codes, scales, f32


def act_quantize(x: np.ndarray):
    x = _f32(x)
    k = x.shape[-1]
    rows = x.size // k
    codes = np.empty((rows, k), np.int8)
    scales = np.empty((rows, k // 32, 2), np.float32)
    lib().fnbo_act_quantize(_p(x), C.c_int64(rows), C.c_int32(k), _p(codes), _p(scales))
    return codes, scales


def kv8_quantize(x: np.ndarray):
    x = _f32(x)
    codes = np.empty(x.size, np.int8)
    scales = np.empty(x.size // 64, np.uint16)
    lib().fnbo_kv8_quantize(_p(x), C.c_int64(x.size), _p(codes), _p(scales))
    return codes, scales


def kv8_dequantize(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """The value each KV8 code stands for: float(code) * f32(FP16 scale of its group of 64), one F32 product, exact
    (fn::quant::kv_q8_value, fn/quant/kv_q8_ref.cpp:95-97; device form fn/kernels/qsa/kv_q8.cuh:61-67)."""
    c = np.ascontiguousarray(codes, np.int8).reshape(-1, 64).astype(np.float32)
    s = np.ascontiguousarray(scales, np.uint16).reshape(-1, 1).view(np.float16).astype(np.float32)
    return (c * s).reshape(-1)


IQ2_TYPE = {"iq2_xxs": 16, "iq2_xs": 17, "iq2_s": 22}   # ggml's type numbers, as the reference's templates use them


def expert_gu_rows(fmt: str, gate: np.ndarray, up: np.ndarray, act: np.ndarray, n: int, r0: int = 0, r1: int | None = None,
                   use_ref: bool = False, want_gu: bool = False):
    """ff[t][r] = silu(gate row r . act[t]) * (up row r . act[t]): weight rows uint8 [rows][n/256*block bytes] of
    fmt "q4_k" (144), "q5_k" (176), "iq3_xxs" (98), "iq3_s" (110), "iq2_xxs" (66), "iq2_xs" (74) or "iq2_s" (82) against Q8_K activations uint8 [nt][n/256*292].  use_ref: the reference's own
    AVX2 kernel (its libm's expf)."""
    gate, up, act = (np.ascontiguousarray(a, np.uint8) for a in (gate, up, act))
    if fmt in IQ2_TYPE:    # one entry point for the three IQ2 formats, told apart by ggml's type number
        rows, nt = gate.shape[0], act.shape[0]
        r1 = rows if r1 is None else r1
        ff = np.zeros((nt, rows), np.float32)
        ty = C.c_int32(IQ2_TYPE[fmt])
        if use_ref:
            ref().ref_iq_gu_rows_iq2(ty, _p(gate), _p(up), C.c_int64(gate.shape[1]), C.c_int32(n), _p(act),
                                     C.c_int64(act.shape[1]), C.c_int32(nt), _p(ff), C.c_int64(rows), C.c_int32(r0), C.c_int32(r1))
            return ff
        gu = np.zeros((2, nt, rows), np.float32) if want_gu else None
        lib().fnbo_expert_gu_rows_iq2(ty, _p(gate), _p(up), C.c_int64(gate.shape[1]), C.c_int32(n), _p(act),
                                      C.c_int64(act.shape[1]), C.c_int32(nt), _p(ff), C.c_int64(rows), _p(gu), C.c_int64(r0),
                                      C.c_int64(r1))
        return (ff, gu) if want_gu else ff
    ref_fn, own_fn = {"q4_k": ("ref_kq_gu_rows_q4_k", "fnbo_expert_gu_rows_q4_k"),
                      "q5_k": ("ref_kq_gu_rows_q5_k", "fnbo_expert_gu_rows_q5_k"),
                      "iq3_xxs": ("ref_iq_gu_rows_iq3_xxs", "fnbo_expert_gu_rows_iq3_xxs"),
                      "iq3_s": ("ref_iq_gu_rows_iq3_s", "fnbo_expert_gu_rows_iq3_s")}[fmt]
    gate, up, act = (np.ascontiguousarray(a, np.uint8) for a in (gate, up, act))
    rows, nt = gate.shape[0], act.shape[0]
    r1 = rows if r1 is None else r1
    ff = np.zeros((nt, rows), np.float32)
    if use_ref:
        getattr(ref(), ref_fn)(_p(gate), _p(up), C.c_int64(gate.shape[1]), C.c_int32(n), _p(act), C.c_int64(act.shape[1]),
                               C.c_int32(nt), _p(ff), C.c_int64(rows), C.c_int32(r0), C.c_int32(r1))
        return ff
    gu = np.zeros((2, nt, rows), np.float32) if want_gu else None
    getattr(lib(), own_fn)(_p(gate), _p(up), C.c_int64(gate.shape[1]), C.c_int32(n), _p(act), C.c_int64(act.shape[1]),
                           C.c_int32(nt), _p(ff), C.c_int64(rows), _p(gu), C.c_int64(r0), C.c_int64(r1))
    return (ff, gu) if want_gu else ff


def expert_gu_rows_q4_k(gate, up, act, n, **kw):
    return expert_gu_rows("q4_k", gate, up, act, n, **kw)


def expert_gu_rows_q5_k(gate, up, act, n, **kw):
    return expert_gu_rows("q5_k", gate, up, act, n, **kw)


def expert_gu_rows_iq3_xxs(gate, up, act, n, **kw):
    return expert_gu_rows("iq3_xxs", gate, up, act, n, **kw)


Q8_K_BYTES = 292


def quantize_q8_k(x: np.ndarray, which: str = "oracle") -> np.ndarray:
    """ggml Q8_K blocks of x (a multiple of 256 values).  which: "oracle" (this restatement), "ggml" (the reference's
    quantize_row_q8_K_ref) or "avx2" (the reference's fn::experts::cpu::quantize_q8_k)."""
    x = _f32(x).reshape(-1)
    out = np.zeros(x.size // 256 * Q8_K_BYTES, np.uint8)
    fn = {"oracle": lambda: lib().fnbo_quantize_row_q8_k, "ggml": lambda: ref().quantize_row_q8_K_ref,
          "avx2": lambda: ref().ref_quantize_q8_k_avx2}[which]()
    fn(_p(x), _p(out), C.c_int64(x.size))
    return out.reshape(-1, Q8_K_BYTES)


DOWN_FMT = {"q5_1": (0, 24, Q8_1_BYTES), "q8_0": (1, Q8_0_BYTES, Q8_0_BYTES), "iq4_nl": (2, 18, Q8_0_BYTES)}   # code, weight block, activation block


def quantize_act_q(x: np.ndarray, use_ref: bool = False):
    """The reference's planar 32-value activation: (codes int8 [rows][n], chunk scales f32 [rows][n/32]) of x [rows][n].
    use_ref: the reference's own AVX2 quantiser (n <= 640, a multiple of 128)."""
    x = _f32(x)
    rows, n = x.shape
    q, s = np.zeros((rows, n), np.int8), np.zeros((rows, n // 32), np.float32)
    for r in range(rows):
        if use_ref:
            ref().ref_quantize_act_q(_p(x[r]), C.c_int32(n), _p(q[r]), _p(s[r]))
        else:
            lib().fnbo_quantize_act_q(_p(x[r]), C.c_int64(n), _p(q[r]), _p(s[r]))
    return q, s


def expert_down_rows_q2_0(w: np.ndarray, n: int, q: np.ndarray = None, scale: np.ndarray = None, r0: int = 0,
                          r1: int | None = None, x: np.ndarray = None) -> np.ndarray:
    """out[t][r] = Q2_0 weight row r (uint8 [rows][n/64*18]) . planar activation row t (codes q, chunk scales scale).
    With x (F32 [nt][n], nt <= 8, n <= 640) instead: the reference's own quantiser and AVX2 rows."""
    w = np.ascontiguousarray(w, np.uint8)
    rows = w.shape[0]
    r1 = rows if r1 is None else r1
    if x is not None:
        x = _f32(x)
        out = np.zeros((x.shape[0], rows), np.float32)
        ref().ref_q2_down_rows(_p(w), C.c_int64(w.shape[1]), C.c_int32(n), _p(x), C.c_int32(x.shape[0]), _p(out),
                               C.c_int64(rows), C.c_int32(r0), C.c_int32(r1))
        return out
    q, scale = np.ascontiguousarray(q, np.int8), _f32(scale)
    out = np.zeros((q.shape[0], rows), np.float32)
    lib().fnbo_expert_down_rows_q2_0(_p(w), C.c_int64(w.shape[1]), C.c_int32(n), _p(q), C.c_int64(q.shape[1]), _p(scale),
                                     C.c_int64(scale.shape[1]), C.c_int32(q.shape[0]), _p(out), C.c_int64(rows),
                                     C.c_int64(r0), C.c_int64(r1))
    return out


def expert_down_rows(fmt: str, w: np.ndarray, act: np.ndarray, n: int, r0: int = 0, r1: int | None = None,
                     use_ref: bool = False) -> np.ndarray:
    """out[t][r] = weight row r . act[t]: w uint8 [rows][n/32 * weight block], act uint8 [nt][n/32 * activation block]
    (Q8_1 blocks for "q5_1" weights, Q8_0 blocks for "q8_0" and "iq4_nl").  use_ref: the reference's own AVX2 kernel."""
    code, wb, ab = DOWN_FMT[fmt]
    w, act = np.ascontiguousarray(w, np.uint8), np.ascontiguousarray(act, np.uint8)
    rows, nt = w.shape[0], act.shape[0]
    assert w.shape[1] == n // 32 * wb and act.shape[1] == n // 32 * ab
    r1 = rows if r1 is None else r1
    out = np.zeros((nt, rows), np.float32)
    fn = ref().ref_kq_down_rows if use_ref else lib().fnbo_expert_down_rows
    last = (C.c_int32(r0), C.c_int32(r1)) if use_ref else (C.c_int64(r0), C.c_int64(r1))
    fn(C.c_int32(code), _p(w), C.c_int64(w.shape[1]), C.c_int32(n), _p(act), C.c_int64(act.shape[1]), C.c_int32(nt),
       _p(out), C.c_int64(rows), *last)
    return out


def rope_kv_append(q, k, v, pos, *, n_rot: int, theta_scale: float, k_cache: np.ndarray, v_cache: np.ndarray,
                   cache_slots: int, slots=None, q_norm_w=None, k_norm_w=None, eps: float = 1e-6,
                   want_k_f32: bool = False, q_out: np.ndarray | None = None, planes=None):
    """q [rows][n_q][hd], k/v [rows][n_kv][hd]; caches are uint8 [cache_slots][n_kv][hd/32*34], updated in place.
    Returns (q_out, k_f32 or None, err)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    rows, n_q, hd = q.shape
    n_kv = k.shape[1]
    pos = np.ascontiguousarray(pos, np.int32)
    slots = None if slots is None else np.ascontiguousarray(slots, np.int32)
    qw = None if q_norm_w is None else _f32(q_norm_w)
    kw = None if k_norm_w is None else _f32(k_norm_w)
    if q_out is None:
        q_out = np.zeros_like(q)
    k_f32 = np.zeros_like(k) if want_k_f32 else None
    err = np.zeros(1, np.uint32)
    a = _RopeArgs(_p(q), _p(k), _p(v), _p(pos), _p(slots), _p(qw), _p(kw), _p(q_out), _p(k_cache), _p(v_cache),
                  _p(k_f32), _p(err), rows, cache_slots, n_q, n_kv, hd, n_rot, theta_scale, eps,
                  _p(None if planes is None else np.ascontiguousarray(planes, np.int32)))
    lib().fnbo_rope_neox_q8_0_append(C.byref(a))
    return q_out, k_f32, int(err[0])


def attend_f64(q, k, v, first, count, scale: float, gate=None) -> np.ndarray:
    """FP64 attention over decoded cache rows: q [rows][n_q][hd], k / v F32 [cells][n_kv][hd] (absolute cells), row t over
    cells first[t] .. first[t] + count[t] - 1.  Returns float64 [rows][n_q][hd]."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    rows, n_q, hd = q.shape
    n_kv = k.shape[1]
    first = np.ascontiguousarray(first, np.int32)
    count = np.ascontiguousarray(count, np.int32)
    g = None if gate is None else _f32(gate)
    out = np.zeros((rows, n_q, hd), np.float64)
    l = lib()
    l.fnbo_attend_f64.restype = None
    l.fnbo_attend_f64.argtypes = [C.c_void_p] * 6 + [C.c_int32] * 4 + [C.c_double, C.c_void_p]
    l.fnbo_attend_f64(_p(q), _p(g), _p(k), _p(v), _p(first), _p(count), rows, n_q, n_kv, hd, scale, _p(out))
    return out


def theta_scale(freq_base: float, n_rot: int) -> float:
    """powf(freq_base, -2/n_rot) in F32, as fn/kernels/qsa/attend.cu:830-832 computes it on the host."""
    l = lib()
    l.fnbo_theta_scale.restype = C.c_float
    return float(l.fnbo_theta_scale(C.c_float(freq_base), C.c_int32(n_rot)))


# ---- multi-threaded row split, for the timed CPU baseline ------------------------------------------------

def parallel_rows(fn, rows: int, threads: int) -> None:
    """Run fn(r0, r1) over an even split of [0, rows) on `threads` host threads (ctypes drops the GIL)."""
    threads = max(1, min(threads, rows))
    cuts = [rows * i // threads for i in range(threads + 1)]
    if threads == 1:
        fn(0, rows)
        return
    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(lambda i: fn(cuts[i], cuts[i + 1]), range(threads)))
