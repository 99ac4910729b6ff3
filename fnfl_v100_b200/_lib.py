"""ctypes binding of libfnb200.so (the C ABI of include/fnb200.h).

There is no fallback: if the CUDA library is missing, import of the product package fails with an error that
says how to build it.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FNB200_LIB") or os.path.join(HERE, "libfnb200.so")   # FNB200_LIB: load another build

OK, REJECTED, LAUNCH_FAILED = 0, 1, 2
ERR_TOKEN, ERR_SLOT, ERR_TIMEOUT = 1, 2, 4


class RopeKvArgs(C.Structure):
    """fnb_rope_kv_args"""
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("pos", C.c_void_p), ("slots", C.c_void_p),
        ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p), ("q_out", C.c_void_p), ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p), ("k_f32", C.c_void_p), ("err", C.c_void_p), ("rows", C.c_int64),
        ("cache_slots", C.c_int64), ("n_q_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("n_rot", C.c_int32), ("theta_scale", C.c_float), ("eps", C.c_float), ("planes", C.c_void_p),
    ]


class EmbedArgs(C.Structure):
    """fnb_embed_args"""
    _fields_ = [
        ("table", C.c_void_p), ("tok", C.c_void_p), ("own", C.c_void_p), ("full", C.c_void_p), ("streams", C.c_void_p),
        ("err", C.c_void_p), ("n_vocab", C.c_int64), ("rows", C.c_int64), ("fmt", C.c_int32), ("n_own", C.c_int32),
        ("n_full", C.c_int32), ("col0", C.c_int32), ("n_streams", C.c_int32),
    ]


TABLE_Q4_K, TABLE_IQ3_XXS, TABLE_Q8_0, TABLE_IQ3_S = 0, 1, 2, 3


class KvReadArgs(C.Structure):
    """fnb_kv_read_args"""
    _fields_ = [("cache", C.c_void_p), ("scale", C.c_void_p), ("cells", C.c_void_p), ("out", C.c_void_p),
                ("err", C.c_void_p), ("rows", C.c_int64), ("cache_slots", C.c_int64), ("cell0", C.c_int64),
                ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32)]


class AttendArgs(C.Structure):
    """fnb_attend_args"""
    _fields_ = [("q", C.c_void_p), ("gate", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
                ("k_scale", C.c_void_p), ("v_scale", C.c_void_p), ("first_cell", C.c_void_p), ("n_cells", C.c_void_p),
                ("out", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("err", C.c_void_p),
                ("cache_slots", C.c_int64), ("range_begin", C.c_int64), ("range_end", C.c_int64), ("rows", C.c_int32),
                ("n_q_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("scale", C.c_float)]


class GgufTensor(C.Structure):
    """fnb_gguf_tensor"""
    _fields_ = [("ne", C.c_int64 * 4), ("offset", C.c_int64), ("row_bytes", C.c_int64), ("n_rows", C.c_int64),
                ("n_dims", C.c_int32), ("type", C.c_int32)]


class RopeKv8Args(C.Structure):
    """fnb_rope_kv8_args"""
    _fields_ = [("base", RopeKvArgs), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p)]


_P, _I64, _I32, _F = C.c_void_p, C.c_int64, C.c_int32, C.c_float

# name -> (restype, argtypes); every symbol include/fnb200.h declares
SIGNATURES = {
    "fnb_version": (_I32, []),
    "fnb_status_name": (C.c_char_p, [_I32]),
    "fnb_rms_norm_f32": (_I32, [_P, _P, _F, _P, _I64, _I32, _P]),
    "fnb_rms_norm_heads_f32": (_I32, [_P, _P, _F, _P, _I64, _I32, _I32, _P]),
    "fnb_swiglu_q8_1": (_I32, [_P, _P, _P, _P, _I64, _I32, _P, _P]),
    "fnb_swiglu_act": (_I32, [_P, _P, _P, _P, _P, _I64, _I32, _P, _P]),
    "fnb_quantize_q8_1": (_I32, [_P, _P, _I64, _I32, _P, _P]),
    "fnb_quantize_q8_0": (_I32, [_P, _P, _I64, _I32, _P, _P]),
    "fnb_act_quantize": (_I32, [_P, _P, _P, _I64, _I32, _P, _P]),
    "fnb_rms_norm_q8_1": (_I32, [_P, _P, _F, _P, _P, _I64, _I32, _P, _P]),
    "fnb_rms_norm_q8_0": (_I32, [_P, _P, _F, _P, _P, _I64, _I32, _P, _P]),
    "fnb_rms_norm_act": (_I32, [_P, _P, _F, _P, _P, _P, _I64, _I32, _P, _P]),
    "fnb_rope_neox_q8_0_append": (_I32, [C.POINTER(RopeKvArgs), _P]),
    "fnb_rope_neox_kv8_append": (_I32, [C.POINTER(RopeKv8Args), _P]),
    "fnb_rope_theta_scale": (_F, [_F, _I32]),
    "fnb_get_rows_q4_k": (_I32, [_P, _I64, _P, _P, _P, _I64, _I32, _P]),
    "fnb_get_rows_rms_norm_q4_k": (_I32, [_P, _I64, _P, _P, _F, _P, _P, _P, _I64, _I32, _P]),
    "fnb_get_rows_rms_norm_iq3_xxs": (_I32, [_P, _I64, _P, _P, _F, _P, _P, _P, _I64, _I32, _P]),
    "fnb_get_rows_iq3_xxs": (_I32, [_P, _I64, _P, _P, _P, _I64, _I32, _P]),
    "fnb_get_rows_q8_0": (_I32, [_P, _I64, _P, _P, _P, _I64, _I32, _P]),
    "fnb_embed_rows": (_I32, [C.POINTER(EmbedArgs), _P]),
    "fnb_embed_join": (_I32, [C.POINTER(EmbedArgs), _P, _I32, _P]),
    "fnb_embed_supply": (_I32, [C.POINTER(EmbedArgs), _P, _I64, _I64, _P]),
    "fnb_kv_read_f32": (_I32, [C.POINTER(KvReadArgs), _P]),
    "fnb_attend_workspace_bytes": (C.c_size_t, [C.POINTER(AttendArgs)]),
    "fnb_attend": (_I32, [C.POINTER(AttendArgs), _P]),
    "fnb_attend_static": (_I32, [C.POINTER(AttendArgs), _P]),
    "fnb_quantize_q8_k": (_I32, [_P, _P, _I64, _I32, _P]),
    "fnb_expert_gate_up_rows_q4_k": (_I32, [_P, _P, _I64, _I32, _P, _I64, _I32, _P, _I64, _P, _I64, _I64, _P]),
    "fnb_expert_gate_up_rows_q5_k": (_I32, [_P, _P, _I64, _I32, _P, _I64, _I32, _P, _I64, _P, _I64, _I64, _P]),
    "fnb_expert_gate_up_rows_iq3_s": (_I32, [_P, _P, _I64, _I32, _P, _I64, _I32, _P, _I64, _P, _I64, _I64, _P]),
    "fnb_expert_gate_up_rows_iq3_xxs": (_I32, [_P, _P, _I64, _I32, _P, _I64, _I32, _P, _I64, _P, _I64, _I64, _P]),
    "fnb_expert_gate_up_rows_iq2_xxs": (_I32, [_P, _P, _I64, _I32, _P, _I64, _I32, _P, _I64, _P, _I64, _I64, _P]),
    "fnb_expert_gate_up_rows_iq2_xs": (_I32, [_P, _P, _I64, _I32, _P, _I64, _I32, _P, _I64, _P, _I64, _I64, _P]),
    "fnb_expert_gate_up_rows_iq2_s": (_I32, [_P, _P, _I64, _I32, _P, _I64, _I32, _P, _I64, _P, _I64, _I64, _P]),
    "fnb_expert_down_rows_q5_1": (_I32, [_P, _I64, _I32, _P, _I64, _I32, _P, _I64, _I64, _I64, _P]),
    "fnb_expert_down_rows_q8_0": (_I32, [_P, _I64, _I32, _P, _I64, _I32, _P, _I64, _I64, _I64, _P]),
    "fnb_quantize_act_q": (_I32, [_P, _P, _P, _I64, _I32, _P]),
    "fnb_expert_down_rows_q2_0": (_I32, [_P, _I64, _I32, _P, _I64, _P, _I64, _I32, _P, _I64, _I64, _I64, _P]),
    "fnb_expert_down_rows_iq4_nl": (_I32, [_P, _I64, _I32, _P, _I64, _I32, _P, _I64, _I64, _I64, _P]),
    "fnb_check_tokens": (_I64, [_P, _I64, _I64]),
    "fnb_prepare_device": (_I32, []),
    "fnb_gguf_open": (_P, [C.c_char_p]),
    "fnb_gguf_close": (None, [_P]),
    "fnb_gguf_n_tensors": (_I64, [_P]),
    "fnb_gguf_find": (_I32, [_P, C.c_char_p, C.POINTER(GgufTensor)]),
    "fnb_gguf_read_rows": (_I32, [_P, C.POINTER(GgufTensor), _I64, _I64, _P]),
}

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "fnfl_v100_b200: the CUDA library %s is missing and there is no fallback path. "
                "Build it with `python -m fnfl_v100_b200.build` (needs nvcc)." % LIB_PATH)
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)  # AttributeError here means header and library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def status_name(code: int) -> str:
    return lib().fnb_status_name(code).decode()
