"""Host-side operators over torch CUDA tensors: thin, checked calls into the C ABI (include/fnb200.h).

The names and argument meaning follow the reference's launcher families (fn::draft::dcp_norm,
fn::experts::glu_finish, fn::act::quantize, fn::qsa::qsp_kv, fn::embed::embed_rows); torch only supplies device
memory and the current stream.  Every function enqueues on `torch.cuda.current_stream()` and returns without
synchronising.  A rejected argument raises ValueError (the reference returns false with nothing enqueued); there
is no CPU or eager fallback.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

Q8_0_BLOCK, Q8_1_BLOCK, Q4_K_BLOCK, IQ3_XXS_BLOCK = 34, 36, 144, 98
ERR_TOKEN, ERR_SLOT, ERR_TIMEOUT = _lib.ERR_TOKEN, _lib.ERR_SLOT, _lib.ERR_TIMEOUT

_TABLE_BLOCK = {"q4_k": (256, Q4_K_BLOCK), "iq3_xxs": (256, IQ3_XXS_BLOCK), "q8_0": (32, Q8_0_BLOCK)}


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _dev(t: torch.Tensor, dtype: torch.dtype, name: str) -> torch.Tensor:
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == dtype and t.is_contiguous()):
        raise ValueError(f"{name}: expected a contiguous CUDA tensor of {dtype}")
    return t


def _same_device(*tensors) -> torch.device:
    """Every tensor of a call lives on one device, which becomes the current device for the launch."""
    devs = {t.device for t in tensors if t is not None}
    if len(devs) != 1:
        raise ValueError("tensors of one call must live on one CUDA device")
    return devs.pop()


def _numel(t: torch.Tensor | None, n: int, name: str) -> None:
    if t is not None and t.numel() != n:
        raise ValueError(f"{name}: expected {n} elements, got {t.numel()}")


def _err(err: torch.Tensor | None) -> torch.Tensor | None:
    if err is not None:
        _dev(err, torch.int32, "err")
    return err


def _check(status: int, what: str) -> None:
    if status == _lib.OK:
        return
    msg = f"{what}: {_lib.status_name(status)}"
    raise ValueError(msg) if status == _lib.REJECTED else RuntimeError(msg)


def new_err(device) -> torch.Tensor:
    """A zeroed device error word (uint32 viewed as int32) for the kernels' data-dependent faults."""
    return torch.zeros(1, dtype=torch.int32, device=device)


# ---- RMSNorm ------------------------------------------------------------------------------------------------

def rms_norm(x: torch.Tensor, w: torch.Tensor | None, eps: float = 1e-6, out: torch.Tensor | None = None):
    """y = (x * scale) * w per row of x [..., cols]; replaces fn::draft::dcp_norm's arithmetic."""
    _dev(x, torch.float32, "x")
    if w is not None:
        _dev(w, torch.float32, "w")
        if w.numel() != x.shape[-1]:
            raise ValueError("w: expected [cols]")
    out = torch.empty_like(x) if out is None else _dev(out, torch.float32, "out")
    cols = x.shape[-1]
    _check(_lib.lib().fnb_rms_norm_f32(_ptr(x), _ptr(w), eps, _ptr(out), x.numel() // cols, cols, _stream()),
           "rms_norm")
    return out


def rms_norm_heads(x: torch.Tensor, w: torch.Tensor | None, eps: float = 1e-6, out: torch.Tensor | None = None):
    """The per-head Q/K norm over x [rows][n_heads][head_dim] with one weight [head_dim]."""
    _dev(x, torch.float32, "x")
    if x.dim() != 3:
        raise ValueError("x: expected [rows][n_heads][head_dim]")
    if w is not None:
        _dev(w, torch.float32, "w")
    out = torch.empty_like(x) if out is None else _dev(out, torch.float32, "out")
    rows, n_heads, hd = x.shape
    _check(_lib.lib().fnb_rms_norm_heads_f32(_ptr(x), _ptr(w), eps, _ptr(out), rows, n_heads, hd, _stream()),
           "rms_norm_heads")
    return out


def rms_norm_quant(x: torch.Tensor, w: torch.Tensor | None, eps: float = 1e-6, fmt: str = "q8_1",
                   out_f32: torch.Tensor | None = None, err: torch.Tensor | None = None):
    """RMSNorm fused with requantisation of its output.  fmt "q8_1" / "q8_0": returns uint8 blocks [rows][cols/32*B];
    fmt "act": returns (codes int8 [rows][cols], scales F32 [rows][cols/32][2])."""
    _dev(x, torch.float32, "x")
    rows, cols = _rows_cols(x)
    if w is not None:
        _dev(w, torch.float32, "w")
        _numel(w, cols, "w")
    if out_f32 is not None:
        _dev(out_f32, torch.float32, "out_f32")
        _numel(out_f32, rows * cols, "out_f32")
    L = _lib.lib()
    with torch.cuda.device(_same_device(x, w, out_f32, _err(err))):
        if fmt == "act":
            codes = torch.empty((rows, cols), dtype=torch.int8, device=x.device)
            scales = torch.empty((rows, cols // 32, 2), dtype=torch.float32, device=x.device)
            _check(L.fnb_rms_norm_act(_ptr(x), _ptr(w), eps, _ptr(codes), _ptr(scales), _ptr(out_f32), rows, cols,
                                      _ptr(err), _stream()), "rms_norm_act")
            return codes, scales
        bb = {"q8_1": Q8_1_BLOCK, "q8_0": Q8_0_BLOCK}[fmt]
        out = torch.empty((rows, cols // 32 * bb), dtype=torch.uint8, device=x.device)
        fn = L.fnb_rms_norm_q8_1 if fmt == "q8_1" else L.fnb_rms_norm_q8_0
        _check(fn(_ptr(x), _ptr(w), eps, _ptr(out), _ptr(out_f32), rows, cols, _ptr(err), _stream()), "rms_norm_" + fmt)
        return out


# ---- SwiGLU + requantisation --------------------------------------------------------------------------------

def _rows_cols(x: torch.Tensor) -> tuple[int, int]:
    cols = x.shape[-1]
    return x.numel() // cols, cols


def swiglu_q8_1(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor | None = None,
                out_f32: torch.Tensor | None = None, err: torch.Tensor | None = None) -> torch.Tensor:
    """silu(gate) * up -> ggml Q8_1 blocks, uint8 [rows][cols / 32 * 36]; replaces fn::experts::glu_finish."""
    _dev(gate, torch.float32, "gate")
    _dev(up, torch.float32, "up")
    if up.shape != gate.shape:
        raise ValueError("gate and up must have one shape")
    rows, cols = _rows_cols(gate)
    with torch.cuda.device(_same_device(gate, up, out, out_f32, _err(err))):
        if out is None:
            out = torch.empty((rows, cols // 32 * Q8_1_BLOCK), dtype=torch.uint8, device=gate.device)
        _dev(out, torch.uint8, "out")
        _numel(out, rows * (cols // 32) * Q8_1_BLOCK, "out")
        if out_f32 is not None:
            _dev(out_f32, torch.float32, "out_f32")
            _numel(out_f32, rows * cols, "out_f32")
        _check(_lib.lib().fnb_swiglu_q8_1(_ptr(gate), _ptr(up), _ptr(out), _ptr(out_f32), rows, cols, _ptr(err),
                                          _stream()), "swiglu_q8_1")
    return out


def swiglu_act(gate: torch.Tensor, up: torch.Tensor, out_f32: torch.Tensor | None = None,
               err: torch.Tensor | None = None):
    """silu(gate) * up -> the reference's activation format: (codes int8 [rows][cols], scales F32 [rows][cols/32][2])."""
    _dev(gate, torch.float32, "gate")
    _dev(up, torch.float32, "up")
    if up.shape != gate.shape:
        raise ValueError("gate and up must have one shape")
    rows, cols = _rows_cols(gate)
    if out_f32 is not None:
        _dev(out_f32, torch.float32, "out_f32")
        _numel(out_f32, rows * cols, "out_f32")
    with torch.cuda.device(_same_device(gate, up, out_f32, _err(err))):
        codes = torch.empty((rows, cols), dtype=torch.int8, device=gate.device)
        scales = torch.empty((rows, cols // 32, 2), dtype=torch.float32, device=gate.device)
        _check(_lib.lib().fnb_swiglu_act(_ptr(gate), _ptr(up), _ptr(codes), _ptr(scales), _ptr(out_f32), rows, cols,
                                         _ptr(err), _stream()), "swiglu_act")
    return codes, scales


def quantize_q8_1(x: torch.Tensor, err: torch.Tensor | None = None) -> torch.Tensor:
    _dev(x, torch.float32, "x")
    rows, cols = _rows_cols(x)
    with torch.cuda.device(_same_device(x, _err(err))):
        out = torch.empty((rows, cols // 32 * Q8_1_BLOCK), dtype=torch.uint8, device=x.device)
        _check(_lib.lib().fnb_quantize_q8_1(_ptr(x), _ptr(out), rows, cols, _ptr(err), _stream()), "quantize_q8_1")
    return out


def quantize_q8_0(x: torch.Tensor, err: torch.Tensor | None = None) -> torch.Tensor:
    _dev(x, torch.float32, "x")
    rows, cols = _rows_cols(x)
    with torch.cuda.device(_same_device(x, _err(err))):
        out = torch.empty((rows, cols // 32 * Q8_0_BLOCK), dtype=torch.uint8, device=x.device)
        _check(_lib.lib().fnb_quantize_q8_0(_ptr(x), _ptr(out), rows, cols, _ptr(err), _stream()), "quantize_q8_0")
    return out


def quantize_q8_k(x: torch.Tensor) -> torch.Tensor:
    """ggml Q8_K blocks (fn::experts::cpu::quantize_q8_k): uint8 [rows][cols/256*292]."""
    _dev(x, torch.float32, "x")
    rows, cols = _rows_cols(x)
    out = torch.empty((rows, cols // 256 * 292), dtype=torch.uint8, device=x.device)
    _check(_lib.lib().fnb_quantize_q8_k(_ptr(x), _ptr(out), rows, cols, _stream()), "quantize_q8_k")
    return out


def act_quantize(x: torch.Tensor, err: torch.Tensor | None = None):
    """fn::act::quantize: F32 [rows][k] -> (codes int8 [rows][k], scales F32 [rows][k/32][2])."""
    _dev(x, torch.float32, "x")
    rows, cols = _rows_cols(x)
    with torch.cuda.device(_same_device(x, _err(err))):
        codes = torch.empty((rows, cols), dtype=torch.int8, device=x.device)
        scales = torch.empty((rows, cols // 32, 2), dtype=torch.float32, device=x.device)
        _check(_lib.lib().fnb_act_quantize(_ptr(x), _ptr(codes), _ptr(scales), rows, cols, _ptr(err), _stream()),
               "act_quantize")
    return codes, scales


# ---- RoPE + KV append -----------------------------------------------------------------------------------------

def theta_scale(freq_base: float, n_rot: int) -> float:
    return float(_lib.lib().fnb_rope_theta_scale(freq_base, n_rot))


def new_kv_cache(cache_slots: int, n_kv_heads: int, head_dim: int, device, fmt: str = "q8_0"):
    """Zeroed cache planes.  q8_0: uint8 [slots][n_kv][head_dim/32*34]; kv8: (codes int8, scales fp16-bits int16)."""
    if fmt == "q8_0":
        return torch.zeros((cache_slots, n_kv_heads, head_dim // 32 * Q8_0_BLOCK), dtype=torch.uint8, device=device)
    codes = torch.zeros((cache_slots, n_kv_heads, head_dim), dtype=torch.int8, device=device)
    scales = torch.zeros((cache_slots, n_kv_heads, head_dim // 64), dtype=torch.int16, device=device)
    return codes, scales


def _rope_args(q, k, v, pos, slots, q_norm_w, k_norm_w, q_out, k_cache, v_cache, k_f32, err, n_rot, ts, eps, planes=None):
    _dev(q, torch.float32, "q")
    _dev(k, torch.float32, "k")
    _dev(v, torch.float32, "v")
    _dev(pos, torch.int32, "pos")
    if q.dim() != 3 or k.dim() != 3 or v.shape != k.shape or q.shape[0] != k.shape[0] or q.shape[2] != k.shape[2]:
        raise ValueError("q [rows][n_q][hd], k and v [rows][n_kv][hd]")
    rows, n_q, hd = q.shape
    if pos.numel() != rows or (slots is not None and slots.numel() != rows):
        raise ValueError("pos / slots: expected [rows]")
    if planes is not None:
        _dev(planes, torch.int32, "planes")
        if planes.numel() != 4 * rows:
            raise ValueError("planes: expected [rows][4]")
    cache_slots = k_cache.shape[0]
    a = _lib.RopeKvArgs(
        _ptr(q).value, _ptr(k).value, _ptr(v).value, _ptr(pos).value, _ptr(slots).value, _ptr(q_norm_w).value,
        _ptr(k_norm_w).value, _ptr(q_out).value, _ptr(k_cache).value, _ptr(v_cache).value, _ptr(k_f32).value,
        _ptr(err).value, rows, cache_slots, n_q, k.shape[1], hd, n_rot, ts, eps, _ptr(planes).value)
    return a


def rope_neox_q8_0_append(q, k, v, pos, *, n_rot: int, theta_scale: float, k_cache, v_cache, slots=None,
                          q_norm_w=None, k_norm_w=None, eps: float = 1e-6, q_out=None, k_f32=None, err=None,
                          planes=None):
    """Per-head norm (optional) + NeoX partial RoPE; Q -> q_out (F32), K/V -> Q8_0 cells at each token's slot.
    Replaces fn::qsa::qsp_kv and the prepare phase of fn::qsa::attn::attend.  Returns q_out."""
    if q_out is None:
        q_out = torch.empty_like(q)
    _dev(k_cache, torch.uint8, "k_cache")
    _dev(v_cache, torch.uint8, "v_cache")
    a = _rope_args(q, k, v, pos, slots, q_norm_w, k_norm_w, q_out, k_cache, v_cache, k_f32, err, n_rot,
                   theta_scale, eps, planes)
    _check(_lib.lib().fnb_rope_neox_q8_0_append(C.byref(a), _stream()), "rope_neox_q8_0_append")
    return q_out


def rope_neox_kv8_append(q, k, v, pos, *, n_rot: int, theta_scale: float, k_cache, v_cache, k_scale, v_scale,
                         slots=None, q_norm_w=None, k_norm_w=None, eps: float = 1e-6, q_out=None, k_f32=None,
                         err=None, planes=None):
    """The same step into the reference's KV8 format (int8 codes + FP16 scale per 64 values)."""
    if q_out is None:
        q_out = torch.empty_like(q)
    _dev(k_cache, torch.int8, "k_cache")
    _dev(v_cache, torch.int8, "v_cache")
    _dev(k_scale, torch.int16, "k_scale")
    _dev(v_scale, torch.int16, "v_scale")
    base = _rope_args(q, k, v, pos, slots, q_norm_w, k_norm_w, q_out, k_cache, v_cache, k_f32, err, n_rot,
                      theta_scale, eps, planes)
    a = _lib.RopeKv8Args(base, _ptr(k_scale).value, _ptr(v_scale).value)
    _check(_lib.lib().fnb_rope_neox_kv8_append(C.byref(a), _stream()), "rope_neox_kv8_append")
    return q_out


# ---- embedding get_rows ---------------------------------------------------------------------------------------

def table_row_bytes(fmt: str, cols: int) -> int:
    values, nbytes = _TABLE_BLOCK[fmt]
    return cols // values * nbytes


def kv_read_f32(cache: torch.Tensor, *, scale: torch.Tensor | None = None, cells: torch.Tensor | None = None,
                cell0: int = 0, rows: int | None = None, out: torch.Tensor | None = None,
                err: torch.Tensor | None = None) -> torch.Tensor:
    """Cache rows widened to F32 exactly as a consumer reads them: out [rows][n_kv][head_dim].  `cache` is a Q8_0 plane
    from new_kv_cache (scale None) or the KV8 codes with `scale` their FP16 plane; rows are cells[t], or cell0 + t."""
    kv8 = scale is not None
    _dev(cache, torch.int8 if kv8 else torch.uint8, "cache")
    slots, n_kv = cache.shape[0], cache.shape[1]
    hd = cache.shape[2] if kv8 else cache.shape[2] // Q8_0_BLOCK * 32
    if kv8:
        _dev(scale, torch.int16, "scale")
    if cells is not None:
        _dev(cells, torch.int32, "cells")
        rows = cells.numel()
    elif rows is None:
        rows = slots - cell0
    if out is None:
        out = torch.empty((rows, n_kv, hd), dtype=torch.float32, device=cache.device)
    _dev(out, torch.float32, "out")
    a = _lib.KvReadArgs(_ptr(cache).value, _ptr(scale).value, _ptr(cells).value, _ptr(out).value, _ptr(err).value,
                        rows, slots, cell0, n_kv, hd)
    _check(_lib.lib().fnb_kv_read_f32(C.byref(a), _stream()), "kv_read_f32")
    return out


def attend(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *, range_begin: int, range_end: int,
           scale: float | None = None, k_scale: torch.Tensor | None = None, v_scale: torch.Tensor | None = None,
           first_cell: torch.Tensor | None = None, n_cells: torch.Tensor | None = None, gate: torch.Tensor | None = None,
           out: torch.Tensor | None = None, workspace: torch.Tensor | None = None, err: torch.Tensor | None = None):
    """Decode attention of q [rows][n_q][hd] over cells [range_begin, range_end) of the cache planes new_kv_cache made
    (Q8_0, or KV8 codes with k_scale / v_scale): the attention phase of fn::qsa::attn::attend for dense cell ranges.
    Row t attends first_cell[t] .. + n_cells[t] (int32 device tensors) when given.  `workspace` (uint8) is reused when it
    is large enough, else allocated.  Returns out [rows][n_q][hd]."""
    _dev(q, torch.float32, "q")
    if q.dim() != 3:
        raise ValueError("q: expected [rows][n_q_heads][head_dim]")
    rows, n_q, hd = q.shape
    kv8 = k_scale is not None or v_scale is not None
    _dev(k_cache, torch.int8 if kv8 else torch.uint8, "k_cache")
    _dev(v_cache, torch.int8 if kv8 else torch.uint8, "v_cache")
    if kv8:
        _dev(k_scale, torch.int16, "k_scale")
        _dev(v_scale, torch.int16, "v_scale")
    slots, n_kv = k_cache.shape[0], k_cache.shape[1]
    if v_cache.shape != k_cache.shape or k_cache.shape[2] != (hd if kv8 else hd // 32 * Q8_0_BLOCK):
        raise ValueError("k_cache / v_cache: expected the planes of new_kv_cache for this head_dim")
    for name, t in (("first_cell", first_cell), ("n_cells", n_cells)):
        if t is not None:
            _dev(t, torch.int32, name)
            _numel(t, rows, name)
    if gate is not None:
        _dev(gate, torch.float32, "gate")
        _numel(gate, q.numel(), "gate")
    with torch.cuda.device(_same_device(q, k_cache, v_cache, k_scale, v_scale, first_cell, n_cells, gate, out, _err(err))):
        if out is None:
            out = torch.empty_like(q)
        _dev(out, torch.float32, "out")
        _numel(out, q.numel(), "out")
        a = _lib.AttendArgs(_ptr(q).value, _ptr(gate).value, _ptr(k_cache).value, _ptr(v_cache).value, _ptr(k_scale).value,
                            _ptr(v_scale).value, _ptr(first_cell).value, _ptr(n_cells).value, _ptr(out).value, None, 0,
                            _ptr(err).value, slots, range_begin, range_end, rows, n_q, n_kv, hd,
                            float(scale) if scale is not None else hd ** -0.5)
        need = int(_lib.lib().fnb_attend_workspace_bytes(C.byref(a)))
        if need == 0:
            raise ValueError("attend: shape outside the contract")
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
        _dev(workspace, torch.uint8, "workspace")
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
        _check(_lib.lib().fnb_attend(C.byref(a), _stream()), "attend")
    return out


def get_rows(fmt: str, table: torch.Tensor, ids: torch.Tensor, cols: int, out: torch.Tensor | None = None,
             err: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = dequantised row ids[t] of `table` (uint8 [n_vocab][row_bytes]); replaces fn::embed::embed_rows."""
    _dev(table, torch.uint8, "table")
    _dev(ids, torch.int32, "ids")
    rb = table_row_bytes(fmt, cols)
    if table.numel() % rb != 0:
        raise ValueError("table: size is not a whole number of rows")
    n_vocab = table.numel() // rb
    if out is None:
        out = torch.empty((ids.numel(), cols), dtype=torch.float32, device=table.device)
    _dev(out, torch.float32, "out")
    fn = getattr(_lib.lib(), "fnb_get_rows_" + fmt)
    _check(fn(_ptr(table), n_vocab, _ptr(ids), _ptr(out), _ptr(err), ids.numel(), cols, _stream()), "get_rows_" + fmt)
    return out


def get_rows_rms_norm(fmt: str, table: torch.Tensor, ids: torch.Tensor, cols: int, w: torch.Tensor | None, eps: float,
                      out: torch.Tensor | None = None, normed: torch.Tensor | None = None,
                      err: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """get_rows and the RMSNorm of each row in one launch (Q4_K and IQ3_XXS tables): returns (rows, normalised rows),
    the same values as get_rows followed by rms_norm."""
    if fmt not in ("q4_k", "iq3_xxs"):
        raise ValueError("get_rows_rms_norm: Q4_K and IQ3_XXS tables")
    _dev(table, torch.uint8, "table")
    _dev(ids, torch.int32, "ids")
    rb = table_row_bytes(fmt, cols)
    if table.numel() % rb != 0:
        raise ValueError("table: size is not a whole number of rows")
    n_vocab = table.numel() // rb
    n = ids.numel()
    if out is None:
        out = torch.empty((n, cols), dtype=torch.float32, device=table.device)
    if normed is None:
        normed = torch.empty((n, cols), dtype=torch.float32, device=table.device)
    _dev(out, torch.float32, "out")
    _dev(normed, torch.float32, "normed")
    _numel(out, n * cols, "out")
    _numel(normed, n * cols, "normed")
    if w is not None:
        _dev(w, torch.float32, "w")
        _numel(w, cols, "w")
    _same_device(table, ids, out, normed, w, err)
    fn = getattr(_lib.lib(), "fnb_get_rows_rms_norm_" + fmt)
    _check(fn(_ptr(table), n_vocab, _ptr(ids), _ptr(w), float(eps), _ptr(out), _ptr(normed), _ptr(err), n, cols, _stream()),
           "get_rows_rms_norm_" + fmt)
    return out, normed


def _embed_args(fmt, table, tok, n_own, own, full, streams, col0, err):
    _dev(table, torch.uint8, "table")
    _dev(tok, torch.int32, "tok")
    code, (bv, bb) = {"iq3_s": (_lib.TABLE_IQ3_S, (256, 110)), "q8_0": (_lib.TABLE_Q8_0, (32, 34))}[fmt]
    n_vocab = table.numel() // (n_own // bv * bb)
    for name, t in (("own", own), ("full", full), ("streams", streams)):
        if t is not None:
            _dev(t, torch.float32, name)
    n_full = full.shape[-1] if full is not None else streams.shape[-1] if streams is not None else n_own
    n_streams = streams.shape[-2] if streams is not None else 0
    return _lib.EmbedArgs(_ptr(table).value, _ptr(tok).value, _ptr(own).value, _ptr(full).value, _ptr(streams).value,
                          _ptr(err).value, n_vocab, tok.numel(), code, n_own, n_full, col0, n_streams)


def embed_rows(fmt: str, table, tok, n_own: int, *, own=None, full=None, streams=None, col0: int = 0, err=None) -> None:
    """fn::embed::embed_rows: decode each token's `n_own` features (IQ3_S or Q8_0 table) into own [rows][n_own], columns
    col0.. of full [rows][n_full] and of every stream of streams [rows][n_streams][n_full]."""
    a = _embed_args(fmt, table, tok, n_own, own, full, streams, col0, err)
    _check(_lib.lib().fnb_embed_rows(C.byref(a), _stream()), "embed_rows")


def embed_join(fmt: str, table, tok, n_own: int, peer, peer_col0: int, *, full=None, streams=None) -> None:
    """fn::embed::embed_join: the peer card's half [rows][n_own] into columns peer_col0.. of full and the streams."""
    _dev(peer, torch.float32, "peer")
    a = _embed_args(fmt, table, tok, n_own, None, full, streams, 0, None)
    _check(_lib.lib().fnb_embed_join(C.byref(a), _ptr(peer), peer_col0, _stream()), "embed_join")


def embed_supply(fmt: str, table, tok, n_own: int, src, row0: int, *, own=None, full=None, streams=None, col0: int = 0):
    """fn::embed::embed_supply: rows row0 .. row0 + len(src) - 1 overwritten from src [n][n_own]."""
    _dev(src, torch.float32, "src")
    a = _embed_args(fmt, table, tok, n_own, own, full, streams, col0, None)
    _check(_lib.lib().fnb_embed_supply(C.byref(a), _ptr(src), row0, src.shape[0], _stream()), "embed_supply")


def expert_gate_up_rows(fmt: str, gate: torch.Tensor, up: torch.Tensor, act: torch.Tensor, n: int, r0: int = 0,
                        r1: int | None = None, out: torch.Tensor | None = None, gu: torch.Tensor | None = None):
    """ff[t][r] = silu(gate row r . act[t]) * (up row r . act[t]), bit for bit the reference's CPU rows: fmt "q4_k"
    / "q5_k" (fn::experts::cpu::kq_gu_rows; rows uint8 [rows][n/256*144] / [rows][n/256*176]) or "iq3_xxs" / "iq3_s" /
    "iq2_xxs" / "iq2_xs" / "iq2_s" (fn::experts::cpu::iq_gu_rows; rows [rows][n/256*98 / 110 / 66 / 74 / 82]), Q8_K activations uint8 [nt][n/256*292]; returns F32 [nt][rows]."""
    entry = {"q4_k": "fnb_expert_gate_up_rows_q4_k", "q5_k": "fnb_expert_gate_up_rows_q5_k", "iq3_xxs": "fnb_expert_gate_up_rows_iq3_xxs",
             "iq3_s": "fnb_expert_gate_up_rows_iq3_s", "iq2_xxs": "fnb_expert_gate_up_rows_iq2_xxs",
             "iq2_xs": "fnb_expert_gate_up_rows_iq2_xs", "iq2_s": "fnb_expert_gate_up_rows_iq2_s"}[fmt]
    _dev(gate, torch.uint8, "gate")
    _dev(up, torch.uint8, "up")
    _dev(act, torch.uint8, "act")
    rows, nt = gate.shape[0], act.shape[0]
    r1 = rows if r1 is None else r1
    if out is None:
        out = torch.zeros((nt, rows), dtype=torch.float32, device=gate.device)
    _dev(out, torch.float32, "out")
    _check(getattr(_lib.lib(), entry)(_ptr(gate), _ptr(up), gate.shape[1], n, _ptr(act), act.shape[1], nt, _ptr(out),
                                      out.shape[1], _ptr(gu), r0, r1, _stream()), "expert_gate_up_rows_" + fmt)
    return out


def expert_gate_up_rows_q4_k(gate, up, act, n, **kw):
    return expert_gate_up_rows("q4_k", gate, up, act, n, **kw)


def expert_gate_up_rows_q5_k(gate, up, act, n, **kw):
    return expert_gate_up_rows("q5_k", gate, up, act, n, **kw)


def expert_gate_up_rows_iq3_xxs(gate, up, act, n, **kw):
    return expert_gate_up_rows("iq3_xxs", gate, up, act, n, **kw)


def expert_down_rows(fmt: str, w: torch.Tensor, act: torch.Tensor, n: int, r0: int = 0, r1: int | None = None,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t][r] = weight row r . activation row t (fn::experts::cpu::kq_down_rows, bit for bit).  fmt "q5_1": Q5_1
    weights uint8 [rows][n/32*24] against Q8_1 activations uint8 [nt][n/32*36]; fmt "q8_0": Q8_0 weights
    [rows][n/32*34] against Q8_0 activations [nt][n/32*34].  Returns F32 [nt][rows] (columns r0 .. r1 - 1 written)."""
    _dev(w, torch.uint8, "w")
    _dev(act, torch.uint8, "act")
    rows, nt = w.shape[0], act.shape[0]
    r1 = rows if r1 is None else r1
    if out is None:
        out = torch.zeros((nt, rows), dtype=torch.float32, device=w.device)
    _dev(out, torch.float32, "out")
    fn = {"q5_1": _lib.lib().fnb_expert_down_rows_q5_1, "q8_0": _lib.lib().fnb_expert_down_rows_q8_0,
          "iq4_nl": _lib.lib().fnb_expert_down_rows_iq4_nl}[fmt]
    _check(fn(_ptr(w), w.shape[1], n, _ptr(act), act.shape[1], nt, _ptr(out), out.shape[1], r0, r1, _stream()),
           "expert_down_rows_" + fmt)
    return out


def quantize_act_q(x: torch.Tensor, codes: torch.Tensor | None = None, scales: torch.Tensor | None = None):
    """The reference's planar 32-value activation (fn::experts::cpu::quantize_act_q): (codes int8 [rows][n], chunk scales
    F32 [rows][n/32]) of x F32 [rows][n]."""
    _dev(x, torch.float32, "x")
    rows, n = x.shape
    if codes is None:
        codes = torch.empty((rows, n), dtype=torch.int8, device=x.device)
    if scales is None:
        scales = torch.empty((rows, n // 32), dtype=torch.float32, device=x.device)
    _dev(codes, torch.int8, "codes")
    _dev(scales, torch.float32, "scales")
    _check(_lib.lib().fnb_quantize_act_q(_ptr(x), _ptr(codes), _ptr(scales), rows, n, _stream()), "quantize_act_q")
    return codes, scales


def expert_down_rows_q2_0(w: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, n: int, r0: int = 0,
                          r1: int | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t][r] = Q2_0 weight row r (uint8 [rows][n/64*18]) . planar activation row t (fn::experts::cpu::q2_down_rows,
    bit for bit).  Returns F32 [nt][rows] (columns r0 .. r1 - 1 written)."""
    _dev(w, torch.uint8, "w")
    _dev(codes, torch.int8, "codes")
    _dev(scales, torch.float32, "scales")
    rows, nt = w.shape[0], codes.shape[0]
    r1 = rows if r1 is None else r1
    if out is None:
        out = torch.zeros((nt, rows), dtype=torch.float32, device=w.device)
    _dev(out, torch.float32, "out")
    _check(_lib.lib().fnb_expert_down_rows_q2_0(_ptr(w), w.shape[1], n, _ptr(codes), codes.shape[1], _ptr(scales),
                                                scales.shape[1], nt, _ptr(out), out.shape[1], r0, r1, _stream()),
           "expert_down_rows_q2_0")
    return out


def expert_down_rows_q5_1(w, act, n, r0=0, r1=None, out=None):
    return expert_down_rows("q5_1", w, act, n, r0, r1, out)


def prepare_device() -> None:
    """One-time kernel attribute set-up for the current device, so that even a first call can sit inside a capture."""
    _check(_lib.lib().fnb_prepare_device(), "prepare_device")


def check_tokens(ids_host: torch.Tensor, n_vocab: int) -> int:
    """Host check before upload (fn::embed::check_tokens): 0, or 1 + the index of the first id outside [0, n_vocab)."""
    if ids_host.is_cuda or ids_host.dtype != torch.int32 or not ids_host.is_contiguous():
        raise ValueError("ids_host: expected a contiguous host int32 tensor")
    return int(_lib.lib().fnb_check_tokens(C.c_void_p(ids_host.data_ptr()), ids_host.numel(), n_vocab))
