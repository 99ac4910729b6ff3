"""Loading a quantised table (e.g. token_embd.weight) from a GGUF model file into device memory, through the
library's host-side reader (fnb_gguf_* in include/fnb200.h).  Only what this path needs of the reference's loader
(fn/loader/loader.h, fn/borrowed/gguf_tensors.h): find the tensor, read its rows, upload."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

GGML_TYPE_NAMES = {0: "f32", 1: "f16", 8: "q8_0", 12: "q4_k", 18: "iq3_xxs", 21: "iq3_s"}


class GgufFile:
    def __init__(self, path: str):
        self._lib = _lib.lib()
        self._h = self._lib.fnb_gguf_open(path.encode())
        if not self._h:
            raise ValueError(f"{path}: not a readable GGUF v2/v3 file")

    def close(self) -> None:
        if self._h:
            self._lib.fnb_gguf_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def n_tensors(self) -> int:
        return int(self._lib.fnb_gguf_n_tensors(self._h))

    def find(self, name: str) -> _lib.GgufTensor:
        t = _lib.GgufTensor()
        if self._lib.fnb_gguf_find(self._h, name.encode(), C.byref(t)) != _lib.OK:
            raise KeyError(name)
        return t

    def read_rows(self, t: _lib.GgufTensor, row0: int = 0, n_rows: int | None = None) -> np.ndarray:
        """uint8 [n_rows][row_bytes] of the tensor's raw blocks."""
        n_rows = int(t.n_rows) - row0 if n_rows is None else n_rows
        out = np.empty((n_rows, int(t.row_bytes)), np.uint8)
        if self._lib.fnb_gguf_read_rows(self._h, C.byref(t), row0, n_rows, C.c_void_p(out.ctypes.data)) != _lib.OK:
            raise ValueError("read_rows: rows outside the tensor, or a type this library does not decode")
        return out


def load_table(path: str, name: str = "token_embd.weight", device=None):
    """Returns (table uint8 tensor [n_vocab][row_bytes], format name, cols).  On `device` when given, else on the host."""
    import torch
    with GgufFile(path) as g:
        t = g.find(name)
        fmt = GGML_TYPE_NAMES.get(int(t.type))
        if fmt is None or t.row_bytes == 0:
            raise ValueError(f"{name}: ggml type {int(t.type)} is not one this library decodes")
        rows = torch.from_numpy(g.read_rows(t))
        if device is not None:
            rows = rows.pin_memory().to(device, non_blocking=True) if torch.cuda.is_available() else rows.to(device)
        return rows, fmt, int(t.ne[0])
