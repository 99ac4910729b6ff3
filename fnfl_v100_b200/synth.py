"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

No dataset is involved in this path: every input is generated from a seed (0x464E464C + the configuration's
index, the reference's seeding convention in fn/quant/synth.h:24-28).  The numpy forms feed both the kernels and
the CPU oracle in parity tests; the torch forms fill large device tensors for full-size runs.
"""
from __future__ import annotations

import numpy as np

SEED_BASE = 0x464E464C


def rng(case: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(SEED_BASE + case))


def _f16_bits(x: np.ndarray) -> np.ndarray:
    return x.astype(np.float16).view(np.uint16)


def q4_k_table(g: np.random.Generator, n_rows: int, cols: int, d_lo: float = 1e-3, d_hi: float = 1e-2) -> np.ndarray:
    """uint8 [n_rows][cols/256*144]: uniform bytes (6-bit scales/mins and nibbles), fp16 d and dmin ~ U(d_lo, d_hi)."""
    nsb = cols // 256
    t = g.integers(0, 256, size=(n_rows, nsb, 144), dtype=np.uint8)
    dm = _f16_bits(g.uniform(d_lo, d_hi, size=(n_rows, nsb, 2)))
    t[:, :, 0:4] = dm.view(np.uint8).reshape(n_rows, nsb, 4)
    return t.reshape(n_rows, nsb * 144)


def q5_k_table(g: np.random.Generator, n_rows: int, cols: int, d_lo: float = 1e-3, d_hi: float = 1e-2) -> np.ndarray:
    """uint8 [n_rows][cols/256*176]: uniform bytes (6-bit scales/mins, high bits, nibbles), fp16 d and dmin ~ U(d_lo, d_hi)."""
    nsb = cols // 256
    t = g.integers(0, 256, size=(n_rows, nsb, 176), dtype=np.uint8)
    dm = _f16_bits(g.uniform(d_lo, d_hi, size=(n_rows, nsb, 2)))
    t[:, :, 0:4] = dm.view(np.uint8).reshape(n_rows, nsb, 4)
    return t.reshape(n_rows, nsb * 176)


def iq3_xxs_table(g: np.random.Generator, n_rows: int, cols: int, d_lo: float = 1e-3, d_hi: float = 1e-2) -> np.ndarray:
    """uint8 [n_rows][cols/256*98]: uniform codebook indices, sign bits and 4-bit scales, fp16 d ~ U(d_lo, d_hi) > 0."""
    nsb = cols // 256
    t = g.integers(0, 256, size=(n_rows, nsb, 98), dtype=np.uint8)
    d = _f16_bits(g.uniform(d_lo, d_hi, size=(n_rows, nsb, 1)))
    t[:, :, 0:2] = d.view(np.uint8).reshape(n_rows, nsb, 2)
    return t.reshape(n_rows, nsb * 98)


def iq3_s_table(g: np.random.Generator, n_rows: int, cols: int, d_lo: float = 1e-3, d_hi: float = 1e-2) -> np.ndarray:
    """uint8 [n_rows][cols/256*110]: uniform indices, high bits, sign bits and 4-bit scales, fp16 d ~ U(d_lo, d_hi)."""
    nsb = cols // 256
    t = g.integers(0, 256, size=(n_rows, nsb, 110), dtype=np.uint8)
    d = _f16_bits(g.uniform(d_lo, d_hi, size=(n_rows, nsb, 1)))
    t[:, :, 0:2] = d.view(np.uint8).reshape(n_rows, nsb, 2)
    return t.reshape(n_rows, nsb * 110)


def iq2_table(fmt: str, g: np.random.Generator, n_rows: int, cols: int, d_lo: float = 1e-3, d_hi: float = 1e-2) -> np.ndarray:
    """uint8 [n_rows][cols/256*B] for fmt "iq2_xxs" (B = 66), "iq2_xs" (74) or "iq2_s" (82): uniform bytes (every index,
    sign and scale pattern is a valid block), fp16 d ~ U(d_lo, d_hi)."""
    bb = {"iq2_xxs": 66, "iq2_xs": 74, "iq2_s": 82}[fmt]
    nsb = cols // 256
    t = g.integers(0, 256, size=(n_rows, nsb, bb), dtype=np.uint8)
    d = _f16_bits(g.uniform(d_lo, d_hi, size=(n_rows, nsb, 1)))
    t[:, :, 0:2] = d.view(np.uint8).reshape(n_rows, nsb, 2)
    return t.reshape(n_rows, nsb * bb)


def q8_0_table(g: np.random.Generator, n_rows: int, cols: int) -> np.ndarray:
    nb = cols // 32
    t = g.integers(0, 256, size=(n_rows, nb, 34), dtype=np.uint8)
    d = _f16_bits(g.uniform(1e-3, 1e-2, size=(n_rows, nb, 1)) * g.choice([-1.0, 1.0], size=(n_rows, nb, 1)))
    t[:, :, 0:2] = d.view(np.uint8).reshape(n_rows, nb, 2)
    return t.reshape(n_rows, nb * 34)


def normal(g: np.random.Generator, shape, scale: float = 1.0) -> np.ndarray:
    return (g.standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)


def q5_1_rows(g: np.random.Generator, rows: int, n: int, d_lo: float = 1e-3, d_hi: float = 1e-2) -> np.ndarray:
    """Random valid ggml Q5_1 rows: uint8 [rows][n/32*24] (fp16 d ~ U(d_lo, d_hi), fp16 m ~ U(-0.1, 0.1), random bits)."""
    nb = n // 32
    t = g.integers(0, 256, (rows, nb, 24)).astype(np.uint8)
    t[:, :, 0:2] = g.uniform(d_lo, d_hi, (rows, nb)).astype(np.float16).view(np.uint8).reshape(rows, nb, 2)
    t[:, :, 2:4] = g.uniform(-0.1, 0.1, (rows, nb)).astype(np.float16).view(np.uint8).reshape(rows, nb, 2)
    return t.reshape(rows, nb * 24)


def iq4_nl_rows(g: np.random.Generator, rows: int, n: int, d_lo: float = 1e-3, d_hi: float = 1e-2) -> np.ndarray:
    """Random valid ggml IQ4_NL rows: uint8 [rows][n/32*18] (fp16 d ~ U(d_lo, d_hi), random nibbles)."""
    nb = n // 32
    t = g.integers(0, 256, (rows, nb, 18)).astype(np.uint8)
    t[:, :, 0:2] = g.uniform(d_lo, d_hi, (rows, nb)).astype(np.float16).view(np.uint8).reshape(rows, nb, 2)
    return t.reshape(rows, nb * 18)


def q2_0_rows(g: np.random.Generator, rows: int, n: int, d_lo: float = 1e-3, d_hi: float = 1e-2) -> np.ndarray:
    """Random valid Q2_0 rows of the reference engine: uint8 [rows][n/64*18] (fp16 d ~ U(d_lo, d_hi), random 2-bit codes)."""
    nb = n // 64
    t = g.integers(0, 256, (rows, nb, 18)).astype(np.uint8)
    t[:, :, 0:2] = g.uniform(d_lo, d_hi, (rows, nb)).astype(np.float16).view(np.uint8).reshape(rows, nb, 2)
    return t.reshape(rows, nb * 18)


def norm_weight(g: np.random.Generator, cols: int) -> np.ndarray:
    """1 + N(0, 0.1), the RMSNorm weight of the first configuration."""
    return (1.0 + 0.1 * g.standard_normal(cols)).astype(np.float32)


def positions(g: np.random.Generator, rows: int, max_offset: int = 258048) -> np.ndarray:
    """offset ~ U[0, max_offset) + 0..rows-1"""
    off = int(g.integers(0, max_offset))
    return (off + np.arange(rows)).astype(np.int32)


# ---- torch forms for full-size device tensors -------------------------------------------------------------

def torch_gen(device, case: int):
    import torch
    gen = torch.Generator(device=device)
    gen.manual_seed(SEED_BASE + case)
    return gen


def torch_normal(gen, shape, scale: float, device):
    import torch
    out = torch.empty(shape, dtype=torch.float32, device=device)
    out.normal_(0.0, scale, generator=gen)
    return out


def torch_table(fmt: str, gen, n_rows: int, cols: int, device, d_lo: float = 1e-3, d_hi: float = 1e-2):
    """Device form of q4_k_table / iq3_xxs_table / an IQ3_S table (same distributions, torch's generator)."""
    import torch
    bv, bb, nd = {"q4_k": (256, 144, 2), "q5_k": (256, 176, 2), "iq3_xxs": (256, 98, 1), "iq3_s": (256, 110, 1)}[fmt]
    nsb = cols // bv
    t = torch.randint(0, 256, (n_rows, nsb, bb), dtype=torch.uint8, device=device, generator=gen)
    d = torch.empty((n_rows, nsb, nd), dtype=torch.float32, device=device).uniform_(d_lo, d_hi, generator=gen)
    t[:, :, 0:2 * nd] = d.to(torch.float16).view(torch.uint8).reshape(n_rows, nsb, 2 * nd)
    return t.reshape(n_rows, nsb * bb)


# ---- counter-based device inputs: any rank can regenerate any row of the job -------------------------------------
# Element (row, col) of stream `sid` is a pure function of (seed, sid, row * cols + col): a splitmix64 finaliser of
# the counter gives two 24-bit uniforms, Box-Muller (F32, on the device) gives one normal.  A shard that holds rows
# [lo, hi) of the job generates exactly the values the unsharded job holds in those rows, so a partitioned run can
# be compared with the whole one byte for byte, and one rank can recompute another rank's slice.

_M64 = (1 << 64) - 1


def _s64(v: int) -> int:
    """An unsigned 64-bit constant as the signed value torch's int64 arithmetic wraps to."""
    v &= _M64
    return v - (1 << 64) if v >> 63 else v


def _lsr(x, n: int):
    """Logical right shift of an int64 tensor (torch's >> is arithmetic)."""
    return (x >> n) & ((1 << (64 - n)) - 1)


def _mix64(x):
    x = (x ^ _lsr(x, 30)) * _s64(0xBF58476D1CE4E5B9)
    x = (x ^ _lsr(x, 27)) * _s64(0x94D049BB133111EB)
    return x ^ _lsr(x, 31)


def _counter_bits(seed: int, sid: int, lo: int, n: int, device):
    import torch
    idx = torch.arange(lo, lo + n, dtype=torch.int64, device=device)
    key = _s64((seed * 0x9E3779B97F4A7C15 + sid * 0xD1B54A32D192ED03) & _M64)
    return _mix64((idx + key) * _s64(0x9E3779B97F4A7C15))


def counter_normal(seed: int, sid: int, row_lo: int, row_hi: int, cols: int, scale: float, device, out=None):
    """F32 [row_hi - row_lo][cols] ~ N(0, scale^2): rows row_lo .. row_hi - 1 of stream `sid`."""
    import math
    import torch
    rows = row_hi - row_lo
    if out is None:
        out = torch.empty((rows, cols), dtype=torch.float32, device=device)
    flat = out.view(-1)
    step = max(1, (1 << 25) // cols)                      # rows per pass: bounded temporaries
    for r in range(0, rows, step):
        n = min(step, rows - r) * cols
        z = _counter_bits(seed, sid, (row_lo + r) * cols, n, device)
        u1 = (_lsr(z, 40).to(torch.float32) + 0.5) * (1.0 / (1 << 24))          # (0, 1)
        u2 = ((z >> 16) & 0xFFFFFF).to(torch.float32) * (1.0 / (1 << 24))        # [0, 1)
        torch.mul(torch.sqrt(-2.0 * torch.log(u1)), torch.cos((2.0 * math.pi) * u2) * scale, out=flat[r * cols:r * cols + n])
    return out


def counter_ids(seed: int, sid: int, row_lo: int, row_hi: int, n_vocab: int, device):
    """I32 [row_hi - row_lo] uniform in [0, n_vocab): token ids of rows row_lo .. row_hi - 1."""
    import torch
    z = _counter_bits(seed, sid, row_lo, row_hi - row_lo, device)
    return (_lsr(z, 11) % n_vocab).to(torch.int32)
