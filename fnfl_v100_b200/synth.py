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
