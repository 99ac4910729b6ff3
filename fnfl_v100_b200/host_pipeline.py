"""The chain driven from HOST buffers: what a caller that owns pinned host tensors sees end to end.

A prefill of T tokens is cut into chunks (8192 rows, the reference's prompt chunk: fn/runtime/prefill.cpp
cuts chunks of at most 8192 rows) and pipelined over three streams - host-to-device copies of chunk c + 1,
the chain's kernels of chunk c, device-to-host copies of chunk c - 1 - with two device slots.  Inputs are the
tensors the kernels consume (ids, positions, q, k, v, gate, up); results returned to the host are what a
host-side consumer needs: the Q8_1 activations, the appended K/V cells and the error word.
"""
from __future__ import annotations

import torch

from . import ops
from .chain import ChainConfig, PrefillChain


class HostChunkPipeline:
    def __init__(self, cfg: ChainConfig, device, chunk: int = 8192, source: PrefillChain | None = None):
        self.cfg, self.device = cfg, torch.device(device)
        T = cfg.tokens
        self.chunk = min(chunk, T)
        self.n_chunks = (T + self.chunk - 1) // self.chunk
        if T % self.chunk != 0:
            raise ValueError("tokens must be a multiple of the chunk")
        src = source if source is not None else PrefillChain(cfg, device)
        self.src = src
        pin = lambda t: t.cpu().pin_memory()  # noqa: E731
        # pinned host inputs (full T) and outputs
        self.h_in = {n: pin(getattr(src, n)) for n in ("ids", "pos", "q", "k", "v", "gate", "up")}
        c = cfg
        self.h_act = torch.empty((T * c.top_k, c.inter // 32 * ops.Q8_1_BLOCK), dtype=torch.uint8).pin_memory()
        cell = c.head_dim // 32 * ops.Q8_0_BLOCK
        self.h_k = torch.empty((T, c.n_kv_heads, cell), dtype=torch.uint8).pin_memory()
        self.h_v = torch.empty_like(self.h_k).pin_memory()
        self.h_err = torch.zeros(1, dtype=torch.int32).pin_memory()
        # two device slots of one chunk each; table, weights and caches are shared with the source chain
        ccfg = ChainConfig(**{**src.describe(), "tokens": self.chunk})
        self.slots = []
        for _ in range(2):
            s = PrefillChain.__new__(PrefillChain)
            s.cfg, s.device = ccfg, self.device
            for n in PrefillChain.SHARED + ("k_cache", "v_cache", "err", "theta_scale"):
                setattr(s, n, getattr(src, n))
            s.first_token = src.first_token
            dev = self.device
            Tc = self.chunk
            s.ids = torch.empty(Tc, dtype=torch.int32, device=dev)
            s.pos = torch.empty(Tc, dtype=torch.int32, device=dev)
            s.q = torch.empty((Tc, c.n_q_heads, c.head_dim), dtype=torch.float32, device=dev)
            s.k = torch.empty((Tc, c.n_kv_heads, c.head_dim), dtype=torch.float32, device=dev)
            s.v = torch.empty_like(s.k)
            s.gate = torch.empty((Tc * c.top_k, c.inter), dtype=torch.float32, device=dev)
            s.up = torch.empty_like(s.gate)
            s.hidden = torch.empty((Tc, c.hidden), dtype=torch.float32, device=dev)
            s.normed_attn = torch.empty_like(s.hidden)
            s.normed_ffn = torch.empty_like(s.hidden)
            s.q_out = torch.empty_like(s.q)
            s.act = torch.empty((Tc * c.top_k, c.inter // 32 * ops.Q8_1_BLOCK), dtype=torch.uint8, device=dev)
            self.slots.append(s)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_done = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]
        self.first_pos = int(src.pos[0].item())
        row_in = {"ids": 4, "pos": 4, "q": c.n_q_heads * c.head_dim * 4, "k": c.n_kv_heads * c.head_dim * 4,
                  "v": c.n_kv_heads * c.head_dim * 4, "gate": c.top_k * c.inter * 4, "up": c.top_k * c.inter * 4}
        self.h2d_bytes = sum(row_in.values()) * T
        self.d2h_bytes = T * (c.top_k * c.inter // 32 * ops.Q8_1_BLOCK + 2 * c.n_kv_heads * cell) + 4

    def step(self, copies_only: bool = False) -> None:
        """One pass over all T tokens from and to host memory; returns with work enqueued (no sync).
        copies_only: the same copies on the same streams with the kernels left out - the ceiling the host link
        and the host's memory system set for this pipeline."""
        c, Tc = self.cfg, self.chunk
        cur = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(cur)
        for ci in range(self.n_chunks):
            s, b = self.slots[ci % 2], ci % 2
            lo, hi = ci * Tc, (ci + 1) * Tc
            with torch.cuda.stream(self.s_in):
                if ci >= 2:
                    self.s_in.wait_event(self.ev_done[b])       # the slot's inputs were consumed
                for n in ("ids", "pos", "q", "k", "v"):
                    getattr(s, n).copy_(self.h_in[n][lo:hi], non_blocking=True)
                for n in ("gate", "up"):
                    getattr(s, n).copy_(self.h_in[n][lo * c.top_k:hi * c.top_k], non_blocking=True)
                self.ev_in[b].record(self.s_in)
            cur.wait_event(self.ev_in[b])
            if ci >= 2:
                cur.wait_event(self.ev_out[b])                   # the slot's previous outputs reached the host
            if not copies_only:
                s.step()
            self.ev_done[b].record(cur)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_done[b])
                self.h_act[lo * c.top_k:hi * c.top_k].copy_(s.act, non_blocking=True)
                p0 = self.first_pos + lo
                self.h_k[lo:hi].copy_(self.src.k_cache[p0:p0 + Tc], non_blocking=True)
                self.h_v[lo:hi].copy_(self.src.v_cache[p0:p0 + Tc], non_blocking=True)
                self.ev_out[b].record(self.s_out)
        with torch.cuda.stream(self.s_out):
            self.h_err.copy_(self.src.err, non_blocking=True)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_in)

    launches_per_step = property(lambda self: PrefillChain.launches_per_step * self.n_chunks)
