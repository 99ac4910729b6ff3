"""The fused-op chain of one prefill chunk on one GPU's shard of token rows.

    ids --get_rows(Q4_K)--> hidden --RMSNorm--> normed_attn         (a QKV projection would consume this)
    q, k, v --per-head RMSNorm + NeoX partial RoPE--> q_out, K/V appended to the Q8_0 cache
    hidden --RMSNorm--> normed_ffn                                   (the expert gate/up products would consume this)
    gate, up --SwiGLU + Q8_1--> activations for the expert down product

Only get_rows -> RMSNorm is truly chained; the tensors a dense product would produce (q, k, v, gate, up) are
seeded synthetic inputs, because contractions are outside this path.  The chained pair is ONE launch (the decoded row
stays in registers between the two steps), so a step is four launches: no host
synchronisation, no allocation after construction, so a step can be captured in a CUDA graph and replayed,
which is how the reference's prompt path replays its unit graphs.

Sharding: a chain object holds rows [first_token, first_token + tokens) of ONE job.  Per-row inputs (ids, q, k, v,
gate, up) are counter-based functions of the job's row index (synth.counter_*), positions are depth + row and the
cache cell of a row is its position, so shards of a job compute exactly the rows the unsharded job computes and
append disjoint cell ranges; the small shared state (table, norm weights) is generated from one seed on every GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict

import torch

from . import ops, synth


@dataclass
class ChainConfig:
    tokens: int = 65536          # rows this object holds (the whole job, or one shard of it)
    hidden: int = 2048
    n_q_heads: int = 16
    n_kv_heads: int = 2
    head_dim: int = 256
    n_rot: int = 64
    freq_base: float = 1e7
    top_k: int = 10              # expert rows per token
    inter: int = 512             # expert intermediate width
    n_vocab: int = 151936
    cache_slots: int = 262144
    depth: int = 196608          # context depth: the first token's position and cache slot
    eps: float = 1e-6
    table_fmt: str = "q4_k"
    seed_case: int = 5

    # algorithmic bytes per token of each stage (compulsory reads + writes)
    def bytes_per_token(self) -> dict:
        row_b = ops.table_row_bytes(self.table_fmt, self.hidden)
        hd, nq, nkv = self.head_dim, self.n_q_heads, self.n_kv_heads
        cell = hd // 32 * ops.Q8_0_BLOCK
        rope = 2 * nq * hd * 4 + 2 * nkv * hd * 4 + 2 * nkv * cell + 4
        glu_rows = self.top_k
        glu = glu_rows * (2 * self.inter * 4 + self.inter // 32 * ops.Q8_1_BLOCK)
        norm = 2 * self.hidden * 4
        return {"get_rows_rms_norm": row_b + 4 + 2 * self.hidden * 4, "get_rows": row_b + 4 + self.hidden * 4,
                "rms_norm_attn": norm, "rope_kv": rope, "rms_norm_ffn": norm, "swiglu_q8_1": glu}


class PrefillChain:
    """Owns every buffer of the chain for one shard; `step()` enqueues the four launches."""

    # get_rows and the attention norm that reads its rows are one launch (the row stays in registers between them);
    # the two separately callable stages remain for tests and for tables in other formats
    STAGES = ("get_rows_rms_norm", "rope_kv", "rms_norm_ffn", "swiglu_q8_1")
    UNFUSED = ("get_rows", "rms_norm_attn", "rope_kv", "rms_norm_ffn", "swiglu_q8_1")

    SHARED = ("table", "w_attn", "w_ffn", "w_q", "w_k")   # replicated on every GPU

    def __init__(self, cfg: ChainConfig, device, first_token: int = 0, shared: "PrefillChain | None" = None):
        """rows [first_token, first_token + cfg.tokens) of the job; `shared` lends its table and norm weights (a
        second shard on the same GPU) instead of generating them again."""
        self.cfg, self.device = cfg, torch.device(device)
        c, dev, T = cfg, self.device, cfg.tokens
        self.first_token = first_token
        if shared is None:
            # state every shard replicates: one seed, the same bits on every GPU of one model
            gen = synth.torch_gen(dev, c.seed_case)
            self.table = synth.torch_table(c.table_fmt, gen, c.n_vocab, c.hidden, dev)
            self.w_attn = 1.0 + 0.1 * synth.torch_normal(gen, (c.hidden,), 1.0, dev)
            self.w_ffn = 1.0 + 0.1 * synth.torch_normal(gen, (c.hidden,), 1.0, dev)
            self.w_q = 1.0 + 0.1 * synth.torch_normal(gen, (c.head_dim,), 1.0, dev)
            self.w_k = 1.0 + 0.1 * synth.torch_normal(gen, (c.head_dim,), 1.0, dev)
        else:
            for n in self.SHARED:
                setattr(self, n, getattr(shared, n))
        # per-row inputs: functions of the job's row index, so any shard regenerates exactly its rows
        seed, lo, hi = synth.SEED_BASE + c.seed_case, first_token, first_token + T
        self.ids = synth.counter_ids(seed, 0, lo, hi, c.n_vocab, dev)
        self.pos = (c.depth + first_token + torch.arange(T, device=dev, dtype=torch.int64)).to(torch.int32)
        qw, kw = c.n_q_heads * c.head_dim, c.n_kv_heads * c.head_dim
        self.q = synth.counter_normal(seed, 1, lo, hi, qw, 1.0, dev).view(T, c.n_q_heads, c.head_dim)
        self.k = synth.counter_normal(seed, 2, lo, hi, kw, 1.0, dev).view(T, c.n_kv_heads, c.head_dim)
        self.v = synth.counter_normal(seed, 3, lo, hi, kw, 1.0, dev).view(T, c.n_kv_heads, c.head_dim)
        self.gate = synth.counter_normal(seed, 4, lo * c.top_k, hi * c.top_k, c.inter, 0.5, dev)
        self.up = synth.counter_normal(seed, 5, lo * c.top_k, hi * c.top_k, c.inter, 0.5, dev)
        self.theta_scale = ops.theta_scale(c.freq_base, c.n_rot)
        # outputs
        self.hidden = torch.empty((T, c.hidden), dtype=torch.float32, device=dev)
        self.normed_attn = torch.empty_like(self.hidden)
        self.normed_ffn = torch.empty_like(self.hidden)
        self.q_out = torch.empty_like(self.q)
        if shared is None:
            self.k_cache = ops.new_kv_cache(c.cache_slots, c.n_kv_heads, c.head_dim, dev)
            self.v_cache = ops.new_kv_cache(c.cache_slots, c.n_kv_heads, c.head_dim, dev)
        else:  # shards on one GPU append disjoint cells of one cache
            self.k_cache, self.v_cache = shared.k_cache, shared.v_cache
        self.act = torch.empty((T * c.top_k, c.inter // 32 * ops.Q8_1_BLOCK), dtype=torch.uint8, device=dev)
        self.err = ops.new_err(dev)

    # ---- stages, individually callable so each can be timed alone ----
    def get_rows_rms_norm(self):
        if self.cfg.table_fmt not in ("q4_k", "iq3_xxs"):
            self.get_rows()
            self.rms_norm_attn()
            return
        ops.get_rows_rms_norm(self.cfg.table_fmt, self.table, self.ids, self.cfg.hidden, self.w_attn, self.cfg.eps, out=self.hidden,
                              normed=self.normed_attn, err=self.err)

    def get_rows(self):
        ops.get_rows(self.cfg.table_fmt, self.table, self.ids, self.cfg.hidden, out=self.hidden, err=self.err)

    def rms_norm_attn(self):
        ops.rms_norm(self.hidden, self.w_attn, self.cfg.eps, out=self.normed_attn)

    def rope_kv(self):
        c = self.cfg
        ops.rope_neox_q8_0_append(self.q, self.k, self.v, self.pos, n_rot=c.n_rot, theta_scale=self.theta_scale,
                                  k_cache=self.k_cache, v_cache=self.v_cache, q_norm_w=self.w_q, k_norm_w=self.w_k,
                                  eps=c.eps, q_out=self.q_out, err=self.err)

    def rms_norm_ffn(self):
        ops.rms_norm(self.hidden, self.w_ffn, self.cfg.eps, out=self.normed_ffn)

    def swiglu_q8_1(self):
        ops.swiglu_q8_1(self.gate, self.up, out=self.act, err=self.err)

    def step(self):
        for name in self.STAGES:
            getattr(self, name)()

    launches_per_step = 4

    def capture(self) -> torch.cuda.CUDAGraph:
        """Record one step into a CUDA graph (the launchers neither synchronise nor allocate)."""
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self.step()  # warm the context before capture
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.step()
        return g

    def kv_cells(self):
        """The cells this shard appended: (K, V) uint8 [tokens][n_kv][cell bytes]."""
        lo = self.cfg.depth + self.first_token
        return self.k_cache[lo:lo + self.cfg.tokens], self.v_cache[lo:lo + self.cfg.tokens]

    def describe(self) -> dict:
        return asdict(self.cfg)
