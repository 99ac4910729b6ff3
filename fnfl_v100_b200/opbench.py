"""Per-operator timing on synthetic inputs: `python -m fnfl_v100_b200.opbench --op swiglu_q8_1 --tokens 65536`.

Follows the reference's bench protocol (fn/kernels/act/act_bench.cpp:18-22, :60-140): warm launches, then timed
launches measured with CUDA events on the launching stream, median and p90 reported, cold (inputs rotated over
more distinct buffers than fit in L2) and hot (same buffers), one JSON line per point with bytes per launch and
the fraction of the HBM peak.  Small `--tokens` make it the target of an `ncu` capture of one kernel.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import ops, synth
from .chain import ChainConfig

OPS = ("get_rows_q4_k", "get_rows_iq3_xxs", "rms_norm", "rms_norm_heads", "rope_kv", "swiglu_q8_1", "swiglu_act",
       "rope_kv8", "quantize_q8_1", "rms_norm_q8_1", "embed_iq3_s", "kv_read_q8_0", "kv_read_kv8",
       "expert_down_q5_1_nt1", "expert_down_q5_1_nt3", "expert_down_q5_1_nt8", "expert_down_q8_0_nt1", "expert_down_q8_0_nt3", "quantize_q8_k",
       "expert_down_q2_0_nt1", "expert_down_q2_0_nt3", "expert_down_q2_0_nt8", "quantize_act_q",
       "expert_down_iq4_nl_nt1", "expert_down_iq4_nl_nt3", "expert_down_iq4_nl_nt8",
       "expert_gate_up_q4_k_nt1", "expert_gate_up_q4_k_nt3", "expert_gate_up_q4_k_nt8",
       "expert_gate_up_q5_k_nt1", "expert_gate_up_q5_k_nt3", "expert_gate_up_q5_k_nt8",
       "expert_gate_up_iq3_s_nt1", "expert_gate_up_iq3_s_nt3", "expert_gate_up_iq3_s_nt8",
       "expert_gate_up_iq3_xxs_nt1", "expert_gate_up_iq3_xxs_nt3", "expert_gate_up_iq3_xxs_nt8",
       "expert_gate_up_iq2_xxs_nt1", "expert_gate_up_iq2_xxs_nt3", "expert_gate_up_iq2_xs_nt1", "expert_gate_up_iq2_s_nt1",
       "attend_q8_0_b1", "attend_q8_0_b3", "attend_q8_0_b5", "attend_kv8_b1", "attend_kv8_b5",
       # shapes that take the general kernels instead of the tuned ones: 64-wide heads with 32 rotated dims, 4096 columns
       "rope_kv_fallback", "get_rows_q4_k_c4096", "get_rows_iq3_xxs_c4096",
       "fused_get_rows_rms_norm_q4_k", "fused_get_rows_rms_norm_iq3_xxs")


def hbm_peak() -> float:
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"])
    except Exception:
        return 6650.0


def make_case(op: str, T: int, dev, gen, c: ChainConfig):
    """Returns (launch, algorithmic bytes)."""
    N = synth.torch_normal
    if op.startswith("fused_get_rows_rms_norm_"):
        fmt = op[len("fused_get_rows_rms_norm_"):]
        table = synth.torch_table(fmt, gen, c.n_vocab, c.hidden, dev)
        ids = torch.randint(0, c.n_vocab, (T,), dtype=torch.int32, device=dev, generator=gen)
        w = 1 + 0.1 * N(gen, (c.hidden,), 1.0, dev)
        out = torch.empty((T, c.hidden), dtype=torch.float32, device=dev)
        normed = torch.empty_like(out)
        err = ops.new_err(dev)
        return (lambda: ops.get_rows_rms_norm(fmt, table, ids, c.hidden, w, c.eps, out=out, normed=normed, err=err),
                T * (ops.table_row_bytes(fmt, c.hidden) + 4 + 2 * c.hidden * 4) + c.hidden * 4)
    if op.startswith("get_rows"):
        fmt, cols = op[len("get_rows_"):], c.hidden
        if fmt.endswith("_c4096"):
            fmt, cols = fmt[:-len("_c4096")], 4096
        table = synth.torch_table(fmt, gen, c.n_vocab, cols, dev)
        ids = torch.randint(0, c.n_vocab, (T,), dtype=torch.int32, device=dev, generator=gen)
        out = torch.empty((T, cols), dtype=torch.float32, device=dev)
        err = ops.new_err(dev)
        return (lambda: ops.get_rows(fmt, table, ids, cols, out=out, err=err),
                T * (ops.table_row_bytes(fmt, cols) + 4 + cols * 4))
    if op == "rope_kv_fallback":
        # 64 heads of 64 (the same bytes a token as the chain's 16 x 256), 32 rotated dims: the row-per-warp kernel
        hq, hk, hd, n_rot = 64, 8, 64, 32
        q, k, v = N(gen, (T, hq, hd), 1.0, dev), N(gen, (T, hk, hd), 1.0, dev), N(gen, (T, hk, hd), 1.0, dev)
        wq, wk = 1 + 0.1 * N(gen, (hd,), 1.0, dev), 1 + 0.1 * N(gen, (hd,), 1.0, dev)
        pos = (c.depth + torch.arange(T, device=dev)).to(torch.int32)
        q_out = torch.empty_like(q)
        err = ops.new_err(dev)
        kc, vc = ops.new_kv_cache(c.cache_slots, hk, hd, dev), ops.new_kv_cache(c.cache_slots, hk, hd, dev)
        ts = ops.theta_scale(c.freq_base, n_rot)
        return (lambda: ops.rope_neox_q8_0_append(q, k, v, pos, n_rot=n_rot, theta_scale=ts, k_cache=kc, v_cache=vc,
                                                  q_norm_w=wq, k_norm_w=wk, eps=c.eps, q_out=q_out, err=err)), \
            T * (2 * hq * hd * 4 + 2 * hk * hd * 4 + 4 + 2 * hk * hd // 32 * ops.Q8_0_BLOCK)
    if op == "embed_iq3_s":
        # the reference's two-card layout (fn/kernels/embed/embed.h:70-87): 1280 own features of 2560, four streams
        n_own, n_full, n_streams, vocab = 1280, 2560, 4, 248320
        table = synth.torch_table("iq3_s", gen, vocab, n_own, dev)
        tok = torch.randint(0, vocab, (T,), dtype=torch.int32, device=dev, generator=gen)
        own = torch.empty((T, n_own), dtype=torch.float32, device=dev)
        full = torch.empty((T, n_full), dtype=torch.float32, device=dev)
        streams = torch.empty((T, n_streams, n_full), dtype=torch.float32, device=dev)
        err = ops.new_err(dev)
        return (lambda: ops.embed_rows("iq3_s", table, tok, n_own, own=own, full=full, streams=streams, col0=0, err=err),
                T * (n_own // 256 * 110 + 4 + (2 + n_streams) * n_own * 4))
    if op.startswith("expert_down_q5_1"):
        # a decode window of nt rows against 16 T Q5_1 weight rows of 640 columns (the reference's down width); random
        # bytes with sane fp16 d / m stand in for weights, SwiGLU-shaped Q8_1 rows for the activations
        nt, n, rows = int(op.rsplit("nt", 1)[1]), 640, 16 * T
        w = torch.randint(0, 256, (rows, n // 32, 24), dtype=torch.uint8, device=dev, generator=gen)
        w.view(torch.float16).reshape(rows, n // 32, 12)[..., 0:2] = 0.01
        w = w.reshape(rows, n // 32 * 24)
        act = ops.quantize_q8_1(N(gen, (nt, n), 0.5, dev))
        out = torch.empty((nt, rows), dtype=torch.float32, device=dev)
        return (lambda: ops.expert_down_rows_q5_1(w, act, n, out=out)), rows * (n // 32 * 24 + nt * 4) + nt * n // 32 * 36
    if op.startswith("expert_down_q8_0"):
        nt, n, rows = int(op.rsplit("nt", 1)[1]), 640, 16 * T
        w = torch.randint(0, 256, (rows, n // 32, 34), dtype=torch.uint8, device=dev, generator=gen)
        w.view(torch.float16).reshape(rows, n // 32, 17)[..., 0] = 0.01
        w = w.reshape(rows, n // 32 * 34)
        act = ops.quantize_q8_0(N(gen, (nt, n), 0.5, dev)).reshape(nt, -1)
        out = torch.empty((nt, rows), dtype=torch.float32, device=dev)
        return (lambda: ops.expert_down_rows("q8_0", w, act, n, out=out)), rows * (n // 32 * 34 + nt * 4) + nt * n // 32 * 34
    if op == "quantize_act_q":
        x = N(gen, (T, 640), 1.0, dev)
        codes, scales = ops.quantize_act_q(x)
        return (lambda: ops.quantize_act_q(x, codes, scales)), T * 640 * 4 + T * 640 + T * 20 * 4
    if op.startswith("expert_down_q2_0"):
        nt, n, rows = int(op.rsplit("nt", 1)[1]), 640, 32 * T
        w = torch.randint(0, 256, (rows, n // 64, 18), dtype=torch.uint8, device=dev, generator=gen)
        w.view(torch.float16).reshape(rows, n // 64, 9)[..., 0] = 0.01
        w = w.reshape(rows, n // 64 * 18)
        codes, scales = ops.quantize_act_q(N(gen, (nt, n), 0.5, dev))
        out = torch.empty((nt, rows), dtype=torch.float32, device=dev)
        return (lambda: ops.expert_down_rows_q2_0(w, codes, scales, n, out=out)), rows * (n // 64 * 18 + nt * 4) + nt * n * 9 // 8
    if op.startswith("expert_down_iq4_nl"):
        nt, n, rows = int(op.rsplit("nt", 1)[1]), 640, 16 * T
        w = torch.randint(0, 256, (rows, n // 32, 18), dtype=torch.uint8, device=dev, generator=gen)
        w.view(torch.float16).reshape(rows, n // 32, 9)[..., 0] = 0.01
        w = w.reshape(rows, n // 32 * 18)
        act = ops.quantize_q8_0(N(gen, (nt, n), 0.5, dev)).reshape(nt, -1)
        out = torch.empty((nt, rows), dtype=torch.float32, device=dev)
        return (lambda: ops.expert_down_rows("iq4_nl", w, act, n, out=out)), rows * (n // 32 * 18 + nt * 4) + nt * n // 32 * 34
    if op.startswith("expert_gate_up_q4_k"):
        # a decode window of nt rows against T gate rows and T up rows of 2560 columns (the reference's d_model)
        nt, n, rows = int(op.rsplit("nt", 1)[1]), 2560, 2 * T
        def table():
            w = torch.randint(0, 256, (rows, n // 256, 144), dtype=torch.uint8, device=dev, generator=gen)
            w.view(torch.float16).reshape(rows, n // 256, 72)[..., 0:2] = 1e-4
            return w.reshape(rows, n // 256 * 144)
        gate, up = table(), table()
        act = ops.quantize_q8_k(N(gen, (nt, n), 1.0, dev))
        out = torch.empty((nt, rows), dtype=torch.float32, device=dev)
        return (lambda: ops.expert_gate_up_rows_q4_k(gate, up, act, n, out=out)), rows * (2 * n // 256 * 144 + nt * 4) + nt * n // 256 * 292
    if op.startswith("expert_gate_up_q5_k"):
        nt, n, rows = int(op.rsplit("nt", 1)[1]), 2560, 2 * T
        gate = synth.torch_table("q5_k", gen, rows, n, dev, 1e-5, 2e-4)
        up = synth.torch_table("q5_k", gen, rows, n, dev, 1e-5, 2e-4)
        act = ops.quantize_q8_k(N(gen, (nt, n), 1.0, dev))
        out = torch.empty((nt, rows), dtype=torch.float32, device=dev)
        return (lambda: ops.expert_gate_up_rows_q5_k(gate, up, act, n, out=out)), rows * (2 * n // 256 * 176 + nt * 4) + nt * n // 256 * 292
    if op.startswith("expert_gate_up_iq3_s"):
        nt, n, rows = int(op.rsplit("nt", 1)[1]), 2560, 2 * T
        gate = synth.torch_table("iq3_s", gen, rows, n, dev, 2e-5, 3e-4)
        up = synth.torch_table("iq3_s", gen, rows, n, dev, 2e-5, 3e-4)
        act = ops.quantize_q8_k(N(gen, (nt, n), 1.0, dev))
        out = torch.empty((nt, rows), dtype=torch.float32, device=dev)
        return (lambda: ops.expert_gate_up_rows("iq3_s", gate, up, act, n, out=out)), rows * (2 * n // 256 * 110 + nt * 4) + nt * n // 256 * 292
    if op.startswith("expert_gate_up_iq2"):
        fmt = op[len("expert_gate_up_"):op.rindex("_nt")]
        nt, n, rows = int(op.rsplit("nt", 1)[1]), 2560, 2 * T
        bb = {"iq2_xxs": 66, "iq2_xs": 74, "iq2_s": 82}[fmt]

        def rows_of():
            t = torch.randint(0, 256, (rows, n // 256, bb), dtype=torch.uint8, device=dev, generator=gen)
            t.view(torch.float16).reshape(rows, n // 256, bb // 2)[..., 0] = 2e-4
            return t.reshape(rows, n // 256 * bb)
        gate, up = rows_of(), rows_of()
        act = ops.quantize_q8_k(N(gen, (nt, n), 1.0, dev))
        out = torch.empty((nt, rows), dtype=torch.float32, device=dev)
        return (lambda: ops.expert_gate_up_rows(fmt, gate, up, act, n, out=out)), rows * (2 * n // 256 * bb + nt * 4) + nt * n // 256 * 292
    if op.startswith("expert_gate_up_iq3_xxs"):
        nt, n, rows = int(op.rsplit("nt", 1)[1]), 2560, 2 * T
        gate = synth.torch_table("iq3_xxs", gen, rows, n, dev, 5e-5, 4e-4)
        up = synth.torch_table("iq3_xxs", gen, rows, n, dev, 5e-5, 4e-4)
        act = ops.quantize_q8_k(N(gen, (nt, n), 1.0, dev))
        out = torch.empty((nt, rows), dtype=torch.float32, device=dev)
        return (lambda: ops.expert_gate_up_rows_iq3_xxs(gate, up, act, n, out=out)), rows * (2 * n // 256 * 98 + nt * 4) + nt * n // 256 * 292
    if op.startswith("attend_"):
        # decode rows over T cells of the cache (16 query heads on 2 KV heads of 256): the roofline counts the cache
        # bytes, which every row of a head's group shares
        rows, kv8 = int(op.rsplit("_b", 1)[1]), "kv8" in op
        q = N(gen, (rows, c.n_q_heads, c.head_dim), 1.0, dev)
        if kv8:
            kc = torch.randint(-127, 128, (T, c.n_kv_heads, c.head_dim), dtype=torch.int8, device=dev, generator=gen)
            vc = torch.randint(-127, 128, (T, c.n_kv_heads, c.head_dim), dtype=torch.int8, device=dev, generator=gen)
            ks = torch.full((T, c.n_kv_heads, c.head_dim // 64), 0.01, dtype=torch.float16, device=dev).view(torch.int16)
            vs = ks.clone()
            cell = c.head_dim + c.head_dim // 64 * 2
        else:
            def plane():
                t = torch.randint(0, 256, (T, c.n_kv_heads, c.head_dim // 32, 34), dtype=torch.uint8, device=dev, generator=gen)
                t.view(torch.float16).reshape(T, c.n_kv_heads, c.head_dim // 32, 17)[..., 0] = 0.01
                return t.reshape(T, c.n_kv_heads, c.head_dim // 32 * 34)
            kc, vc, ks, vs = plane(), plane(), None, None
            cell = c.head_dim // 32 * 34
        out = torch.empty_like(q)
        ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
        return (lambda: ops.attend(q, kc, vc, k_scale=ks, v_scale=vs, range_begin=0, range_end=T, out=out, workspace=ws),
                T * c.n_kv_heads * 2 * cell + 2 * q.numel() * 4)
    if op == "quantize_q8_k":
        x = N(gen, (T, 2560), 1.0, dev)                      # the reference's d_model
        return (lambda: ops.quantize_q8_k(x)), T * 2560 * 4 + T * 2560 // 256 * 292
    if op.startswith("kv_read"):
        # T consecutive cells of a cache the append has filled (random bytes stand in: every byte pattern is a valid cell)
        if op == "kv_read_q8_0":
            cache = torch.randint(0, 256, (T, c.n_kv_heads, c.head_dim // 32 * 34), dtype=torch.uint8, device=dev, generator=gen)
            cache.view(torch.float16).reshape(T, c.n_kv_heads, c.head_dim // 32, 17)[..., 0] = 0.01
            scale, cell = None, c.head_dim // 32 * 34
        else:
            cache = torch.randint(-127, 128, (T, c.n_kv_heads, c.head_dim), dtype=torch.int8, device=dev, generator=gen)
            scale = torch.full((T, c.n_kv_heads, c.head_dim // 64), 0.01, dtype=torch.float16, device=dev).view(torch.int16)
            cell = c.head_dim + c.head_dim // 64 * 2
        out = torch.empty((T, c.n_kv_heads, c.head_dim), dtype=torch.float32, device=dev)
        return (lambda: ops.kv_read_f32(cache, scale=scale, out=out)), T * c.n_kv_heads * (cell + c.head_dim * 4)
    if op == "rms_norm":
        x, w = N(gen, (T, c.hidden), 1.0, dev), 1 + 0.1 * N(gen, (c.hidden,), 1.0, dev)
        y = torch.empty_like(x)
        return (lambda: ops.rms_norm(x, w, c.eps, out=y)), T * c.hidden * 8 + c.hidden * 4
    if op == "rms_norm_q8_1":
        x, w = N(gen, (T, c.hidden), 1.0, dev), 1 + 0.1 * N(gen, (c.hidden,), 1.0, dev)
        return (lambda: ops.rms_norm_quant(x, w, c.eps, "q8_1")), T * c.hidden * 4 + T * c.hidden // 32 * 36 + c.hidden * 4
    if op == "rms_norm_heads":
        h = c.n_q_heads + c.n_kv_heads
        x, w = N(gen, (T, h, c.head_dim), 1.0, dev), 1 + 0.1 * N(gen, (c.head_dim,), 1.0, dev)
        y = torch.empty_like(x)
        return (lambda: ops.rms_norm_heads(x, w, c.eps, out=y)), T * h * c.head_dim * 8
    if op in ("rope_kv", "rope_kv8"):
        q = N(gen, (T, c.n_q_heads, c.head_dim), 1.0, dev)
        k = N(gen, (T, c.n_kv_heads, c.head_dim), 1.0, dev)
        v = N(gen, (T, c.n_kv_heads, c.head_dim), 1.0, dev)
        wq, wk = 1 + 0.1 * N(gen, (c.head_dim,), 1.0, dev), 1 + 0.1 * N(gen, (c.head_dim,), 1.0, dev)
        pos = (c.depth + torch.arange(T, device=dev)).to(torch.int32)
        q_out = torch.empty_like(q)
        err = ops.new_err(dev)
        ts = ops.theta_scale(c.freq_base, c.n_rot)
        io = 2 * c.n_q_heads * c.head_dim * 4 + 2 * c.n_kv_heads * c.head_dim * 4 + 4
        if op == "rope_kv":
            kc = ops.new_kv_cache(c.cache_slots, c.n_kv_heads, c.head_dim, dev)
            vc = ops.new_kv_cache(c.cache_slots, c.n_kv_heads, c.head_dim, dev)
            cell = c.head_dim // 32 * ops.Q8_0_BLOCK
            return (lambda: ops.rope_neox_q8_0_append(q, k, v, pos, n_rot=c.n_rot, theta_scale=ts, k_cache=kc,
                                                      v_cache=vc, q_norm_w=wq, k_norm_w=wk, eps=c.eps, q_out=q_out,
                                                      err=err)), T * (io + 2 * c.n_kv_heads * cell)
        kc, ks = ops.new_kv_cache(c.cache_slots, c.n_kv_heads, c.head_dim, dev, fmt="kv8")
        vc, vs = ops.new_kv_cache(c.cache_slots, c.n_kv_heads, c.head_dim, dev, fmt="kv8")
        cell = c.head_dim + c.head_dim // 64 * 2
        return (lambda: ops.rope_neox_kv8_append(q, k, v, pos, n_rot=c.n_rot, theta_scale=ts, k_cache=kc, v_cache=vc,
                                                 k_scale=ks, v_scale=vs, q_norm_w=wq, k_norm_w=wk, eps=c.eps,
                                                 q_out=q_out, err=err)), T * (io + 2 * c.n_kv_heads * cell)
    rows = T * c.top_k
    gate, up = N(gen, (rows, c.inter), 0.5, dev), N(gen, (rows, c.inter), 0.5, dev)
    if op == "swiglu_q8_1":
        out = torch.empty((rows, c.inter // 32 * 36), dtype=torch.uint8, device=dev)
        return (lambda: ops.swiglu_q8_1(gate, up, out=out)), rows * (c.inter * 8 + c.inter // 32 * 36)
    if op == "swiglu_act":
        return (lambda: ops.swiglu_act(gate, up)), rows * (c.inter * 8 + c.inter // 32 * 40)
    if op == "quantize_q8_1":
        return (lambda: ops.quantize_q8_1(gate)), rows * (c.inter * 4 + c.inter // 32 * 36)
    raise SystemExit("unknown op " + op)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=OPS + ("all",), default="all")
    ap.add_argument("--tokens", type=int, default=65536)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--sets", type=int, default=1, help="distinct input sets rotated between launches (cold when > 1)")
    ap.add_argument("--graph", type=int, default=0, metavar="N",
                    help="time N launches replayed from one CUDA graph (device time without the host's launch cost; "
                         "for launches of a few microseconds)")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    peak = hbm_peak()
    cfg = ChainConfig(tokens=args.tokens)
    for op in (OPS if args.op == "all" else (args.op,)):
        gen = synth.torch_gen(dev, 7)
        cases = [make_case(op, args.tokens, dev, gen, cfg) for _ in range(args.sets)]
        nbytes = cases[0][1]
        for i in range(args.warmup):
            cases[i % args.sets][0]()
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.iters)]
        if args.graph > 0:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for i in range(args.graph):
                        cases[i % args.sets][0]()
            torch.cuda.current_stream(dev).wait_stream(side)
            graph.replay()
            torch.cuda.synchronize()
            for a, b in evs:
                a.record()
                graph.replay()
                b.record()
            torch.cuda.synchronize()
            ms = sorted(a.elapsed_time(b) / args.graph for a, b in evs)
        else:
            for i, (a, b) in enumerate(evs):
                a.record()
                cases[i % args.sets][0]()
                b.record()
            torch.cuda.synchronize()
            ms = sorted(a.elapsed_time(b) for a, b in evs)
        med, p90 = ms[len(ms) // 2], ms[min(len(ms) - 1, int(len(ms) * 0.9))]
        gbs = nbytes / (med * 1e-3) / 1e9
        print(json.dumps({"op": op, "tokens": args.tokens, "sets": args.sets, "graph": args.graph, "median_ms": round(med, 4),
                          "p90_ms": round(p90, 4), "min_ms": round(ms[0], 4), "bytes": nbytes, "gbs": round(gbs, 1),
                          "frac_of_hbm_peak": round(gbs / peak, 4), "tokens_per_s": round(args.tokens / (med * 1e-3))}))
        del cases
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
