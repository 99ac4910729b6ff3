#!/usr/bin/env python3
"""Benchmark of the fused row-wise chain (embedding get_rows -> RMSNorm -> per-head norm + RoPE + Q8_0 KV append
-> RMSNorm -> SwiGLU + Q8_1) on synthetic inputs, one process per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

The job is ONE prefill chunk of T = 65536 tokens.  With N GPUs it is partitioned by token rows: rank r holds rows
shard.row_range(T, r, N) of every per-row tensor and appends its own range of cache cells; the table and the norm
weights are replicated; the data path has no collective (strong scaling).  A step is one pass of the chain over the
job, replayed from a CUDA graph of the rank's four launches.  Rank 0 prints ONE JSON line:

  value         whole-job tokens/s: T x K / (device time of K graph replays, CUDA events, max over ranks)
  step          median / p90 / mean of the K replays
  ops           per fused op, replayed alone from its own graph (after a short idle): median / p90 / mean ms, GB/s of the algorithmic
                bytes, fraction of the measured and of the nominal HBM peak.  At N = 1 also the configurations the
                chain does not run at their stated sizes (get_rows IQ3_XXS at T, RoPE + KV at 4096 tokens with
                random offsets, SwiGLU + Q8_1 at 40960 rows, RMSNorm at 512 rows), cold (inputs rotated over more
                bytes than L2 holds) and hot
  roofline      the dominant kernel (SwiGLU + Q8_1) against the measured HBM copy bandwidth
  sustained     at least a second of back-to-back chain steps (outside value) with the clocks sampled meanwhile
  e2e           the same metric through the host-buffer pipeline (pinned host inputs in, results out, copies timed),
                and the same copies without the kernels (the ceiling the host link sets)
  gather_ms,    N > 1: all-gather of the quantised outputs (Q8_1 activations, K / V cells), timed beside value; rank 0
  shard_check   recomputes a sample of every other rank's rows and compares it with the gathered bytes
  cpu_baseline  N = 1: the CPU oracle (a port of the reference's CPU definition) on a bounded sample, all host threads
`--impl reference` times only that CPU path on the whole job and prints the same line shape with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fused row-wise chain throughput at T=65536 tokens (per-op GB/s and fraction of HBM peak in ops)"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0
L2_BYTES = 126 * 1024 * 1024


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def ncu_traffic(kernel: str):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "roofline_traffic.json")) as f:
            return json.load(f).get(kernel)
    except Exception:
        return None


def job_config(args) -> dict:
    """The workload, spelled identically by both arms."""
    from fnfl_v100_b200.chain import ChainConfig
    c = ChainConfig(tokens=args.tokens)
    return {"workload": "fused-op chain of one prefill chunk: get_rows(Q4_K) -> RMSNorm -> Q/K head norm + NeoX RoPE + "
                        "Q8_0 KV append -> RMSNorm -> SwiGLU + Q8_1",
            "tokens": args.tokens, "hidden": c.hidden, "q_heads": c.n_q_heads, "kv_heads": c.n_kv_heads,
            "head_dim": c.head_dim, "n_rot": c.n_rot, "experts_per_token": c.top_k, "expert_inter": c.inter,
            "n_vocab": c.n_vocab, "cache_slots": c.cache_slots, "depth": c.depth, "shards": args.gpus,
            "sharding": "contiguous token-row ranges, no collective on the data path",
            "l2": "every step streams more than the 126 MB L2 per GPU between two launches of the same kernel; "
                  "no flush needed"}


def stats(ms: list) -> dict:
    s = sorted(ms)
    n = len(s)
    return {"median_ms": s[n // 2] if n % 2 else 0.5 * (s[n // 2 - 1] + s[n // 2]),
            "p90_ms": s[min(n - 1, int(math.ceil(0.9 * n)) - 1)], "mean_ms": sum(s) / n, "min_ms": s[0], "n": n}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi (read-only queries) from before the warm-up
    on; window(t0, t1) summarises the samples taken inside a wall-clock window.  A window shorter than the sampling
    period falls back to every sample taken so far, and says so."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, index: int):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "10"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def window(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.03)  # let the line that was sampled during the window arrive
        ok = [(t, r) for t, r in list(self.rows) if len(r) >= 6 and r[0].isdigit()]
        inside, where = [r for t, r in ok if t0 <= t <= t1 + 0.02], "the window itself"
        if not inside:
            inside, where = [r for t, r in ok if t <= t1 + 0.02], "everything sampled up to the window's end"
        sm = sorted(int(r[0]) for r in inside)
        mx = [int(r[1]) for r in inside if r[1].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for r in inside for n, v in zip(names, r[2:6]) if v.lower() == "active"})
        watts = [float(r[6]) for r in inside if len(r) > 6 and r[6].replace(".", "", 1).isdigit()]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "window": where,
                "power_w_max": max(watts) if watts else None}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass


# ---- the CPU arm ---------------------------------------------------------------------------------------------

class CpuChain:
    """The oracle's chain on rows [0, tokens) of the job (full row widths, the full table), rows split over host
    threads.  Inputs are the job's own counter-based rows, generated on the host."""

    def __init__(self, tokens: int, libm: bool = True):
        import ctypes as C
        import numpy as np
        import torch
        from fnfl_v100_b200 import synth
        from fnfl_v100_b200.chain import ChainConfig
        from oracle import oracle as O
        O.use_libm(libm)
        self.O, self.C, self.tokens = O, C, tokens
        c = self.c = ChainConfig(tokens=tokens)
        g = synth.rng(c.seed_case)
        seed = synth.SEED_BASE + c.seed_case
        self.vocab = c.n_vocab
        self.table = synth.q4_k_table(g, self.vocab, c.hidden)
        self.w1, self.w2 = synth.norm_weight(g, c.hidden), synth.norm_weight(g, c.hidden)
        self.wq, self.wk = synth.norm_weight(g, c.head_dim), synth.norm_weight(g, c.head_dim)
        torch.set_num_threads(os.cpu_count() or 1)
        N = lambda sid, rows, cols, sc: synth.counter_normal(seed, sid, 0, rows, cols, sc, "cpu").numpy()  # noqa: E731
        self.ids = synth.counter_ids(seed, 0, 0, tokens, c.n_vocab, "cpu").numpy()
        self.q = N(1, tokens, c.n_q_heads * c.head_dim, 1.0).reshape(tokens, c.n_q_heads, c.head_dim)
        self.k = N(2, tokens, c.n_kv_heads * c.head_dim, 1.0).reshape(tokens, c.n_kv_heads, c.head_dim)
        self.v = N(3, tokens, c.n_kv_heads * c.head_dim, 1.0).reshape(tokens, c.n_kv_heads, c.head_dim)
        self.gate = N(4, tokens * c.top_k, c.inter, 0.5)
        self.up = N(5, tokens * c.top_k, c.inter, 0.5)
        self.pos = (c.depth + np.arange(tokens)).astype(np.int32)
        self.slot = np.arange(tokens).astype(np.int32)          # a cache of `tokens` cells: the cells this job appends
        self.ts = O.theta_scale(c.freq_base, c.n_rot)
        self.kc = np.zeros((tokens, c.n_kv_heads, 272), np.uint8)
        self.vc = np.zeros_like(self.kc)
        self.hidden = np.zeros((tokens, c.hidden), np.float32)
        self.n1, self.n2, self.q_out = np.zeros_like(self.hidden), np.zeros_like(self.hidden), np.zeros_like(self.q)
        self.act = np.zeros((tokens * c.top_k, c.inter // 32 * 36), np.uint8)

    def _work(self, r0, r1):
        import numpy as np
        O, C, c, L = self.O, self.C, self.c, self.O.lib()
        n, k = r1 - r0, self.c.top_k
        err = np.zeros(1, np.uint32)
        L.fnbo_get_rows_q4_k(O._p(self.table), C.c_int64(self.vocab), O._p(self.ids[r0:r1]), O._p(self.hidden[r0:r1]),
                             O._p(err), C.c_int64(n), C.c_int32(c.hidden))
        L.fnbo_rms_norm_f32(O._p(self.hidden[r0:r1]), O._p(self.w1), C.c_float(c.eps), O._p(self.n1[r0:r1]),
                            C.c_int64(n), C.c_int32(c.hidden))
        a = O._RopeArgs(O._p(self.q[r0:r1]), O._p(self.k[r0:r1]), O._p(self.v[r0:r1]), O._p(self.pos[r0:r1]),
                        O._p(self.slot[r0:r1]), O._p(self.wq), O._p(self.wk), O._p(self.q_out[r0:r1]), O._p(self.kc),
                        O._p(self.vc), None, O._p(err), n, self.tokens, c.n_q_heads, c.n_kv_heads, c.head_dim,
                        c.n_rot, self.ts, c.eps)
        L.fnbo_rope_neox_q8_0_append(C.byref(a))
        L.fnbo_rms_norm_f32(O._p(self.hidden[r0:r1]), O._p(self.w2), C.c_float(c.eps), O._p(self.n2[r0:r1]),
                            C.c_int64(n), C.c_int32(c.hidden))
        L.fnbo_swiglu_q8_1(O._p(self.gate[r0 * k:r1 * k]), O._p(self.up[r0 * k:r1 * k]), O._p(self.act[r0 * k:r1 * k]),
                           None, C.c_int64(n * k), C.c_int32(c.inter))

    def run(self, threads: int) -> float:
        """One pass; returns seconds."""
        t0 = time.perf_counter()
        self.O.parallel_rows(self._work, self.tokens, threads)
        return time.perf_counter() - t0


CPU_BUILD = "oracle built -O3 -ffp-contract=off (no -march=native), host libm expf / sinf / cosf"


def cpu_baseline(threads: int, job_tokens: int) -> dict:
    """A bounded sample (about 10-30 s of CPU work with its set-up) of the same job on all host threads."""
    sample = min(16384, job_tokens)
    ch = CpuChain(sample)
    ch.run(threads)
    best = min(ch.run(threads) for _ in range(5))
    return {"value": sample / best, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"rows [0, {sample}) of the job (full row widths, the full {ch.vocab}-row table), best of 5 "
                      f"passes ({best:.3f} s); {CPU_BUILD}, rows split over {threads} host threads"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    if not os.path.exists(O.ORACLE_SO):
        O.build(with_ref=False)
    threads = os.cpu_count() or 1
    T = args.tokens
    ch = CpuChain(T)
    for _ in range(max(1, args.warmup)):
        ch.run(threads)
    dts = [ch.run(threads) for _ in range(args.steps)]
    dt = sum(dts)
    tps = T * args.steps / dt
    desc = (f"the whole job ({T} tokens) per step on {threads} host threads; the reference ships no CPU code for the "
            f"whole path, so this is the oracle port: {CPU_BUILD}")
    emit({
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": max(1, args.warmup), "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded, counter-based rows)",
        "config": job_config(args), "step": stats([d * 1e3 for d in dts]),
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })


# ---- the GPU arm -----------------------------------------------------------------------------------------------

def capture(fn):
    """`fn` (launches only, no allocation) recorded into a CUDA graph; one warm call first."""
    import torch
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


EVENT_TICK_MS = 0.002048   # the device clock CUDA events read advances in steps of about 2 us on this GPU
MIN_SAMPLE_MS = 0.4        # a timed sample is at least this long, so that the tick is under 1 % of it


def time_replays(graphs: list, k: int, warm: int = 3) -> list:
    """k samples of the time of one replay in ms (graphs taken in turn).  A sample is a run of back-to-back replays
    between two events, long enough that the event clock's tick does not show, divided by its length."""
    import torch
    cur = torch.cuda.current_stream()
    for i in range(max(warm, len(graphs))):
        graphs[i % len(graphs)].replay()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(cur)
    for i in range(8):
        graphs[i % len(graphs)].replay()
    b.record(cur)
    torch.cuda.synchronize()
    est = max(a.elapsed_time(b) / 8, EVENT_TICK_MS)
    per = max(1, int(math.ceil(MIN_SAMPLE_MS / est)))
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(k + 1)]
    torch.cuda.synchronize()
    ev[0].record(cur)
    n = 0
    for i in range(k):
        for _ in range(per):
            graphs[n % len(graphs)].replay()
            n += 1
        ev[i + 1].record(cur)
    torch.cuda.synchronize()
    return [ev[i].elapsed_time(ev[i + 1]) / per for i in range(k)]


def op_report(ms: list, nbytes: int, peak: float) -> dict:
    st = stats(ms)
    gbs = nbytes / (st["median_ms"] * 1e-3) / 1e9
    return {"median_ms": round(st["median_ms"], 5), "p90_ms": round(st["p90_ms"], 5), "mean_ms": round(st["mean_ms"], 5),
            "bytes": nbytes, "gbs": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak, 4),
            "frac_of_nominal_8tbs": round(gbs / NOMINAL_HBM_GBS, 4)}


def extra_configs(dev, k: int, peak: float, rest_s: float) -> dict:
    """The stated configurations the chain does not run at their own sizes, each replayed from graphs: cold (instances
    rotated so that more bytes than L2 holds pass between two replays of one instance) and hot (one instance), with
    one graph per launch and, `*_in_stream`, with the launches following one another inside one graph."""
    import torch
    from fnfl_v100_b200 import ops, synth
    from fnfl_v100_b200.chain import ChainConfig
    c = ChainConfig()
    out = {}

    def rotate(make, nbytes: int):
        n_inst = max(2, int(math.ceil(2.5 * L2_BYTES / nbytes)))
        return [make(i) for i in range(n_inst)], n_inst

    def both(name, make, nbytes, note):
        fns, n_inst = rotate(make, nbytes)
        graphs = [capture(f) for f in fns]
        time.sleep(rest_s)
        r = {"cold": op_report(time_replays(graphs, k), nbytes, peak), "hot": op_report(time_replays(graphs[:1], k), nbytes, peak),
             "instances_rotated": n_inst, "what": note}
        # the same launches as their caller issues them: one after the other in a stream (here: one graph of two
        # rounds over the instances), so that a launch's start-up overlaps its predecessor's end
        per = 2 * n_inst

        def in_stream(one: bool):
            def run():
                for j in range(per):
                    fns[0 if one else j % n_inst]()
            return run
        for key, one in (("cold_in_stream", False), ("hot_in_stream", True)):
            g = capture(in_stream(one))
            r[key] = op_report([t / per for t in time_replays([g], k)], nbytes, peak)
            del g
        r["launches_per_in_stream_graph"] = per
        out[name] = r

    seed = synth.SEED_BASE
    # configuration 4, the other table format, at T = 65536 (one launch streams 589 MB: cold by construction)
    gen = synth.torch_gen(dev, 4)
    T = 65536
    table = synth.torch_table("iq3_xxs", gen, c.n_vocab, c.hidden, dev)
    ids = synth.counter_ids(seed + 4, 0, 0, T, c.n_vocab, dev)
    rows_out = torch.empty((T, c.hidden), dtype=torch.float32, device=dev)
    err = ops.new_err(dev)
    nb = T * (ops.table_row_bytes("iq3_xxs", c.hidden) + 4 + c.hidden * 4)
    g = capture(lambda: ops.get_rows("iq3_xxs", table, ids, c.hidden, out=rows_out, err=err))
    out["get_rows_iq3_xxs_T65536"] = {"cold": op_report(time_replays([g], k), nb, peak),
                                      "what": "configuration 4, IQ3_XXS table [151936][2048], 65536 uniform ids"}
    del table, rows_out, g

    # configuration 2: 4096 tokens, positions = offset ~ U[0, 258048) + t, cache of 262144 slots
    T2 = 4096
    kc, vc = ops.new_kv_cache(c.cache_slots, c.n_kv_heads, c.head_dim, dev), ops.new_kv_cache(c.cache_slots, c.n_kv_heads, c.head_dim, dev)
    ts = ops.theta_scale(c.freq_base, c.n_rot)
    rg = synth.rng(2)

    def make_rope(i):
        q = synth.counter_normal(seed + 2, 10 + 3 * i, 0, T2, c.n_q_heads * c.head_dim, 1.0, dev).view(T2, c.n_q_heads, c.head_dim)
        kk = synth.counter_normal(seed + 2, 11 + 3 * i, 0, T2, c.n_kv_heads * c.head_dim, 1.0, dev).view(T2, c.n_kv_heads, c.head_dim)
        v = synth.counter_normal(seed + 2, 12 + 3 * i, 0, T2, c.n_kv_heads * c.head_dim, 1.0, dev).view(T2, c.n_kv_heads, c.head_dim)
        pos = torch.from_numpy(synth.positions(rg, T2)).to(dev)
        q_out = torch.empty_like(q)
        return lambda: ops.rope_neox_q8_0_append(q, kk, v, pos, n_rot=c.n_rot, theta_scale=ts, k_cache=kc, v_cache=vc,
                                                 q_out=q_out, err=err)
    cell = c.head_dim // 32 * ops.Q8_0_BLOCK
    nb2 = T2 * (2 * c.n_q_heads * c.head_dim * 4 + 2 * c.n_kv_heads * c.head_dim * 4 + 2 * c.n_kv_heads * cell + 4)
    both("rope_kv_q8_0_T4096", make_rope, nb2, "configuration 2: Q [4096][16][256], K / V [4096][2][256], no head norm, "
                                               "offsets U[0, 258048)")

    # configuration 3: 40960 rows of 512
    R3 = 40960

    def make_glu(i):
        gate = synth.counter_normal(seed + 3, 2 * i, 0, R3, c.inter, 0.5, dev)
        up = synth.counter_normal(seed + 3, 2 * i + 1, 0, R3, c.inter, 0.5, dev)
        act = torch.empty((R3, c.inter // 32 * ops.Q8_1_BLOCK), dtype=torch.uint8, device=dev)
        return lambda: ops.swiglu_q8_1(gate, up, out=act, err=err)
    both("swiglu_q8_1_R40960", make_glu, R3 * (2 * c.inter * 4 + c.inter // 32 * ops.Q8_1_BLOCK),
         "configuration 3: gate, up [40960][512]")

    # configuration 1: 512 rows of 2048 (plumbing size: launch-bound)
    R1 = 512
    w = 1.0 + 0.1 * synth.counter_normal(seed + 1, 0, 0, 1, c.hidden, 1.0, dev).view(-1)

    def make_norm(i):
        x = synth.counter_normal(seed + 1, 1 + i, 0, R1, c.hidden, 1.0, dev)
        y = torch.empty_like(x)
        return lambda: ops.rms_norm(x, w, c.eps, out=y)
    both("rms_norm_R512", make_norm, 2 * R1 * c.hidden * 4 + c.hidden * 4, "configuration 1: x [512][2048]")
    del kc, vc

    # the consumer of the cache the chain appends to: decode attention of 1 and 5 rows over the chain's depth (196608
    # cells, 2 KV heads under 16 query heads); the roofline counts the cache bytes, read once whatever the row count
    cells = c.depth

    def plane():
        t = torch.randint(0, 256, (cells, c.n_kv_heads, c.head_dim // 32, ops.Q8_0_BLOCK), dtype=torch.uint8, device=dev, generator=gen)
        t.view(torch.float16).reshape(cells, c.n_kv_heads, c.head_dim // 32, ops.Q8_0_BLOCK // 2)[..., 0] = 0.01
        return t.reshape(cells, c.n_kv_heads, c.head_dim // 32 * ops.Q8_0_BLOCK)
    ka, va = plane(), plane()
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    att = {"what": "fnb_attend over 196608 Q8_0 cells x 2 KV heads, 16 query heads of 256 (tcgen05.mma); bytes = the cache read once"}
    for rows in (1, 5):
        qa = synth.counter_normal(seed + 6, rows, 0, rows, c.n_q_heads * c.head_dim, 1.0, dev).view(rows, c.n_q_heads, c.head_dim)
        oa = torch.empty_like(qa)
        g = capture(lambda: ops.attend(qa, ka, va, range_begin=0, range_end=cells, out=oa, workspace=ws, err=err))
        time.sleep(rest_s)
        att["rows%d" % rows] = op_report(time_replays([g], k), cells * c.n_kv_heads * 2 * cell + 2 * qa.numel() * 4, peak)
    out["attend_q8_0_C196608"] = att
    if int(err.item()) != 0:
        raise RuntimeError("device error word %d in the extra configurations" % int(err.item()))
    return out


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    import fnfl_v100_b200 as fnb
    from fnfl_v100_b200 import ops, shard
    from fnfl_v100_b200.chain import ChainConfig, PrefillChain
    from fnfl_v100_b200.host_pipeline import HostChunkPipeline

    fnb.require()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this path has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # rank 0 prints exactly one JSON line on stdout: whatever NCCL logs goes to stderr
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values: list) -> list:
        t = torch.tensor(values, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t]

    T = args.tokens
    lo, hi = shard.row_range(T, rank, world)
    Tl = hi - lo
    cfg = ChainConfig(tokens=Tl)
    sampler = ClockSampler(local) if rank == 0 else None
    ops.prepare_device()
    chain = PrefillChain(cfg, dev, first_token=lo)
    bpt = cfg.bytes_per_token()
    stages = PrefillChain.STAGES
    peak, peak_kind = hbm_peak()
    cur = torch.cuda.current_stream()
    W, K = max(args.warmup, 3), args.steps

    # ---- the timed region: K replays of the step graph ----
    step_graph = chain.capture()
    for _ in range(W):
        step_graph.replay()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(K + 1)]
    barrier()
    t_begin = time.time()
    ev[0].record(cur)
    for i in range(K):
        step_graph.replay()
        ev[i + 1].record(cur)
    barrier()
    t_end = time.time()
    total_ms = ev[0].elapsed_time(ev[K])
    step_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(K)]
    clocks = sampler.window(t_begin, t_end) if sampler else None
    if int(chain.err.item()) != 0:
        raise SystemExit("bench.py: the chain reported a device error word of %d" % int(chain.err.item()))
    total_ms, = max_over_ranks([total_ms])
    step_stats = stats(step_ms)
    step_stats = dict(zip(step_stats, max_over_ranks([float(v) for v in step_stats.values()])))

    # ---- every stage alone, replayed from its own graph ----
    # (and the two stages the step's first launch fuses, each alone: configuration 4 and the hidden norm as stated)
    timed = stages + tuple(n for n in PrefillChain.UNFUSED if n not in stages)
    stage_ms = {}
    for name in timed:
        time.sleep(args.rest_s)          # each leg alone: let the board's power controller forget the previous one
        g = capture(getattr(chain, name))
        stage_ms[name] = time_replays([g], K, W)
        del g
    flat = max_over_ranks([v for name in timed for v in (stats(stage_ms[name])["median_ms"], stats(stage_ms[name])["p90_ms"],
                                                         stats(stage_ms[name])["mean_ms"])])
    ops_report = {}
    for i, name in enumerate(timed):
        med, p90, mean = flat[3 * i:3 * i + 3]
        nbytes = bpt[name] * math.ceil(T / world)            # the largest shard's bytes against the slowest rank's time
        gbs = nbytes / (med * 1e-3) / 1e9
        ops_report[name] = {"median_ms": round(med, 5), "p90_ms": round(p90, 5), "mean_ms": round(mean, 5),
                            "bytes": nbytes, "gbs": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak, 4),
                            "frac_of_nominal_8tbs": round(gbs / NOMINAL_HBM_GBS, 4), "in_step": name in stages,
                            "l2": "cold: one launch streams more than twice the L2" if nbytes > 2 * L2_BYTES else
                                  "the launch's bytes could partly sit in L2 between replays"}

    # ---- the stated configurations the chain does not run at their own sizes (one GPU only) ----
    extras = None
    if world == 1 and not args.no_extras:
        try:
            extras = extra_configs(dev, K, peak, args.rest_s)
        except Exception as e:  # the headline does not depend on them
            extras = {"error": repr(e)}

    # ---- sustained: at least a second of back-to-back steps, stage events on the last hundred ----
    n_sus = max(100, int(math.ceil(args.sustain_s * 1e3 / (total_ms / K)))) if args.sustain_s > 0 else 0
    n_ev = min(100, n_sus)
    sev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(stages) + 1)] for _ in range(n_ev)]
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    ts0 = time.time()
    s0.record(cur)
    for i in range(n_sus):
        j = i - (n_sus - n_ev)
        if j < 0:
            step_graph.replay()
            continue
        sev[j][0].record(cur)
        for si, name in enumerate(stages):
            getattr(chain, name)()
            sev[j][si + 1].record(cur)
    s1.record(cur)
    torch.cuda.synchronize()
    ts1 = time.time()
    sus_clocks = sampler.window(ts0 + 0.5 * (ts1 - ts0), ts1) if sampler else None
    sustained = None
    if rank == 0 and n_sus > 0:
        mhz = (sus_clocks or {}).get("sm_mhz")
        per = {}
        for si, name in enumerate(stages):
            ms = stats([sev[j][si].elapsed_time(sev[j][si + 1]) for j in range(n_ev)])["median_ms"]
            gbs = bpt[name] * Tl / (ms * 1e-3) / 1e9
            per[name] = {"median_ms": round(ms, 5), "gbs": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak, 4),
                         "ms_x_sm_mhz": round(ms * mhz, 2) if mhz else None}
        sustained = {"steps": n_sus, "seconds": round(s0.elapsed_time(s1) * 1e-3, 3),
                     "ms_per_step": round(s0.elapsed_time(s1) / n_sus, 5),
                     "stages_last_%d_steps" % n_ev: per, "clocks_second_half": sus_clocks,
                     "note": "rank 0's shard; graph replays, then eager launches with an event between stages"}

    # ---- end to end from pinned host memory ----
    e2e = None
    if not args.no_e2e:
        chunk = min(8192, max(256, (Tl // 4) // 256 * 256))
        while Tl % chunk != 0:
            chunk //= 2
        pipe = HostChunkPipeline(cfg, dev, chunk=chunk, source=chain)
        e2e_steps = max(1, min(args.e2e_steps, K))

        def timed(fn, n):
            fn()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(cur)
            for _ in range(n):
                fn()
            b.record(cur)
            barrier()
            return max_over_ranks([a.elapsed_time(b) / n])[0]

        e2e_ms = timed(pipe.step, e2e_steps)
        copy_ms = timed(lambda: pipe.step(copies_only=True), e2e_steps)
        if int(pipe.h_err.item()) != 0:
            raise SystemExit("bench.py: the host pipeline reported a device error word of %d" % int(pipe.h_err.item()))
        h2d, d2h = max_over_ranks([float(pipe.h2d_bytes), float(pipe.d2h_bytes)])
        e2e = {"value": T / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "bytes_are": "per GPU (the largest shard)", "ms_per_step": e2e_ms, "chunk_tokens": pipe.chunk,
               "launches_per_step": pipe.launches_per_step * world,
               "copies_only_ms_per_step": copy_ms, "copies_only_value": T / (copy_ms * 1e-3),
               "frac_of_copies_only": copy_ms / e2e_ms,
               "host_link_gbs_per_gpu": (h2d + d2h) / (copy_ms * 1e-3) / 1e9}
        del pipe

    # ---- N > 1: gather of the quantised outputs, timed beside value, and the cross-rank check ----
    gather_ms, shard_check = None, None
    if world > 1:
        k_cells, v_cells = chain.kv_cells()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        full_act = shard.gather_rows(chain.act, T * cfg.top_k)       # warm (communicator set-up)
        del full_act
        barrier()
        g0.record(cur)
        full_act = shard.gather_rows(chain.act, T * cfg.top_k)
        full_k = shard.gather_rows(k_cells, T)
        full_v = shard.gather_rows(v_cells, T)
        g1.record(cur)
        barrier()
        gather_ms, = max_over_ranks([g0.elapsed_time(g1)])
        if rank == 0:
            n_check, bad, checked = 256, 0, 0
            for r in range(1, world):
                rlo, rhi = shard.row_range(T, r, world)
                n = min(n_check, rhi - rlo)
                s = rlo + (rhi - rlo - n) // 2
                part = PrefillChain(ChainConfig(tokens=n), dev, first_token=s, shared=chain)
                part.step()
                torch.cuda.synchronize()
                pk, pv = part.kv_cells()
                bad += int((part.act != full_act[s * cfg.top_k:(s + n) * cfg.top_k]).sum())
                bad += int((pk != full_k[s:s + n]).sum()) + int((pv != full_v[s:s + n]).sum())
                bad += int(part.err.item() != 0)
                checked += n
            shard_check = {"mismatches": bad, "rows_checked": checked,
                           "what": "rank 0 regenerates %d rows from the middle of every other rank's range, runs the chain "
                                   "on them and compares Q8_1 bytes and K / V cells with the gathered ones" % n_check}
        gathered_bytes = int(full_act.numel() + full_k.numel() + full_v.numel())
        del full_act, full_k, full_v

    # ---- N > 1: the replicated form (every rank the whole job), for comparison with earlier records ----
    replicas = None
    if world > 1 and not args.no_replicas:
        del chain, step_graph
        torch.cuda.empty_cache()
        rep = PrefillChain(ChainConfig(tokens=T), dev, first_token=0)
        rg = rep.capture()
        for _ in range(W):
            rg.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record(cur)
        for _ in range(K):
            rg.replay()
        b.record(cur)
        barrier()
        rep_ms, = max_over_ranks([a.elapsed_time(b)])
        replicas = {"value": T * world * K / (rep_ms * 1e-3), "unit": UNIT, "tokens_per_gpu": T, "ms_per_step": rep_ms / K,
                    "note": "REPLICAS, not a partition: every rank runs the whole job on its own copy (weak scaling); "
                            "not the headline"}

    if rank == 0:
        dom = "swiglu_q8_1"
        dom_bytes = ops_report[dom]["bytes"]
        achieved = dom_bytes / (ops_report[dom]["mean_ms"] * 1e-3) / 1e9
        traffic = ncu_traffic("glu_quant_kernel")
        chain_bytes = sum(bpt[name] for name in stages) * T   # the step's launches, the fused first one as it is
        ms_per_step = total_ms / K
        line = {
            "metric": METRIC, "value": T * K / (total_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded, counter-based rows)",
            "config": job_config(args),
            "tokens_per_gpu": math.ceil(T / world),
            "timing": "CUDA-graph replays (%d warm, %d timed), CUDA events on the launching stream, max over ranks" % (W, K),
            "step": {k: round(v, 5) for k, v in step_stats.items()},
            "chain_gbs": chain_bytes / (ms_per_step * 1e-3) / 1e9,
            "chain_frac_of_measured_peak_x_gpus": chain_bytes / (ms_per_step * 1e-3) / 1e9 / (peak * world),
            "chain_frac_of_nominal_8tbs_x_gpus": chain_bytes / (ms_per_step * 1e-3) / 1e9 / (NOMINAL_HBM_GBS * world),
            "ops": ops_report,
            "configs": extras,
            "roofline": {"kernel": "glu_quant_kernel (SwiGLU + Q8_1)", "bound": "hbm", "achieved": achieved,
                         "peak": peak, "peak_source": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         "frac_of_nominal_8tbs": achieved / NOMINAL_HBM_GBS,
                         "traffic": traffic * dom_bytes / (bpt[dom] * 65536) if traffic else None,
                         "algorithmic_bytes": dom_bytes,
                         "how": "mean of the kernel's %d graph replays alone (ops.swiglu_q8_1.mean_ms); its time inside a "
                                "long run of the chain is sustained.stages_*.swiglu_q8_1" % K},
            "sustained": sustained,
            "e2e": e2e,
            "gpu_launches": PrefillChain.launches_per_step * K * world,
            "clocks": clocks,
        }
        if world > 1:
            line["gather_ms"] = gather_ms
            line["gather_bytes"] = gathered_bytes
            line["shard_check"] = shard_check
            line["replicas"] = replicas
        if world == 1 and not args.no_cpu:
            try:
                line["cpu_baseline"] = cpu_baseline(os.cpu_count() or 1, T)
            except Exception as e:
                line["cpu_baseline"] = {"error": repr(e)}
        emit(line)
    if sampler:
        sampler.stop()
    if world > 1:
        dist.destroy_process_group()


_RESULT_FD = None


def claim_stdout() -> None:
    """The contract is ONE JSON line on stdout.  Libraries print there too (NCCL's version banner at some debug
    levels, whatever a C extension writes), so file descriptor 1 is pointed at stderr for the whole run and the result
    line alone goes to the descriptor that was stdout."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main() -> None:
    claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3, help="warm-up steps (at least 3 are run)")
    ap.add_argument("--tokens", type=int, default=65536, help="token rows of the whole job (partitioned over the GPUs)")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--sustain-s", type=float, default=1.2, help="length of the sustained leg in seconds (0: skip it)")
    ap.add_argument("--rest-s", type=float, default=0.3,
                    help="idle time before each per-op leg (outside every timed region), so that a kernel timed alone "
                         "is not timed under the power cap its predecessor drove the board into")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (for profiler runs)")
    ap.add_argument("--no-extras", action="store_true", help="skip the stated configurations outside the chain")
    ap.add_argument("--no-replicas", action="store_true", help="N > 1: skip the replicated (weak) form")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
