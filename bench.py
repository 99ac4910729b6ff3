#!/usr/bin/env python3
"""Benchmark of the fused row-wise chain (embedding get_rows -> RMSNorm -> per-head norm + RoPE + Q8_0 KV append
-> RMSNorm -> SwiGLU + Q8_1) on synthetic inputs, one process per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

A step is one pass of the chain over T = 65536 tokens per GPU (weak scaling: every rank owns T token rows of a
longer prompt; the path has no collective).  Rank 0 prints ONE JSON line:
  value        whole-job tokens/s, inputs resident in HBM, CUDA events, max over ranks
  ops          per fused op: ms per launch, effective GB/s (algorithmic bytes), fraction of the measured HBM peak
  roofline     the dominant kernel (SwiGLU + Q8_1) against the measured HBM copy bandwidth
  e2e          the same metric through the host-buffer pipeline (pinned host inputs in, results out, copies timed)
  cpu_baseline the CPU oracle (a port of the reference's CPU definition) on a bounded sample, all host threads
`--impl reference` times only that CPU path and prints the same line shape with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fused row-wise chain throughput at T=65536 tokens per GPU (per-op GB/s and fraction of HBM peak in ops)"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0


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


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi.  It is started before the warm-up steps
    (nvidia-smi takes tens of milliseconds to produce its first line); the samples that arrive between begin() and
    end() are the timed region's.  A region shorter than the sampling period falls back to the samples taken while
    the same kernels were running in warm-up, and says so in `window`."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.t0, self.t1 = [], None, None, None
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

    def begin(self):
        self.t0 = time.time()

    def end(self):
        self.t1 = time.time()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.03)  # let the line that was sampled during the region arrive
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        ok = [(t, r) for t, r in self.rows if len(r) >= 6 and r[0].isdigit()]
        inside = [r for t, r in ok if self.t0 is not None and self.t0 <= t <= (self.t1 or t) + 0.02]
        window = "timed region"
        if not inside:
            inside, window = [r for t, r in ok if self.t0 is None or t <= (self.t1 or t) + 0.02], "warm-up + timed region"
        sm = sorted(int(r[0]) for r in inside)
        mx = [int(r[1]) for r in inside if r[1].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for r in inside for n, v in zip(names, r[2:6]) if v.lower() == "active"})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "window": window}


# ---- the CPU arm ---------------------------------------------------------------------------------------------

class CpuChain:
    """The oracle's chain on `tokens` tokens (full row widths), rows split over host threads."""

    def __init__(self, tokens: int, libm: bool = True):
        import ctypes as C
        import numpy as np
        from fnfl_v100_b200 import synth
        from fnfl_v100_b200.chain import ChainConfig
        from oracle import oracle as O
        O.use_libm(libm)
        self.O, self.C, self.tokens = O, C, tokens
        c = self.c = ChainConfig(tokens=tokens)
        g = synth.rng(5)
        self.vocab = 4096                               # rows actually touched; the decode cost per row is the same
        self.table = synth.q4_k_table(g, self.vocab, c.hidden)
        self.ids = g.integers(0, self.vocab, tokens).astype(np.int32)
        self.w1, self.w2 = synth.norm_weight(g, c.hidden), synth.norm_weight(g, c.hidden)
        self.wq, self.wk = synth.norm_weight(g, c.head_dim), synth.norm_weight(g, c.head_dim)
        self.q = synth.normal(g, (tokens, c.n_q_heads, c.head_dim))
        self.k = synth.normal(g, (tokens, c.n_kv_heads, c.head_dim))
        self.v = synth.normal(g, (tokens, c.n_kv_heads, c.head_dim))
        self.gate = synth.normal(g, (tokens * c.top_k, c.inter), 0.5)
        self.up = synth.normal(g, (tokens * c.top_k, c.inter), 0.5)
        self.pos = (c.depth + np.arange(tokens)).astype(np.int32)
        self.slot = np.arange(tokens).astype(np.int32)
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


def _cpu_sample_size(threads: int, target_s: float, cap: int) -> int:
    probe = CpuChain(256)
    probe.run(threads)
    per_tok = probe.run(threads) / 256
    n = int(min(cap, max(256, target_s / per_tok)))
    return n - n % 64


def cpu_baseline(threads: int) -> dict:
    sample = _cpu_sample_size(threads, 1.0, 16384)
    ch = CpuChain(sample)
    ch.run(threads)
    best = min(ch.run(threads) for _ in range(5))
    return {"value": sample / best, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{sample} tokens of the same chain (full row widths), best of 5 passes ({best:.3f} s); "
                      "oracle built -O2 -ffp-contract=off, host libm expf/sinf/cosf, rows split over host threads"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    if not os.path.exists(O.ORACLE_SO):
        O.build(with_ref=False)
    threads = os.cpu_count() or 1
    sample = _cpu_sample_size(threads, 1.0, 16384)
    ch = CpuChain(sample)
    for _ in range(args.warmup):
        ch.run(threads)
    dt = sum(ch.run(threads) for _ in range(args.steps))
    tps = sample * args.steps / dt
    desc = (f"{sample} tokens per step of the same chain on the host cores (the reference has no CPU code for the "
            "whole path in its tree: this is the oracle port, -O2 -ffp-contract=off, host libm)")
    emit({
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded)",
        "config": {"workload": "fused-op chain, hidden 2048, 16 Q / 2 KV heads x 256, 10 experts x 512", "sample": desc},
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })


# ---- the GPU arm -----------------------------------------------------------------------------------------------

def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    import fnfl_v100_b200 as fnb
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
        # rank 0 prints exactly one JSON line on stdout: whatever NCCL logs (its version banner at the VERSION and
        # WARN levels, everything at INFO) goes to stderr
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    T = args.tokens
    cfg = ChainConfig(tokens=T)
    chain = PrefillChain(cfg, dev, first_token=0)
    bpt = cfg.bytes_per_token()
    stages = PrefillChain.STAGES
    peak, peak_kind = hbm_peak()

    sampler = ClockSampler(local) if rank == 0 else None
    for _ in range(max(args.warmup, 3)):
        chain.step()
    barrier()
    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(stages) + 1)] for _ in range(K)]
    cur = torch.cuda.current_stream()
    barrier()
    if sampler:
        sampler.begin()
    for k in range(K):
        ev[k][0].record(cur)
        for i, name in enumerate(stages):
            getattr(chain, name)()
            ev[k][i + 1].record(cur)
    barrier()
    if sampler:
        sampler.end()
    total_ms = ev[0][0].elapsed_time(ev[K - 1][len(stages)])
    stage_ms = [sum(ev[k][i].elapsed_time(ev[k][i + 1]) for k in range(K)) / K for i in range(len(stages))]
    clocks = sampler.stop() if sampler else None
    if int(chain.err.item()) != 0:
        raise SystemExit("bench.py: the chain reported a device error word of %d" % int(chain.err.item()))

    t = torch.tensor([total_ms] + stage_ms, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, stage_ms = float(t[0]), [float(x) for x in t[1:]]

    # end to end from pinned host memory (chunks of 8192 tokens over three streams)
    e2e_steps = max(1, min(args.e2e_steps, K))
    e2e = None
    if not args.no_e2e:
        pipe = HostChunkPipeline(cfg, dev, chunk=min(8192, T), source=chain)
        pipe.step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(cur)
        for _ in range(e2e_steps):
            pipe.step()
        e1.record(cur)
        barrier()
        e2e_ms = torch.tensor([e0.elapsed_time(e1) / e2e_steps], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
        e2e_ms = float(e2e_ms)
        if int(pipe.h_err.item()) != 0:
            raise SystemExit("bench.py: the host pipeline reported a device error word of %d" % int(pipe.h_err.item()))
        e2e = {"value": T * world / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": pipe.h2d_bytes,
               "d2h_bytes_per_step": pipe.d2h_bytes, "ms_per_step": e2e_ms, "chunk_tokens": pipe.chunk,
               "launches_per_step": pipe.launches_per_step}

    # optional final gather of the quantised outputs over NVLink (not part of the timed chain)
    gather_ms = None
    if world > 1 and args.gather:
        from fnfl_v100_b200 import shard
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        g0.record(cur)
        full = shard.gather_rows(chain.act, T * cfg.top_k * world)
        g1.record(cur)
        barrier()
        gather_ms = g0.elapsed_time(g1)
        del full

    if rank == 0:
        ops_report = {}
        for name, ms in zip(stages, stage_ms):
            gbs = bpt[name] * T / (ms * 1e-3) / 1e9
            ops_report[name] = {"ms": round(ms, 4), "gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 4),
                                "bytes": bpt[name] * T}
        dom = "swiglu_q8_1"
        dom_bytes = bpt[dom] * T
        dom_ms = stage_ms[stages.index(dom)]
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        traffic = ncu_traffic("glu_quant_kernel")
        line = {
            "metric": METRIC, "value": T * world * K / (total_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded)",
            "config": {"workload": "fused-op chain: get_rows(Q4_K) -> RMSNorm -> Q/K head norm + NeoX RoPE + Q8_0 KV "
                                   "append -> RMSNorm -> SwiGLU + Q8_1",
                       "tokens_per_gpu": T, "hidden": cfg.hidden, "q_heads": cfg.n_q_heads, "kv_heads": cfg.n_kv_heads,
                       "head_dim": cfg.head_dim, "n_rot": cfg.n_rot, "experts_per_token": cfg.top_k,
                       "expert_inter": cfg.inter, "n_vocab": cfg.n_vocab, "cache_slots": cfg.cache_slots,
                       "depth": cfg.depth, "sharding": f"token rows, {world} shard(s), no collective",
                       "l2": "every stage streams more than the 126 MB L2 per launch; no flush needed"},
            "chain_gbs": sum(bpt.values()) * T / (total_ms / K * 1e-3) / 1e9,
            "chain_frac_of_hbm_peak": sum(bpt.values()) * T / (total_ms / K * 1e-3) / 1e9 / peak,
            "ops": ops_report,
            "roofline": {"kernel": "glu_quant_kernel (SwiGLU + Q8_1)", "bound": "hbm", "achieved": achieved,
                         "peak": peak, "peak_source": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "algorithmic_bytes": dom_bytes},
            "e2e": e2e,
            "gpu_launches": 5 * K * world,
            "clocks": clocks,
        }
        if gather_ms is not None:
            line["gather_ms"] = gather_ms
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(os.cpu_count() or 1)
        emit(line)
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
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=65536, help="token rows per GPU")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--gather", action="store_true", help="also time an all-gather of the Q8_1 outputs (N > 1)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (for profiler runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
