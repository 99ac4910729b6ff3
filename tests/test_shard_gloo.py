"""The multi-GPU form on CPU: two gloo ranks each process their row_range shard (the oracle stands in for the
kernels here - this tests the partition and the gather, not the arithmetic) and gather_rows must reproduce the
unsharded result; a host-injected failure on one rank must be seen by both and skip the gather."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fnfl_v100_b200 import shard, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_row_range_is_a_balanced_partition():
    for total in (0, 1, 7, 65536, 65537):
        for world in (1, 2, 3, 4, 8):
            cuts = [shard.row_range(total, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            sizes = shard.shard_sizes(total, world)
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard.row_range(10, 2, 2)


def _worker(rank, world, port, rows, fail_rank, q):
    sys.path.insert(0, ROOT)
    from oracle import oracle as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = synth.rng(5)
        table = synth.q4_k_table(g, 64, 512)
        ids = g.integers(0, 64, rows).astype(np.int32)
        w = synth.norm_weight(g, 512)
        lo, hi = shard.row_range(rows, rank, world)
        hidden, err = O.get_rows("q4_k", table, 64, ids[lo:hi], 512)
        normed = O.rms_norm(hidden, w, 1e-6)
        act = O.quantize_q8_1(normed).reshape(hi - lo, -1)
        failed = shard.any_rank_failed(err != 0 or rank == fail_rank, torch.device("cpu"))
        if failed:
            q.put((rank, "skipped", None, None))
            return
        full_normed = shard.gather_rows(torch.from_numpy(normed), rows)
        full_act = shard.gather_rows(torch.from_numpy(act), rows)
        want_h, _ = O.get_rows("q4_k", table, 64, ids, 512)
        want_n = O.rms_norm(want_h, w, 1e-6)
        want_a = O.quantize_q8_1(want_n).reshape(rows, -1)
        ok = np.array_equal(full_normed.numpy().view(np.uint32), want_n.view(np.uint32)) and \
            np.array_equal(full_act.numpy(), want_a)
        q.put((rank, "ok" if ok else "mismatch", tuple(full_normed.shape), tuple(full_act.shape)))
    finally:
        dist.destroy_process_group()


def _run(rows, fail_rank, port):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, rows, fail_rank, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=180) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    return res


def test_two_ranks_gather_equals_unsharded():
    res = _run(rows=37, fail_rank=-1, port=29671)     # odd row count: shards of 18 and 19
    assert [r[1] for r in res] == ["ok", "ok"]
    assert res[0][2] == (37, 512) and res[0][3] == (37, 16 * 36)


def test_two_ranks_gather_of_equal_shards():
    res = _run(rows=64, fail_rank=-1, port=29675)     # equal shards take the single-collective path
    assert [r[1] for r in res] == ["ok", "ok"]
    assert res[0][2] == (64, 512) and res[0][3] == (64, 16 * 36)


def test_failure_on_one_rank_skips_the_gather_on_all():
    res = _run(rows=16, fail_rank=1, port=29673)
    assert [r[1] for r in res] == ["skipped", "skipped"]
