"""Row sharding on a device: a job partitioned with shard.row_range reproduces the unsharded job's bytes.

One GPU stands in for 2, 4 and 8: the shards of a job run one after another on cuda:0, each a PrefillChain that
holds only its row range (counter-based inputs, positions depth + row, cells appended at the row's position), and
the concatenated outputs and the appended cache cells must equal the unsharded run bit for bit.  That is the
property the multi-GPU bench relies on: no row reads another row, so a partition changes nothing.
"""
import numpy as np
import pytest
import torch

from fnfl_v100_b200 import ChainConfig, PrefillChain, shard

pytestmark = pytest.mark.gpu

OUTPUTS = ("hidden", "normed_attn", "normed_ffn", "q_out", "act")


def _cfg(tokens):
    return ChainConfig(tokens=tokens, n_vocab=4096, cache_slots=8192, depth=1500)


@pytest.mark.parametrize("total", [4096, 1000 + 7])
def test_partitioned_job_equals_the_whole_job(dev, total):
    whole = PrefillChain(_cfg(total), dev)
    whole.step()
    torch.cuda.synchronize()
    assert int(whole.err.item()) == 0
    want = {n: getattr(whole, n).clone() for n in OUTPUTS}
    want_k, want_v = whole.k_cache.clone(), whole.v_cache.clone()
    lo0 = whole.cfg.depth
    assert bool(want_k[lo0:lo0 + total].any()) and not bool(want_k[:lo0].any()) and not bool(want_k[lo0 + total:].any())

    for world in (2, 4, 8):
        whole.k_cache.zero_()
        whole.v_cache.zero_()
        parts = {n: [] for n in OUTPUTS}
        covered = 0
        for rank in range(world):
            lo, hi = shard.row_range(total, rank, world)
            assert lo == covered
            covered = hi
            part = PrefillChain(_cfg(hi - lo), dev, first_token=lo, shared=whole)   # same table, weights and cache
            # the shard's inputs are the job's rows lo .. hi - 1
            assert torch.equal(part.ids, whole.ids[lo:hi]) and torch.equal(part.q, whole.q[lo:hi])
            assert torch.equal(part.gate, whole.gate[lo * 10:hi * 10]) and torch.equal(part.pos, whole.pos[lo:hi])
            part.step()
            torch.cuda.synchronize()
            assert int(part.err.item()) == 0
            k_cells, v_cells = part.kv_cells()
            assert torch.equal(k_cells, want_k[lo0 + lo:lo0 + hi]) and torch.equal(v_cells, want_v[lo0 + lo:lo0 + hi])
            for n in OUTPUTS:
                parts[n].append(getattr(part, n))
        assert covered == total
        for n in OUTPUTS:
            got = torch.cat(parts[n], dim=0)
            assert torch.equal(got.view(torch.uint8), want[n].view(torch.uint8)), (world, n)
        assert torch.equal(whole.k_cache, want_k) and torch.equal(whole.v_cache, want_v), world


def test_counter_inputs_do_not_depend_on_the_slice(dev):
    from fnfl_v100_b200 import synth
    a = synth.counter_normal(11, 3, 0, 5000, 512, 0.5, dev)
    for lo, hi in ((0, 1), (17, 4097), (4999, 5000)):
        assert torch.equal(synth.counter_normal(11, 3, lo, hi, 512, 0.5, dev), a[lo:hi])
    ids = synth.counter_ids(11, 0, 0, 100000, 151936, dev)
    assert torch.equal(synth.counter_ids(11, 0, 777, 9000, 151936, dev), ids[777:9000])
    assert 0 <= int(ids.min()) and int(ids.max()) < 151936
    m, s = float(a.mean()), float(a.std())
    assert abs(m) < 2e-3 and abs(s - 0.5) < 2e-3
