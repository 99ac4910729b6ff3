"""The benchmark configurations at their full sizes: checked against the oracle on a seeded sample of rows
(the oracle finishes those in seconds) and through size-independent properties over the whole output
(equal ids give equal rows; decode(quantise) stays within half a step; every appended cell is written and
every other cell untouched)."""
import numpy as np
import pytest
import torch

from fnfl_v100_b200 import ops, synth

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.mark.parametrize("fmt", ["q4_k", "iq3_xxs"])
def test_get_rows_full_table(dev, oracle, fmt):
    V, cols, T = 151936, 2048, 65536
    gen = synth.torch_gen(dev, 4)
    table = synth.torch_table(fmt, gen, V, cols, dev)
    ids = torch.randint(0, V, (T,), dtype=torch.int32, device=dev, generator=gen)
    ids[:64] = ids[64:128]                                   # guaranteed repeats
    ids[-1], ids[-2] = V - 1, 0
    err = ops.new_err(dev)
    out = ops.get_rows(fmt, table, ids, cols, err=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert torch.equal(out[:64], out[64:128])                # equal ids -> equal rows
    assert bool(torch.isfinite(out).all())
    pick = torch.randperm(T, device=dev, generator=gen)[:768]
    pick[0], pick[1] = T - 1, T - 2
    rows = table[ids[pick].long()].cpu().numpy()
    deq = oracle.dequantize_q4_k if fmt == "q4_k" else oracle.dequantize_iq3_xxs
    want = deq(rows).reshape(len(pick), cols)
    assert np.array_equal(bits(out[pick].cpu().numpy()), bits(want))


def test_rms_norm_full(dev, oracle):
    T, cols = 65536, 2048
    gen = synth.torch_gen(dev, 1)
    x = synth.torch_normal(gen, (T, cols), 1.0, dev)
    w = 1.0 + 0.1 * synth.torch_normal(gen, (cols,), 1.0, dev)
    y = ops.rms_norm(x, w, 1e-6)
    torch.cuda.synchronize()
    # property over everything: mean((y / w)^2) is 1 to within eps and rounding
    ms = ((y / w).double() ** 2).mean(-1)
    assert float((ms - 1).abs().max()) < 1e-5
    pick = torch.randperm(T, device=dev, generator=gen)[:512]
    want = oracle.rms_norm(x[pick].cpu().numpy(), w.cpu().numpy(), 1e-6)
    got = y[pick].cpu().numpy()
    assert np.abs(bits(got).astype(np.int64) - bits(want).astype(np.int64)).max() <= 2


def test_swiglu_q8_1_full(dev, oracle):
    rows, cols = 65536 * 10, 512
    gen = synth.torch_gen(dev, 3)
    gate = synth.torch_normal(gen, (rows, cols), 0.5, dev)
    up = synth.torch_normal(gen, (rows, cols), 0.5, dev)
    out = ops.swiglu_q8_1(gate, up)
    torch.cuda.synchronize()
    pick = torch.cat([torch.randperm(rows, device=dev, generator=gen)[:1022], torch.tensor([0, rows - 1], device=dev)])
    want = oracle.swiglu_q8_1(gate[pick].cpu().numpy(), up[pick].cpu().numpy())
    assert np.array_equal(out[pick].cpu().numpy(), want)
    # property over everything: |decode(block) - glu| <= d / 2 (+ rounding of d to fp16), checked on the device
    blk = out.view(rows * cols // 32, 36)
    d = blk[:, 0:2].contiguous().view(torch.float16).float()
    qs = blk[:, 4:].contiguous().view(torch.int8).float()
    glu = (torch.nn.functional.silu(gate) * up).view(-1, 32)
    amax = glu.abs().max(-1, keepdim=True).values
    assert bool(((qs * d - glu).abs() <= 0.5 * d + amax * 2.0 ** -11 + 1e-30).all())
    assert bool((qs.abs().max(-1).values[amax[:, 0] > 1e-20] == 127).all())   # the largest value maps to +-127


def test_rope_kv_append_full_configuration(dev, oracle):
    T, nq, nkv, hd, n_rot, slots = 4096, 16, 2, 256, 64, 262144
    g = synth.rng(2)
    q, k, v = synth.normal(g, (T, nq, hd)), synth.normal(g, (T, nkv, hd)), synth.normal(g, (T, nkv, hd))
    pos = synth.positions(g, T)
    ts = oracle.theta_scale(1e7, n_rot)
    D = lambda a: torch.from_numpy(a).to(dev)  # noqa: E731
    kc = ops.new_kv_cache(slots, nkv, hd, dev)
    vc = ops.new_kv_cache(slots, nkv, hd, dev)
    err = ops.new_err(dev)
    q_out = ops.rope_neox_q8_0_append(D(q), D(k), D(v), D(pos), n_rot=n_rot, theta_scale=ts, k_cache=kc, v_cache=vc,
                                      err=err)
    torch.cuda.synchronize()
    lo = int(pos[0])
    wk = np.zeros((T, nkv, 272), np.uint8)      # the oracle writes the same T consecutive cells, rebased to 0
    wv = np.zeros_like(wk)
    wq, _, werr = oracle.rope_kv_append(q, k, v, pos, n_rot=n_rot, theta_scale=ts, k_cache=wk, v_cache=wv,
                                        cache_slots=T, slots=(pos - lo).astype(np.int32))
    assert werr == 0 and int(err.item()) == 0
    assert np.array_equal(bits(q_out.cpu().numpy()), bits(wq))
    assert np.array_equal(kc[lo:lo + T].cpu().numpy(), wk) and np.array_equal(vc[lo:lo + T].cpu().numpy(), wv)
    assert not bool(kc[:lo].any()) and not bool(kc[lo + T:].any())        # every other cell untouched
    assert not bool(vc[:lo].any()) and not bool(vc[lo + T:].any())
    # round trip over every appended cell: reading V back gives the oracle's decode of its own cells, and lies within
    # half a quantisation step (+ the FP16 rounding of d) of the V that went in
    back = ops.kv_read_f32(vc, cell0=lo, rows=T)
    assert np.array_equal(bits(back.cpu().numpy().reshape(-1)), bits(oracle.dequantize_q8_0(wv)))
    vin = D(v)
    amax = vin.reshape(T, nkv, hd // 32, 32).abs().amax(-1, keepdim=True)
    bound = amax / 127 * (0.5 + 127 * 2.0 ** -11) + 1e-30
    assert bool(((back.reshape(T, nkv, hd // 32, 32) - vin.reshape(T, nkv, hd // 32, 32)).abs() <= bound).all())
