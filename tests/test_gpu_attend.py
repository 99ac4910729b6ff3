"""Decode attention over the appended cache against the FP64 oracle, through the C ABI.

The protocol is the reference's (fn/kernels/qsa/qa2_test.cpp:469-520): an FP64 evaluation over the DECODED cache
(the oracle's own dequantisers, the same values fnb_kv_read_f32 gives) and the bound max |error| / max |reference|
<= 1e-5 per row and query head.  Cases: both cache formats, both head widths, one to five rows (one to four 16-row
tiles: the two work splits of the kernel), ragged per-row ranges that start and end inside tiles, rows with no cell,
the output gate, many work units, and the chain itself: q_out and the cells written by fnb_rope_neox_q8_0_append.
"""
import numpy as np
import pytest
import torch

from fnfl_v100_b200 import ops, synth

pytestmark = pytest.mark.gpu
BOUND = 1e-5


def to_dev(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def make_cache(oracle, g, cells, n_kv, hd, fmt, scale=1.0):
    """Random K / V rows quantised by the oracle into cache planes; returns (device planes..., decoded F32 k, v)."""
    k = synth.normal(g, (cells, n_kv, hd), scale)
    v = synth.normal(g, (cells, n_kv, hd), scale)
    if fmt == "q8_0":
        kq = oracle.quantize_q8_0(k).reshape(cells, n_kv, hd // 32 * 34)
        vq = oracle.quantize_q8_0(v).reshape(cells, n_kv, hd // 32 * 34)
        return (kq, vq, None, None), oracle.dequantize_q8_0(kq).reshape(k.shape), oracle.dequantize_q8_0(vq).reshape(v.shape)
    kc, ks = oracle.kv8_quantize(k)
    vc, vs = oracle.kv8_quantize(v)
    planes = (kc.reshape(cells, n_kv, hd), vc.reshape(cells, n_kv, hd), ks.view(np.int16).reshape(cells, n_kv, hd // 64),
              vs.view(np.int16).reshape(cells, n_kv, hd // 64))
    return planes, oracle.kv8_dequantize(kc, ks).reshape(k.shape), oracle.kv8_dequantize(vc, vs).reshape(v.shape)


def check(out, ref, what):
    out = out.astype(np.float64)
    worst = 0.0
    for t in range(ref.shape[0]):
        for h in range(ref.shape[1]):
            top = np.abs(ref[t, h]).max()
            e = np.abs(out[t, h] - ref[t, h]).max()
            worst = max(worst, e / top if top > 0 else e)
    print("attend %s: worst max|error| / max|reference| over rows and heads %.3g" % (what, worst))
    assert worst <= BOUND, what
    return worst


@pytest.mark.parametrize("fmt,hd,rows,n_q,n_kv,cells", [
    ("q8_0", 256, 1, 16, 2, 1000),     # one row: one 16-row tile a KV head (8 of its rows live), halves split
    ("q8_0", 256, 3, 16, 2, 777),      # 24 rows a head: two tiles
    ("q8_0", 256, 5, 16, 2, 2051),     # 40 rows: three tiles, whole-tile warps
    ("q8_0", 256, 5, 12, 1, 600),      # the reference's shape: 12 heads on one KV head, five rows (60 rows, four tiles)
    ("kv8", 256, 1, 12, 1, 900), ("kv8", 256, 4, 16, 2, 1500),
    ("q8_0", 128, 2, 8, 2, 640), ("kv8", 128, 5, 8, 1, 333),
])
def test_attend_matches_fp64_reference(dev, oracle, fmt, hd, rows, n_q, n_kv, cells):
    g = synth.rng(31)
    planes, kf, vf = make_cache(oracle, g, cells + 70, n_kv, hd, fmt)
    q = synth.normal(g, (rows, n_q, hd), 1.0)
    first = g.integers(0, 60, rows).astype(np.int32)                    # ragged starts inside the first tile
    count = (cells - g.integers(0, 50, rows)).astype(np.int32)          # ragged ends
    lo, hi = int(first.min()), int((first + count).max())
    gate = synth.normal(g, (rows, n_q, hd), 1.5)
    d = [None if p is None else to_dev(p, dev) for p in planes]
    err = ops.new_err(dev)
    out = ops.attend(to_dev(q, dev), d[0], d[1], k_scale=d[2], v_scale=d[3], range_begin=lo, range_end=hi,
                     first_cell=to_dev(first, dev), n_cells=to_dev(count, dev), gate=to_dev(gate, dev), err=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = oracle.attend_f64(q, kf, vf, first, count, hd ** -0.5, gate=gate)
    check(out.cpu().numpy(), ref, "%s hd %d rows %d heads %d/%d cells %d" % (fmt, hd, rows, n_q, n_kv, cells))
    # bitwise reruns (the reference's bound includes them), with and without a caller-held workspace
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    again = ops.attend(to_dev(q, dev), d[0], d[1], k_scale=d[2], v_scale=d[3], range_begin=lo, range_end=hi,
                       first_cell=to_dev(first, dev), n_cells=to_dev(count, dev), gate=to_dev(gate, dev), workspace=ws)
    assert torch.equal(out, again)


def test_attend_many_units_no_gate_whole_range(dev, oracle):
    """A range long enough for several hundred work units, every row over the whole range (no per-row arrays), peaked
    scores (a few cells dominate) and no gate."""
    g = synth.rng(32)
    cells, n_kv, hd, rows, n_q = 40000, 2, 256, 2, 16
    planes, kf, vf = make_cache(oracle, g, cells, n_kv, hd, "q8_0")
    q = synth.normal(g, (rows, n_q, hd), 3.0)
    d = [None if p is None else to_dev(p, dev) for p in planes]
    out = ops.attend(to_dev(q, dev), d[0], d[1], range_begin=0, range_end=cells)
    torch.cuda.synchronize()
    ref = oracle.attend_f64(q, kf, vf, np.zeros(rows, np.int32), np.full(rows, cells, np.int32), hd ** -0.5)
    check(out.cpu().numpy(), ref, "40000 cells, whole range")


@pytest.mark.parametrize("fmt,rows,q_scale", [("q8_0", 1, 1.0), ("q8_0", 5, 3.0), ("kv8", 3, 2.0)])
def test_attend_full_depth_cache(dev, oracle, fmt, rows, q_scale):
    """The bench's depth: 196 608 cells of 2 KV heads under 16 query heads, whole range: every work unit is at its
    longest (the most accumulation steps between two partial results), flat and peaked scores."""
    g = synth.rng(35 + rows)
    cells, n_kv, hd, n_q = 196608, 2, 256, 16
    planes, kf, vf = make_cache(oracle, g, cells, n_kv, hd, fmt)
    q = synth.normal(g, (rows, n_q, hd), q_scale)
    d = [None if p is None else to_dev(p, dev) for p in planes]
    err = ops.new_err(dev)
    out = ops.attend(to_dev(q, dev), d[0], d[1], k_scale=d[2], v_scale=d[3], range_begin=0, range_end=cells, err=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = oracle.attend_f64(q, kf, vf, np.zeros(rows, np.int32), np.full(rows, cells, np.int32), hd ** -0.5)
    check(out.cpu().numpy(), ref, "%s, 196608 cells, %d rows, q x %g" % (fmt, rows, q_scale))


def test_attend_empty_rows_bad_ranges_and_rejections(dev, oracle):
    g = synth.rng(33)
    cells, n_kv, hd, rows, n_q = 512, 1, 256, 4, 4
    planes, kf, vf = make_cache(oracle, g, cells, n_kv, hd, "q8_0")
    q = synth.normal(g, (rows, n_q, hd), 1.0)
    first = np.array([10, 100, 300, 500], np.int32)
    count = np.array([200, 0, 100, 100], np.int32)          # row 1 has no cell; row 3 runs past the cache (600 > 512)
    d = [None if p is None else to_dev(p, dev) for p in planes]
    err = ops.new_err(dev)
    out = ops.attend(to_dev(q, dev), d[0], d[1], range_begin=0, range_end=cells, first_cell=to_dev(first, dev),
                     n_cells=to_dev(count, dev), err=err).cpu().numpy()
    torch.cuda.synchronize()
    assert int(err.item()) == ops.ERR_SLOT
    count_ok = count.copy()
    count_ok[3] = 0                                          # a refused row attends nothing: zeros
    ref = oracle.attend_f64(q, kf, vf, first, count_ok, hd ** -0.5)
    assert not out[1].any() and not out[3].any()
    check(out[[0, 2]], ref[[0, 2]], "ragged rows beside an empty and a refused one")
    # outside the contract: nothing enqueued
    with pytest.raises(ValueError):
        ops.attend(to_dev(q, dev), d[0], d[1], range_begin=0, range_end=cells + 1)           # range past the cache
    with pytest.raises(ValueError):
        ops.attend(to_dev(synth.normal(g, (17, n_q, hd)), dev), d[0], d[1], range_begin=0, range_end=cells)  # 68 rows a head


def test_attend_over_the_cells_the_append_wrote(dev, oracle):
    """The chain's own hand-over: q_out and the K / V cells of fnb_rope_neox_q8_0_append feed fnb_attend; the reference
    is the FP64 attention over the oracle's decode of the very cells the kernel wrote, with the kernel's own q_out."""
    g = synth.rng(34)
    hist, rows, n_q, n_kv, hd = 1200, 3, 16, 2, 256
    total = hist + rows
    q = synth.normal(g, (total, n_q, hd))
    k, v = synth.normal(g, (total, n_kv, hd)), synth.normal(g, (total, n_kv, hd))
    wq, wk = synth.norm_weight(g, hd), synth.norm_weight(g, hd)
    pos = np.arange(total).astype(np.int32)
    kc, vc = ops.new_kv_cache(2048, n_kv, hd, dev), ops.new_kv_cache(2048, n_kv, hd, dev)
    ts = ops.theta_scale(1e7, 64)
    q_out = ops.rope_neox_q8_0_append(to_dev(q, dev), to_dev(k, dev), to_dev(v, dev), to_dev(pos, dev), n_rot=64,
                                      theta_scale=ts, k_cache=kc, v_cache=vc, q_norm_w=to_dev(wq, dev), k_norm_w=to_dev(wk, dev))
    # the last `rows` tokens are the decode rows: row t attends cells 0 .. hist + t (causal)
    first = np.zeros(rows, np.int32)
    count = (hist + 1 + np.arange(rows)).astype(np.int32)
    out = ops.attend(q_out[hist:].contiguous(), kc, vc, range_begin=0, range_end=total, first_cell=to_dev(first, dev),
                     n_cells=to_dev(count, dev))
    torch.cuda.synchronize()
    kf = oracle.dequantize_q8_0(kc.cpu().numpy()[:total]).reshape(total, n_kv, hd)
    vf = oracle.dequantize_q8_0(vc.cpu().numpy()[:total]).reshape(total, n_kv, hd)
    ref = oracle.attend_f64(q_out[hist:].cpu().numpy(), kf, vf, first, count, hd ** -0.5)
    check(out.cpu().numpy(), ref, "causal rows over appended cells")


@pytest.mark.parametrize("seed", range(32))
def test_attend_random_shapes(dev, oracle, seed):
    """Shapes and ranges drawn at random: both formats and head widths, 1 to 5 rows, 1 to 4 KV heads, groups of up to 64
    query rows, ranges from a single cell to a few thousand that start and end anywhere, with and without the gate."""
    g = synth.rng(1000 + seed)
    fmt = ("q8_0", "kv8")[int(g.integers(0, 2))]
    hd = (128, 256)[int(g.integers(0, 2))]
    rows = int(g.integers(1, 6))
    n_kv = int(g.integers(1, 5))
    n_rep = int(g.integers(1, 64 // rows + 1))
    n_q = n_kv * n_rep
    cells = int(g.integers(1, 5000))
    lo = int(g.integers(0, cells))
    hi = int(g.integers(lo + 1, cells + 1))
    planes, kf, vf = make_cache(oracle, g, cells, n_kv, hd, fmt)
    q = synth.normal(g, (rows, n_q, hd), float(g.uniform(0.5, 2.5)))
    first = g.integers(lo, hi, rows).astype(np.int32)
    count = np.array([int(g.integers(0, hi - f + 1)) for f in first], np.int32)
    gate = synth.normal(g, (rows, n_q, hd), 1.0) if g.integers(0, 2) else None
    d = [None if p is None else to_dev(p, dev) for p in planes]
    err = ops.new_err(dev)
    out = ops.attend(to_dev(q, dev), d[0], d[1], k_scale=d[2], v_scale=d[3], range_begin=lo, range_end=hi,
                     first_cell=to_dev(first, dev), n_cells=to_dev(count, dev),
                     gate=None if gate is None else to_dev(gate, dev), err=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = oracle.attend_f64(q, kf, vf, first, count, hd ** -0.5, gate=gate)
    check(out.cpu().numpy(), ref, "%s hd %d rows %d heads %d/%d range [%d, %d)" % (fmt, hd, rows, n_q, n_kv, lo, hi))
