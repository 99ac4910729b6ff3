"""The bulk-copy pipelines' ring discipline, on a GPU.

1. Wide rows of the fused RMSNorm + requantise kernel leave room for fewer shared-memory stages than there are
   consumer groups; the kernel then runs fewer groups.  Enough rows to refill every stage many times, compared
   with the oracle, at the widths where that happens (3072, 4096) and at the benchmark width.
2. The give-up path of the bounded barrier waits (the reference bounds its device waits the same way:
   fn/kernels/qsa/attend.cu:264-281).  A second build of the three pipeline kernels gives every data-path wait a
   limit of two polls, while the waits a producer makes for its own copies to land keep the production limit.  A
   launch of that build ends by itself with FNB_ERR_TIMEOUT in the error word; nothing is left spinning, no copy is
   left in flight, the process carries on, and the next launch through the production library is bit-correct.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from fnfl_v100_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu


def to_dev(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("cols,fmt", [(4096, "q8_1"), (3072, "q8_0"), (3072, "act"), (2048, "q8_1"), (2560, "act")])
def test_fused_norm_refills_every_stage_many_times(dev, oracle, cols, fmt):
    rows = 148 * 3 * 8 * 8 + 5          # every CTA takes 64 tiles of three rows and a ragged end
    g = synth.rng(77)
    x = synth.normal(g, (rows, cols), 1.5)
    w = synth.norm_weight(g, cols)
    err = ops.new_err(dev)
    dx, dw = to_dev(x, dev), to_dev(w, dev)
    y_dev = torch.empty((rows, cols), dtype=torch.float32, device=dev)
    res = ops.rms_norm_quant(dx, dw, 1e-6, fmt, out_f32=y_dev, err=err)
    res2 = ops.rms_norm_quant(dx, dw, 1e-6, fmt, err=err)       # the form without the F32 copy: another instantiation
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    got_y, want_y = y_dev.cpu().numpy(), oracle.rms_norm(x, w, 1e-6)
    ia, ib = got_y.view(np.int32).astype(np.int64), want_y.view(np.int32).astype(np.int64)
    bad_rows = np.nonzero((np.abs(ia - ib) > 2).any(axis=1))[0]       # (same sign wherever the values are not tiny)
    assert bad_rows.size == 0, "%d rows differ, the first at %s (tiles %s)" % (bad_rows.size, bad_rows[:12], bad_rows[:12] // 3)
    # the blocks are exactly the CPU quantiser of the kernel's own F32 rows: a stale or foreign row cannot pass
    if fmt == "act":
        codes, scales = (t.cpu().numpy() for t in res)
        wc, ws = oracle.act_quantize(got_y)
        assert np.array_equal(codes, wc) and np.array_equal(scales.view(np.uint32), ws.view(np.uint32))
        assert torch.equal(res2[0], res[0]) and torch.equal(res2[1], res[1])
    else:
        q = oracle.quantize_q8_1 if fmt == "q8_1" else oracle.quantize_q8_0
        assert np.array_equal(res.cpu().numpy().reshape(-1), q(got_y).reshape(-1))
        assert torch.equal(res2, res)


def _expect_timeout(launch, err, tries=3):
    """Runs `launch` up to `tries` times; each launch must end by itself; returns once the error word holds
    FNB_ERR_TIMEOUT."""
    for _ in range(tries):
        assert launch() == _lib.OK
        torch.cuda.synchronize()        # returns: the kernel gave up and unwound, nothing is left spinning
        if int(err.item()) & _lib.ERR_TIMEOUT:
            return
    raise AssertionError("no wait gave up in %d launches of the two-poll build" % tries)


@pytest.mark.parametrize("rows", [256, 148 * 8 * 8])
def test_swiglu_wait_gives_up_and_reports_it(dev, oracle, shortwait_lib, rows):
    cols = 512
    g = synth.rng(3)
    gate, up = synth.normal(g, (rows, cols), 0.5), synth.normal(g, (rows, cols), 0.5)
    dg, du = to_dev(gate, dev), to_dev(up, dev)
    out = torch.zeros((rows, cols // 32 * 36), dtype=torch.uint8, device=dev)
    err = ops.new_err(dev)
    ops.swiglu_q8_1(dg, du, out=out, err=err)          # the production build first (also sets the kernel attribute)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    _expect_timeout(lambda: shortwait_lib.fnb_swiglu_q8_1(_p(dg), _p(du), _p(out), None, rows, cols, _p(err), _stream()),
                    err)
    # without an error word the same launch also ends by itself
    assert shortwait_lib.fnb_swiglu_q8_1(_p(dg), _p(du), _p(out), None, rows, cols, None, _stream()) == _lib.OK
    torch.cuda.synchronize()
    # the process carries on and the production library is bit-correct on the next launch
    err.zero_()
    out.fill_(0x5A)
    ops.swiglu_q8_1(dg, du, out=out, err=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert np.array_equal(out.cpu().numpy().reshape(-1), oracle.swiglu_q8_1(gate, up).reshape(-1))


def test_requantiser_and_fused_norm_waits_give_up_and_report_it(dev, oracle, shortwait_lib):
    rows, cols = 148 * 3 * 8 * 2, 2048
    g = synth.rng(4)
    x = synth.normal(g, (rows, cols), 1.0)
    w = synth.norm_weight(g, cols)
    dx, dw = to_dev(x, dev), to_dev(w, dev)
    out = torch.zeros((rows, cols // 32 * 36), dtype=torch.uint8, device=dev)
    err = ops.new_err(dev)
    want_q = ops.quantize_q8_1(dx, err=err)
    want_n = ops.rms_norm_quant(dx, dw, 1e-6, "q8_1", err=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    _expect_timeout(lambda: shortwait_lib.fnb_quantize_q8_1(_p(dx), _p(out), rows, cols, _p(err), _stream()), err)
    err.zero_()
    _expect_timeout(lambda: shortwait_lib.fnb_rms_norm_q8_1(_p(dx), _p(dw), 1e-6, _p(out), None, rows, cols, _p(err),
                                                            _stream()), err)
    err.zero_()
    again_q = ops.quantize_q8_1(dx, err=err)
    again_n = ops.rms_norm_quant(dx, dw, 1e-6, "q8_1", err=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert torch.equal(again_q, want_q) and torch.equal(again_n, want_n)
    assert np.array_equal(again_q.cpu().numpy().reshape(-1), oracle.quantize_q8_1(x))


@pytest.mark.parametrize("rows", [64, 148 * 2 * 4 * 3])
def test_rope_append_wait_gives_up_and_reports_it(dev, oracle, shortwait_lib, rows):
    n_q, n_kv, hd, n_rot, slots = 16, 2, 256, 64, 8192
    g = synth.rng(5)
    q, k, v = (synth.normal(g, (rows, h, hd)) for h in (n_q, n_kv, n_kv))
    pos = (np.arange(rows) + 1000).astype(np.int32)
    ts = ops.theta_scale(1e7, n_rot)
    dq, dk, dv, dpos = (to_dev(a, dev) for a in (q, k, v, pos))
    kc, vc = ops.new_kv_cache(slots, n_kv, hd, dev), ops.new_kv_cache(slots, n_kv, hd, dev)
    q_out = torch.empty_like(dq)
    err = ops.new_err(dev)
    ops.rope_neox_q8_0_append(dq, dk, dv, dpos, n_rot=n_rot, theta_scale=ts, k_cache=kc, v_cache=vc, q_out=q_out, err=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    want = (q_out.clone(), kc.clone(), vc.clone())
    a = _lib.RopeKvArgs(_p(dq).value, _p(dk).value, _p(dv).value, _p(dpos).value, None, None, None, _p(q_out).value,
                        _p(kc).value, _p(vc).value, None, _p(err).value, rows, slots, n_q, n_kv, hd, n_rot, ts, 1e-6)
    _expect_timeout(lambda: shortwait_lib.fnb_rope_neox_q8_0_append(C.byref(a), _stream()), err)
    err.zero_()
    q_out.fill_(0)
    kc.zero_()
    vc.zero_()
    ops.rope_neox_q8_0_append(dq, dk, dv, dpos, n_rot=n_rot, theta_scale=ts, k_cache=kc, v_cache=vc, q_out=q_out, err=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert torch.equal(q_out, want[0]) and torch.equal(kc, want[1]) and torch.equal(vc, want[2])
