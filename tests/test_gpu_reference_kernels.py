"""This library's kernels held to the REFERENCE'S OWN GPU kernels for the three F32 operations it has no CPU code for.

oracle/_ref/libfnb_ref_gpu.so is three of the reference's translation units compiled where they lie for sm_100a
(oracle/Makefile ref-gpu, oracle/ref_gpu_shim.cu): hidden RMSNorm (fn::draft::dcp_norm), SwiGLU into the activation
format (fn::experts::glu_finish) and K / V into the KV8 cache (fn::qsa::qsp_kv, text rows and image-row position
planes).  Those kernels evaluate the same definitions with the device's own expf / sincosf and fmaf chains, so their
bits are not the CPU definition's everywhere: the tests bound the difference as the reference's own tests do (one code
step, one FP16 unit) and print how many codes differ.  Where no transcendental or long sum is involved (the V half of
the KV8 append) the bytes must be equal.  Skipped when the library was not built (no reference tree at build time).
"""
import ctypes as C

import numpy as np
import pytest
import torch

from fnfl_v100_b200 import ops, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(oracle):
    lib = oracle.ref_gpu()
    if lib is None:
        pytest.skip("oracle/_ref/libfnb_ref_gpu.so was not built")
    return lib


def to_dev(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    # the reference's launchers refuse the null stream
    return C.c_void_p(torch.cuda.current_stream().cuda_stream or 0)


@pytest.fixture()
def side_stream(dev):
    s = torch.cuda.Stream(dev)
    with torch.cuda.stream(s):
        yield s
    s.synchronize()


def f16_steps(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in FP16 units in the last place between two int16 bit patterns of finite halves."""
    def key(x):
        x = x.to(torch.int32) & 0xFFFF
        return torch.where(x >= 0x8000, 0x8000 - x, x)
    return (key(a) - key(b)).abs()


def test_hidden_rms_norm_against_the_reference_kernel(dev, ref, side_stream):
    rows, D = 96, 2560
    g = synth.rng(0xD0)
    emb = synth.normal(g, (rows, D), 3.0)
    hidden = synth.normal(g, (rows, 4, D), 3.0)
    pred = synth.normal(g, (4, D), 3.0)
    enorm = g.uniform(0.5, 1.5, D).astype(np.float32)
    hnorm = g.uniform(0.5, 1.5, (4, D)).astype(np.float32)
    d = {n: to_dev(a, dev) for n, a in dict(emb=emb, hidden=hidden, pred=pred, enorm=enorm, hnorm=hnorm).items()}
    e16 = torch.zeros((rows, D), dtype=torch.int16, device=dev)
    h16 = torch.zeros((rows, 4, D), dtype=torch.int16, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    torch.cuda.current_stream().wait_stream(torch.cuda.default_stream())
    assert ref.fnbr_dcp_norm(rows, _p(d["emb"]), _p(d["hidden"]), _p(d["pred"]), _p(d["enorm"]), _p(d["hnorm"]), _p(e16),
                             _p(h16), _p(err), _stream()) == 0
    # this library: the same rows through fnb_rms_norm_f32, rounded to FP16 as the reference stores them
    ours_e = ops.rms_norm(d["emb"], d["enorm"], 1e-6).to(torch.float16).view(torch.int16)
    x_h = torch.cat([d["pred"][None], d["hidden"][:-1]], dim=0)            # row t's input is hidden row t - 1
    ours_h = torch.stack([ops.rms_norm(x_h[:, s].contiguous(), d["hnorm"][s].contiguous(), 1e-6) for s in range(4)], dim=1)
    ours_h = ours_h.to(torch.float16).view(torch.int16)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    for name, got, want in (("embedding rows", ours_e, e16), ("stream rows", ours_h, h16)):
        steps = f16_steps(got, want)
        differing = int((steps != 0).sum())
        print("rms_norm vs fn::draft::dcp_norm, %s: %d of %d FP16 codes differ, largest distance %d"
              % (name, differing, steps.numel(), int(steps.max())))
        assert int(steps.max()) <= 1 and differing <= 0.01 * steps.numel()


def test_swiglu_act_against_the_reference_kernel(dev, ref, side_stream):
    n, cols = 50, 320
    g = synth.rng(0xE1)
    gs, us = synth.normal(g, (n, cols), 2.0), synth.normal(g, (n, cols), 1.5)
    dg, du = to_dev(gs, dev), to_dev(us, dev)
    codes = torch.zeros((n, cols), dtype=torch.int8, device=dev)
    scales = torch.zeros((n, cols // 32, 2), dtype=torch.float32, device=dev)
    torch.cuda.current_stream().wait_stream(torch.cuda.default_stream())
    assert ref.fnbr_glu_finish(_p(dg), _p(du), n, _p(codes), _p(scales), _stream()) == 0
    oc, osc = ops.swiglu_act(dg, du)
    torch.cuda.synchronize()
    diff = (oc.to(torch.int32) - codes.to(torch.int32)).abs()
    differing = int((diff != 0).sum())
    d_rel = ((osc[..., 0] - scales[..., 0]).abs() / scales[..., 0].abs().clamp_min(1e-30)).max()
    print("swiglu_act vs fn::experts::glu_finish: %d of %d codes differ (largest step %d), largest relative "
          "difference of d %.3g" % (differing, diff.numel(), int(diff.max()), float(d_rel)))
    assert int(diff.max()) <= 1 and differing <= 0.01 * diff.numel()
    assert float(d_rel) <= 1e-6
    # s = d * sum(q): equal up to the codes that differ
    s_err = (osc[..., 1] - scales[..., 1]).abs()
    allowed = scales[..., 0].abs() * (diff.view(n, cols // 32, 32).sum(-1).float() + 1e-3) + 1e-6 * scales[..., 1].abs()
    assert bool((s_err <= allowed).all())


@pytest.mark.parametrize("with_planes", [False, True])
def test_kv8_append_against_the_reference_kernel(dev, ref, side_stream, with_planes):
    rows, hd, pos0, cells, rope_off = 512, 256, 1000, 4096, 0
    g = synth.rng(0xF2 + int(with_planes))
    k, v = synth.normal(g, (rows, 1, hd)), synth.normal(g, (rows, 1, hd))
    k_norm = synth.norm_weight(g, hd)
    planes = g.integers(0, 200000, (rows, 4)).astype(np.int32) if with_planes else None
    dk, dv, dw = to_dev(k, dev), to_dev(v, dev), to_dev(k_norm, dev)
    dpl = to_dev(planes, dev) if with_planes else None
    rk = torch.zeros((cells, hd), dtype=torch.int8, device=dev)
    rv = torch.zeros_like(rk)
    rks = torch.zeros((cells, 64), dtype=torch.int16, device=dev)      # the reference's scale parts: 64 halves a cell
    rvs = torch.zeros_like(rks)
    torch.cuda.current_stream().wait_stream(torch.cuda.default_stream())
    assert ref.fnbr_qsp_kv8(_p(dk), _p(dv), _p(dw), rows, pos0, cells, _p(rk), _p(rv), _p(rks), _p(rvs), rope_off, _p(dpl),
                            _stream()) == 0
    ts = ops.theta_scale(1e7, 64)
    assert ts == ref.fnbr_rope_theta_scale()
    (kc, ks), (vc, vs) = ops.new_kv_cache(cells, 1, hd, dev, fmt="kv8"), ops.new_kv_cache(cells, 1, hd, dev, fmt="kv8")
    q = torch.zeros((rows, 1, hd), dtype=torch.float32, device=dev)     # the entry point wants a Q tensor; unused here
    pos = to_dev((pos0 + rope_off + np.arange(rows)).astype(np.int32), dev)
    slots = to_dev((pos0 + np.arange(rows)).astype(np.int32), dev)
    err = ops.new_err(dev)
    ops.rope_neox_kv8_append(q, dk, dv, pos, n_rot=64, theta_scale=ts, k_cache=kc, v_cache=vc, k_scale=ks, v_scale=vs,
                             slots=slots, k_norm_w=dw, eps=1e-6, err=err, planes=dpl)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    sl = slice(pos0, pos0 + rows)
    # V has no transcendental and no long sum: the same bytes, and nothing outside the appended cells
    assert torch.equal(vc[sl, 0], rv[sl]) and torch.equal(vs[sl, 0], rvs[sl, :4])
    assert not bool(vc[:pos0].any()) and not bool(vc[pos0 + rows:].any())
    diff = (kc[sl, 0].to(torch.int32) - rk[sl].to(torch.int32)).abs()
    sdiff = f16_steps(ks[sl, 0], rks[sl, :4])
    print("rope + KV8 append vs fn::qsa::qsp_kv (%s): %d of %d K codes differ (largest step %d), %d of %d scales "
          "(largest distance %d)" % ("position planes" if with_planes else "text rows", int((diff != 0).sum()), diff.numel(),
                                     int(diff.max()), int((sdiff != 0).sum()), sdiff.numel(), int(sdiff.max())))
    assert int(sdiff.max()) <= 1
    # a scale one FP16 unit apart moves every code of its group by up to a step; beyond that one step is the bound
    assert int(diff.max()) <= 2 and int((diff > 1).sum()) <= 0.001 * diff.numel()
    assert int((diff != 0).sum()) <= 0.02 * diff.numel()
