"""Parity of the CUDA path with the CPU oracle, through the C ABI (fnfl_v100_b200.ops -> libfnb200.so).

Bars: bit-exact for quantised bytes, dequantised embeddings and every F32 value whose CPU definition is a fixed
sequence of IEEE operations; RMSNorm outputs (whose sum of squares is reduced in a different order than the
CPU's sequential sum) within 2 ULP.  Outputs are poisoned before each launch and guard rows around them are
checked afterwards, so an unwritten or overrun value cannot pass.
"""
import os

import numpy as np
import pytest
import torch

from fnfl_v100_b200 import ops, synth

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
POISON = 0x5A


def to_dev(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def ulp_diff(a, b):
    """Distance in units in the last place between two float32 arrays (same sign assumed where it matters)."""
    ia = bits(a).astype(np.int64)
    ib = bits(b).astype(np.int64)
    ia = np.where(ia & 0x80000000, 0x80000000 - ia, ia)
    ib = np.where(ib & 0x80000000, 0x80000000 - ib, ib)
    return np.abs(ia - ib)


class Guarded:
    """A device output with poisoned guard rows before and after the live region."""

    def __init__(self, shape, dtype, dev, guard_rows=16):   # 16 rows keep the live region 16-byte aligned
        self.g = guard_rows
        full = (shape[0] + 2 * guard_rows,) + tuple(shape[1:])
        self.full = torch.empty(full, dtype=torch.uint8 if dtype == torch.uint8 else dtype, device=dev)
        self.full.view(torch.uint8).fill_(POISON)
        self.live = self.full[guard_rows:guard_rows + shape[0]]

    def check_guards(self):
        raw = self.full.view(torch.uint8).reshape(self.full.shape[0], -1)
        assert bool((raw[: self.g] == POISON).all()) and bool((raw[-self.g:] == POISON).all()), "guard rows overwritten"

    def numpy(self):
        return self.live.cpu().numpy()


# ---- RMSNorm ---------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("rows,cols", [(512, 2048), (1, 2048), (7, 2048), (33, 256), (1030, 256), (5, 128),
                                       (9, 512), (6, 1024), (3, 2560), (3, 4096), (5, 320), (4, 36), (2, 8192)])
def test_rms_norm_matches_oracle(dev, oracle, rows, cols):
    g = synth.rng(1)
    x = synth.normal(g, (rows, cols))
    w = synth.norm_weight(g, cols)
    out = Guarded((rows, cols), torch.float32, dev)
    ops.rms_norm(to_dev(x, dev), to_dev(w, dev), 1e-6, out=out.live)
    torch.cuda.synchronize()
    want = oracle.rms_norm(x, w, 1e-6)
    got = out.numpy()
    out.check_guards()
    d = ulp_diff(got, want)
    assert d.max() <= 2, f"max ulp {d.max()}"
    assert (d == 0).mean() >= 0.9999


def test_rms_norm_without_weight_and_heads_form(dev, oracle):
    g = synth.rng(1)
    x = synth.normal(g, (40, 16, 256), 3.0)
    w = synth.norm_weight(g, 256)
    got = ops.rms_norm_heads(to_dev(x, dev), to_dev(w, dev), 1e-6).cpu().numpy()
    assert ulp_diff(got, oracle.rms_norm(x, w, 1e-6)).max() <= 2
    got = ops.rms_norm(to_dev(x, dev), None, 1e-6).cpu().numpy()
    assert ulp_diff(got, oracle.rms_norm(x, None, 1e-6)).max() <= 2


# ---- SwiGLU + Q8_1 and the requantisers ------------------------------------------------------------------------------

@pytest.mark.parametrize("rows,cols", [(2048, 512), (1, 32), (7, 96), (33, 320), (50, 320), (3, 2048), (129, 512)])
def test_swiglu_q8_1_bytes_and_f32_bit_exact(dev, oracle, rows, cols):
    g = synth.rng(3)
    gate, up = synth.normal(g, (rows, cols), 0.5), synth.normal(g, (rows, cols), 0.5)
    out = Guarded((rows, cols // 32 * 36), torch.uint8, dev)
    f32 = Guarded((rows, cols), torch.float32, dev)
    ops.swiglu_q8_1(to_dev(gate, dev), to_dev(up, dev), out=out.live, out_f32=f32.live)
    torch.cuda.synchronize()
    want, want_f32 = oracle.swiglu_q8_1(gate, up, want_f32=True)
    got, got_f32 = out.numpy(), f32.numpy()
    out.check_guards()
    f32.check_guards()
    assert np.array_equal(bits(got_f32), bits(want_f32)), "F32 GLU differs from the CPU definition"
    # the reference's protocol: codes are the CPU quantiser of the kernel's own F32 ...
    assert np.array_equal(got.reshape(-1), oracle.quantize_q8_1(got_f32))
    # ... and end to end against the all-CPU oracle the mismatch count is zero
    assert int((got != want).sum()) == 0
    # without the optional F32 output the bytes are the same
    out2 = ops.swiglu_q8_1(to_dev(gate, dev), to_dev(up, dev)).cpu().numpy()
    assert np.array_equal(out2, want)


def test_swiglu_extreme_gates(dev, oracle):
    gate = np.array([[-200.0, -104.0, -103.5, -90.0, -88.0, -20.0, -1e-3, 0.0, 1e-30, 20.0, 88.0, 89.0, 100.0, 3e4,
                      -3e4, 1.0] * 2], np.float32)
    up = np.ones_like(gate)
    f32 = torch.empty((1, 32), dtype=torch.float32, device=dev)
    got = ops.swiglu_q8_1(to_dev(gate, dev), to_dev(up, dev), out_f32=f32).cpu().numpy()
    want, want_f32 = oracle.swiglu_q8_1(gate, up, want_f32=True)
    assert np.array_equal(bits(f32.cpu().numpy()), bits(want_f32))
    assert np.array_equal(got, want)


def test_requantisers_match_reference_golden_bytes(dev, oracle):
    """Inputs and expected bytes were produced by the reference's own quantize_row_q8_0_ref / _q8_1_ref and
    act_quantize_ref (tests/golden/make_golden.py): midpoints, zeros, subnormals, 127 x 65504, random runs."""
    gold = np.load(os.path.join(GOLD, "quant.npz"))
    x = to_dev(gold["x"], dev)
    assert np.array_equal(ops.quantize_q8_0(x).cpu().numpy(), gold["q8_0"])
    assert np.array_equal(ops.quantize_q8_1(x).cpu().numpy(), gold["q8_1"])
    codes, scales = ops.act_quantize(x)
    assert np.array_equal(codes.cpu().numpy(), gold["act_codes"])
    assert np.array_equal(bits(scales.cpu().numpy().reshape(-1, 2)), bits(gold["act_scales"]))


def test_swiglu_act_format_matches_oracle(dev, oracle):
    g = synth.rng(3)
    gate, up = synth.normal(g, (50, 320), 0.5), synth.normal(g, (50, 320), 0.5)
    codes, scales = ops.swiglu_act(to_dev(gate, dev), to_dev(up, dev))
    wc, ws, _ = oracle.swiglu_act(gate, up)
    assert np.array_equal(codes.cpu().numpy(), wc)
    assert np.array_equal(bits(scales.cpu().numpy()), bits(ws))


# ---- RoPE + KV append ------------------------------------------------------------------------------------------------

def _rope_case(g, rows, nq, nkv, hd, norm):
    q, k, v = synth.normal(g, (rows, nq, hd)), synth.normal(g, (rows, nkv, hd)), synth.normal(g, (rows, nkv, hd))
    wq = synth.norm_weight(g, hd) if norm else None
    wk = synth.norm_weight(g, hd) if norm else None
    return q, k, v, wq, wk


@pytest.mark.parametrize("rows,nq,nkv,hd,n_rot,norm", [
    (256, 16, 2, 256, 64, False),   # the rope + KV configuration, reduced rows
    (256, 16, 2, 256, 64, True),    # with the per-head Q/K norm fused, as the chain runs it
    (1, 16, 2, 256, 64, True), (7, 12, 1, 256, 64, True), (33, 3, 1, 256, 256, False), (5, 4, 4, 256, 0, True),
    (19, 8, 2, 128, 64, True), (19, 8, 2, 64, 32, False), (3, 40, 2, 256, 64, False),
])
def test_rope_kv_append_matches_oracle(dev, oracle, rows, nq, nkv, hd, n_rot, norm):
    g = synth.rng(2)
    q, k, v, wq, wk = _rope_case(g, rows, nq, nkv, hd, norm)
    slots_total = 4096
    pos = synth.positions(g, rows)                       # offsets up to 258 048: the large-argument sin/cos path
    slot = (g.permutation(slots_total - 8)[:rows] + 4).astype(np.int32)
    ts = oracle.theta_scale(1e7, max(n_rot, 2))
    cell = hd // 32 * 34
    kc = Guarded((slots_total, nkv, cell), torch.uint8, dev)
    vc = Guarded((slots_total, nkv, cell), torch.uint8, dev)
    qo = Guarded((rows, nq, hd), torch.float32, dev)
    kf = Guarded((rows, nkv, hd), torch.float32, dev)
    err = ops.new_err(dev)
    D = lambda a: None if a is None else to_dev(a, dev)  # noqa: E731
    ops.rope_neox_q8_0_append(D(q), D(k), D(v), D(pos), n_rot=n_rot, theta_scale=ts, k_cache=kc.live, v_cache=vc.live,
                              slots=D(slot), q_norm_w=D(wq), k_norm_w=D(wk), q_out=qo.live, k_f32=kf.live, err=err)
    torch.cuda.synchronize()
    wkc = np.full((slots_total, nkv, cell), POISON, np.uint8)
    wvc = wkc.copy()
    wq_out, wk_f32, werr = oracle.rope_kv_append(q, k, v, pos, n_rot=n_rot, theta_scale=ts, k_cache=wkc, v_cache=wvc,
                                                 cache_slots=slots_total, slots=slot, q_norm_w=wq, k_norm_w=wk,
                                                 want_k_f32=True)
    assert int(err.item()) == werr == 0
    for o in (kc, vc, qo, kf):
        o.check_guards()
    got_q, got_k = qo.numpy(), kf.numpy()
    if norm:
        assert ulp_diff(got_q, wq_out).max() <= 2 and ulp_diff(got_k, wk_f32).max() <= 2
        assert (ulp_diff(got_q, wq_out) == 0).mean() >= 0.9999
    else:
        assert np.array_equal(bits(got_q), bits(wq_out)), "rope output differs from the CPU definition"
        assert np.array_equal(bits(got_k), bits(wk_f32))
    # V cells are bit-exact unconditionally; K cells are the CPU quantiser of the kernel's own F32 k, and equal
    # the all-CPU oracle's bytes end to end
    assert np.array_equal(vc.numpy(), wvc)
    assert np.array_equal(kc.numpy()[slot].reshape(-1), oracle.quantize_q8_0(got_k))
    assert int((kc.numpy() != wkc).sum()) == 0


@pytest.mark.parametrize("rows,nq,nkv,hd", [(130, 16, 2, 256), (9, 12, 1, 256), (21, 1, 0, 256), (17, 8, 2, 128)])
def test_rope_position_planes_match_oracle(dev, oracle, rows, nq, nkv, hd):
    """Image rows: every rotary pair takes its position from one of four planes (fn/kernels/qsa/imrope.cuh:15-24).  Bit
    for bit the CPU definition, in the pipelined kernel and (one Q head and no K / V) in the row-per-warp kernel; text
    rows, whose four planes hold one integer, give exactly what no planes give."""
    g = synth.rng(6)
    q, k, v, _, _ = _rope_case(g, rows, nq, nkv, hd, False)
    planes = g.integers(0, 258048, (rows, 4)).astype(np.int32)
    pos = (100 + np.arange(rows)).astype(np.int32)            # with planes only the cache slot
    ts = oracle.theta_scale(1e7, 64)
    cell = hd // 32 * 34

    def run(pl, rot_pos):
        kc = Guarded((512, max(nkv, 1), cell), torch.uint8, dev)
        vc = Guarded((512, max(nkv, 1), cell), torch.uint8, dev)
        qo = Guarded((rows, nq, hd), torch.float32, dev)
        err = ops.new_err(dev)
        D = lambda a: None if a is None else to_dev(a, dev)  # noqa: E731
        ops.rope_neox_q8_0_append(D(q), D(k), D(v), D(rot_pos), n_rot=64, theta_scale=ts, k_cache=kc.live[:, :nkv],
                                  v_cache=vc.live[:, :nkv], slots=D(pos), q_out=qo.live, err=err, planes=D(pl))
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        for o in (kc, vc, qo):
            o.check_guards()
        return qo.numpy(), kc.numpy()[:, :nkv], vc.numpy()[:, :nkv]

    got_q, got_k, got_v = run(planes, pos)
    wkc = np.full((512, nkv, cell), POISON, np.uint8)
    wvc = wkc.copy()
    want_q, _, werr = oracle.rope_kv_append(q, k, v, pos, n_rot=64, theta_scale=ts, k_cache=wkc, v_cache=wvc,
                                            cache_slots=512, slots=pos, planes=planes)
    assert werr == 0
    assert np.array_equal(bits(got_q), bits(want_q))
    assert np.array_equal(got_k, wkc) and np.array_equal(got_v, wvc)
    # a text row: the same integer in all four planes is plain NeoX at that position
    same = np.repeat(planes[:, :1], 4, axis=1)
    q_a, k_a, _ = run(same, pos)
    q_b, k_b, _ = run(None, np.ascontiguousarray(planes[:, 0]))
    assert np.array_equal(bits(q_a), bits(q_b)) and np.array_equal(k_a, k_b)


def test_rope_slot_is_position_by_default_and_bad_slot_is_flagged(dev, oracle):
    g = synth.rng(2)
    q, k, v, _, _ = _rope_case(g, 6, 4, 2, 256, False)
    pos = np.array([10, 11, 70000, 12, -1, 13], np.int32)   # 70000 and -1 are outside a 64-slot cache
    ts = oracle.theta_scale(1e7, 64)
    kc = Guarded((64, 2, 272), torch.uint8, dev)
    vc = Guarded((64, 2, 272), torch.uint8, dev)
    qo = Guarded((6, 4, 256), torch.float32, dev)
    err = ops.new_err(dev)
    ops.rope_neox_q8_0_append(to_dev(q, dev), to_dev(k, dev), to_dev(v, dev), to_dev(pos, dev), n_rot=64,
                              theta_scale=ts, k_cache=kc.live, v_cache=vc.live, q_out=qo.live, err=err)
    torch.cuda.synchronize()
    wkc = np.full((64, 2, 272), POISON, np.uint8)
    wvc = wkc.copy()
    wq = np.full((6, 4, 256), 0, np.float32)
    wq.view(np.uint8)[:] = POISON
    wq, _, werr = oracle.rope_kv_append(q, k, v, pos, n_rot=64, theta_scale=ts, k_cache=wkc, v_cache=wvc,
                                        cache_slots=64, q_out=wq)
    assert int(err.item()) == werr == ops.ERR_SLOT
    assert np.array_equal(kc.numpy(), wkc) and np.array_equal(vc.numpy(), wvc)
    assert np.array_equal(bits(qo.numpy()), bits(wq))       # rows 2 and 4 stay poisoned in both
    for o in (kc, vc, qo):
        o.check_guards()


def test_rope_kv8_format_matches_reference_rule(dev, oracle):
    g = synth.rng(2)
    rows, nq, nkv, hd = 64, 12, 1, 256
    q, k, v, wq, wk = _rope_case(g, rows, nq, nkv, hd, True)
    # V rows: the reference's own KV8 stress rows (half steps, FP16-subnormal scales, underflow, huge magnitudes)
    gold = np.load(os.path.join(GOLD, "quant.npz"))
    stress = gold["x"].reshape(-1)[-(rows * hd):].reshape(rows, nkv, hd)
    v = np.ascontiguousarray(stress)
    pos = synth.positions(g, rows, 4096 - rows)
    ts = oracle.theta_scale(1e7, 64)
    kc, ks = ops.new_kv_cache(4096, nkv, hd, dev, fmt="kv8")
    vc, vs = ops.new_kv_cache(4096, nkv, hd, dev, fmt="kv8")
    kf = torch.empty((rows, nkv, hd), dtype=torch.float32, device=dev)
    ops.rope_neox_kv8_append(to_dev(q, dev), to_dev(k, dev), to_dev(v, dev), to_dev(pos, dev), n_rot=64,
                             theta_scale=ts, k_cache=kc, v_cache=vc, k_scale=ks, v_scale=vs, q_norm_w=to_dev(wq, dev),
                             k_norm_w=to_dev(wk, dev), k_f32=kf)
    torch.cuda.synchronize()
    got_k = kf.cpu().numpy()
    wc, wsc = oracle.kv8_quantize(got_k)
    pos = torch.from_numpy(pos).long().to(dev)
    assert np.array_equal(kc[pos].cpu().numpy().reshape(-1), wc)
    assert np.array_equal(ks[pos].cpu().numpy().view(np.uint16).reshape(-1), wsc)
    wc, wsc = oracle.kv8_quantize(v)
    assert np.array_equal(vc[pos].cpu().numpy().reshape(-1), wc)
    assert np.array_equal(vs[pos].cpu().numpy().view(np.uint16).reshape(-1), wsc)


# ---- reading the cache back ------------------------------------------------------------------------------------------

def test_kv_read_matches_reference_decode_on_golden_cells(dev, oracle):
    """Cells filled with the reference's own quantised stress rows: the read-back equals its decode bit for bit."""
    gold = np.load(os.path.join(GOLD, "quant.npz"))
    # KV8: 856 groups of 64 = 214 rows of 256
    codes = gold["kv8_codes"].reshape(214, 1, 256)
    scales = gold["kv8_scales"].reshape(214, 1, 4)
    got = ops.kv_read_f32(to_dev(codes, dev), scale=to_dev(scales.view(np.int16), dev)).cpu().numpy()
    assert np.array_equal(bits(got.reshape(-1)), bits(gold["kv8_values"].reshape(-1)))
    # Q8_0: 1712 blocks = 214 rows of 8 blocks
    cells = gold["q8_0"].reshape(214, 1, 272)
    got = ops.kv_read_f32(to_dev(cells, dev)).cpu().numpy()
    assert np.array_equal(bits(got.reshape(-1)), bits(oracle.dequantize_q8_0(cells)))


@pytest.mark.parametrize("fmt,hd,nkv", [("q8_0", 256, 2), ("kv8", 256, 2), ("q8_0", 128, 3), ("kv8", 128, 1),
                                        ("q8_0", 64, 2), ("kv8", 64, 5)])
def test_append_then_read_back(dev, oracle, fmt, hd, nkv):
    """What the append wrote, read back through a list of cells (bad cells flagged, their rows untouched), equals the
    oracle's quantise-then-decode of the same V rows; cells nobody wrote read as zeros."""
    g = synth.rng(21)
    rows, nq, slots = 77, 4, 512
    q, k, v, _, _ = _rope_case(g, rows, nq, nkv, hd, False)
    pos = synth.positions(g, rows, slots - rows)
    ts = oracle.theta_scale(1e7, 64)
    D = lambda a: to_dev(a, dev)  # noqa: E731
    if fmt == "q8_0":
        kc, vc = ops.new_kv_cache(slots, nkv, hd, dev), ops.new_kv_cache(slots, nkv, hd, dev)
        ops.rope_neox_q8_0_append(D(q), D(k), D(v), D(pos), n_rot=min(64, hd), theta_scale=ts, k_cache=kc, v_cache=vc)
        want = oracle.dequantize_q8_0(oracle.quantize_q8_0(v)).reshape(rows, nkv, hd)
        scale = None
    else:
        (kc, ks), (vc, vs) = ops.new_kv_cache(slots, nkv, hd, dev, fmt="kv8"), ops.new_kv_cache(slots, nkv, hd, dev, fmt="kv8")
        ops.rope_neox_kv8_append(D(q), D(k), D(v), D(pos), n_rot=min(64, hd), theta_scale=ts, k_cache=kc, v_cache=vc,
                                 k_scale=ks, v_scale=vs)
        want = oracle.kv8_dequantize(*oracle.kv8_quantize(v)).reshape(rows, nkv, hd)
        scale = vs
    cells = np.concatenate([pos, [-1, slots, int(pos.max()) + 1]]).astype(np.int32)   # two bad cells, one unwritten
    out = Guarded((len(cells), nkv, hd), torch.float32, dev)
    err = ops.new_err(dev)
    ops.kv_read_f32(vc, scale=scale, cells=D(cells), out=out.live, err=err)
    torch.cuda.synchronize()
    out.check_guards()
    got = out.numpy()
    assert int(err.item()) == ops.ERR_SLOT
    assert np.array_equal(bits(got[:rows]), bits(want))
    assert (got[rows:rows + 2].view(np.uint8) == POISON).all()
    assert not got[rows + 2].any()
    # contiguous form: cells cell0 .. cell0 + n - 1
    lo = int(pos.min())
    span = ops.kv_read_f32(vc, scale=scale, cell0=lo, rows=16).cpu().numpy()
    full = np.zeros((slots, nkv, hd), np.float32)
    full[pos] = want
    assert np.array_equal(bits(span), bits(full[lo:lo + 16]))


def test_quantize_q8_k_bit_exact(dev, oracle):
    """The reference's stress blocks (golden, from ggml's own quantiser) and a large random tensor."""
    gold = np.load(os.path.join(GOLD, "q8_k.npz"))
    got = ops.quantize_q8_k(to_dev(gold["x"], dev)).cpu().numpy()
    assert np.array_equal(got.reshape(-1, 292), gold["blocks"])
    g = synth.rng(41)
    x = synth.normal(g, (1000, 2560), 1.5)
    x[::7, ::5] = 0
    out = Guarded((1000, 2560 // 256 * 292), torch.uint8, dev)
    st = _lib_call_quantize_q8_k(to_dev(x, dev), out.live)
    torch.cuda.synchronize()
    out.check_guards()
    assert st == 0 and np.array_equal(out.numpy().reshape(-1, 292), oracle.quantize_q8_k(x))


def _lib_call_quantize_q8_k(x, out):
    import ctypes as C
    from fnfl_v100_b200 import _lib
    return _lib.lib().fnb_quantize_q8_k(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), x.shape[0], x.shape[1],
                                        C.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_expert_gate_up_rows_equal_the_reference_avx2_kernel_on_golden(dev):
    gold = np.load(os.path.join(GOLD, "gate_up_rows.npz"))
    got = ops.expert_gate_up_rows_q4_k(to_dev(gold["gate"], dev), to_dev(gold["up"], dev), to_dev(gold["act"], dev), 2560)
    assert np.array_equal(bits(got.cpu().numpy()), bits(gold["ff"]))


@pytest.mark.parametrize("n,rows,nt", [(2560, 320, 1), (2560, 999, 3), (2560, 130, 8), (256, 37, 2), (1024, 65, 13)])
def test_expert_gate_up_rows_bit_exact(dev, oracle, n, rows, nt):
    """RMSNorm -> Q8_K on the device (the path's hand-over), Q4_K gate and up rows: ff, and g and u themselves, carry
    every bit of the oracle's lane-for-lane restatement; rows outside [r0, r1) stay untouched."""
    g = synth.rng(33)
    x = synth.normal(g, (nt, n), 1.0)
    act = ops.quantize_q8_k(to_dev(x, dev))
    assert np.array_equal(act.cpu().numpy().reshape(-1, 292), oracle.quantize_q8_k(x))
    gate, up = synth.q4_k_table(g, rows, n, 1e-5, 3e-4), synth.q4_k_table(g, rows, n, 1e-5, 3e-4)
    r0, r1 = 2, rows - 1
    out = torch.full((nt, rows), float("nan"), dtype=torch.float32, device=dev)
    gu = torch.zeros((2, nt, rows), dtype=torch.float32, device=dev) if nt <= 8 else None
    ops.expert_gate_up_rows_q4_k(to_dev(gate, dev), to_dev(up, dev), act, n, r0=r0, r1=r1, out=out, gu=gu)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    want, wgu = oracle.expert_gu_rows_q4_k(gate, up, act.cpu().numpy(), n, r0=r0, r1=r1, want_gu=True)
    assert np.array_equal(bits(got[:, r0:r1]), bits(want[:, r0:r1]))
    assert np.isnan(got[:, :r0]).all() and np.isnan(got[:, r1:]).all()
    if gu is not None:
        assert np.array_equal(bits(gu.cpu().numpy()[:, :, r0:r1]), bits(wgu[:, :, r0:r1]))
    assert np.abs(want[:, r0:r1]).max() < 1e3 and np.abs(wgu[0][:, r0:r1]).std() > 0.3   # gates of order one: the GLU is exercised


def test_expert_gate_up_rows_q5_k_equal_the_reference_avx2_kernel_on_golden(dev):
    gold = np.load(os.path.join(GOLD, "gate_up_rows_q5_k.npz"))
    got = ops.expert_gate_up_rows_q5_k(to_dev(gold["gate"], dev), to_dev(gold["up"], dev), to_dev(gold["act"], dev), 2560)
    assert np.array_equal(bits(got.cpu().numpy()), bits(gold["ff"]))


@pytest.mark.parametrize("n,rows,nt", [(2560, 320, 1), (2560, 999, 3), (2560, 130, 8), (256, 37, 2), (1024, 65, 13)])
def test_expert_gate_up_rows_q5_k_bit_exact(dev, oracle, n, rows, nt):
    """As the Q4_K test, with Q5_K rows: the high bits from qh and the mins as one scalar per (row, window row)."""
    g = synth.rng(34)
    x = synth.normal(g, (nt, n), 1.0)
    act = ops.quantize_q8_k(to_dev(x, dev))
    d_hi = 1.5e-4 * (2560 / n) ** 0.5
    gate, up = synth.q5_k_table(g, rows, n, d_hi / 10, d_hi), synth.q5_k_table(g, rows, n, d_hi / 10, d_hi)
    r0, r1 = 2, rows - 1
    out = torch.full((nt, rows), float("nan"), dtype=torch.float32, device=dev)
    gu = torch.zeros((2, nt, rows), dtype=torch.float32, device=dev) if nt <= 8 else None
    ops.expert_gate_up_rows_q5_k(to_dev(gate, dev), to_dev(up, dev), act, n, r0=r0, r1=r1, out=out, gu=gu)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    want, wgu = oracle.expert_gu_rows_q5_k(gate, up, act.cpu().numpy(), n, r0=r0, r1=r1, want_gu=True)
    assert np.array_equal(bits(got[:, r0:r1]), bits(want[:, r0:r1]))
    assert np.isnan(got[:, :r0]).all() and np.isnan(got[:, r1:]).all()
    if gu is not None:
        assert np.array_equal(bits(gu.cpu().numpy()[:, :, r0:r1]), bits(wgu[:, :, r0:r1]))
    assert np.abs(want[:, r0:r1]).max() < 1e4 and np.abs(wgu[0][:, r0:r1]).std() > 0.3


def test_expert_gate_up_rows_iq3_xxs_equal_the_reference_avx2_kernel_on_golden(dev):
    """The reference's own iq_gu_rows outputs, also for a window holding -128 codes (the kernel's other sign path)."""
    gold = np.load(os.path.join(GOLD, "gate_up_rows_iq3_xxs.npz"))
    gate, up = to_dev(gold["gate"], dev), to_dev(gold["up"], dev)
    for act, want in ((gold["act"], gold["ff"]), (gold["act_m128"], gold["ff_m128"])):
        got = ops.expert_gate_up_rows_iq3_xxs(gate, up, to_dev(act, dev), 2560)
        assert np.array_equal(bits(got.cpu().numpy()), bits(want))


@pytest.mark.parametrize("n,rows,nt,m128", [(2560, 320, 1, False), (2560, 999, 3, False), (2048, 130, 8, False),
                                            (512, 37, 2, True), (1024, 65, 13, False), (4096, 70, 5, True),
                                            (5632, 41, 2, False), (16384, 9, 7, False)])
def test_expert_gate_up_rows_iq3_xxs_bit_exact(dev, oracle, n, rows, nt, m128):
    """Q8_K on the device, IQ3_XXS gate and up rows: ff, and g and u themselves, carry every bit of the oracle's
    lane-for-lane restatement; rows outside [r0, r1) stay untouched.  Covers rows staged whole (up to 2560 columns) and
    in chunks with a ragged last one (5632 = 8 + 8 + 6 super-blocks), every row alignment within 16 bytes (2560 columns:
    980-byte rows), windows of several passes, and -128 codes."""
    g = synth.rng(35)
    x = synth.normal(g, (nt, n), 1.0)
    act = ops.quantize_q8_k(to_dev(x, dev))
    if m128:
        a = act.cpu().numpy().reshape(nt, -1, 292)
        codes = a[:, :, 4:260]
        codes[g.integers(0, 7, size=codes.shape) == 0] = 0x80
        act = to_dev(a.reshape(nt, -1), dev)
    d_hi = 4e-4 * (2560 / n) ** 0.5
    gate, up = synth.iq3_xxs_table(g, rows, n, d_hi / 8, d_hi), synth.iq3_xxs_table(g, rows, n, d_hi / 8, d_hi)
    r0, r1 = 2, rows - 1
    out = torch.full((nt, rows), float("nan"), dtype=torch.float32, device=dev)
    gu = torch.zeros((2, nt, rows), dtype=torch.float32, device=dev) if nt <= 8 else None
    ops.expert_gate_up_rows_iq3_xxs(to_dev(gate, dev), to_dev(up, dev), act, n, r0=r0, r1=r1, out=out, gu=gu)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    want, wgu = oracle.expert_gu_rows_iq3_xxs(gate, up, act.cpu().numpy(), n, r0=r0, r1=r1, want_gu=True)
    assert np.array_equal(bits(got[:, r0:r1]), bits(want[:, r0:r1]))
    assert np.isnan(got[:, :r0]).all() and np.isnan(got[:, r1:]).all()
    if gu is not None:
        assert np.array_equal(bits(gu.cpu().numpy()[:, :, r0:r1]), bits(wgu[:, :, r0:r1]))
    assert np.abs(want[:, r0:r1]).max() < 1e3 and np.abs(wgu[0][:, r0:r1]).std() > 0.3   # gates of order one: the GLU is exercised


def test_expert_gate_up_rows_iq3_s_equal_the_reference_avx2_kernel_on_golden(dev):
    gold = np.load(os.path.join(GOLD, "gate_up_rows_iq3_s.npz"))
    gate, up = to_dev(gold["gate"], dev), to_dev(gold["up"], dev)
    for act, want in ((gold["act"], gold["ff"]), (gold["act_m128"], gold["ff_m128"])):
        got = ops.expert_gate_up_rows("iq3_s", gate, up, to_dev(act, dev), 2560)
        assert np.array_equal(bits(got.cpu().numpy()), bits(want))


@pytest.mark.parametrize("n,rows,nt,m128", [(2560, 320, 1, False), (2560, 999, 3, True), (2048, 130, 8, False),
                                            (512, 37, 2, True), (5632, 41, 13, False), (16384, 9, 7, False)])
def test_expert_gate_up_rows_iq3_s_bit_exact(dev, oracle, n, rows, nt, m128):
    """As the IQ3_XXS test, with IQ3_S rows (9-bit indices, plain sign bits, a scale per 32 values)."""
    g = synth.rng(37)
    act = ops.quantize_q8_k(to_dev(synth.normal(g, (nt, n), 1.0), dev))
    if m128:
        a = act.cpu().numpy().reshape(nt, -1, 292)
        codes = a[:, :, 4:260]
        codes[g.integers(0, 7, size=codes.shape) == 0] = 0x80
        act = to_dev(a.reshape(nt, -1), dev)
    d_hi = 3e-4 * (2560 / n) ** 0.5
    gate, up = synth.iq3_s_table(g, rows, n, d_hi / 15, d_hi), synth.iq3_s_table(g, rows, n, d_hi / 15, d_hi)
    r0, r1 = 2, rows - 1
    out = torch.full((nt, rows), float("nan"), dtype=torch.float32, device=dev)
    gu = torch.zeros((2, nt, rows), dtype=torch.float32, device=dev) if nt <= 8 else None
    ops.expert_gate_up_rows("iq3_s", to_dev(gate, dev), to_dev(up, dev), act, n, r0=r0, r1=r1, out=out, gu=gu)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    want, wgu = oracle.expert_gu_rows("iq3_s", gate, up, act.cpu().numpy(), n, r0=r0, r1=r1, want_gu=True)
    assert np.array_equal(bits(got[:, r0:r1]), bits(want[:, r0:r1]))
    assert np.isnan(got[:, :r0]).all() and np.isnan(got[:, r1:]).all()
    if gu is not None:
        assert np.array_equal(bits(gu.cpu().numpy()[:, :, r0:r1]), bits(wgu[:, :, r0:r1]))
    assert np.abs(wgu[0][:, r0:r1]).std() > 0.3


@pytest.mark.parametrize("fmt", ["iq2_xxs", "iq2_xs", "iq2_s"])
def test_expert_gate_up_rows_iq2_equal_the_reference_avx2_kernel_on_golden(dev, fmt):
    """The reference's own iq_gu_rows outputs for the three IQ2 formats, also for a window holding -128 codes."""
    gold = np.load(os.path.join(GOLD, "gate_up_rows_iq2.npz"))
    gate, up = to_dev(gold[fmt + "_gate"], dev), to_dev(gold[fmt + "_up"], dev)
    for act, want in ((gold[fmt + "_act"], gold[fmt + "_ff"]), (gold[fmt + "_act_m128"], gold[fmt + "_ff_m128"])):
        got = ops.expert_gate_up_rows(fmt, gate, up, to_dev(act, dev), 2560)
        assert np.array_equal(bits(got.cpu().numpy()), bits(want))


@pytest.mark.parametrize("fmt", ["iq2_xxs", "iq2_xs", "iq2_s"])
@pytest.mark.parametrize("n,rows,nt,m128", [(2560, 320, 1, False), (2560, 999, 3, True), (2048, 130, 8, False),
                                            (512, 37, 2, True), (5632, 41, 13, False), (16384, 9, 7, False)])
def test_expert_gate_up_rows_iq2_bit_exact(dev, oracle, fmt, n, rows, nt, m128):
    """As the IQ3 tests, with IQ2 rows: eight-magnitude codebook entries, a scale per 16 or 32 values, both reduction
    orders.  Rows staged whole and in chunks, every row alignment, windows of several passes, -128 codes."""
    g = synth.rng(39)
    act = ops.quantize_q8_k(to_dev(synth.normal(g, (nt, n), 1.0), dev))
    if m128:
        a = act.cpu().numpy().reshape(nt, -1, 292)
        codes = a[:, :, 4:260]
        codes[g.integers(0, 7, size=codes.shape) == 0] = 0x80
        act = to_dev(a.reshape(nt, -1), dev)
    d_hi = 2.5e-4 * (2560 / n) ** 0.5
    gate, up = synth.iq2_table(fmt, g, rows, n, d_hi / 8, d_hi), synth.iq2_table(fmt, g, rows, n, d_hi / 8, d_hi)
    r0, r1 = 2, rows - 1
    out = torch.full((nt, rows), float("nan"), dtype=torch.float32, device=dev)
    gu = torch.zeros((2, nt, rows), dtype=torch.float32, device=dev) if nt <= 8 else None
    ops.expert_gate_up_rows(fmt, to_dev(gate, dev), to_dev(up, dev), act, n, r0=r0, r1=r1, out=out, gu=gu)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    want, wgu = oracle.expert_gu_rows(fmt, gate, up, act.cpu().numpy(), n, r0=r0, r1=r1, want_gu=True)
    assert np.array_equal(bits(got[:, r0:r1]), bits(want[:, r0:r1]))
    assert np.isnan(got[:, :r0]).all() and np.isnan(got[:, r1:]).all()
    if gu is not None:
        assert np.array_equal(bits(gu.cpu().numpy()[:, :, r0:r1]), bits(wgu[:, :, r0:r1]))
    assert np.abs(wgu[0][:, r0:r1]).std() > 0.1       # gates of order one: the GLU is exercised


@pytest.mark.parametrize("fmt", ["q4_k", "q5_k", "iq3_xxs", "iq3_s"])
def test_expert_ffn_for_a_decode_window_stage_by_stage(dev, oracle, fmt):
    """One routed expert for a window of three rows, every hand-over on the device: RMSNorm -> Q8_K -> gate / up mat-vec
    with the GLU (Q4_K, Q5_K or IQ3_XXS) -> Q8_1 -> down mat-vec (Q5_1).  Each stage is checked bit for bit against the
    oracle applied to the previous stage's device output, and the end against the all-CPU chain."""
    g = synth.rng(77)
    nt, d_model, d_ff = 3, 2560, 640
    x, w = synth.normal(g, (nt, d_model), 1.0), synth.norm_weight(g, d_model)
    table, d_lo, d_hi = {"q4_k": (synth.q4_k_table, 1e-5, 3e-4), "q5_k": (synth.q5_k_table, 1e-5, 1.5e-4),
                         "iq3_xxs": (synth.iq3_xxs_table, 5e-5, 4e-4), "iq3_s": (synth.iq3_s_table, 2e-5, 3e-4)}[fmt]
    gate, up = table(g, d_ff, d_model, d_lo, d_hi), table(g, d_ff, d_model, d_lo, d_hi)
    down = synth.q5_1_rows(g, d_model, d_ff)
    D = lambda a: to_dev(a, dev)  # noqa: E731
    normed = ops.rms_norm(D(x), D(w), 1e-6)
    q8k = ops.quantize_q8_k(normed)
    ff = ops.expert_gate_up_rows(fmt, D(gate), D(up), q8k, d_model)
    q81 = ops.quantize_q8_1(ff)
    out = ops.expert_down_rows("q5_1", D(down), q81, d_ff)
    torch.cuda.synchronize()
    H = lambda t: t.cpu().numpy()  # noqa: E731
    assert ulp_diff(H(normed), oracle.rms_norm(x, w, 1e-6)).max() <= 2
    assert np.array_equal(H(q8k).reshape(-1, 292), oracle.quantize_q8_k(H(normed)))
    assert np.array_equal(bits(H(ff)), bits(oracle.expert_gu_rows(fmt, gate, up, H(q8k), d_model)))
    assert np.array_equal(H(q81).reshape(-1), oracle.quantize_q8_1(H(ff)).reshape(-1))
    assert np.array_equal(bits(H(out)), bits(oracle.expert_down_rows("q5_1", down, H(q81).reshape(nt, -1), d_ff)))
    # the all-CPU chain (its RMSNorm sums in another order: the device result may sit an ulp away, and a code with it)
    c_norm = oracle.rms_norm(x, w, 1e-6)
    c_ff = oracle.expert_gu_rows(fmt, gate, up, oracle.quantize_q8_k(c_norm).reshape(nt, -1), d_model)
    c_out = oracle.expert_down_rows("q5_1", down, oracle.quantize_q8_1(c_ff).reshape(nt, -1), d_ff)
    assert np.abs(H(out) - c_out).max() <= 1e-3 * np.abs(c_out).max()


# ---- the consumer of the Q8_1 blocks: the experts' down mat-vec ---------------------------------------------------------

def test_expert_down_rows_equal_the_reference_avx2_kernel_on_golden(dev):
    gold = np.load(os.path.join(GOLD, "down_rows.npz"))
    for key in ("q5_1_640", "q5_1_64", "q8_0_640"):
        fmt, n = key.rsplit("_", 1)[0], int(key.rsplit("_", 1)[1])
        w, act, want = gold[key + "|w"], gold[key + "|act"], gold[key + "|out"]
        got = ops.expert_down_rows(fmt, to_dev(w, dev), to_dev(act, dev), n).cpu().numpy()
        assert np.array_equal(bits(got), bits(want)), key


@pytest.mark.parametrize("n,rows,nt", [(640, 2560, 1), (640, 2560, 3), (640, 1000, 8), (512, 333, 5), (32, 40, 2),
                                       (2048, 129, 13)])
def test_expert_down_rows_bit_exact(dev, oracle, n, rows, nt):
    """SwiGLU's own Q8_1 output as the activations (the path's real hand-over), Q5_1 weights: every bit of the oracle's
    lane-for-lane restatement; rows outside [r0, r1) stay untouched."""
    g = synth.rng(31)
    gate, up = synth.normal(g, (nt, n), 0.5), synth.normal(g, (nt, n), 0.5)
    act = ops.swiglu_q8_1(to_dev(gate, dev), to_dev(up, dev))
    assert np.array_equal(act.cpu().numpy(), oracle.swiglu_q8_1(gate, up))
    w = synth.q5_1_rows(g, rows, n)
    r0, r1 = 5, rows - 3
    out = torch.full((nt, rows), float("nan"), dtype=torch.float32, device=dev)
    ops.expert_down_rows_q5_1(to_dev(w, dev), act, n, r0=r0, r1=r1, out=out)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    want = oracle.expert_down_rows("q5_1", w, act.cpu().numpy(), n, r0=r0, r1=r1)
    assert np.array_equal(bits(got[:, r0:r1]), bits(want[:, r0:r1]))
    assert np.isnan(got[:, :r0]).all() and np.isnan(got[:, r1:]).all()


@pytest.mark.parametrize("n,rows,nt", [(640, 2560, 1), (640, 777, 5), (128, 40, 2), (2048, 129, 11)])
def test_expert_down_rows_q8_0_bit_exact(dev, oracle, n, rows, nt):
    """Q8_0 weights against the Q8_0 blocks fnb_quantize_q8_0 writes."""
    g = synth.rng(32)
    x = synth.normal(g, (nt, n), 2.0)
    act = ops.quantize_q8_0(to_dev(x, dev))
    assert np.array_equal(act.cpu().numpy().reshape(-1), oracle.quantize_q8_0(x).reshape(-1))
    w = synth.q8_0_table(g, rows, n)
    got = ops.expert_down_rows("q8_0", to_dev(w, dev), act, n).cpu().numpy()
    want = oracle.expert_down_rows("q8_0", w, act.cpu().numpy().reshape(nt, -1), n)
    assert np.array_equal(bits(got), bits(want))


def test_expert_down_rows_iq4_nl_equal_the_reference_avx2_kernel_on_golden(dev):
    gold = np.load(os.path.join(GOLD, "down_rows_iq4_nl.npz"))
    for key in sorted({k.split("|")[0] for k in gold.files}):
        n = int(key.rsplit("_", 1)[1])
        got = ops.expert_down_rows("iq4_nl", to_dev(gold[key + "|w"], dev), to_dev(gold[key + "|act"], dev), n).cpu().numpy()
        assert np.array_equal(bits(got), bits(gold[key + "|out"])), key


@pytest.mark.parametrize("n,rows,nt,raw", [(640, 2560, 1, False), (640, 777, 5, False), (64, 40, 2, True), (2048, 129, 11, False),
                                           (320, 1001, 3, True), (8192, 21, 8, False)])
def test_expert_down_rows_iq4_nl_bit_exact(dev, oracle, n, rows, nt, raw):
    """IQ4_NL weights against Q8_0 blocks: the ones fnb_quantize_q8_0 writes, or (raw) random blocks with -128 codes
    among them; rows outside [r0, r1) stay untouched; every row offset within 16 bytes (320 columns: 180-byte rows)."""
    g = synth.rng(36)
    if raw:
        act = to_dev(synth.q8_0_table(g, nt, n), dev)
    else:
        act = ops.quantize_q8_0(to_dev(synth.normal(g, (nt, n), 2.0), dev)).reshape(nt, -1)
    w = synth.iq4_nl_rows(g, rows, n)
    r0, r1 = 3, rows - 2
    out = torch.full((nt, rows), float("nan"), dtype=torch.float32, device=dev)
    ops.expert_down_rows("iq4_nl", to_dev(w, dev), act, n, r0=r0, r1=r1, out=out)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    want = oracle.expert_down_rows("iq4_nl", w, act.cpu().numpy().reshape(nt, -1), n, r0=r0, r1=r1)
    assert np.array_equal(bits(got[:, r0:r1]), bits(want[:, r0:r1]))
    assert np.isnan(got[:, :r0]).all() and np.isnan(got[:, r1:]).all()


def test_planar_activation_and_q2_0_down_rows_equal_the_reference_on_golden(dev):
    gold = np.load(os.path.join(GOLD, "down_rows_q2_0.npz"))
    codes, scales = ops.quantize_act_q(to_dev(gold["x"], dev))
    assert np.array_equal(codes.cpu().numpy(), gold["codes"]) and np.array_equal(bits(scales.cpu().numpy()), bits(gold["scales"]))
    got = ops.expert_down_rows_q2_0(to_dev(gold["w"], dev), codes, scales, 640).cpu().numpy()
    assert np.array_equal(bits(got), bits(gold["out"]))


@pytest.mark.parametrize("n,rows,nt", [(640, 2560, 1), (640, 777, 5), (128, 40, 2), (2048, 129, 11), (384, 1001, 3),
                                       (8192, 21, 8)])
def test_q2_0_down_rows_bit_exact(dev, oracle, n, rows, nt):
    """Planar activation on the device (codes and scales equal the oracle's), Q2_0 rows against it; rows outside
    [r0, r1) stay untouched."""
    g = synth.rng(38)
    x = synth.normal(g, (nt, n), 2.0)
    x[0, :32] = 0.0
    codes, scales = ops.quantize_act_q(to_dev(x, dev))
    wq, ws = oracle.quantize_act_q(x)
    assert np.array_equal(codes.cpu().numpy(), wq) and np.array_equal(bits(scales.cpu().numpy()), bits(ws))
    w = synth.q2_0_rows(g, rows, n)
    r0, r1 = 3, rows - 2
    out = torch.full((nt, rows), float("nan"), dtype=torch.float32, device=dev)
    ops.expert_down_rows_q2_0(to_dev(w, dev), codes, scales, n, r0=r0, r1=r1, out=out)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    want = oracle.expert_down_rows_q2_0(w, n, wq, ws, r0=r0, r1=r1)
    assert np.array_equal(bits(got[:, r0:r1]), bits(want[:, r0:r1]))
    assert np.isnan(got[:, :r0]).all() and np.isnan(got[:, r1:]).all()


def test_quantize_act_q_ragged_grid(dev, oracle):
    """Row counts whose last warp is partly past the end."""
    g = synth.rng(39)
    for rows, n in ((1, 32), (3, 96), (7, 160), (1001, 64)):
        x = synth.normal(g, (rows, n), 1.0)
        codes, scales = ops.quantize_act_q(to_dev(x, dev))
        wq, ws = oracle.quantize_act_q(x)
        assert np.array_equal(codes.cpu().numpy(), wq) and np.array_equal(bits(scales.cpu().numpy()), bits(ws)), (rows, n)


def test_expert_ffn_in_the_iq_formats_stage_by_stage(dev, oracle):
    """The IQ-format expert for a window of three rows, every hand-over on the device: RMSNorm -> Q8_K -> IQ3_XXS gate / up
    with the GLU -> Q8_0 -> IQ4_NL down; each stage bit for bit against the oracle on the previous stage's device output."""
    g = synth.rng(78)
    nt, d_model, d_ff = 3, 2560, 640
    x, w = synth.normal(g, (nt, d_model), 1.0), synth.norm_weight(g, d_model)
    gate, up = synth.iq3_xxs_table(g, d_ff, d_model, 5e-5, 4e-4), synth.iq3_xxs_table(g, d_ff, d_model, 5e-5, 4e-4)
    down = synth.iq4_nl_rows(g, d_model, d_ff)
    D = lambda a: to_dev(a, dev)  # noqa: E731
    H = lambda t: t.cpu().numpy()  # noqa: E731
    q8k = ops.quantize_q8_k(ops.rms_norm(D(x), D(w), 1e-6))
    ff = ops.expert_gate_up_rows("iq3_xxs", D(gate), D(up), q8k, d_model)
    q80 = ops.quantize_q8_0(ff).reshape(nt, -1)
    out = ops.expert_down_rows("iq4_nl", D(down), q80, d_ff)
    torch.cuda.synchronize()
    assert np.array_equal(bits(H(ff)), bits(oracle.expert_gu_rows("iq3_xxs", gate, up, H(q8k), d_model)))
    assert np.array_equal(H(q80).reshape(-1), oracle.quantize_q8_0(H(ff)).reshape(-1))
    assert np.array_equal(bits(H(out)), bits(oracle.expert_down_rows("iq4_nl", down, H(q80), d_ff)))
    assert np.abs(H(out)).max() > 1e-3


# ---- get_rows ----------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("fmt,cols,vocab,rows", [
    ("q4_k", 2048, 1000, 777), ("iq3_xxs", 2048, 1000, 777), ("q8_0", 2048, 500, 300),
    ("q4_k", 256, 64, 1), ("q4_k", 4096, 64, 7), ("q4_k", 2560, 64, 33), ("iq3_xxs", 4096, 64, 33),
    ("iq3_xxs", 256, 64, 9), ("iq3_xxs", 768, 64, 5),
    ("q8_0", 1280, 64, 5), ("q8_0", 32, 64, 9),
])
def test_get_rows_bit_exact_and_bad_ids(dev, oracle, fmt, cols, vocab, rows):
    g = synth.rng(4)
    table = {"q4_k": synth.q4_k_table, "iq3_xxs": synth.iq3_xxs_table, "q8_0": synth.q8_0_table}[fmt](g, vocab, cols)
    ids = g.integers(0, vocab, rows).astype(np.int32)
    if rows >= 5:
        ids[1], ids[rows - 2] = -1, vocab        # out of range on both sides
    out = Guarded((rows, cols), torch.float32, dev)
    err = ops.new_err(dev)
    ops.get_rows(fmt, to_dev(table, dev), to_dev(ids, dev), cols, out=out.live, err=err)
    torch.cuda.synchronize()
    if fmt == "q8_0":
        want = np.zeros((rows, cols), np.float32)
        want.view(np.uint8)[:] = POISON
        werr = 0
        for t, i in enumerate(ids):
            if 0 <= i < vocab:
                want[t] = oracle.dequantize_q8_0(table[i])
            else:
                werr = oracle.ERR_TOKEN
    else:
        want = np.zeros((rows, cols), np.float32)
        want.view(np.uint8)[:] = POISON
        want, werr = oracle.get_rows(fmt, table, vocab, ids, cols, want)
    out.check_guards()
    assert int(err.item()) == werr
    assert np.array_equal(bits(out.numpy()), bits(want))


@pytest.mark.parametrize("fmt", ["q4_k", "iq3_xxs"])
def test_get_rows_many_rows_per_warp_with_bad_ids(dev, oracle, fmt):
    """More rows than the grid has warps (each warp decodes several rows, fetching one ahead), bad ids sprinkled in:
    every good row equals the oracle's decode of its table row, every bad row stays untouched."""
    vocab, cols, rows = 1024, 2048, 150001
    g = synth.rng(11)
    table = {"q4_k": synth.q4_k_table, "iq3_xxs": synth.iq3_xxs_table}[fmt](g, vocab, cols)
    deq = oracle.dequantize_q4_k if fmt == "q4_k" else oracle.dequantize_iq3_xxs
    decoded = to_dev(deq(table).reshape(vocab, cols).view(np.int32), dev)
    ids = g.integers(0, vocab, rows).astype(np.int32)
    bad = np.arange(7, rows, 1001)
    ids[bad[::2]], ids[bad[1::2]] = -3, vocab + 5
    ids[-1] = vocab                                             # the last row of the last warp too
    ids_d = to_dev(ids, dev)
    out = torch.full((rows, cols), 0x5a5a5a5a, dtype=torch.int32, device=dev)
    err = ops.new_err(dev)
    ops.get_rows(fmt, to_dev(table, dev), ids_d, cols, out=out.view(torch.float32), err=err)
    torch.cuda.synchronize()
    assert int(err.item()) == oracle.ERR_TOKEN
    ok = (ids_d >= 0) & (ids_d < vocab)
    assert torch.equal(out[ok], decoded[ids_d[ok].long()])
    assert bool((out[~ok] == 0x5a5a5a5a).all())


def test_get_rows_matches_reference_golden_decode(dev):
    """Blocks generated by the reference's fn::quant::synth_blocks and decoded by its dequantize_row_* (golden)."""
    gold = np.load(os.path.join(GOLD, "decode.npz"))
    for fmt, bv, per_row in (("q4_k", 256, 8), ("iq3_xxs", 256, 8), ("q8_0", 32, 8)):
        blocks, values = gold[fmt + "_blocks"], gold[fmt + "_values"]
        n_rows = blocks.shape[0] // per_row
        table = blocks.reshape(n_rows, -1)
        ids = np.arange(n_rows - 1, -1, -1).astype(np.int32)
        got = ops.get_rows(fmt, to_dev(table, dev), to_dev(ids, dev), per_row * bv).cpu().numpy()
        want = values.reshape(n_rows, per_row * bv)[ids]
        assert np.array_equal(bits(got), bits(want)), fmt


# ---- the chain, and graph replay -----------------------------------------------------------------------------------

def test_chain_matches_oracle_and_replays_in_a_graph(dev, oracle):
    from fnfl_v100_b200 import ChainConfig, PrefillChain
    cfg = ChainConfig(tokens=96, n_vocab=512, cache_slots=1024, depth=700, top_k=10)
    ch = PrefillChain(cfg, dev)
    ch.step()
    torch.cuda.synchronize()
    H = lambda t: t.cpu().numpy()  # noqa: E731
    hidden, err = oracle.get_rows("q4_k", H(ch.table), cfg.n_vocab, H(ch.ids), cfg.hidden)
    assert err == 0 and int(ch.err.item()) == 0
    assert np.array_equal(bits(H(ch.hidden)), bits(hidden))
    assert ulp_diff(H(ch.normed_attn), oracle.rms_norm(hidden, H(ch.w_attn), cfg.eps)).max() <= 2
    assert ulp_diff(H(ch.normed_ffn), oracle.rms_norm(hidden, H(ch.w_ffn), cfg.eps)).max() <= 2
    kc = np.zeros((cfg.cache_slots, cfg.n_kv_heads, 272), np.uint8)
    vc = np.zeros_like(kc)
    q_out, _, werr = oracle.rope_kv_append(H(ch.q), H(ch.k), H(ch.v), H(ch.pos), n_rot=cfg.n_rot,
                                           theta_scale=ch.theta_scale, k_cache=kc, v_cache=vc,
                                           cache_slots=cfg.cache_slots, q_norm_w=H(ch.w_q), k_norm_w=H(ch.w_k))
    assert werr == 0
    assert ulp_diff(H(ch.q_out), q_out).max() <= 2
    assert np.array_equal(H(ch.k_cache), kc) and np.array_equal(H(ch.v_cache), vc)
    assert np.array_equal(H(ch.act), oracle.swiglu_q8_1(H(ch.gate), H(ch.up)))
    # one graph replay over poisoned outputs reproduces the same bytes
    snap = [H(t).copy() for t in (ch.hidden, ch.normed_attn, ch.q_out, ch.k_cache, ch.act)]
    graph = ch.capture()
    for t in (ch.hidden, ch.normed_attn, ch.q_out, ch.act):
        t.view(torch.uint8).fill_(POISON)
    graph.replay()
    torch.cuda.synchronize()
    for a, t in zip(snap, (ch.hidden, ch.normed_attn, ch.q_out, ch.k_cache, ch.act)):
        assert np.array_equal(a.view(np.uint8), H(t).view(np.uint8))


def test_first_calls_can_be_captured_after_prepare_device(dev, oracle):
    """In a fresh process: prepare_device, then the very first call of a pipeline kernel happens inside a stream capture
    (no launcher may then do anything but launch) and the replayed graph gives the oracle's bytes."""
    import subprocess
    import sys
    import textwrap
    code = textwrap.dedent("""
        import numpy as np, torch
        from fnfl_v100_b200 import ops, synth
        from oracle import oracle as O
        dev = torch.device("cuda:0")
        g = synth.rng(3)
        gate, up = synth.normal(g, (64, 512), 0.5), synth.normal(g, (64, 512), 0.5)
        x, w = synth.normal(g, (9, 2048)), synth.norm_weight(g, 2048)
        dg, du, dx, dw = (torch.from_numpy(a).to(dev) for a in (gate, up, x, w))
        out = torch.empty((64, 16 * 36), dtype=torch.uint8, device=dev)
        # the experts' kernels that raise their shared-memory limit: IQ3_XXS gate / up, IQ4_NL and Q2_0 down
        n, ff_rows = 2560, 24
        wg, wu = synth.iq3_xxs_table(g, ff_rows, n, 5e-5, 4e-4), synth.iq3_xxs_table(g, ff_rows, n, 5e-5, 4e-4)
        q8k = O.quantize_q8_k(synth.normal(g, (2, n), 1.0)).reshape(2, -1)
        w4, a80 = synth.iq4_nl_rows(g, 40, 640), O.quantize_q8_0(synth.normal(g, (2, 640), 2.0)).reshape(2, -1)
        w2 = synth.q2_0_rows(g, 40, 640)
        qc, qs = O.quantize_act_q(synth.normal(g, (2, 640), 2.0))
        D = lambda a: torch.from_numpy(a).to(dev)
        dwg, dwu, dq8k, dw4, da80, dw2, dqc, dqs = (D(a) for a in (wg, wu, q8k, w4, a80, w2, qc, qs))
        ff = torch.zeros((2, ff_rows), dtype=torch.float32, device=dev)
        o4 = torch.zeros((2, 40), dtype=torch.float32, device=dev)
        o2 = torch.zeros((2, 40), dtype=torch.float32, device=dev)
        ops.prepare_device()
        torch.cuda.synchronize()
        s = torch.cuda.Stream(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(s):
            with torch.cuda.graph(graph, stream=s):
                ops.swiglu_q8_1(dg, du, out=out)          # first call of this kernel in the process
                blocks = ops.rms_norm_quant(dx, dw, 1e-6, "q8_1")
                ops.expert_gate_up_rows("iq3_xxs", dwg, dwu, dq8k, n, out=ff)
                ops.expert_down_rows("iq4_nl", dw4, da80, 640, out=o4)
                ops.expert_down_rows_q2_0(dw2, dqc, dqs, 640, out=o2)
        graph.replay()
        torch.cuda.synchronize()
        bits = lambda a: np.ascontiguousarray(a).view(np.uint32)
        assert np.array_equal(bits(ff.cpu().numpy()), bits(O.expert_gu_rows("iq3_xxs", wg, wu, q8k, n)))
        assert np.array_equal(bits(o4.cpu().numpy()), bits(O.expert_down_rows("iq4_nl", w4, a80, 640)))
        assert np.array_equal(bits(o2.cpu().numpy()), bits(O.expert_down_rows_q2_0(w2, 640, qc, qs)))
        want = O.swiglu_q8_1(gate, up)
        assert np.array_equal(out.cpu().numpy().reshape(-1), want.reshape(-1))
        again = ops.rms_norm_quant(dx, dw, 1e-6, "q8_1")       # the same launch outside a capture
        assert torch.equal(blocks, again) and bool(blocks.any())
        print("captured-first-call ok")
    """)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=root, timeout=600)
    assert r.returncode == 0 and "captured-first-call ok" in r.stdout, r.stdout + r.stderr


def test_glu_fast_path_equals_generic_path_on_its_whole_domain(dev, selftest_lib):
    """Every gate of the fast domain, |gate| in [2^-40, 64) (2 x 46 x 2^23 of them; everything before the product with
    `up` depends on the gate alone), each with a pseudo-random `up`: the eight-operation expf and the shortened
    written-out division must give the same bits as the generic path (expf operation for operation, __fdiv_rn)."""
    import ctypes as C
    bad = torch.zeros(1, dtype=torch.int64, device=dev)
    st = selftest_lib.fnbt_selftest_glu_math(0, 12345, C.c_void_p(bad.data_ptr()),
                                          C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0
    torch.cuda.synchronize()
    assert int(bad.item()) == 0


def test_q8_rule_divisions_written_out_equal_ieee_division_for_every_amax(dev, selftest_lib):
    """Every non-negative float as a block's amax (and infinity, and NaNs): d and id of the Q8_0 / Q8_1 rule as the
    kernels compute them are the bits of amax / 127 and 1 / d."""
    import ctypes as C
    bad = torch.zeros(1, dtype=torch.int64, device=dev)
    st = selftest_lib.fnbt_selftest_q8_rule(C.c_void_p(bad.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0
    torch.cuda.synchronize()
    assert int(bad.item()) == 0


def test_fused_expf_equals_the_definition_for_every_float(dev, selftest_lib):
    """All 2 x 0x42b00000 floats |x| < 88: the 8-operation evaluation rounds to the same float as the 12-operation one."""
    import ctypes as C
    bad = torch.zeros(1, dtype=torch.int64, device=dev)
    st = selftest_lib.fnbt_selftest_expf(C.c_void_p(bad.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0
    torch.cuda.synchronize()
    assert int(bad.item()) == 0


def test_kv8_written_out_division_equals_ieee_division(dev, selftest_lib):
    """Every positive finite FP16 scale x 2^27 pseudo-random values (half on exact half steps): same codes as __fdiv_rn."""
    import ctypes as C
    bad = torch.zeros(1, dtype=torch.int64, device=dev)
    st = selftest_lib.fnbt_selftest_kv8_math(1 << 27, 777, C.c_void_p(bad.data_ptr()),
                                          C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0
    torch.cuda.synchronize()
    assert int(bad.item()) == 0


@pytest.mark.parametrize("rows,cols,fmt", [(512, 2048, "q8_1"), (7, 2048, "q8_0"), (33, 2560, "q8_1"), (5, 4096, "q8_1"),
                                           (9, 1024, "act"), (3, 320, "act"), (1, 32, "q8_1"), (130, 2048, "act")])
def test_rms_norm_fused_with_requantisation(dev, oracle, rows, cols, fmt):
    g = synth.rng(1)
    x = synth.normal(g, (rows, cols), 2.0)
    w = synth.norm_weight(g, cols)
    y = Guarded((rows, cols), torch.float32, dev)
    res = ops.rms_norm_quant(to_dev(x, dev), to_dev(w, dev), 1e-6, fmt, out_f32=y.live)
    torch.cuda.synchronize()
    y.check_guards()
    got_y = y.numpy()
    want_y = oracle.rms_norm(x, w, 1e-6)
    assert ulp_diff(got_y, want_y).max() <= 2
    # blocks are the CPU quantiser of the kernel's own F32 row, and equal the all-CPU result end to end
    if fmt == "act":
        codes, scales = (t.cpu().numpy() for t in res)
        wc, ws = oracle.act_quantize(got_y)
        assert np.array_equal(codes, wc) and np.array_equal(bits(scales), bits(ws))
        ec, es = oracle.act_quantize(want_y)
        assert int((codes != ec).sum()) == 0 and np.array_equal(bits(scales), bits(es))
    else:
        q = oracle.quantize_q8_1 if fmt == "q8_1" else oracle.quantize_q8_0
        got = res.cpu().numpy().reshape(-1)
        assert np.array_equal(got, q(got_y))
        assert int((got != q(want_y)).sum()) == 0
    # same bytes without the optional F32 output
    res2 = ops.rms_norm_quant(to_dev(x, dev), to_dev(w, dev), 1e-6, fmt)
    a = res2[0] if fmt == "act" else res2
    b = res[0] if fmt == "act" else res
    assert torch.equal(a, b)


@pytest.mark.parametrize("fmt,rows", [("iq3_s", 1), ("iq3_s", 7), ("iq3_s", 1536), ("q8_0", 33)])
def test_reference_embedding_layout_two_cards(dev, oracle, fmt, rows):
    """The reference's pe-test (fn/kernels/ple/ple_prompt_test.cpp:27-147) restated: two card tables of 1280 features,
    every output row of own, full and the four streams on both cards must be memcmp-equal to the CPU decode; then the
    join of the peer half, a supplied-row overwrite, and a bad id that leaves its rows unwritten."""
    n_own, n_full, n_streams, vocab = 1280, 2560, 4, 4096
    gold = np.load(os.path.join(GOLD, "decode.npz"))
    g = synth.rng(0x454d42)
    bb, bv = (110, 256) if fmt == "iq3_s" else (34, 32)
    pool = gold[fmt + "_blocks"]                                      # blocks made by the reference's synth_blocks
    tables = [pool[g.integers(0, len(pool), (vocab, n_own // bv))].reshape(vocab, -1).copy() for _ in range(2)]
    deq = oracle.dequantize_iq3_s if fmt == "iq3_s" else oracle.dequantize_q8_0
    tok = g.integers(0, vocab, rows).astype(np.int32)
    if rows >= 7:
        tok[3] = vocab                                                 # out of range
    good = (tok >= 0) & (tok < vocab)
    want_half = [np.where(good[:, None], deq(t[np.clip(tok, 0, vocab - 1)]).reshape(rows, n_own), np.nan).astype(np.float32)
                 for t in tables]
    dtok = to_dev(tok, dev)
    outs = []
    for card in (0, 1):
        own = Guarded((rows, n_own), torch.float32, dev)
        full = Guarded((rows, n_full), torch.float32, dev)
        streams = Guarded((rows, n_streams, n_full), torch.float32, dev)
        err = ops.new_err(dev)
        ops.embed_rows(fmt, to_dev(tables[card], dev), dtok, n_own, own=own.live, full=full.live, streams=streams.live,
                       col0=card * n_own, err=err)
        torch.cuda.synchronize()
        assert int(err.item()) == (0 if good.all() else ops.ERR_TOKEN)
        outs.append((own, full, streams))
    poison = np.frombuffer(bytes([POISON] * 4), np.float32)[0]
    for card in (0, 1):
        own, full, streams = outs[card]
        peer = outs[1 - card][0]
        ops.embed_join(fmt, to_dev(tables[card], dev), dtok, n_own, peer.live, (1 - card) * n_own, full=full.live,
                       streams=streams.live)
        torch.cuda.synchronize()
        for o in (own, full, streams):
            o.check_guards()
        want_full = np.full((rows, n_full), poison, np.float32)
        for c in (0, 1):
            want_full[good, c * n_own:(c + 1) * n_own] = want_half[c][good]
        assert np.array_equal(bits(own.numpy())[good], bits(want_half[card])[good])
        assert (bits(own.numpy())[~good] == bits(np.array([poison]))[0]).all()       # unwritten
        assert np.array_equal(bits(full.numpy()), bits(want_full))
        for s in range(n_streams):
            assert np.array_equal(bits(streams.numpy()[:, s]), bits(want_full))
    if rows >= 7:   # supplied rows (an image's) over rows 2..4 of card 0, the bad row included
        own, full, streams = outs[0]
        src = synth.normal(g, (3, n_own))
        ops.embed_supply(fmt, to_dev(tables[0], dev), dtok, n_own, to_dev(src, dev), 2, own=own.live, full=full.live,
                         streams=streams.live, col0=0)
        torch.cuda.synchronize()
        assert np.array_equal(bits(own.numpy()[2:5]), bits(src))
        assert np.array_equal(bits(full.numpy()[2:5, :n_own]), bits(src))
        assert np.array_equal(bits(streams.numpy()[2:5, 3, :n_own]), bits(src))


@pytest.mark.parametrize("fmt", ["q4_k", "iq3_xxs"])
@pytest.mark.parametrize("rows,cols", [(1, 2048), (37, 2048), (3000, 2048), (65, 1024), (40, 4096)])
def test_get_rows_rms_norm_is_get_rows_then_rms_norm(dev, oracle, fmt, rows, cols):
    """The fused launch against the oracle (rows bit for bit, normalised rows within 2 units in the last place: the
    double sum runs in another order) and against the two stand-alone kernels; a refused id leaves both rows unwritten
    at the fused width."""
    g = synth.rng(77 + rows)
    n_vocab = 5000
    table = {"q4_k": synth.q4_k_table, "iq3_xxs": synth.iq3_xxs_table}[fmt](g, n_vocab, cols)
    ids = g.integers(0, n_vocab, rows).astype(np.int32)
    w = synth.norm_weight(g, cols)
    eps = 1e-6
    d_table, d_ids, d_w = (torch.from_numpy(a).to(dev) for a in (table, ids, w))
    err = ops.new_err(dev)
    out, normed = ops.get_rows_rms_norm(fmt, d_table, d_ids, cols, d_w, eps, err=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    want_rows, _ = oracle.get_rows(fmt, table, n_vocab, ids, cols)
    want_norm = oracle.rms_norm(want_rows, w, eps)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want_rows.view(np.uint32))
    got = normed.cpu().numpy()
    assert np.abs(got.view(np.int32).astype(np.int64) - want_norm.view(np.int32)).max() <= 2
    alone_rows = ops.get_rows(fmt, d_table, d_ids, cols)
    alone_norm = ops.rms_norm(alone_rows, d_w, eps)
    assert torch.equal(out, alone_rows)
    differing = int((normed.view(torch.int32) != alone_norm.view(torch.int32)).sum())
    print("get_rows_rms_norm %d x %d: %d of %d normalised values differ from the stand-alone kernel's" % (rows, cols, differing, normed.numel()))
    assert differing <= 1e-4 * normed.numel()
    if cols == 2048 and rows >= 3:
        bad = ids.copy()
        bad[1] = n_vocab
        out2 = torch.full((rows, cols), 7.0, dtype=torch.float32, device=dev)
        norm2 = torch.full((rows, cols), 9.0, dtype=torch.float32, device=dev)
        ops.get_rows_rms_norm(fmt, d_table, torch.from_numpy(bad).to(dev), cols, d_w, eps, out=out2, normed=norm2, err=err)
        torch.cuda.synchronize()
        assert int(err.item()) == ops.ERR_TOKEN
        assert bool((out2[1] == 7.0).all()) and bool((norm2[1] == 9.0).all())
        assert torch.equal(out2[0], out[0]) and torch.equal(norm2[2], normed[2])


# ---- the four launches of the path at shapes drawn at random ------------------------------------------------------------

@pytest.mark.parametrize("seed", range(16))
def test_hot_path_random_shapes(dev, oracle, seed):
    """Each seed draws its own shape for every kernel of the path (ragged row counts, widths from one block up, head
    counts and rotary widths that are no power of two) and holds it to the same bar as the fixed cases above."""
    g = synth.rng(1000 + seed)
    D = lambda a: None if a is None else to_dev(a, dev)  # noqa: E731

    # RMSNorm
    rows, cols = int(g.integers(1, 700)), 4 * int(g.integers(1, 1200))
    x, w = synth.normal(g, (rows, cols)), synth.norm_weight(g, cols)
    out = Guarded((rows, cols), torch.float32, dev)
    ops.rms_norm(D(x), D(w), 1e-6, out=out.live)
    torch.cuda.synchronize()
    out.check_guards()
    d = ulp_diff(out.numpy(), oracle.rms_norm(x, w, 1e-6))
    assert d.max() <= 2, f"rms_norm {rows} x {cols}: max ulp {d.max()}"

    # SwiGLU + Q8_1
    rows, cols = int(g.integers(1, 900)), 32 * int(g.integers(1, 40))
    gate, up = synth.normal(g, (rows, cols), 2.0), synth.normal(g, (rows, cols), 0.5)
    q = Guarded((rows, cols // 32 * 36), torch.uint8, dev)
    f32 = Guarded((rows, cols), torch.float32, dev)
    ops.swiglu_q8_1(D(gate), D(up), out=q.live, out_f32=f32.live)
    torch.cuda.synchronize()
    q.check_guards()
    f32.check_guards()
    want, want_f32 = oracle.swiglu_q8_1(gate, up, want_f32=True)
    assert np.array_equal(bits(f32.numpy()), bits(want_f32)), f"swiglu {rows} x {cols}"
    assert np.array_equal(q.numpy(), want), f"swiglu {rows} x {cols}"

    # head norm + RoPE + Q8_0 append
    hd = int(g.choice([64, 128, 256]))
    rows, nq, nkv = int(g.integers(1, 300)), int(g.integers(1, 21)), int(g.integers(1, 5))
    n_rot = 2 * (hd // 32) * int(g.integers(0, 16 + 1))
    norm = bool(g.integers(0, 2))
    qx, kx, vx, wq, wk = _rope_case(g, rows, nq, nkv, hd, norm)
    slots_total = 1024
    pos = synth.positions(g, rows)
    slot = (g.permutation(slots_total - 8)[:rows] + 4).astype(np.int32)
    ts = oracle.theta_scale(1e7, max(n_rot, 2))
    cell = hd // 32 * 34
    kc = Guarded((slots_total, nkv, cell), torch.uint8, dev)
    vc = Guarded((slots_total, nkv, cell), torch.uint8, dev)
    qo = Guarded((rows, nq, hd), torch.float32, dev)
    err = ops.new_err(dev)
    ops.rope_neox_q8_0_append(D(qx), D(kx), D(vx), D(pos), n_rot=n_rot, theta_scale=ts, k_cache=kc.live, v_cache=vc.live,
                              slots=D(slot), q_norm_w=D(wq), k_norm_w=D(wk), q_out=qo.live, err=err)
    torch.cuda.synchronize()
    wkc = np.full((slots_total, nkv, cell), POISON, np.uint8)
    wvc = wkc.copy()
    want_q, _, werr = oracle.rope_kv_append(qx, kx, vx, pos, n_rot=n_rot, theta_scale=ts, k_cache=wkc, v_cache=wvc,
                                            cache_slots=slots_total, slots=slot, q_norm_w=wq, k_norm_w=wk)
    what = f"rope rows {rows} heads {nq}+{nkv} x {hd} n_rot {n_rot} norm {norm}"
    assert int(err.item()) == werr == 0, what
    for o in (kc, vc, qo):
        o.check_guards()
    if norm:
        assert ulp_diff(qo.numpy(), want_q).max() <= 2, what
    else:
        assert np.array_equal(bits(qo.numpy()), bits(want_q)), what
    assert np.array_equal(vc.numpy(), wvc), what
    assert int((kc.numpy() != wkc).sum()) == 0, what

    # get_rows, alone and with the norm
    for fmt in ("q4_k", "iq3_xxs"):
        rows, cols, vocab = int(g.integers(1, 500)), 256 * int(g.integers(1, 17)), int(g.integers(1, 300))
        table = {"q4_k": synth.q4_k_table, "iq3_xxs": synth.iq3_xxs_table}[fmt](g, vocab, cols)
        ids = g.integers(0, vocab, rows).astype(np.int32)
        w = synth.norm_weight(g, cols)
        out = Guarded((rows, cols), torch.float32, dev)
        ops.get_rows(fmt, D(table), D(ids), cols, out=out.live, err=err)
        torch.cuda.synchronize()
        out.check_guards()
        want_rows, werr = oracle.get_rows(fmt, table, vocab, ids, cols)
        what = f"get_rows {fmt} {rows} x {cols} of {vocab}"
        assert int(err.item()) == werr == 0, what
        assert np.array_equal(bits(out.numpy()), bits(want_rows)), what
        out2, normed = Guarded((rows, cols), torch.float32, dev), Guarded((rows, cols), torch.float32, dev)
        ops.get_rows_rms_norm(fmt, D(table), D(ids), cols, D(w), 1e-6, out=out2.live, normed=normed.live, err=err)
        torch.cuda.synchronize()
        out2.check_guards()
        normed.check_guards()
        assert np.array_equal(bits(out2.numpy()), bits(want_rows)), what
        assert ulp_diff(normed.numpy(), oracle.rms_norm(want_rows, w, 1e-6)).max() <= 2, what
