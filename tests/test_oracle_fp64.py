"""rms_norm, swiglu and rope have no CPU source in the reference tree; the oracle's restatements are held to
FP64 statements of the same formulas with the bounds the reference's own tests use
(fn/kernels/qsa/qa2_test.cpp:230-259, :508; fn/kernels/draft/draft_prompt_test.cpp:66-75;
fn/kernels/dense/dense_test.cpp:730-740)."""
import numpy as np

from fnfl_v100_b200 import synth


def test_rms_norm_against_fp64(oracle):
    g = synth.rng(1)
    x = synth.normal(g, (64, 2048))
    w = synth.norm_weight(g, 2048)
    y = oracle.rms_norm(x, w, 1e-6)
    x64 = x.astype(np.float64)
    ref = x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + 1e-6) * w.astype(np.float64)
    err = np.abs(y - ref).max(-1) / np.abs(ref).max(-1)
    assert err.max() <= 1e-6
    # three roundings (scale, x * scale, * w) on top of the FP64 value: a few ULP elementwise
    ulp = np.spacing(np.abs(ref).astype(np.float32))
    assert (np.abs(y - ref) <= 4 * ulp).all()


def test_rms_norm_no_weight_and_heads(oracle):
    g = synth.rng(1)
    x = synth.normal(g, (32, 256), 3.0)
    y = oracle.rms_norm(x, None, 1e-6)
    x64 = x.astype(np.float64)
    ref = x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + 1e-6)
    assert np.abs(y - ref).max() <= 1e-6 * np.abs(ref).max()


def test_swiglu_against_fp64_and_q8_1_of_own_output(oracle):
    g = synth.rng(3)
    gate, up = synth.normal(g, (40, 512), 0.5), synth.normal(g, (40, 512), 0.5)
    blocks, f32 = oracle.swiglu_q8_1(gate, up, want_f32=True)
    g64, u64 = gate.astype(np.float64), up.astype(np.float64)
    ref = g64 / (1 + np.exp(-g64)) * u64
    assert np.abs(f32 - ref).max() <= 1e-5 * np.abs(ref).max()          # the reference's GLU bound
    assert (np.abs(f32 - ref) <= 4 * np.spacing(np.abs(ref).astype(np.float32)) + 1e-45).all()
    assert np.array_equal(blocks.reshape(-1), oracle.quantize_q8_1(f32))   # codes are the quantiser of the F32 GLU


def _rope_fp64(x, w, pos, ts, n_rot, eps):
    x64 = x.astype(np.float64)
    y = x64 if w is None else x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + eps) * w.astype(np.float64)
    half = n_rot // 2
    th = np.empty((len(pos), half), np.float32)
    t = pos.astype(np.float32)
    for i in range(half):          # the F32 product chain
        th[:, i] = t
        t = (t * np.float32(ts)).astype(np.float32)
    c, s = np.cos(th.astype(np.float64))[:, None, :], np.sin(th.astype(np.float64))[:, None, :]
    out = y.copy()
    x0, x1 = y[..., :half], y[..., half:n_rot]
    out[..., :half] = x0 * c - x1 * s
    out[..., half:n_rot] = x0 * s + x1 * c
    return out, np.abs(x0 * c) + np.abs(x1 * s), np.abs(x0 * s) + np.abs(x1 * c)


def test_rope_kv_append_against_fp64(oracle):
    g = synth.rng(2)
    rows, nq, nkv, hd, n_rot, slots = 48, 16, 2, 256, 64, 4096
    q, k, v = synth.normal(g, (rows, nq, hd)), synth.normal(g, (rows, nkv, hd)), synth.normal(g, (rows, nkv, hd))
    pos = (200000 + np.arange(rows)).astype(np.int32)
    slot = np.arange(100, 100 + rows).astype(np.int32)
    wq, wk = synth.norm_weight(g, hd), synth.norm_weight(g, hd)
    ts = oracle.theta_scale(1e7, n_rot)
    kc = np.zeros((slots, nkv, 8 * 34), np.uint8)
    vc = np.zeros_like(kc)
    q_out, k_f32, err = oracle.rope_kv_append(q, k, v, pos, n_rot=n_rot, theta_scale=ts, k_cache=kc, v_cache=vc,
                                              cache_slots=slots, slots=slot, q_norm_w=wq, k_norm_w=wk,
                                              want_k_f32=True)
    assert err == 0
    for got, x, w in ((q_out, q, wq), (k_f32, k, wk)):
        ref, m0, m1 = _rope_fp64(x, w, pos, ts, n_rot, 1e-6)
        row_max = np.abs(ref).max(-1, keepdims=True)
        assert (np.abs(got - ref) <= 1e-6 * row_max).all()      # qa2-test's bound: 1e-6 of the row maximum
    # cells: K is the Q8_0 quantiser of the F32 k, V of the raw v; untouched slots stay zero
    want_k = oracle.quantize_q8_0(k_f32).reshape(rows, nkv, 272)
    want_v = oracle.quantize_q8_0(v).reshape(rows, nkv, 272)
    assert np.array_equal(kc[100:100 + rows], want_k) and np.array_equal(vc[100:100 + rows], want_v)
    assert not kc[:100].any() and not kc[100 + rows:].any()


def test_rope_bad_slot_sets_error_and_writes_nothing(oracle):
    g = synth.rng(2)
    q, k, v = synth.normal(g, (3, 2, 256)), synth.normal(g, (3, 1, 256)), synth.normal(g, (3, 1, 256))
    pos = np.array([5, 70, 6], np.int32)
    kc = np.zeros((64, 1, 272), np.uint8)
    vc = np.zeros_like(kc)
    q_out = np.full_like(q, 9.0)
    q_out, _, err = oracle.rope_kv_append(q, k, v, pos, n_rot=64, theta_scale=oracle.theta_scale(1e7, 64), k_cache=kc,
                                          v_cache=vc, cache_slots=64, q_out=q_out)
    assert err == oracle.ERR_SLOT
    assert (q_out[1] == 9.0).all() and kc[5].any() and kc[6].any() and kc.sum(axis=(1, 2)).astype(bool).sum() == 2
