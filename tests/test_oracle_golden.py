"""The CPU oracle against the golden vectors recorded from the reference's own CPU sources
(tests/golden/make_golden.py) and, where the reference build is present, against that build directly."""
import ctypes as C
import os

import numpy as np
import pytest

from fnfl_v100_b200 import synth

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def quant():
    return np.load(os.path.join(GOLD, "quant.npz"))


@pytest.fixture(scope="module")
def decode():
    return np.load(os.path.join(GOLD, "decode.npz"))


def test_q8_0_matches_reference_bytes(oracle, quant):
    got = oracle.quantize_q8_0(quant["x"]).reshape(-1, 34)
    assert np.array_equal(got, quant["q8_0"])


def test_q8_1_matches_reference_bytes(oracle, quant):
    got = oracle.quantize_q8_1(quant["x"]).reshape(-1, 36)
    assert np.array_equal(got, quant["q8_1"])


def test_act_format_matches_reference(oracle, quant):
    codes, scales = oracle.act_quantize(quant["x"])
    assert np.array_equal(codes, quant["act_codes"])
    assert np.array_equal(scales.reshape(-1, 2).view(np.uint32), quant["act_scales"].view(np.uint32))


def test_kv8_matches_reference(oracle, quant):
    codes, scales = oracle.kv8_quantize(quant["x"])
    assert np.array_equal(codes.reshape(-1, 64), quant["kv8_codes"])
    assert np.array_equal(scales, quant["kv8_scales"])


def test_kv8_decode_matches_reference(oracle, quant):
    """value = float(code) * f32(scale): bit for bit the reference's kv_q8_value over its stress rows."""
    got = oracle.kv8_dequantize(quant["kv8_codes"], quant["kv8_scales"])
    assert np.array_equal(got.view(np.uint32), quant["kv8_values"].reshape(-1).view(np.uint32))


@pytest.mark.parametrize("fmt", ["q4_k", "iq3_xxs", "q8_0", "iq3_s"])
def test_decoders_match_reference_bits(oracle, decode, fmt):
    fn = {"q4_k": oracle.dequantize_q4_k, "iq3_xxs": oracle.dequantize_iq3_xxs, "q8_0": oracle.dequantize_q8_0,
          "iq3_s": oracle.dequantize_iq3_s}[fmt]
    got = fn(decode[fmt + "_blocks"])
    assert np.array_equal(got.view(np.uint32), decode[fmt + "_values"].reshape(-1).view(np.uint32))


def test_q8_midpoints_round_half_away(oracle):
    # amax 127 -> d = 1, id = 1: x = k + 0.5 must round away from zero (roundf), not to even
    x = np.zeros(32, np.float32)
    x[:8] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, 127.0]
    b = oracle.quantize_q8_0(x)
    assert list(b[2:10].view(np.int8)) == [1, 2, 3, -1, -2, -3, 127, 127]
    assert b[:2].view(np.uint16)[0] == 0x3C00  # d = 1.0


def test_q8_1_sum_field(oracle):
    g = np.random.default_rng(3)
    x = g.standard_normal(32 * 50).astype(np.float32)
    b = oracle.quantize_q8_1(x).reshape(-1, 36)
    for blk, xs in zip(b, x.reshape(-1, 32)):
        d = np.float32(np.abs(xs).max()) / np.float32(127)
        s = np.float32(int(blk[4:].view(np.int8).astype(np.int32).sum())) * d
        assert blk[2:4].view(np.uint16)[0] == np.float32(s).astype(np.float16).view(np.uint16)


def test_get_rows_is_row_decode_and_flags_bad_ids(oracle, decode):
    blocks = decode["q4_k_blocks"]            # 96 blocks = 12 rows of 2048
    table = blocks.reshape(12, 8 * 144)
    ids = np.array([3, 0, 11, -1, 12, 7], np.int32)
    out = np.full((6, 2048), 7.0, np.float32)
    out, err = oracle.get_rows("q4_k", table, 12, ids, 2048, out)
    vals = decode["q4_k_values"].reshape(12, 2048)
    assert err == oracle.ERR_TOKEN
    for t, i in enumerate(ids):
        if 0 <= i < 12:
            assert np.array_equal(out[t], vals[i])
        else:
            assert np.all(out[t] == 7.0)      # unwritten


def test_f16_conversion_against_numpy(oracle):
    g = np.random.default_rng(5)
    x = np.concatenate([g.standard_normal(2000) * 10.0 ** g.uniform(-9, 6, 2000),
                        [0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001,
                         6.1e-5, 5.96e-8]]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(oracle.f32_to_f16_bits(x), want)
    h = np.arange(0, 0x7C00, 7, dtype=np.uint16)
    assert np.array_equal(oracle.f16_bits_to_f32(h), h.view(np.float16).astype(np.float32))
    assert oracle.lib().fnbo_f32_to_f16(float("nan")) & 0x7FFF == 0x7E00


@pytest.mark.skipif(not __import__("oracle.oracle", fromlist=["x"]).have_ref(), reason="reference build absent")
def test_oracle_equals_live_reference_build(oracle):
    """Wider than the fixtures: 20k random blocks through the reference library itself."""
    r = oracle.ref()
    g = np.random.default_rng(11)
    x = (g.standard_normal(32 * 20000) * 10.0 ** g.uniform(-5, 4, 32 * 20000)).astype(np.float32)
    a = oracle.quantize_q8_0(x)
    b = np.empty_like(a)
    r.quantize_row_q8_0_ref(oracle._p(x), oracle._p(b), C.c_int64(x.size))
    assert np.array_equal(a, b)
    a = oracle.quantize_q8_1(x)
    b = np.empty_like(a)
    r.quantize_row_q8_1_ref(oracle._p(x), oracle._p(b), C.c_int64(x.size))
    assert np.array_equal(a, b)
    from fnfl_v100_b200 import synth
    for fmt, mk, dq, fn in (("q4_k", synth.q4_k_table, oracle.dequantize_q4_k, r.dequantize_row_q4_K),
                            ("iq3_xxs", synth.iq3_xxs_table, oracle.dequantize_iq3_xxs, r.dequantize_row_iq3_xxs)):
        t = mk(synth.rng(4), 256, 2048)
        a = dq(t)
        b = np.empty_like(a)
        fn(oracle._p(t), oracle._p(b), C.c_int64(a.size))
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), fmt


def test_expert_down_rows_match_the_reference_avx2_kernel(oracle):
    """tests/golden/down_rows.npz: outputs of the reference's own kq_down_rows (compiled with its flags); the scalar
    restatement reproduces every bit, for Q5_1 x Q8_1 and Q8_0 x Q8_0, also on a sub-range of rows."""
    gold = np.load(os.path.join(GOLD, "down_rows.npz"))
    for key in sorted({k.split("|")[0] for k in gold.files}):
        fmt, n = key.rsplit("_", 1)[0], int(key.rsplit("_", 1)[1])
        w, act, want = gold[key + "|w"], gold[key + "|act"], gold[key + "|out"]
        got = oracle.expert_down_rows(fmt, w, act, n)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), key
        part = oracle.expert_down_rows(fmt, w, act, n, r0=3, r1=8)
        assert np.array_equal(part[:, 3:8].view(np.uint32), want[:, 3:8].view(np.uint32)) and not part[:, :3].any()


def test_expert_down_rows_iq4_nl_match_the_reference_avx2_kernel(oracle):
    """tests/golden/down_rows_iq4_nl.npz: outputs of the reference's own iq4nl_down_rows, one case with -128 codes."""
    gold = np.load(os.path.join(GOLD, "down_rows_iq4_nl.npz"))
    for key in sorted({k.split("|")[0] for k in gold.files}):
        n = int(key.rsplit("_", 1)[1])
        got = oracle.expert_down_rows("iq4_nl", gold[key + "|w"], gold[key + "|act"], n)
        assert np.array_equal(got.view(np.uint32), gold[key + "|out"].view(np.uint32)), key


def test_planar_activation_and_q2_0_down_rows_match_the_reference(oracle):
    """tests/golden/down_rows_q2_0.npz: codes and scales of the reference's quantize_act_q and outputs of its
    q2_down_rows; the restatements reproduce every bit, also on a sub-range of rows."""
    gold = np.load(os.path.join(GOLD, "down_rows_q2_0.npz"))
    q, s = oracle.quantize_act_q(gold["x"])
    assert np.array_equal(q, gold["codes"]) and np.array_equal(s.view(np.uint32), gold["scales"].view(np.uint32))
    out = oracle.expert_down_rows_q2_0(gold["w"], 640, q, s)
    assert np.array_equal(out.view(np.uint32), gold["out"].view(np.uint32))
    part = oracle.expert_down_rows_q2_0(gold["w"], 640, q, s, r0=3, r1=8)
    assert np.array_equal(part[:, 3:8].view(np.uint32), gold["out"][:, 3:8].view(np.uint32)) and not part[:, :3].any()


def test_q8_k_matches_ggml_and_the_reference_avx2_form(oracle):
    """tests/golden/q8_k.npz: blocks from ggml's quantize_row_q8_K_ref, equal to the reference's AVX2 quantize_q8_k."""
    gold = np.load(os.path.join(GOLD, "q8_k.npz"))
    assert np.array_equal(oracle.quantize_q8_k(gold["x"]), gold["blocks"])


def test_expert_gate_up_rows_q5_k_match_the_reference_avx2_kernel(oracle):
    """tests/golden/gate_up_rows_q5_k.npz: ff of the reference's own kq_gu_rows (fmt q5_k, GLU included)."""
    gold = np.load(os.path.join(GOLD, "gate_up_rows_q5_k.npz"))
    got = oracle.expert_gu_rows_q5_k(gold["gate"], gold["up"], gold["act"], 2560)
    assert np.array_equal(got.view(np.uint32), gold["ff"].view(np.uint32))


def test_expert_gate_up_rows_iq3_xxs_match_the_reference_avx2_kernel(oracle):
    """tests/golden/gate_up_rows_iq3_xxs.npz: ff of the reference's own iq_gu_rows (fmt iq3_xxs, GLU included), also for
    activations holding -128 codes, which its sign step leaves as they are; the restatement reproduces every bit."""
    gold = np.load(os.path.join(GOLD, "gate_up_rows_iq3_xxs.npz"))
    gate, up = gold["gate"], gold["up"]
    for act, want in ((gold["act"], gold["ff"]), (gold["act_m128"], gold["ff_m128"])):
        got = oracle.expert_gu_rows_iq3_xxs(gate, up, act, 2560)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    part = oracle.expert_gu_rows_iq3_xxs(gate, up, gold["act"], 2560, r0=7, r1=19)
    assert np.array_equal(part[:, 7:19].view(np.uint32), gold["ff"][:, 7:19].view(np.uint32)) and not part[:, :7].any()
    assert not np.array_equal(gold["ff"], gold["ff_m128"])


def test_expert_gate_up_rows_iq3_s_match_the_reference_avx2_kernel(oracle):
    """tests/golden/gate_up_rows_iq3_s.npz: ff of the reference's own iq_gu_rows (fmt iq3_s), also with -128 codes."""
    gold = np.load(os.path.join(GOLD, "gate_up_rows_iq3_s.npz"))
    for act, want in ((gold["act"], gold["ff"]), (gold["act_m128"], gold["ff_m128"])):
        got = oracle.expert_gu_rows("iq3_s", gold["gate"], gold["up"], act, 2560)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("fmt", ["iq2_xxs", "iq2_xs", "iq2_s"])
def test_expert_gate_up_rows_iq2_match_the_reference_avx2_kernel(oracle, fmt):
    """tests/golden/gate_up_rows_iq2.npz: ff of the reference's own iq_gu_rows for the three IQ2 formats, also with -128
    codes; the scalar restatement reproduces every bit."""
    gold = np.load(os.path.join(GOLD, "gate_up_rows_iq2.npz"))
    gate, up = gold[fmt + "_gate"], gold[fmt + "_up"]
    for act, want in ((gold[fmt + "_act"], gold[fmt + "_ff"]), (gold[fmt + "_act_m128"], gold[fmt + "_ff_m128"])):
        got = oracle.expert_gu_rows(fmt, gate, up, act, 2560)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert not np.array_equal(gold[fmt + "_ff"], gold[fmt + "_ff_m128"])


def test_expert_gate_up_rows_match_the_reference_avx2_kernel(oracle):
    """tests/golden/gate_up_rows.npz: ff of the reference's own kq_gu_rows (fmt q4_k, GLU included); the scalar
    restatement reproduces every bit, also on a sub-range of rows."""
    gold = np.load(os.path.join(GOLD, "gate_up_rows.npz"))
    gate, up, act, want = gold["gate"], gold["up"], gold["act"], gold["ff"]
    got = oracle.expert_gu_rows_q4_k(gate, up, act, 2560)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    part = oracle.expert_gu_rows_q4_k(gate, up, act, 2560, r0=7, r1=19)
    assert np.array_equal(part[:, 7:19].view(np.uint32), want[:, 7:19].view(np.uint32)) and not part[:, :7].any()


def test_attention_reference_against_numpy_and_the_kv_decoders(oracle):
    """The FP64 attention the GPU tests hold fnb_attend to, against the same sum written in numpy over cells decoded
    by the oracle's cache decoders (pinned above to fn::quant::kv_q8_value and ggml's Q8_0 decode): ragged ranges, a
    row with no cell, the output gate, both cache formats."""
    g = synth.rng(0xA77)
    cells, n_kv, n_q, hd, rows = 300, 2, 6, 128, 4
    q = synth.normal(g, (rows, n_q, hd), 1.5)
    gate = synth.normal(g, (rows, n_q, hd), 1.0)
    first = np.array([0, 17, 120, 50], np.int32)
    count = np.array([300, 100, 0, 250], np.int32)
    for fmt in ("q8_0", "kv8"):
        k, v = synth.normal(g, (cells, n_kv, hd)), synth.normal(g, (cells, n_kv, hd))
        if fmt == "q8_0":
            kf = oracle.dequantize_q8_0(oracle.quantize_q8_0(k)).reshape(k.shape)
            vf = oracle.dequantize_q8_0(oracle.quantize_q8_0(v)).reshape(v.shape)
        else:
            kf = oracle.kv8_dequantize(*oracle.kv8_quantize(k)).reshape(k.shape)
            vf = oracle.kv8_dequantize(*oracle.kv8_quantize(v)).reshape(v.shape)
        got = oracle.attend_f64(q, kf, vf, first, count, hd ** -0.5, gate=gate)
        want = np.zeros((rows, n_q, hd))
        for t in range(rows):
            lo, hi = int(first[t]), int(first[t] + count[t])
            if hi == lo:
                continue
            for h in range(n_q):
                kk, vv = kf[lo:hi, h // (n_q // n_kv)].astype(np.float64), vf[lo:hi, h // (n_q // n_kv)].astype(np.float64)
                s = kk @ q[t, h].astype(np.float64) * hd ** -0.5
                p = np.exp(s - s.max())
                want[t, h] = (p / p.sum()) @ vv / (1.0 + np.exp(-np.float64(gate[t, h])))
        assert not got[2].any()
        assert np.abs(got - want).max() <= 1e-12 * max(1.0, np.abs(want).max())
