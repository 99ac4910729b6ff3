#!/usr/bin/env python3
"""Generate tests/golden/*.npz from the reference's own CPU sources.

Runs only where the reference tree is present: oracle/Makefile compiles ggml/src/ggml-quants.c and
fn/quant/*.cpp from the reference into oracle/_ref/libfnb_ref.so, and this script records that library's outputs
on seeded inputs.  The committed .npz files are what the tests read, so the tests need neither the reference
tree nor the reference build.

    python tests/golden/make_golden.py

quant.npz    inputs F32 [n][32] (stress + random runs) and, from the reference: Q8_0 and Q8_1 blocks
             (quantize_row_q8_0_ref / quantize_row_q8_1_ref, ggml-quants.c:274, :300), the activation format
             (fn::quant::act_quantize_ref, act_ref.cpp:8-30) and KV8 (fn::quant::kv_q8_quantize,
             kv_q8_ref.cpp:72-97; rows of 64)
decode.npz   seeded synthetic blocks (fn::quant::synth_blocks with the reference's seeds, synth.h:24-28) of
             Q4_K, IQ3_XXS, Q8_0 and IQ3_S and their decode by dequantize_row_q4_K / _iq3_xxs / _q8_0 / _iq3_s
             (ggml-quants.c:1527, :2573, :551, :2605), cross-checked against fn::quant::decode_row (decode.cpp)
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def stress_blocks() -> np.ndarray:
    g = np.random.Generator(np.random.Philox(0x43324143))  # the seed of the reference's act-test
    out = []
    # random runs: per-run magnitude 1e-6 .. 1e3, one value in 64 an outlier x20 (act_test.cpp:104-120's recipe)
    n = 1536
    mag = 10.0 ** g.uniform(-6, 3, size=(n, 1))
    x = g.standard_normal((n, 32)) * mag
    x = np.where(g.random((n, 32)) < 1 / 64, x * 20, x)
    out.append(x.astype(np.float32))
    # all zeros; one large value; one tiny value
    z = np.zeros((4, 32), np.float32)
    z[1, 7] = 1000.0
    z[2, 31] = -3.5e-5
    z[3, 0] = 65504.0 * 127
    out.append(z)
    # exact rounding midpoints: amax 127 -> id 1 (x = k + 0.5); amax 254 -> id 0.5 (x = 2k + 1)
    m = np.zeros((4, 32), np.float32)
    m[0, :] = np.arange(32) + 0.5
    m[0, 31] = 127.0
    m[1, :] = -(np.arange(32) + 0.5)
    m[1, 31] = -127.0
    m[2, :] = 2 * np.arange(32) + 1
    m[2, 31] = 254.0
    m[3, :] = -(2 * np.arange(32) + 1)
    m[3, 0] = 254.0
    out.append(m)
    # the reference's KV8 stress rows (kv_q8_ref.cpp:99-169): half steps, FP16-subnormal scales, scale underflow,
    # F32 subnormal inputs, magnitudes up to 127 x 65504, random ranges
    r = O.ref()
    cnt = r.ref_kv_q8_stress_rows(C.c_uint64(0x464E464C + 8), C.c_int32(16), None, C.c_int64(0))
    buf = np.empty(cnt, np.float32)
    r.ref_kv_q8_stress_rows(C.c_uint64(0x464E464C + 8), C.c_int32(16), O._p(buf), C.c_int64(cnt))
    out.append(buf.reshape(-1, 32))
    x = np.concatenate(out, 0)
    assert x.shape[0] % 2 == 0
    return np.ascontiguousarray(x)


def model_file() -> None:
    """A small model file written by the reference's OWN gguf writer (ggml/src/gguf.cpp): the fixture the reader is
    pinned against.  The tensors' bytes and the offsets the reference's own reader reports go into model_tiny.npz."""
    from fnfl_v100_b200 import synth
    O.build_ref_gguf()
    g = synth.rng(0x464E464C & 0xffff)
    tensors = [
        ("output_norm.weight", 0, (256,), synth.norm_weight(g, 256).view(np.uint8)),
        ("token_embd.weight", 12, (256, 24), synth.q4_k_table(g, 24, 256)),
        ("blk.0.ffn_gate_exps.weight", 18, (256, 8), synth.iq3_xxs_table(g, 8, 256)),
        ("blk.0.attn_k.weight", 8, (64, 5), synth.q8_0_table(g, 5, 64)),
        ("blk.0.ffn_down.weight", 14, (256, 2), g.integers(0, 256, 2 * 210).astype(np.uint8)),   # Q6_K: listed only
    ]
    path = os.path.join(HERE, "model_tiny.gguf")
    O.ref_gguf_write(path, tensors, alignment=32)   # the writer lays data out on its default 32 whatever the key says
    rec = {}
    for name, typ, dims, raw in tensors:
        off, t2, nb, cnt = O.ref_gguf_find(path, name)
        assert t2 == typ and cnt == len(tensors) and nb == np.asarray(raw).size
        rec[name + "|bytes"] = np.ascontiguousarray(raw, np.uint8).reshape(-1)
        rec[name + "|offset"] = np.int64(off)
        rec[name + "|type"] = np.int32(typ)
    np.savez_compressed(os.path.join(HERE, "model_tiny.npz"), **rec)
    print("model_tiny.gguf", os.path.getsize(path), "bytes")


def down_rows() -> None:
    """The reference's own AVX2 down mat-vec (fn::experts::cpu::kq_down_rows) on seeded weights and activations."""
    from fnfl_v100_b200 import synth
    g = synth.rng(0x4d45)
    rec = {}
    for fmt, n, rows, nt in (("q5_1", 640, 67, 5), ("q5_1", 64, 9, 11), ("q8_0", 640, 67, 5)):
        x = synth.normal(g, (nt, n), 2.0)
        if fmt == "q5_1":
            w, act = synth.q5_1_rows(g, rows, n), O.quantize_q8_1(x).reshape(nt, -1)
        else:
            w, act = synth.q8_0_table(g, rows, n), O.quantize_q8_0(x).reshape(nt, -1)
        key = f"{fmt}_{n}"
        rec[key + "|w"], rec[key + "|act"] = w, act
        rec[key + "|out"] = O.expert_down_rows(fmt, w, act, n, use_ref=True)
    np.savez_compressed(os.path.join(HERE, "down_rows.npz"), **rec)
    print("down_rows.npz", os.path.getsize(os.path.join(HERE, "down_rows.npz")), "bytes")


def down_rows_iq4_nl() -> None:
    """The reference's own AVX2 IQ4_NL down mat-vec (fn::experts::cpu::iq4nl_down_rows) on seeded weights and Q8_0
    activations; the second case's activations are random blocks, -128 codes among them (its sign step leaves them)."""
    from fnfl_v100_b200 import synth
    g = synth.rng(0x344e4c)
    rec = {}
    for key, n, rows, nt in (("quantised", 640, 67, 5), ("random", 128, 19, 8)):
        w = synth.iq4_nl_rows(g, rows, n)
        act = O.quantize_q8_0(synth.normal(g, (nt, n), 2.0)).reshape(nt, -1) if key == "quantised" else synth.q8_0_table(g, nt, n)
        rec[f"{key}_{n}|w"], rec[f"{key}_{n}|act"] = w, act
        rec[f"{key}_{n}|out"] = O.expert_down_rows("iq4_nl", w, act, n, use_ref=True)
    assert (rec["random_128|act"].reshape(8, -1, 34)[:, :, 2:] == 0x80).sum() > 0
    np.savez_compressed(os.path.join(HERE, "down_rows_iq4_nl.npz"), **rec)
    print("down_rows_iq4_nl.npz", os.path.getsize(os.path.join(HERE, "down_rows_iq4_nl.npz")), "bytes")


def down_rows_q2_0() -> None:
    """The reference's own planar activation quantiser and Q2_0 down rows (fn::experts::cpu::quantize_act_q,
    q2_down_rows) on seeded inputs: an all-zero chunk, a large outlier and exact half steps among them."""
    from fnfl_v100_b200 import synth
    g = synth.rng(0x5132)
    n, rows, nt = 640, 67, 5
    x = synth.normal(g, (nt, n), 2.0)
    x[0, :32] = 0.0
    x[1, 7] = 1e3
    x[2, 64:96] = np.arange(32, dtype=np.float32) * 0.5 - 8.0   # amax 8: x / s = 127 x / 8 lands on .5 steps
    w = synth.q2_0_rows(g, rows, n)
    q, s = O.quantize_act_q(x, use_ref=True)
    out = O.expert_down_rows_q2_0(w, n, x=x)
    np.savez_compressed(os.path.join(HERE, "down_rows_q2_0.npz"), x=x, w=w, codes=q, scales=s, out=out)
    print("down_rows_q2_0.npz", os.path.getsize(os.path.join(HERE, "down_rows_q2_0.npz")), "bytes")


def q8_k() -> None:
    """ggml's quantize_row_q8_K_ref and the reference's AVX2 quantize_q8_k on stress blocks (ties between +a and -a in
    both orders, zeros, tiny and huge magnitudes, constant blocks, half steps) and random ones; the two must agree."""
    from fnfl_v100_b200 import synth
    g = synth.rng(0x51384b)
    x = synth.normal(g, (96, 256), 3.0)
    x[1] = 0
    x[2, 5], x[2, 200] = 7.5, -7.5        # tie, the positive one first
    x[3, 5], x[3, 200] = -7.5, 7.5        # tie, the negative one first
    x[4] *= np.float32(1e-30)
    x[5] *= np.float32(1e20)
    x[6, :] = 0.5
    x[7, ::2] = -1.25
    x[8] = np.round(x[8] * 4) / 4          # many exact half steps after scaling by 127 / max
    x[8, 17] = 127.0 / 4
    x[9, :] = 0
    x[9, 255] = -3.0                       # the maximum in the last lane's last slot
    x[10, 0] = np.float32(np.abs(x[10]).max() * 2)   # and in the first
    a, b = O.quantize_q8_k(x, "ggml"), O.quantize_q8_k(x, "avx2")
    assert np.array_equal(a, b)
    np.savez_compressed(os.path.join(HERE, "q8_k.npz"), x=x, blocks=a)
    print("q8_k.npz", os.path.getsize(os.path.join(HERE, "q8_k.npz")), "bytes")


def gate_up_rows() -> None:
    """The reference's own AVX2 gate / up mat-vec with the GLU (fn::experts::cpu::kq_gu_rows, fmt q4_k) on seeded Q4_K rows
    and Q8_K activations.  Its expf is the host C library's; generate with
    GLIBC_TUNABLES=glibc.cpu.hwcaps=-AVX2_Usable,-FMA_Usable,-FMA4_Usable,-AVX2,-FMA,-FMA4 so that libm runs its generic
    build, the one the oracle restates (the assert below checks it)."""
    from fnfl_v100_b200 import synth
    g = synth.rng(0x4755)
    n, rows, nt = 2560, 45, 5
    gate, up = synth.q4_k_table(g, rows, n, 1e-5, 2e-4), synth.q4_k_table(g, rows, n, 1e-5, 2e-4)
    act = O.quantize_q8_k(synth.normal(g, (nt, n), 1.0), "ggml").reshape(nt, -1)
    ff = O.expert_gu_rows_q4_k(gate, up, act, n, use_ref=True)
    O.use_libm(False)
    assert np.array_equal(ff.view(np.uint32), O.expert_gu_rows_q4_k(gate, up, act, n).view(np.uint32)), "libm is not the generic build"
    np.savez_compressed(os.path.join(HERE, "gate_up_rows.npz"), gate=gate, up=up, act=act, ff=ff)
    print("gate_up_rows.npz", os.path.getsize(os.path.join(HERE, "gate_up_rows.npz")), "bytes; |ff| max", float(np.abs(ff).max()))


def gate_up_rows_q5_k() -> None:
    """The same for Q5_K rows (fn::experts::cpu::kq_gu_rows, fmt q5_k).  Same libm note as above."""
    from fnfl_v100_b200 import synth
    g = synth.rng(0x5135)
    n, rows, nt = 2560, 45, 5
    gate, up = synth.q5_k_table(g, rows, n, 1e-5, 1e-4), synth.q5_k_table(g, rows, n, 1e-5, 1e-4)
    act = O.quantize_q8_k(synth.normal(g, (nt, n), 1.0), "ggml").reshape(nt, -1)
    ff = O.expert_gu_rows_q5_k(gate, up, act, n, use_ref=True)
    O.use_libm(False)
    assert np.array_equal(ff.view(np.uint32), O.expert_gu_rows_q5_k(gate, up, act, n).view(np.uint32)), "libm is not the generic build"
    path = os.path.join(HERE, "gate_up_rows_q5_k.npz")
    np.savez_compressed(path, gate=gate, up=up, act=act, ff=ff)
    print("gate_up_rows_q5_k.npz", os.path.getsize(path), "bytes; |ff| max", float(np.abs(ff).max()))


def gate_up_rows_iq3_xxs() -> None:
    """The same for IQ3_XXS rows (fn::experts::cpu::iq_gu_rows, fmt iq3_xxs), and once more with one activation code in
    ten set to -128, which the reference's sign step (_mm256_sign_epi8) leaves as it is.  Same libm note as above."""
    from fnfl_v100_b200 import synth
    g = synth.rng(0x4933)
    n, rows, nt = 2560, 45, 5
    gate, up = synth.iq3_xxs_table(g, rows, n, 5e-5, 4e-4), synth.iq3_xxs_table(g, rows, n, 5e-5, 4e-4)
    act = O.quantize_q8_k(synth.normal(g, (nt, n), 1.0), "ggml").reshape(nt, -1)
    act_m128 = act.copy()
    codes = act_m128.reshape(nt, -1, 292)[:, :, 4:260]
    codes[g.integers(0, 10, size=codes.shape) == 0] = 0x80
    assert (act_m128 != act).sum() > 1000
    ff = O.expert_gu_rows_iq3_xxs(gate, up, act, n, use_ref=True)
    ff_m128 = O.expert_gu_rows_iq3_xxs(gate, up, act_m128, n, use_ref=True)
    O.use_libm(False)
    for a, f in ((act, ff), (act_m128, ff_m128)):
        assert np.array_equal(f.view(np.uint32), O.expert_gu_rows_iq3_xxs(gate, up, a, n).view(np.uint32)), "libm is not the generic build"
    path = os.path.join(HERE, "gate_up_rows_iq3_xxs.npz")
    np.savez_compressed(path, gate=gate, up=up, act=act, ff=ff, act_m128=act_m128, ff_m128=ff_m128)
    print("gate_up_rows_iq3_xxs.npz", os.path.getsize(path), "bytes; |ff| max", float(np.abs(ff).max()))


def gate_up_rows_iq3_s() -> None:
    """The same for IQ3_S rows (fn::experts::cpu::iq_gu_rows, fmt iq3_s), also with -128 codes.  Same libm note."""
    from fnfl_v100_b200 import synth
    g = synth.rng(0x4953)
    n, rows, nt = 2560, 45, 5
    gate, up = synth.iq3_s_table(g, rows, n, 2e-5, 3e-4), synth.iq3_s_table(g, rows, n, 2e-5, 3e-4)
    act = O.quantize_q8_k(synth.normal(g, (nt, n), 1.0), "ggml").reshape(nt, -1)
    act_m128 = act.copy()
    codes = act_m128.reshape(nt, -1, 292)[:, :, 4:260]
    codes[g.integers(0, 10, size=codes.shape) == 0] = 0x80
    ff = O.expert_gu_rows("iq3_s", gate, up, act, n, use_ref=True)
    ff_m128 = O.expert_gu_rows("iq3_s", gate, up, act_m128, n, use_ref=True)
    O.use_libm(False)
    for a, f in ((act, ff), (act_m128, ff_m128)):
        assert np.array_equal(f.view(np.uint32), O.expert_gu_rows("iq3_s", gate, up, a, n).view(np.uint32)), "libm is not the generic build"
    path = os.path.join(HERE, "gate_up_rows_iq3_s.npz")
    np.savez_compressed(path, gate=gate, up=up, act=act, ff=ff, act_m128=act_m128, ff_m128=ff_m128)
    print("gate_up_rows_iq3_s.npz", os.path.getsize(path), "bytes; |ff| max", float(np.abs(ff).max()))


def gate_up_rows_iq2() -> None:
    """The same for the three IQ2 formats (fn::experts::cpu::iq_gu_rows, fmt iq2_xxs / iq2_xs / iq2_s), each also with -128
    codes.  Same libm note."""
    from fnfl_v100_b200 import synth
    out = {}
    for fmt, seed, d_hi in (("iq2_xxs", 0x4932, 2.5e-4), ("iq2_xs", 0x4958, 2.5e-4), ("iq2_s", 0x4953 + 1, 2.5e-4)):
        g = synth.rng(seed)
        n, rows, nt = 2560, 33, 5
        gate, up = synth.iq2_table(fmt, g, rows, n, d_hi / 8, d_hi), synth.iq2_table(fmt, g, rows, n, d_hi / 8, d_hi)
        act = O.quantize_q8_k(synth.normal(g, (nt, n), 1.0), "ggml").reshape(nt, -1)
        act_m128 = act.copy()
        codes = act_m128.reshape(nt, -1, 292)[:, :, 4:260]
        codes[g.integers(0, 10, size=codes.shape) == 0] = 0x80
        O.use_libm(True)
        ff = O.expert_gu_rows(fmt, gate, up, act, n, use_ref=True)
        ff_m128 = O.expert_gu_rows(fmt, gate, up, act_m128, n, use_ref=True)
        O.use_libm(False)
        for a, f in ((act, ff), (act_m128, ff_m128)):
            assert np.array_equal(f.view(np.uint32), O.expert_gu_rows(fmt, gate, up, a, n).view(np.uint32)), fmt + ": restatement differs"
        for k, v in dict(gate=gate, up=up, act=act, ff=ff, act_m128=act_m128, ff_m128=ff_m128).items():
            out[fmt + "_" + k] = v
        print(fmt, "|ff| max", float(np.abs(ff).max()), "g std", float(np.std(O.expert_gu_rows(fmt, gate, up, act, n, want_gu=True)[1][0])))
    path = os.path.join(HERE, "gate_up_rows_iq2.npz")
    np.savez_compressed(path, **out)
    print("gate_up_rows_iq2.npz", os.path.getsize(path), "bytes")


def main() -> None:
    O.build(with_ref=True)
    model_file()
    down_rows()
    down_rows_iq4_nl()
    down_rows_q2_0()
    q8_k()
    gate_up_rows()
    gate_up_rows_q5_k()
    gate_up_rows_iq3_xxs()
    gate_up_rows_iq3_s()
    gate_up_rows_iq2()
    r = O.ref()
    x = stress_blocks()
    n = x.shape[0]
    q80 = np.empty(n * 34, np.uint8)
    q81 = np.empty(n * 36, np.uint8)
    r.quantize_row_q8_0_ref(O._p(x), O._p(q80), C.c_int64(x.size))
    r.quantize_row_q8_1_ref(O._p(x), O._p(q81), C.c_int64(x.size))
    codes = np.empty((n, 32), np.int8)
    scales = np.empty((n, 2), np.float32)
    r.ref_act_quantize(O._p(x), C.c_int32(n), C.c_int32(32), O._p(codes), O._p(scales))
    kv_codes = np.empty(x.size, np.int8)
    kv_scales = np.empty(x.size // 64, np.uint16)
    r.ref_kv_q8_quantize(O._p(x), C.c_int32(x.size), O._p(kv_codes), O._p(kv_scales))
    kv_values = np.empty(x.size, np.float32)
    r.ref_kv_q8_values(O._p(kv_codes), O._p(kv_scales), C.c_int64(x.size), O._p(kv_values))
    np.savez_compressed(os.path.join(HERE, "quant.npz"), x=x, q8_0=q80.reshape(n, 34), q8_1=q81.reshape(n, 36),
                        act_codes=codes, act_scales=scales, kv8_codes=kv_codes.reshape(-1, 64), kv8_scales=kv_scales,
                        kv8_values=kv_values.reshape(-1, 64))

    dec = {}
    nblk = 96
    for i, (fmt, bb, bv, fn) in enumerate((("q4_k", 144, 256, r.dequantize_row_q4_K),
                                           ("iq3_xxs", 98, 256, r.dequantize_row_iq3_xxs),
                                           ("q8_0", 34, 32, r.dequantize_row_q8_0),
                                           ("iq3_s", 110, 256, r.dequantize_row_iq3_s))):
        blk = np.empty(nblk * bb, np.uint8)
        assert r.ref_synth_blocks(fmt.encode(), C.c_uint64(0x464E464C + i), C.c_int64(nblk), O._p(blk)) == 0
        y = np.empty(nblk * bv, np.float32)
        fn(O._p(blk), O._p(y), C.c_int64(y.size))
        y2 = np.empty_like(y)
        assert r.ref_decode_row(fmt.encode(), O._p(blk), O._p(y2), C.c_int64(y.size)) == 0
        assert np.array_equal(y.view(np.uint32), y2.view(np.uint32)), fmt  # two in-tree statements agree
        dec[fmt + "_blocks"] = blk.reshape(nblk, bb)
        dec[fmt + "_values"] = y.reshape(nblk, bv)
    np.savez_compressed(os.path.join(HERE, "decode.npz"), **dec)
    for f in ("quant.npz", "decode.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
