"""The host-side GGUF reader against files written here from the format's specification: header, skipped metadata of
every value kind, alignment, tensor directory, row reads; malformed files are refused."""
import os
import struct

import numpy as np
import pytest

from fnfl_v100_b200 import build, gguf, synth


def _s(x: bytes) -> bytes:
    return struct.pack("<Q", len(x)) + x


def write_gguf(path, tensors, alignment=64, version=3):
    """tensors: list of (name, ggml type, dims (ne0, ne1, ...), raw bytes)."""
    kv = [
        (b"general.architecture", 8, _s(b"qwen4exp")),
        (b"general.alignment", 4, struct.pack("<I", alignment)),
        (b"some.float", 6, struct.pack("<f", 1.5)),
        (b"some.bool", 7, b"\x01"),
        (b"some.i64", 11, struct.pack("<q", -5)),
        (b"tokenizer.tokens", 9, struct.pack("<IQ", 8, 3) + _s(b"a") + _s(b"bc") + _s(b"")),       # array of strings
        (b"tokenizer.scores", 9, struct.pack("<IQ", 6, 4) + struct.pack("<4f", 1, 2, 3, 4)),      # array of f32
    ]
    out = struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(kv))
    for k, t, v in kv:
        out += _s(k) + struct.pack("<I", t) + v
    off, infos, blobs = 0, b"", []
    for name, typ, dims, raw in tensors:
        infos += _s(name.encode()) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", typ, off)
        blobs.append((off, raw))
        off = (off + len(raw) + alignment - 1) // alignment * alignment
    out += infos
    out += b"\0" * ((-len(out)) % alignment)
    start = len(out)
    for o, raw in blobs:
        out += b"\0" * (start + o - len(out)) + raw
    with open(path, "wb") as f:
        f.write(out)


@pytest.fixture(scope="module", autouse=True)
def _built():
    build.build()


def test_reads_directory_and_rows(tmp_path):
    g = synth.rng(9)
    q4 = synth.q4_k_table(g, 37, 2048)
    iq = synth.iq3_xxs_table(g, 11, 512)
    norm = synth.norm_weight(g, 2048)
    path = str(tmp_path / "m.gguf")
    write_gguf(path, [("output_norm.weight", 0, (2048,), norm.tobytes()),
                      ("token_embd.weight", 12, (2048, 37), q4.tobytes()),
                      ("other.weight", 18, (512, 11), iq.tobytes()),
                      ("unknown.weight", 14, (256, 2), b"\0" * 420)])       # Q6_K: listed, not decodable here
    with gguf.GgufFile(path) as f:
        assert f.n_tensors == 4
        t = f.find("token_embd.weight")
        assert (t.type, t.n_dims, t.ne[0], t.ne[1], t.row_bytes, t.n_rows) == (12, 2, 2048, 37, 1152, 37)
        assert np.array_equal(f.read_rows(t), q4)
        assert np.array_equal(f.read_rows(t, 5, 3), q4[5:8])
        t2 = f.find("other.weight")
        assert np.array_equal(f.read_rows(t2), iq)
        tn = f.find("output_norm.weight")
        assert np.array_equal(f.read_rows(tn).view(np.float32).reshape(-1), norm)
        assert f.find("unknown.weight").row_bytes == 0
        with pytest.raises(ValueError):
            f.read_rows(f.find("unknown.weight"))
        with pytest.raises(ValueError):
            f.read_rows(t, 30, 10)
        with pytest.raises(KeyError):
            f.find("missing")
    table, fmt, cols = gguf.load_table(path)
    assert fmt == "q4_k" and cols == 2048 and np.array_equal(table.numpy(), q4)


GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_reads_the_file_the_reference_writer_wrote():
    """tests/golden/model_tiny.gguf was written by the reference's own gguf writer (ggml/src/gguf.cpp, through
    oracle/ref_gguf_shim.cpp); model_tiny.npz holds each tensor's bytes and the file offset the reference's own READER
    reports for it.  This reader must find the same offsets and return the same bytes."""
    rec = np.load(os.path.join(GOLD, "model_tiny.npz"))
    names = sorted({k.split("|")[0] for k in rec.files})
    raw = open(os.path.join(GOLD, "model_tiny.gguf"), "rb").read()
    with gguf.GgufFile(os.path.join(GOLD, "model_tiny.gguf")) as f:
        assert f.n_tensors == len(names) == 5
        for name in names:
            t = f.find(name)
            want = rec[name + "|bytes"]
            off = int(rec[name + "|offset"])
            assert int(t.type) == int(rec[name + "|type"])
            assert raw[off:off + want.size] == want.tobytes()          # the fixture is self-consistent
            if int(t.type) == 14:                                      # Q6_K: listed, not decodable by this library
                assert t.row_bytes == 0
                continue
            got = f.read_rows(t)
            assert got.size == want.size and np.array_equal(got.reshape(-1), want)
            row = f.read_rows(t, int(t.n_rows) - 1, 1)                 # last row alone: offsets inside the tensor
            assert np.array_equal(row.reshape(-1), want[-int(t.row_bytes):])
    table, fmt, cols = gguf.load_table(os.path.join(GOLD, "model_tiny.gguf"))
    assert fmt == "q4_k" and cols == 256 and table.shape == (24, 144)


def test_python_writer_agrees_with_the_reference_reader(tmp_path):
    """The files the other tests write from the format specification are also what the reference's reader accepts
    (runs only where the reference tree was present to build its gguf code)."""
    from oracle import oracle as O
    if not O.have_ref_gguf():
        pytest.skip("reference gguf library not built here")
    g = synth.rng(5)
    q4 = synth.q4_k_table(g, 6, 512)
    norm = synth.norm_weight(g, 512)
    path = str(tmp_path / "m.gguf")
    write_gguf(path, [("output_norm.weight", 0, (512,), norm.tobytes()), ("token_embd.weight", 12, (512, 6), q4.tobytes())],
               alignment=32)
    off, typ, nb, cnt = O.ref_gguf_find(path, "token_embd.weight")
    assert (typ, nb, cnt) == (12, q4.size, 2)
    with gguf.GgufFile(path) as f:
        t = f.find("token_embd.weight")
        assert np.array_equal(f.read_rows(t), q4)
    assert open(path, "rb").read()[off:off + nb] == q4.tobytes()


def test_refuses_malformed_files(tmp_path):
    p = str(tmp_path / "bad.gguf")
    open(p, "wb").write(b"GGML" + b"\0" * 64)
    with pytest.raises(ValueError):
        gguf.GgufFile(p)
    g = synth.rng(9)
    q4 = synth.q4_k_table(g, 4, 256)
    write_gguf(p, [("token_embd.weight", 12, (256, 4), q4.tobytes())])
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-100])                       # tensor data runs past the end of the file
    with pytest.raises(ValueError):
        gguf.GgufFile(p)
    with pytest.raises(ValueError):
        gguf.GgufFile(str(tmp_path / "absent.gguf"))


@pytest.mark.gpu
def test_table_from_gguf_decodes_on_gpu(tmp_path, dev, oracle):
    import torch
    from fnfl_v100_b200 import ops
    g = synth.rng(9)
    q4 = synth.q4_k_table(g, 300, 2048)
    path = str(tmp_path / "m.gguf")
    write_gguf(path, [("token_embd.weight", 12, (2048, 300), q4.tobytes())])
    table, fmt, cols = gguf.load_table(path, device=dev)
    ids = torch.arange(299, -1, -1, dtype=torch.int32, device=dev)
    out = ops.get_rows(fmt, table, ids, cols).cpu().numpy()
    want = oracle.dequantize_q4_k(q4[::-1].copy()).reshape(300, 2048)
    assert np.array_equal(out.view(np.uint32), want.view(np.uint32))
