"""fnb_attend_static: attention for callers that cannot pass or allocate a workspace (a plug-in whose host forbids
device allocation on the serving path, an engine whose memory was all handed out at load).  Its partial results live
in a fixed array inside the library, so the test checks, through the C ABI, that

  * its output equals fnb_attend's with a caller workspace bit for bit, on two calls in a row (the second call finds
    the first call's leftovers in the shared array and must not be disturbed by them), with a different shape in
    between so that the leftovers are of another layout;
  * a shape whose partial results exceed the built-in 16 MiB is refused and nothing is written.

The file sorts last so that a run stopping at the first failure has already run every other test; it also passes
alone in a fresh process (the first call on the device performs the address look-up itself).
"""
import ctypes as C

import numpy as np
import pytest
import torch

from fnfl_v100_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu


def _args(q, kc, vc, out, lo, hi, ws=None):
    rows, n_q, hd = q.shape
    return _lib.AttendArgs(q.data_ptr(), None, kc.data_ptr(), vc.data_ptr(), None, None, None, None, out.data_ptr(),
                           None if ws is None else ws.data_ptr(), 0 if ws is None else ws.numel(), None, kc.shape[0], lo, hi,
                           rows, n_q, kc.shape[1], hd, hd ** -0.5)


def _case(dev, seed, rows, n_q, n_kv, cells, hd=256):
    g = synth.rng(seed)
    plane = lambda: torch.from_numpy(g.integers(0, 256, (cells, n_kv, hd // 32, 34), dtype=np.uint8))  # noqa: E731
    kc, vc = plane(), plane()
    for t in (kc, vc):      # sane fp16 block scales under the random codes
        t.view(torch.float16).reshape(cells, n_kv, hd // 32, 17)[..., 0] = torch.from_numpy(
            g.uniform(0.005, 0.02, (cells, n_kv, hd // 32)).astype(np.float16))
    q = torch.from_numpy(synth.normal(g, (rows, n_q, hd)))
    return q.to(dev), kc.reshape(cells, n_kv, -1).to(dev), vc.reshape(cells, n_kv, -1).to(dev)


def test_static_scratch_attention_equals_the_workspace_form_twice_in_a_row(dev):
    L = _lib.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    cases = [_case(dev, 41, 3, 16, 2, 5000), _case(dev, 42, 1, 12, 1, 1777), _case(dev, 41, 3, 16, 2, 5000)]
    for q, kc, vc in cases:
        cells = kc.shape[0]
        want = torch.full_like(q, float("nan"))
        a = _args(q, kc, vc, want, 0, cells)
        need = int(L.fnb_attend_workspace_bytes(C.byref(a)))
        assert 0 < need <= 16 << 20
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        assert L.fnb_attend(C.byref(_args(q, kc, vc, want, 0, cells, ws)), stream) == _lib.OK
        for _ in range(2):                                   # two calls in a row through the new entry point
            got = torch.full_like(q, float("nan"))
            assert L.fnb_attend_static(C.byref(_args(q, kc, vc, got, 0, cells)), stream) == _lib.OK
            torch.cuda.synchronize()
            assert not bool(torch.isnan(got).any())
            assert torch.equal(got.view(torch.int32), want.view(torch.int32))


def test_static_scratch_attention_refuses_what_does_not_fit(dev, capfd):
    L = _lib.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    q, kc, vc = _case(dev, 43, 4, 256, 16, 40000)           # 64 query rows a group, sixteen KV heads, a long range: over 16 MiB of partials
    out = torch.full_like(q, 7.0)
    a = _args(q, kc, vc, out, 0, kc.shape[0])
    assert int(L.fnb_attend_workspace_bytes(C.byref(a))) > 16 << 20
    assert L.fnb_attend_static(C.byref(a), stream) == _lib.REJECTED
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())                          # nothing was enqueued
    assert "fnb_attend_static" in capfd.readouterr().err
