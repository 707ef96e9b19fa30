"""The delta prefill entry point that carries its own scratch memory, called through the C ABI.

Some users of this library cannot allocate when they call it: an operator hook in a serving runtime gets pointers and a
stream and nothing else, and work being recorded into a CUDA graph may not call the allocator. For them
pgb_aspin_delta_prefill_noscratch_fwd keeps the per-chunk inverses in a fixed array inside the library. This test calls it
twice in a row and checks both results against the ordinary entry point (which takes the caller's scratch buffer) on the
same inputs; the second call runs on an array that still holds the first call's contents. This file is named so that
pytest collects it after every other test file.
"""
import ctypes

import pytest
import torch

from pragnosia_b200 import _lib, synth

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _run(entry, q, k, v, la, be, S0, scratch=None):
    B, H, T, D = q.shape
    o = torch.empty(B, H, T, D, device=DEV, dtype=torch.float32)
    S = torch.empty(B, H, D, D, device=DEV, dtype=torch.float32)
    L = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    head = (_ptr(q), _ptr(k), _ptr(v), _ptr(la), _ptr(be), _ptr(S0), None, None, 0.0, _ptr(o), _lib.F32, _ptr(S), None)
    if entry == "noscratch":
        rc = L.pgb_aspin_delta_prefill_noscratch_fwd(*head, B, H, T, D, stream)
    else:
        rc = L.pgb_aspin_delta_prefill_fwd(*head, _ptr(scratch), scratch.numel(), B, H, T, D, stream)
    _lib.check(rc, entry)
    return o, S


@pytest.mark.parametrize("D", [64, 128])
def test_noscratch_entry_matches_the_scratch_entry_twice(D):
    L = _lib.lib()
    outs = []
    for call, (B, H, T) in enumerate(((2, 3, 333), (3, 2, 200))):            # two calls in a row, different shapes
        x = synth.assoc_op_inputs(B, H, T, D, seed=40 + call + D, delta=True, with_state=True)
        q, k, v = (x[n].to(torch.bfloat16).to(DEV) for n in "qkv")
        la, be, S0 = x["la"].to(DEV), x["beta"].to(DEV), x["S0"].to(DEV)
        scratch = torch.empty(L.pgb_aspin_delta_scratch_bytes(B, H, T), device=DEV, dtype=torch.uint8)
        o_ref, S_ref = _run("scratch", q, k, v, la, be, S0, scratch)
        o, S = _run("noscratch", q, k, v, la, be, S0)
        torch.cuda.synchronize()
        # the same kernels on the same inputs: identical, far inside the 2e-3 / 1e-4 the parity tests use
        assert torch.isfinite(o).all() and torch.isfinite(S).all()
        eo = ((o - o_ref).abs().max() / o_ref.abs().max()).item()
        es = ((S - S_ref).abs().max() / S_ref.abs().max()).item()
        assert eo <= 2e-3 and es <= 1e-4, (call, eo, es)
        outs.append((eo, es))
    assert outs[0] == (0.0, 0.0) and outs[1] == (0.0, 0.0), outs


def test_noscratch_entry_rejects_what_does_not_fit():
    L = _lib.lib()
    one = ctypes.c_void_p(0x1000)
    # 4 x 16 x ceil(4096/64) = 4096 chunk inverses > the 2048 the built-in array holds: refused on the host
    rc = L.pgb_aspin_delta_prefill_noscratch_fwd(one, one, one, one, one, None, None, None, 0.0, one, 0, one, None, 4, 16, 4096, 64, None)
    assert rc == 7 and b"2048" in L.pgb_status_string(rc)
    assert L.pgb_aspin_delta_prefill_noscratch_fwd(one, one, one, one, None, None, None, None, 0.0, one, 0, one, None, 1, 1, 64, 64, None) == 1
