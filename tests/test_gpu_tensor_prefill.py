"""The tcgen05 / TMEM / TMA chunked-prefill kernel (bf16 inputs, plain rule) against the CPU oracle on the same
bf16-rounded inputs, and against the fp32 kernel. Tolerances: output 2e-3, carried state 1e-4 (max|d| / max|ref|)."""
import ctypes

import pytest
import torch

import oracle
from oracle import rel_err
from pragnosia_b200 import ops, synth, _lib

pytestmark = pytest.mark.gpu
torch.set_grad_enabled(False)
DEV = "cuda"
TC = _lib.PREFILL_TENSOR


@pytest.fixture(autouse=True, params=[0, 1], ids=["pipelined", "single-role"])
def tc_variant(request):
    """Every case runs on both plain-rule tensor-core kernels: the warp-specialised pipeline (head dim 64 default) and the
    single-role kernel (always used at head dim 128)."""
    _lib.check(_lib.lib().pgb_tc_set_variant(request.param), "pgb_tc_set_variant")
    yield request.param
    _lib.lib().pgb_tc_set_variant(0)


def flag():
    out = ctypes.c_int(-1)
    _lib.check(_lib.lib().pgb_tc_error_flag(ctypes.byref(out)), "pgb_tc_error_flag")
    return out.value


def inputs(B, H, T, D, seed, with_state=True):
    x = synth.assoc_op_inputs(B, H, T, D, seed=seed, with_state=with_state)
    q = oracle.rotate(x["q"], x["theta"], x["pos"]).to(torch.bfloat16)
    k = oracle.rotate(x["k"], x["theta"], x["pos"]).to(torch.bfloat16)
    return q, k, x["v"].to(torch.bfloat16), x["la"], x.get("S0")


def run(q, k, v, la, S0, **kw):
    d = lambda t: None if t is None else t.to(DEV)
    return ops.prefill(d(q), d(k), d(v), d(la), None, d(S0), precision=TC, **kw)


def check(o, S, ro, rS, what):
    assert torch.isfinite(o).all() and torch.isfinite(S).all(), what
    eo, es = rel_err(o.float().cpu(), ro), rel_err(S.cpu(), rS)
    assert eo <= 2e-3 and es <= 1e-4, f"{what}: o {eo:.2e} S {es:.2e}"
    return eo, es


def test_cfg0_shape_bf16_tensor_cores():
    q, k, v, la, _ = inputs(2, 12, 512, 64, seed=0, with_state=False)
    ro, rS = oracle.assoc_scan(q.float(), k.float(), v.float(), la, None)
    o, S, _ = run(q, k, v, la, None, out_dtype=torch.float32)
    eo, es = check(o, S, ro, rS, "cfg0")
    assert eo < 2e-4, eo                                     # hi/lo operand splitting: far inside the bf16 budget
    o16, S16, _ = run(q, k, v, la, None)
    assert o16.dtype == torch.bfloat16 and torch.equal(o16, o.to(torch.bfloat16)) and torch.equal(S, S16)
    o2, S2, _ = run(q, k, v, la, None, out_dtype=torch.float32)
    assert torch.equal(o, o2) and torch.equal(S, S2)         # deterministic
    assert flag() == 0


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("T", [1, 63, 64, 65, 200, 333, 512])
def test_lengths_states_and_sent(D, T):
    q, k, v, la, S0 = inputs(2, 3, T, D, seed=100 + T + D)
    ro, rS = oracle.assoc_scan(q.float(), k.float(), v.float(), la, S0)
    o, S, sent = run(q, k, v, la, S0, out_dtype=torch.float32, want_sent=True)
    check(o, S, ro, rS, f"D{D} T{T}")
    NC = (T + 63) // 64
    assert tuple(sent.shape) == (2, 3, NC, D, D)
    assert torch.equal(sent[:, :, 0].cpu(), S0.to(torch.bfloat16))
    if NC > 1:
        _, S64 = oracle.assoc_scan(q[:, :, :64].float(), k[:, :, :64].float(), v[:, :, :64].float(), la[:, :, :64], S0)
        assert rel_err(sent[:, :, 1].float().cpu(), S64) < 1e-2
    # against the fp32 kernel on the same inputs
    of, Sf, _ = ops.prefill(q.to(DEV), k.to(DEV), v.to(DEV), la.to(DEV), None, S0.to(DEV), precision=_lib.PREFILL_FP32,
                            out_dtype=torch.float32)
    assert rel_err(o.cpu(), of.cpu()) < 2e-4 and rel_err(S.cpu(), Sf.cpu()) < 1e-4
    assert flag() == 0


def test_rebase_and_windows():
    q, k, v, la, S0 = inputs(2, 3, 300, 64, seed=7)
    th = torch.rand(3, 32) * 0.5
    o, S, _ = run(q, k, v, la, S0, theta=th.to(DEV), shift=41.0, out_dtype=torch.float32)
    ro, rS = oracle.assoc_scan(q.float(), k.float(), v.float(), la, oracle.decode_rebase(S0, th, 41.0))
    check(o, S, ro, rS, "rebase")
    a = run(q[:, :, :130], k[:, :, :130], v[:, :, :130], la[:, :, :130], S0, out_dtype=torch.float32)
    b = ops.prefill(q[:, :, 130:].to(DEV), k[:, :, 130:].to(DEV), v[:, :, 130:].to(DEV), la[:, :, 130:].to(DEV), None, a[1],
                    precision=TC, out_dtype=torch.float32)
    r2, rS2 = oracle.assoc_scan(q.float(), k.float(), v.float(), la, S0)
    check(torch.cat([a[0], b[0]], 2), b[1], r2, rS2, "two windows")
    assert flag() == 0


def test_extreme_decay_and_many_chains():
    g = torch.Generator().manual_seed(3)
    q = torch.randn(4, 12, 512, 64, generator=g).to(torch.bfloat16)
    k = torch.randn(4, 12, 512, 64, generator=g).to(torch.bfloat16)
    v = torch.randn(4, 12, 512, 64, generator=g).to(torch.bfloat16)
    la = -torch.rand(4, 12, 512, generator=g) * 40
    o, S, _ = run(q, k, v, la, None, out_dtype=torch.float32)
    ro, rS = oracle.assoc_scan(q.float(), k.float(), v.float(), la, None)
    check(o, S, ro, rS, "extreme decay")
    assert flag() == 0


# ------------------------------------------------------------------------------------------------ delta rule
def delta_inputs(B, H, T, D, seed):
    x = synth.assoc_op_inputs(B, H, T, D, seed=seed, delta=True, with_state=True)
    q = oracle.rotate(x["q"], x["theta"], x["pos"]).to(torch.bfloat16)
    k = oracle.rotate(x["k"], x["theta"], x["pos"]).to(torch.bfloat16)
    return q, k, x["v"].to(torch.bfloat16), x["la"], x["beta"], x["S0"]


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("T", [1, 63, 64, 65, 200, 333, 512])
def test_delta_tensor_cores(D, T):
    """The delta rule on the tensor cores (X by exact fp32 substitution, then W = X rhs) against the chunked CPU form and
    the literal per-token recurrence, on the same bf16-rounded inputs: output 2e-3, state 1e-4."""
    q, k, v, la, be, S0 = delta_inputs(2, 3, T, D, seed=200 + T + D)
    d = lambda t: t.to(DEV)
    ro, rS = oracle.assoc_scan(q.float(), k.float(), v.float(), la, S0, beta=be)
    o, S, sent = ops.prefill(d(q), d(k), d(v), d(la), d(be), d(S0), out_dtype=torch.float32, want_sent=True)
    check(o, S, ro, rS, f"delta D{D} T{T}")
    lo, lS = oracle.delta_literal(q[:1, :1].double(), k[:1, :1].double(), v[:1, :1].double(), la[:1, :1].double(),
                                  be[:1, :1].double(), S0[:1, :1].double())
    check(o[:1, :1], S[:1, :1], lo.float(), lS.float(), f"delta literal D{D} T{T}")
    assert torch.equal(sent[:, :, 0].cpu(), S0.to(torch.bfloat16))
    of, Sf, _ = ops.prefill(d(q), d(k), d(v), d(la), d(be), d(S0), precision=_lib.PREFILL_FP32, out_dtype=torch.float32)
    assert rel_err(o.cpu(), of.cpu()) < 5e-4 and rel_err(S.cpu(), Sf.cpu()) < 1e-4
    o2, S2, _ = ops.prefill(d(q), d(k), d(v), d(la), d(be), d(S0), out_dtype=torch.float32)
    assert torch.equal(o, o2) and torch.equal(S, S2)
    assert flag() == 0


def test_delta_known_answers_tensor_cores(golden):
    """Repeated key with beta -> 1 (the case that broke reduced-precision inverses, src/assoc_kernel.py:577-582), 256
    correlated writes with beta = 1, and the rebase + two-window split."""
    import torch.nn.functional as F
    R = golden("delta_kat")["repeated"]
    k = R["k"].expand(1, 1, 128, 64).contiguous().to(torch.bfloat16)
    qq, vv = R["q"].to(torch.bfloat16), R["v"].to(torch.bfloat16)
    be = torch.full((1, 1, 128), 0.99999); la = torch.full((1, 1, 128), -1e-4)
    ro, rS = oracle.assoc_scan(qq.double(), k.double(), vv.double(), la.double(), None, beta=be.double())
    o, S, _ = ops.prefill(qq.to(DEV), k.to(DEV), vv.to(DEV), la.to(DEV), be.to(DEV), None, out_dtype=torch.float32)
    assert S.abs().max().item() < 3.0
    check(o, S, ro.float(), rS.float(), "repeated key")
    g = torch.Generator().manual_seed(1)
    Kr = F.normalize(torch.randn(2, 4, 256, 64, generator=g), dim=-1).to(torch.bfloat16)
    Vr = F.normalize(torch.randn(2, 4, 256, 64, generator=g), dim=-1).to(torch.bfloat16)
    z, one = torch.zeros(2, 4, 256), torch.ones(2, 4, 256)
    ro, rS = oracle.assoc_scan(Kr.float(), Kr.float(), Vr.float(), z, None, beta=one)
    o, S, _ = ops.prefill(Kr.to(DEV), Kr.to(DEV), Vr.to(DEV), z.to(DEV), one.to(DEV), None, out_dtype=torch.float32)
    assert S.abs().max().item() < 2.0
    check(o, S, ro, rS, "correlated writes")
    q, k, v, la, be, S0 = delta_inputs(2, 3, 300, 128, seed=9)
    th = torch.rand(3, 64) * 0.5
    d = lambda t: t.to(DEV)
    o, S, _ = ops.prefill(d(q), d(k), d(v), d(la), d(be), d(S0), theta=d(th), shift=41.0, out_dtype=torch.float32)
    ro, rS = oracle.assoc_scan(q.float(), k.float(), v.float(), la, oracle.decode_rebase(S0, th, 41.0), beta=be)
    check(o, S, ro, rS, "delta rebase")
    a = ops.prefill(d(q[:, :, :130]), d(k[:, :, :130]), d(v[:, :, :130]), d(la[:, :, :130]), d(be[:, :, :130]), d(S0), out_dtype=torch.float32)
    b = ops.prefill(d(q[:, :, 130:]), d(k[:, :, 130:]), d(v[:, :, 130:]), d(la[:, :, 130:]), d(be[:, :, 130:]), a[1], out_dtype=torch.float32)
    r2, rS2 = oracle.assoc_scan(q.float(), k.float(), v.float(), la, S0, beta=be)
    check(torch.cat([a[0], b[0]], 2), b[1], r2, rS2, "delta two windows")
    assert flag() == 0


def test_a_wait_that_runs_out_sets_the_flag_and_leaves_the_context_usable():
    """Failure detection without a fault: a wait on an mbarrier that nothing sets gives up after its cycle limit, the
    kernel returns normally, the flag reads 99 once (reading clears it), and the next launch works as usual."""
    L = _lib.lib()
    assert flag() == 0
    _lib.check(L.pgb_tc_wait_selftest(1 << 20, None), "pgb_tc_wait_selftest")       # about half a millisecond
    torch.cuda.synchronize()
    assert flag() == 99 and flag() == 0
    assert L.pgb_tc_wait_selftest(0, None) == 2
    q, k, v, la, _ = inputs(1, 2, 128, 64, seed=5, with_state=False)
    ro, rS = oracle.assoc_scan(q.float(), k.float(), v.float(), la, None)
    o, S, _ = run(q, k, v, la, None, out_dtype=torch.float32)
    check(o, S, ro, rS, "after the timed-out wait")
    assert flag() == 0
