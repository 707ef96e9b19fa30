"""Parity of the CUDA kernels (called through the C ABI) against the CPU oracle and the reference-generated fixtures."""
import ctypes

import pytest
import torch
import torch.nn.functional as F

import oracle
from oracle import rel_err
from pragnosia_b200 import ops, synth, _lib

pytestmark = pytest.mark.gpu
torch.set_grad_enabled(False)
DEV = "cuda"


def cu(x):
    if isinstance(x, (tuple, list)):
        return type(x)(cu(t) for t in x)
    return x.to(DEV) if torch.is_tensor(x) else x


def close(a, b, tol, what=""):
    a, b = a.detach().cpu(), b.detach().cpu()
    assert a.shape == b.shape, (a.shape, b.shape)
    assert torch.isfinite(a).all(), f"{what}: non-finite"
    e = rel_err(a, b)
    assert e <= tol, f"{what}: rel err {e:.3e} > {tol}"
    return e


# ------------------------------------------------------------------------------------------------ lambda scan
@pytest.mark.parametrize("ts", [0, 1, 2, 4, 8, 16, 32])
def test_lambda_scan_d300_carried_state(golden, ts):
    """tests/test_spin.py:225-236 of the reference: B2 T45 D300, carried h0, vs the fp64 definition, < 1e-5 absolute."""
    g = torch.Generator().manual_seed(6)
    u = torch.randn(2, 45, 300, generator=g); lm = -torch.rand(2, 45, 300, generator=g) * 8; an = torch.randn(2, 45, 300, generator=g)
    h0 = (torch.randn(2, 300, generator=g), torch.randn(2, 300, generator=g))
    G = golden("lambda_scan")["d300"]
    y, (hr, hi) = ops.lambda_scan(cu(u), cu(lm), cu(an), cu(h0), time_segments=ts)
    assert (y.cpu() - G["y"].float()).abs().max().item() < 1e-5
    assert (hr.cpu() - G["hr"].float()).abs().max().item() < 1e-5
    assert (hi.cpu() - G["hi"].float()).abs().max().item() < 1e-5
    y0, _ = ops.lambda_scan(cu(u), cu(lm), cu(an), None, time_segments=ts)
    r0, _ = oracle.lambda_literal(u.double(), lm.double(), an.double())
    assert (y0.cpu() - r0.float()).abs().max().item() < 1e-5


@pytest.mark.parametrize("D,T", [(6, 45), (302, 17), (768, 1), (96, 2048), (768, 300)])
def test_lambda_scan_shapes_and_broadcast_angle(D, T):
    x = synth.lambda_scan_inputs(2, T, D, seed=4, with_state=True)
    ref_y, (rr, ri) = oracle.lambda_literal(x["u"].double(), x["logmag"].double(), x["ang"].double(),
                                            (x["h0"][0].double(), x["h0"][1].double()))
    y, (hr, hi) = ops.lambda_scan(cu(x["u"]), cu(x["logmag"]), cu(x["ang"]), cu(x["h0"]))
    close(y, ref_y.float(), 2e-5, "y"); close(hr, rr.float(), 2e-5, "hr"); close(hi, ri.float(), 2e-5, "hi")
    # one angle per channel, passed as a zero-stride expanded view (what the fspin layer passes)
    xb = synth.lambda_scan_inputs(2, T, D, seed=5, with_state=True, per_channel_angle=True)
    ang_dev = cu(xb["ang"][0, 0].contiguous()).expand(2, T, D)
    ref_y, (rr, ri) = oracle.lambda_literal(xb["u"].double(), xb["logmag"].double(), xb["ang"].double(),
                                            (xb["h0"][0].double(), xb["h0"][1].double()))
    y, (hr, hi) = ops.lambda_scan(cu(xb["u"]), cu(xb["logmag"]), ang_dev, cu(xb["h0"]))
    close(y, ref_y.float(), 2e-5, "y bcast"); close(hi, ri.float(), 2e-5, "hi bcast")


def test_lambda_scan_sequential_mode_and_windows():
    """One time segment per warp is the literal recurrence; two carried windows equal one pass; extreme decay is finite."""
    x = synth.lambda_scan_inputs(3, 333, 128, seed=9, with_state=True)
    a = ops.lambda_scan(cu(x["u"]), cu(x["logmag"]), cu(x["ang"]), cu(x["h0"]), time_segments=1)
    b = ops.lambda_scan(cu(x["u"]), cu(x["logmag"]), cu(x["ang"]), cu(x["h0"]), time_segments=1)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1][1], b[1][1])                       # deterministic
    c = ops.lambda_scan(cu(x["u"]), cu(x["logmag"]), cu(x["ang"]), cu(x["h0"]), time_segments=8)
    close(c[0], a[0], 1e-5, "parallel vs sequential")
    w1 = ops.lambda_scan(cu(x["u"][:, :100]), cu(x["logmag"][:, :100]), cu(x["ang"][:, :100]), cu(x["h0"]))
    w2 = ops.lambda_scan(cu(x["u"][:, 100:]), cu(x["logmag"][:, 100:]), cu(x["ang"][:, 100:]), w1[1])
    close(torch.cat([w1[0], w2[0]], 1), a[0], 1e-5, "windows"); close(w2[1][1], a[1][1], 1e-5, "windows Im")
    lmx = torch.full((2, 512, 8), -40.0)
    yx, _ = ops.lambda_scan(cu(torch.randn(2, 512, 8)), cu(lmx), cu(torch.randn(2, 512, 8)))
    assert torch.isfinite(yx).all()


# ------------------------------------------------------------------------------------------------ prep, rotate
def prep_ref(qp, kp, vp, gl, theta, pos):
    q_, k_, v_ = [F.normalize(t.transpose(1, 2).float(), dim=-1) for t in (qp, kp, vp)]
    if gl is not None:
        k_ = k_ * torch.sigmoid(gl.float()).transpose(1, 2).unsqueeze(-1)
    return oracle.rotate(q_, theta, pos), oracle.rotate(k_, theta, pos), v_


@pytest.mark.parametrize("D,T,gate,p0", [(64, 2048, True, 0), (64, 333, False, 1000), (128, 512, True, 4096)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_prep_kernel(D, T, gate, p0, dt):
    """tests/test_assoc.py:196-212 of the reference (forward part), bf16 outputs < 1e-2; fp32 in/out < 1e-5."""
    g = torch.Generator().manual_seed(0)
    H = 3
    mk = lambda: (torch.randn(2, T, H, D, generator=g) * 3).to(dt)
    qp, kp, vp = mk(), mk(), mk()
    gl = (torch.randn(2, T, H, generator=g) * 2).to(dt) if gate else None
    th = synth.rope_theta(H, D); pos = p0 + torch.arange(T)
    refs = prep_ref(qp, kp, vp, gl, th, pos)
    outs = ops.prep(cu(qp), cu(kp), cu(vp), cu(gl), cu(th), cu(pos), out_dtype=dt)
    for o_, r_, n in zip(outs, refs, "qkv"):
        assert o_.dtype == dt and tuple(o_.shape) == (2, H, T, D)
        close(o_.float(), r_, 1e-2 if dt == torch.bfloat16 else 1e-5, n)
    # the same through views into one fused projection (strided input)
    fused = torch.cat([qp.flatten(2), kp.flatten(2), vp.flatten(2), torch.zeros(2, T, 8, dtype=dt)], -1).to(DEV)
    d = H * D
    views = [fused[..., i * d:(i + 1) * d].unflatten(-1, (H, D)) for i in range(3)]
    outs2 = ops.prep(*views, cu(gl), cu(th), cu(pos), out_dtype=dt)
    for a, b in zip(outs, outs2):
        assert torch.equal(a, b)


def test_rotate_matches_and_is_relative():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 3, 45, 64, generator=g); th = torch.rand(3, 32, generator=g) * 0.3
    pos = torch.arange(1000, 1045)
    close(ops.rotate(cu(x), cu(th), cu(pos)), oracle.rotate(x, th, pos), 1e-5, "rotate")
    qq, kk, t1 = torch.randn(1, 1, 1, 8, generator=g), torch.randn(1, 1, 1, 8, generator=g), torch.rand(1, 4, generator=g) * 0.3
    r = lambda v, p: ops.rotate(cu(v), cu(t1), cu(torch.tensor([p]))).cpu()
    assert abs((r(qq, 10) * r(kk, 3)).sum().item() - (r(qq, 107) * r(kk, 100)).sum().item()) < 1e-4


# ------------------------------------------------------------------------------------------------ chunked prefill
def run_prefill(x, delta=False, dtype=torch.float32, S0=True, **kw):
    qr, kr = oracle.rotate(x["q"], x["theta"], x["pos"]), oracle.rotate(x["k"], x["theta"], x["pos"])
    q, k, v = (t.to(dtype) for t in (qr, kr, x["v"]))
    beta = x.get("beta") if delta else None
    s0 = x.get("S0") if S0 else None
    out = ops.prefill(cu(q), cu(k), cu(v), cu(x["la"]), cu(beta), cu(s0), **kw)
    ref = oracle.assoc_scan(q.float(), k.float(), v.float(), x["la"], s0, chunk=64, beta=beta)
    return out, ref


def test_prefill_cfg0_full_size_fp32(golden):
    """Configuration 0: B2 T512 H12 D64, fp32: output (2,512,768) within 2e-3 and state within 1e-4 of the reference's CPU
    result (measured far inside both)."""
    G = golden("cfg0")
    x = synth.assoc_op_inputs(2, 12, 512, 64, seed=0)
    (o, S, _), _ = run_prefill(x, S0=False)
    assert tuple(o.transpose(1, 2).reshape(2, 512, 768).shape) == (2, 512, 768)
    e1 = close(o[:, :, ::8], G["o_sub"], 2e-3, "o"); e2 = close(S, G["S"], 1e-4, "S")
    close(o[:, :, ::8], G["o_sub_literal"], 2e-3, "o vs literal"); close(S, G["S_literal"], 1e-4, "S vs literal")
    assert e1 < 1e-5 and e2 < 1e-5, (e1, e2)                        # the fp32 kernel is an fp32 computation
    (o2, S2, _), _ = run_prefill(x, S0=False)
    assert torch.equal(o, o2) and torch.equal(S, S2)                # run twice, bit-identical


def test_prefill_cfg0_bf16_inputs(golden):
    """bf16 I/O: compared with the oracle on the same bf16-rounded inputs. The fp32 output of the kernel must be within
    2e-3 (state 1e-4); the bf16 output must be exactly that result rounded to nearest."""
    x = synth.assoc_op_inputs(2, 12, 512, 64, seed=0)
    (o32, S, _), (ro, rS) = run_prefill(x, dtype=torch.bfloat16, S0=False, out_dtype=torch.float32)
    close(o32, ro, 2e-3, "o"); close(S, rS, 1e-4, "S")
    (o16, S16, _), _ = run_prefill(x, dtype=torch.bfloat16, S0=False)
    assert o16.dtype == torch.bfloat16 and torch.equal(o16, o32.to(torch.bfloat16)) and torch.equal(S, S16)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("delta", [False, True])
def test_prefill_ragged_carried(golden, D, delta):
    """T=333 (partial last chunk), carried S0, both rules, both head dims: the reference's kernel tests
    (tests/test_assoc.py:146-185) against its CPU two-pass form; here also against the literal recurrence."""
    G = golden("ragged")[D]
    x = synth.assoc_op_inputs(2, 3, 333, D, seed=10 + D, delta=True, with_state=True)
    (o, S, sent), (ro, rS) = run_prefill(x, delta=delta, want_sent=True)
    close(o[:, :, ::4], G["od" if delta else "o"], 2e-5, "o golden"); close(S, G["Sd" if delta else "S"], 2e-5, "S golden")
    close(o, ro, 2e-5, "o oracle")
    assert tuple(sent.shape) == (2, 3, 6, D, D) and sent.dtype == torch.bfloat16
    # entering states: chunk 0 is S0; chunk c is the state after 64c tokens
    close(sent[:, :, 0].float(), x["S0"].to(torch.bfloat16).float(), 1e-6, "sent[0]")
    qr, kr = oracle.rotate(x["q"], x["theta"], x["pos"]), oracle.rotate(x["k"], x["theta"], x["pos"])
    _, S128 = oracle.assoc_scan(qr[:, :, :128], kr[:, :, :128], x["v"][:, :, :128], x["la"][:, :, :128], x["S0"],
                                beta=x["beta"][:, :, :128] if delta else None)
    close(sent[:, :, 2].float(), S128, 1e-2, "sent[2]")
    # bf16 inputs
    (ob, Sb, _), (rob, rSb) = run_prefill(x, delta=delta, dtype=torch.bfloat16, out_dtype=torch.float32)
    close(ob, rob, 2e-3, "o bf16-in"); close(Sb, rSb, 1e-4, "S bf16-in")


@pytest.mark.parametrize("T", [1, 2, 63, 64, 65, 128, 200])
@pytest.mark.parametrize("delta", [False, True])
def test_prefill_lengths_and_windows(T, delta):
    x = synth.assoc_op_inputs(2, 2, T, 64, seed=T, delta=True, with_state=True)
    (o, S, _), (ro, rS) = run_prefill(x, delta=delta)
    close(o, ro, 2e-5, "o"); close(S, rS, 2e-5, "S")
    lo, lS = (oracle.delta_literal if delta else oracle.plain_literal)(
        *[t.double() for t in (oracle.rotate(x["q"], x["theta"], x["pos"]), oracle.rotate(x["k"], x["theta"], x["pos"]),
                               x["v"], x["la"])], *([x["beta"].double()] if delta else []), x["S0"].double())
    close(o, lo.float(), 2e-5, "o literal"); close(S, lS.float(), 2e-5, "S literal")
    if T >= 64:                                                      # two carried windows == one pass
        cut = 40
        qr, kr = oracle.rotate(x["q"], x["theta"], x["pos"]), oracle.rotate(x["k"], x["theta"], x["pos"])
        be = x["beta"] if delta else None
        a = ops.prefill(cu(qr[:, :, :cut]), cu(kr[:, :, :cut]), cu(x["v"][:, :, :cut]), cu(x["la"][:, :, :cut]),
                        cu(be[:, :, :cut]) if delta else None, cu(x["S0"]))
        b = ops.prefill(cu(qr[:, :, cut:]), cu(kr[:, :, cut:]), cu(x["v"][:, :, cut:]), cu(x["la"][:, :, cut:]),
                        cu(be[:, :, cut:]) if delta else None, a[1])
        close(torch.cat([a[0], b[0]], 2), o, 2e-5, "windows o"); close(b[1], S, 2e-5, "windows S")


def test_prefill_rebase_rotates_the_carried_state():
    x = synth.assoc_op_inputs(2, 3, 70, 64, seed=21, with_state=True)
    th = torch.rand(3, 32) * 0.5
    o, S, _ = ops.prefill(cu(x["q"]), cu(x["k"]), cu(x["v"]), cu(x["la"]), None, cu(x["S0"]), theta=cu(th), shift=37.0)
    ro, rS = oracle.assoc_scan(x["q"], x["k"], x["v"], x["la"], oracle.decode_rebase(x["S0"], th, 37.0))
    close(o, ro, 2e-5, "o"); close(S, rS, 2e-5, "S")
    o2, S2, _ = ops.prefill(cu(x["q"]), cu(x["k"]), cu(x["v"]), cu(x["la"]), None, cu(x["S0"]), theta=cu(th),
                            shift=torch.tensor(37.0, device=DEV))
    assert torch.equal(o, o2) and torch.equal(S, S2)


def test_delta_known_answers(golden):
    """tests/test_assoc.py:118-139 of the reference: a key written twice reads back the second value; 256 correlated
    writes with beta = 1 stay bounded; one key repeated 128 times with beta -> 1 (src/assoc_kernel.py:577-582)."""
    G = golden("delta_kat")
    K4, V4 = G["overwrite"]["K"].float(), G["overwrite"]["V"].float()
    pad = lambda t: F.pad(t, (0, 60))
    K, V = pad(K4), pad(V4)
    z, one = torch.zeros(1, 1, 3), torch.ones(1, 1, 3)
    od, _, _ = ops.prefill(cu(K), cu(K), cu(V), cu(z), cu(one), None)
    op, _, _ = ops.prefill(cu(K), cu(K), cu(V), cu(z), None, None)
    assert torch.allclose(od.cpu()[0, 0, 1, :4], V4[0, 0, 1], atol=1e-6)
    assert torch.allclose(op.cpu()[0, 0, 1, :4], V4[0, 0, 0] + V4[0, 0, 1], atol=1e-6)
    g = torch.Generator().manual_seed(1)
    Kr = F.normalize(torch.randn(2, 4, 256, 64, generator=g), dim=-1); Vr = F.normalize(torch.randn(2, 4, 256, 64, generator=g), dim=-1)
    y, S, _ = ops.prefill(cu(Kr), cu(Kr), cu(Vr), cu(torch.zeros(2, 4, 256)), cu(torch.ones(2, 4, 256)), None)
    assert S.abs().max().item() < 2.0
    close(y[:, :, ::8], G["correlated"]["y16"], 2e-5, "correlated y"); close(S, G["correlated"]["S16"], 2e-5, "correlated S")
    R = G["repeated"]
    k = R["k"].expand(1, 1, 128, 64).contiguous().float()
    be = torch.full((1, 1, 128), 0.99999); la = torch.full((1, 1, 128), -1e-4)
    o, S, _ = ops.prefill(cu(R["q"].float()), cu(k), cu(R["v"].float()), cu(la), cu(be), None)
    close(o, R["o"].float(), 1e-4, "repeated o"); close(S, R["S"].float(), 1e-4, "repeated S")
    assert S.abs().max().item() < 3.0


def test_prefill_extreme_decay_is_finite():
    g = torch.Generator().manual_seed(3)
    q = torch.randn(2, 4, 512, 64, generator=g)
    la = -torch.rand(2, 4, 512, generator=g) * 40
    o, S, _ = ops.prefill(cu(q), cu(torch.randn(2, 4, 512, 64, generator=g)), cu(torch.randn(2, 4, 512, 64, generator=g)), cu(la))
    assert torch.isfinite(o).all() and torch.isfinite(S).all()


# ------------------------------------------------------------------------------------------------ decode step
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("delta", [False, True])
@pytest.mark.parametrize("B", [1, 64])
@pytest.mark.parametrize("variant", [1, 2])
def test_decode_step_against_oracle(D, delta, B, variant):
    """variant 1: one CTA per (sequence, head) everywhere; 2: head dim 64 runs one warp per (sequence, head)."""
    if variant == 2 and D == 128:
        pytest.skip("head dim 128 has one kernel")
    _lib.check(_lib.lib().pgb_decode_set_variant(variant), "pgb_decode_set_variant")
    try:
        _decode_step_against_oracle(D, delta, B)
    finally:
        _lib.check(_lib.lib().pgb_decode_set_variant(0), "pgb_decode_set_variant")


def _decode_step_against_oracle(D, delta, B):
    H = 3
    g = torch.Generator().manual_seed(D + B)
    qp, kp, vp = (torch.randn(B, H, D, generator=g) * 2 for _ in range(3))
    gate = torch.randn(B, H, generator=g); araw = torch.randn(B, H, generator=g); A = torch.randn(H, generator=g) - 3
    S = torch.randn(B, H, D, D, generator=g) * 0.2
    th = torch.rand(H, D // 2, generator=g) * 0.4
    w = torch.rand(D, generator=g) + 0.5
    # oracle on prepared vectors
    q, k, v = (F.normalize(t, dim=-1) for t in (qp, kp, vp))
    la = -F.softplus(araw) * A.exp()
    if delta:
        o_ref, S_ref = oracle.decode_step(S, 29.0, q, k, v, la, th, torch.sigmoid(gate))
    else:
        o_ref, S_ref = oracle.decode_step(S, 29.0, q, k * torch.sigmoid(gate)[..., None], v, la, th)
    eps = 1.1920929e-07
    o_norm = o_ref * torch.rsqrt(o_ref.pow(2).mean(-1, keepdim=True) + eps) * w
    Sd = cu(S)
    o, S1 = ops.decode_step(cu(qp), cu(kp), cu(vp), cu(araw), Sd, cu(th), gate=cu(gate), delta=delta, decay_A=cu(A), shift=29.0)
    close(o, o_ref, 1e-5, "o"); close(S1, S_ref, 1e-5, "S")
    assert torch.equal(Sd.cpu(), S)                                  # functional by default: the input state is untouched
    o2, _ = ops.decode_step(cu(qp), cu(kp), cu(vp), cu(araw), Sd, cu(th), gate=cu(gate), delta=delta, decay_A=cu(A),
                            shift=torch.tensor(29.0, device=DEV), rms_weight=cu(w), rms_eps=eps)
    close(o2, o_norm, 1e-5, "o rms")
    # in place, bf16 vectors in a fused row (strided), log-decay given directly
    row = torch.cat([qp.flatten(1), kp.flatten(1), vp.flatten(1), la, gate, torch.zeros(B, 2)], 1).to(torch.bfloat16).to(DEV)
    d = H * D
    views = [row[:, i * d:(i + 1) * d].unflatten(1, (H, D)) for i in range(3)]
    o3, S3 = ops.decode_step(*views, row[:, 3 * d:3 * d + H], Sd, cu(th), gate=row[:, 3 * d + H:3 * d + 2 * H], delta=delta,
                             shift=29.0, S_out=Sd, out_dtype=torch.float32)
    assert S3.data_ptr() == Sd.data_ptr()
    rq, rk, rv = (F.normalize(t.to(torch.bfloat16).float(), dim=-1) for t in (qp, kp, vp))
    rg, rla = torch.sigmoid(gate.to(torch.bfloat16).float()), la.to(torch.bfloat16).float()
    o_r, S_r = oracle.decode_step(S, 29.0, rq, rk if delta else rk * rg[..., None], rv, rla, th, rg if delta else None)
    close(o3, o_r, 1e-5, "o in-place"); close(Sd, S_r, 1e-5, "S in-place")


# ------------------------------------------------------------------------------------------------ fused pieces
@pytest.mark.parametrize("D", [64, 128])
def test_prefill_fused_epilogue_and_decay_gate(D):
    """Decay gate from logits, per-head RMS norm and token-major output fused into the tensor-core prefill."""
    B, H, T = 2, 3, 200
    x = synth.assoc_op_inputs(B, H, T, D, seed=31 + D, with_state=True)
    q, k, v = (t.to(torch.bfloat16) for t in (x["q"], x["k"], x["v"]))
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(B, T, H + 3, generator=g).to(torch.bfloat16)           # a view with a padded last dim
    A = torch.randn(H, generator=g) - 2
    w = torch.rand(D, generator=g) + 0.5
    la = (-F.softplus(logits[..., :H].float()) * A.exp()).transpose(1, 2)
    ro, rS = oracle.assoc_scan(q.float(), k.float(), v.float(), la, x["S0"])
    eps = 1e-6
    rn = ro * torch.rsqrt(ro.pow(2).mean(-1, keepdim=True) + eps) * w
    o, S, _ = ops.prefill_fused(cu(q), cu(k), cu(v), cu(logits)[..., :H], cu(A), cu(x["S0"]), rms_weight=cu(w), rms_eps=eps,
                                out_dtype=torch.float32)
    assert tuple(o.shape) == (B, T, H * D)
    close(o.view(B, T, H, D).transpose(1, 2), rn, 2e-3, "fused o"); close(S, rS, 1e-4, "fused S")
    o2, S2, _ = ops.prefill_fused(cu(q), cu(k), cu(v), cu(logits)[..., :H], cu(A), cu(x["S0"]), out_dtype=torch.float32)
    close(o2.view(B, T, H, D).transpose(1, 2), ro, 2e-3, "fused o, no norm")
    Sd = cu(x["S0"]).clone()
    _, S3, _ = ops.prefill_fused(cu(q), cu(k), cu(v), cu(logits)[..., :H], cu(A), Sd, S_out=Sd)
    assert S3.data_ptr() == Sd.data_ptr() and torch.equal(Sd, S)                 # in-place state update


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("d", [64, 768, 1024])
def test_add_norm(dt, d):
    g = torch.Generator().manual_seed(d)
    x = (torch.randn(5, 37, d, generator=g) * 2).to(dt); dl = torch.randn(5, 37, d, generator=g).to(dt)
    for norm in (torch.nn.RMSNorm(d), torch.nn.LayerNorm(d)):
        norm.weight.data = torch.rand(d, generator=g) + 0.5
        if hasattr(norm, "bias") and norm.bias is not None:
            norm.bias.data = torch.randn(d, generator=g) * 0.1
        norm = norm.to(dt)
        y_ref = x + dl
        z_ref = norm(y_ref)
        y, z = ops.add_norm(cu(x), cu(dl), norm.to(DEV))
        assert torch.equal(y.cpu(), y_ref)
        close(z.float(), z_ref.float(), 1e-2 if dt == torch.bfloat16 else 1e-5, f"z {type(norm).__name__}")
        y0, z0 = ops.add_norm(cu(x), None, norm)
        assert y0.data_ptr() == cu(x).data_ptr() or torch.equal(y0.cpu(), x)
        close(z0.float(), norm.cpu()(x).float(), 1e-2 if dt == torch.bfloat16 else 1e-5, "z without delta")


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("gate", [True, False])
def test_layer_prefill_raw_projections(D, gate):
    """The whole between-GEMMs kernel: raw (B,T,H,D) projection views in, normalised per-head read out, against
    prep_ref + the CPU scan + an fp32 RMS norm on the same bf16 inputs."""
    B, H, T = 2, 3, 333
    g = torch.Generator().manual_seed(17 + D)
    d = H * D
    ld = 3 * d + 2 * H + 2                                                       # padded row, a multiple of 8
    assert ld % 8 == 0
    proj = (torch.randn(B, T, ld, generator=g) * 2).to(torch.bfloat16)
    S0 = torch.randn(B, H, D, D, generator=g) * 0.1
    A = torch.randn(H, generator=g) - 2
    w = torch.rand(D, generator=g) + 0.5
    th = synth.rope_theta(H, D) * (1 + 0.1 * torch.rand(H, D // 2, generator=g))
    qp, kp, vp = (proj[..., i * d:(i + 1) * d].unflatten(-1, (H, D)) for i in range(3))
    dl, gl = proj[..., 3 * d:3 * d + H], proj[..., 3 * d + H:3 * d + 2 * H]
    q, k, v = prep_ref(qp, kp, vp, gl if gate else None, th, torch.arange(T))
    q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))                  # the operands are rounded to bf16
    la = (-F.softplus(dl.float()) * A.exp()).transpose(1, 2)
    ro, rS = oracle.assoc_scan(q, k, v, la, oracle.decode_rebase(S0, th, 50.0))
    eps = 1e-6
    rn = ro * torch.rsqrt(ro.pow(2).mean(-1, keepdim=True) + eps) * w
    pd = cu(proj)
    qd, kd, vd = (pd[..., i * d:(i + 1) * d].unflatten(-1, (H, D)) for i in range(3))
    table = ops.rot_table(cu(th), 512)                                         # covers T rounded up to whole chunks
    o, S, _ = ops.layer_prefill(qd, kd, vd, pd[..., 3 * d + H:3 * d + 2 * H] if gate else None, pd[..., 3 * d:3 * d + H], cu(A),
                                table, cu(S0), theta=cu(th), shift=50.0, rms_weight=cu(w), rms_eps=eps, out_dtype=torch.float32)
    close(o.view(B, T, H, D).transpose(1, 2), rn, 3e-3, "layer o"); close(S, rS, 2e-3, "layer S")
    # and bit-identical to the two-kernel route (prep kernel, then the fused prefill on its output)
    q2, k2, v2 = ops.prep(qd, kd, vd, pd[..., 3 * d + H:3 * d + 2 * H] if gate else None, cu(th), cu(torch.arange(T)))
    o2, S2, _ = ops.prefill_fused(q2, k2, v2, pd[..., 3 * d:3 * d + H], cu(A), cu(S0), theta=cu(th), shift=50.0,
                                  rms_weight=cu(w), rms_eps=eps, out_dtype=torch.float32)
    close(o, o2, 3e-3, "layer vs two-kernel o"); close(S, S2, 2e-3, "layer vs two-kernel S")


@pytest.mark.parametrize("B", [1, 3, 8])
@pytest.mark.parametrize("K,N", [(768, 2328), (3072, 768), (768, 8192)])
@pytest.mark.parametrize("norm,act", [(None, None), ("rms", "gelu"), ("ln", None)])
def test_skinny_linear(B, K, N, norm, act):
    """The fused small-batch linear layer (residual add + norm + linear + bias + GELU in one launch) against the same
    chain of separate torch ops in bf16 (src/model.py:552-560, src/assoc.py:388-451 at T = 1)."""
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(B * 1000 + K + N)
    bf = lambda t: t.to(DEV).to(torch.bfloat16)
    x, delta = bf(torch.randn(B, K, generator=g)), bf(0.5 * torch.randn(B, K, generator=g))
    W, bias = bf(torch.randn(N, K, generator=g) * K ** -0.5), bf(0.1 * torch.randn(N, generator=g))
    mod = None
    if norm is not None:
        mod = (torch.nn.RMSNorm(K) if norm == "rms" else torch.nn.LayerNorm(K)).to(DEV).to(torch.bfloat16)
        with torch.no_grad():
            mod.weight.copy_(bf(1.0 + 0.2 * torch.randn(K, generator=g)))
            if norm == "ln":
                mod.bias.copy_(bf(0.1 * torch.randn(K, generator=g)))
    for dl in (delta, None):
        s = x if dl is None else x + dl
        z = s if mod is None else mod(s)
        ref = F.linear(z, W, bias)
        if act == "gelu":
            ref = F.gelu(ref)
        y, s2 = ops.skinny_linear(x, W, bias, delta=dl, norm=mod, act=act, want_sum=True)
        assert y.dtype == torch.bfloat16 and tuple(y.shape) == (B, N)
        assert torch.equal(s2, s)                                             # the residual stream, bit for bit
        exact = F.linear(z.float(), W.float(), bias.float())                  # same rounded operands, fp32 accumulate
        exact = exact.to(torch.bfloat16).float()
        if act == "gelu":
            exact = F.gelu(exact)
        assert rel_err(y.float().cpu(), exact.cpu()) <= 4e-3                  # one bf16 ulp of the largest value
        assert rel_err(y.float().cpu(), ref.float().cpu()) <= 8e-3
    y0 = ops.skinny_linear(x, W)                                              # no bias, nothing fused
    assert rel_err(y0.float().cpu(), F.linear(x.float(), W.float()).cpu()) <= 4e-3


def test_decode_embed_and_sampler():
    """The single-launch ends of the decode step: embedding sum; Gumbel-max draws that are greedy at temperature 0,
    reproducible from (seed, step), recorded at the running index, and distributed as softmax(logits / temp)."""
    g = torch.Generator().manual_seed(3)
    E = torch.randn(50, 64, generator=g).to(DEV).to(torch.bfloat16)
    P = torch.randn(12, 64, generator=g).to(DEV).to(torch.bfloat16)
    tok = torch.tensor([[3], [49], [0]], device=DEV)
    pos = torch.tensor([7], device=DEV)
    assert torch.equal(ops.decode_embed(tok, pos, E, P), E[tok.view(-1)] + P[7])
    B, V, n = 64, 16, 400
    p = torch.softmax(torch.randn(V, generator=g) * 1.5, -1)
    logits = p.log().expand(B, V).contiguous().to(DEV)
    def run(seed, temp):
        t = torch.zeros(B, dtype=torch.long, device=DEV)
        cnt = torch.zeros(1, dtype=torch.long, device=DEV)
        ticket = torch.zeros(1, dtype=torch.int32, device=DEV)
        hist = torch.full((B, n), -1, dtype=torch.long, device=DEV)
        posd = torch.tensor([10], device=DEV); shift = torch.tensor(5.0, device=DEV)
        for i in range(n):
            ops.decode_sample(logits * temp, temp, seed, t, cnt, ticket, hist=hist, pos=posd, shift=shift, ctx=12)
            if i == 0:
                assert posd.item() == 10 and shift.item() == 5.0          # the first draw leaves the prompt's position alone
        assert cnt.item() == n and ticket.item() == 0 and posd.item() == (10 + n - 1) % 12 and shift.item() == 1.0
        assert torch.equal(hist[:, -1], t)
        return hist
    h1, h2, h3 = run(1, 1.0), run(1, 1.0), run(2, 0.5)
    assert torch.equal(h1, h2) and not torch.equal(h1, h3)
    for h in (h1, h3):                                                    # temperature cancels: same target distribution
        freq = torch.bincount(h.reshape(-1).cpu(), minlength=V).double() / h.numel()
        sigma = (p.double() * (1 - p.double()) / h.numel()).sqrt()
        assert ((freq - p.double()).abs() <= 5 * sigma + 1e-4).all(), (freq, p)
    t = torch.zeros(B, dtype=torch.long, device=DEV)
    lg = torch.randn(B, 1000, generator=g).to(DEV)
    ops.decode_sample(lg.to(torch.bfloat16), 0.0, 9, t, torch.zeros(1, dtype=torch.long, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV))
    assert torch.equal(t, lg.to(torch.bfloat16).float().argmax(-1))


@pytest.mark.parametrize("M,K,N", [(8192, 768, 3072), (300, 768, 3072), (128, 64, 256), (1000, 200, 520)])
@pytest.mark.parametrize("act", ["gelu", None])
def test_linear_act_tensor_core_gemm(M, K, N, act):
    """The fused Linear + bias + erf-GELU GEMM (the MLP up-projection of src/model.py:552-560) against the separate torch
    ops in bf16 and against the fp32 product of the same rounded operands; ragged M, K, N exercise the zero-filled tiles."""
    g = torch.Generator().manual_seed(M + K + N)
    bf = lambda t: t.to(DEV).to(torch.bfloat16)
    x, W, b = bf(torch.randn(M, K, generator=g)), bf(torch.randn(N, K, generator=g) * K ** -0.5), bf(0.2 * torch.randn(N, generator=g))
    y = ops.linear_act(x, W, b, act=act)
    assert y.dtype == torch.bfloat16 and tuple(y.shape) == (M, N)
    pre = F.linear(x.float(), W.float(), b.float()).to(torch.bfloat16).float()
    exact = F.gelu(pre) if act == "gelu" else pre
    assert rel_err(y.float().cpu(), exact.cpu()) <= 8e-3                      # two bf16 ulps of the largest value
    ref = F.linear(x, W, b)
    ref = F.gelu(ref) if act == "gelu" else ref
    assert rel_err(y.float().cpu(), ref.float().cpu()) <= 8e-3
    assert torch.equal(y, ops.linear_act(x, W, b, act=act))                   # deterministic
    y3 = ops.linear_act(x.view(-1, 1, K) if M % 1 == 0 else x, W, None, act=act)
    assert tuple(y3.shape) == (M, 1, N)
    # tiles 256 and 192 columns wide, on one SM and on a pair of SMs (two-CTA cluster, tcgen05.mma.cta_group::2): the same bits
    try:
        for variant in (2, 4, 1, 3, 5):
            _lib.check(_lib.lib().pgb_linear_act_set_variant(variant), "pgb_linear_act_set_variant")
            assert torch.equal(y, ops.linear_act(x, W, b, act=act)), variant
    finally:
        _lib.check(_lib.lib().pgb_linear_act_set_variant(0), "pgb_linear_act_set_variant")
    out = ctypes.c_int(-1)
    _lib.check(_lib.lib().pgb_tc_error_flag(ctypes.byref(out)), "pgb_tc_error_flag")
    assert out.value == 0


def test_windowed_walks_equal_single_calls():
    """pragnosia_b200.sharded on one GPU (gather disabled): walking a sequence window by window with the carried state
    gives the single call's outputs and final state, for the prefill (both rules) and the lambda scan."""
    from pragnosia_b200 import sharded
    d = lambda t: t.to(DEV)
    x = synth.assoc_op_inputs(2, 3, 320, 64, seed=31, delta=True, with_state=True)
    q, k, v = (d(x[n]).to(torch.bfloat16) for n in "qkv")
    la, be, S0 = d(x["la"]), d(x["beta"]), d(x["S0"])
    for beta in (None, be):
        o, S, _ = ops.prefill(q, k, v, la, beta, S0, out_dtype=torch.bfloat16)
        outs, Sw = sharded.prefill_windows(q, k, v, la, 128, beta=beta, S0=S0)
        assert [t.shape[2] for t in outs] == [128, 128, 64]
        assert rel_err(torch.cat(outs, 2).float().cpu(), o.float().cpu()) <= 1e-5 and rel_err(Sw.cpu(), S.cpu()) <= 1e-5
    y = synth.lambda_scan_inputs(3, 300, 96, seed=32, with_state=True)
    u, lm, an, h0 = d(y["u"]), d(y["logmag"]), d(y["ang"]), tuple(d(t) for t in y["h0"])
    full, hf = ops.lambda_scan(u, lm, an, h0=h0)
    ys, hw = sharded.lambda_scan_windows(u, lm, an, 128, h0=h0)
    assert rel_err(torch.cat(ys, 1).cpu(), full.cpu()) <= 1e-5
    assert rel_err(hw[0].cpu(), hf[0].cpu()) <= 1e-5 and rel_err(hw[1].cpu(), hf[1].cpu()) <= 1e-5
    got = sharded.run_windows(lambda w: u[:, w * 100:(w + 1) * 100].contiguous(), 3)
    assert torch.equal(torch.cat(got, 1), u)


@pytest.mark.parametrize("B,K,N,bias,act", [(64, 768, 2328, True, None), (9, 768, 768, False, None), (128, 3072, 768, True, None),
                                            (33, 768, 3072, True, "gelu"), (64, 768, 8192, False, None), (5, 128, 392, True, None),
                                            (16, 200, 24, True, "gelu")])
def test_batch_linear_tensor_core(B, K, N, bias, act):
    """The decode step's linear layer for 5..128 rows as one tcgen05 launch, against the fp32 product of the same bf16
    operands with the separate ops' roundings (bf16 pre-activation, erf-GELU, bf16)."""
    g = torch.Generator().manual_seed(B * 7 + N)
    x = torch.randn(B, K, generator=g).to(DEV).to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g) / K ** 0.5).to(DEV).to(torch.bfloat16)
    b = (torch.randn(N, generator=g) * 0.3).to(DEV).to(torch.bfloat16) if bias else None
    y = ops.batch_linear(x, W, b, act=act)
    ref = x.float() @ W.float().t()
    if bias:
        ref = ref + b.float()
    ref = ref.to(torch.bfloat16).float()
    if act == "gelu":
        ref = torch.nn.functional.gelu(ref).to(torch.bfloat16).float()
    assert y.shape == (B, N) and y.dtype == torch.bfloat16
    assert rel_err(y.float().cpu(), ref.cpu()) <= 4e-3
    assert torch.equal(y, ops.batch_linear(x, W, b, act=act))           # run twice: bit-identical


@pytest.mark.parametrize("norm_cls", [torch.nn.LayerNorm, torch.nn.RMSNorm])
def test_batch_linear_folded_norm_and_residual(norm_cls):
    """The linear layer that takes over the add + norm launches around it: the norm folded into the weight and applied on
    the accumulator from row sums, the residual add and the next norm's row sums in the epilogue."""
    g = torch.Generator().manual_seed(31)
    B, K, N = 48, 768, 2328
    stream = (torch.randn(B, K, generator=g) * 1.5 + 0.3).to(DEV).to(torch.bfloat16)
    norm = norm_cls(K).to(DEV)
    with torch.no_grad():
        norm.weight.copy_(1.0 + 0.2 * torch.randn(K, generator=g).to(DEV))
        if getattr(norm, "bias", None) is not None:
            norm.bias.copy_(0.2 * torch.randn(K, generator=g).to(DEV))
    norm = norm.to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g) / K ** 0.5).to(DEV).to(torch.bfloat16)
    b = (torch.randn(N, generator=g) * 0.3).to(DEV).to(torch.bfloat16)
    sums = torch.stack([stream.float().sum(1), (stream.float() ** 2).sum(1)], 1)[None].contiguous()
    Wf, c1, c2, kind, eps = ops.fold_norm(norm, W, b)
    out = ops.batch_linear(stream, Wf, act="gelu", folded=(sums, c1, c2, kind, eps))
    ref = F.gelu(F.linear(norm.float()(stream.float()), W.float(), b.float()))
    assert rel_err(out.float().cpu(), ref.cpu()) <= 8e-3                      # bf16 roundings of the weight and the output
    # the sums may arrive in parts
    parts = torch.stack([torch.stack([stream[:, i::3].float().sum(1), (stream[:, i::3].float() ** 2).sum(1)], 1) for i in range(3)]).contiguous()
    out3 = ops.batch_linear(stream, Wf, act="gelu", folded=(parts, c1, c2, kind, eps))
    assert rel_err(out3.float().cpu(), out.float().cpu()) <= 4e-3
    # residual add and the row sums of the new stream
    o = torch.randn(B, K, generator=g).to(DEV).to(torch.bfloat16)
    Wo = (torch.randn(K, K, generator=g) / K ** 0.5).to(DEV).to(torch.bfloat16)
    bo = (torch.randn(K, generator=g) * 0.1).to(DEV).to(torch.bfloat16)
    new, psums = ops.batch_linear(o, Wo, bo, resid=stream, want_sums=True)
    lin = F.linear(o.float(), Wo.float(), bo.float()).to(torch.bfloat16)
    want = (stream.float() + lin.float()).to(torch.bfloat16)
    assert rel_err(new.float().cpu(), want.float().cpu()) <= 4e-3
    assert tuple(psums.shape) == (K // 16, B, 2)
    tot = psums.sum(0)
    assert torch.allclose(tot[:, 0].cpu(), new.float().sum(1).cpu(), rtol=1e-4, atol=1e-2)
    assert torch.allclose(tot[:, 1].cpu(), (new.float() ** 2).sum(1).cpu(), rtol=1e-4, atol=1e-2)
    xe, se = ops.decode_embed(torch.arange(B, device=DEV), torch.tensor([3], device=DEV), W[:64].contiguous(), W[100:120].contiguous(), want_sums=True)
    assert torch.allclose(se[0, :, 0].cpu(), xe.float().sum(1).cpu(), rtol=1e-4, atol=1e-3)
    assert torch.allclose(se[0, :, 1].cpu(), (xe.float() ** 2).sum(1).cpu(), rtol=1e-4, atol=1e-3)


def test_every_kernel_bench_case_launches():
    """The timed cases of pragnosia_b200.kernel_bench (what bench.py's per-kernel table and the profiling commands run):
    each one builds its inputs, launches once and leaves the wait-error flag clear."""
    from pragnosia_b200 import kernel_bench as kb
    with torch.no_grad():
        for name in sorted(kb.CASES):
            fn, alg = kb.CASES[name][0]()
            fn()
            torch.cuda.synchronize()
            assert alg > 0, name
            del fn
    out = ctypes.c_int(-1)
    _lib.check(_lib.lib().pgb_tc_error_flag(ctypes.byref(out)), "pgb_tc_error_flag")
    assert out.value == 0
