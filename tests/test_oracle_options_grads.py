"""The CPU oracle's layer options and gradient checkers against outputs of the reference itself (options.pt, grads.pt
made by tests/golden/make_golden.py)."""
import pytest
import torch

import oracle
from oracle import rel_err

torch.set_grad_enabled(False)

CASES = (("topk", dict(key_topk=8), False), ("floor", dict(hl_floor=True), False), ("write_all", dict(write_all=True), False),
         ("write_all_delta", dict(write_all=True), True), ("pos_wrap", dict(pos_wrap=16), False), ("beta_scale", {}, True),
         ("sconv", {}, False), ("sconv_delta_topk", dict(key_topk=16), True))


def checksum(*ts):
    return float(sum(t.double().abs().sum() for t in ts))


def option_inputs(name, delta):
    """The same draws as the fixture generator: parameters, (for sconv) the convolution weights, the input."""
    g = torch.Generator().manual_seed(1000 + len(name))
    d, heads = 128, 2
    P = oracle.init_assoc_params({}, "", d, heads, delta, g, jitter=0.3)
    if name.startswith("sconv"):
        w = torch.zeros(3 * d, 4); w[:, -1] = 1.0
        P["sconv"] = w + 0.3 * torch.randn(3 * d, 4, generator=g)
    x = torch.randn(2, 70, d, generator=g)
    extra = torch.rand(2, heads, 70, generator=g) if name == "beta_scale" else None
    return P, x, extra


@pytest.mark.parametrize("name,kw,delta", CASES)
def test_layer_options_match_the_reference(golden, name, kw, delta):
    G = golden("options")[name]
    P, x, bs = option_inputs(name, delta)
    assert abs(checksum(x, *P.values()) - G["check"]) < 1e-6 * G["check"]
    run = lambda xx, h0=None, **more: oracle.assoc_layer(P, "", xx, h0, heads=2, delta=delta, **kw, **more)
    if name == "beta_scale":
        y, st = run(x, beta_scale=bs)
        assert rel_err(y, G["y"]) <= 1e-5 and rel_err(st[0], G["S"]) <= 1e-5
        return
    y, st = run(x)
    assert rel_err(y, G["y"]) <= 1e-5 and rel_err(st[0], G["S"]) <= 1e-5
    ya, sa = run(x[:, :30]); yb, sb = run(x[:, 30:], sa)
    assert rel_err(torch.cat([ya, yb], 1), G["y_windows"]) <= 1e-5 and rel_err(sb[0], G["S_windows"]) <= 1e-5
    cur, steps = sa, []
    for t in range(30, 40):
        yt, cur = run(x[:, t:t + 1], cur); steps.append(yt)
    assert rel_err(torch.cat(steps, 1), G["y_steps"]) <= 1e-5 and rel_err(cur[0], G["S_steps"]) <= 1e-5
    if name.startswith("sconv"):
        assert len(st) == 3 and rel_err(st[2], G["cc"]) <= 1e-6 and rel_err(cur[2], G["cc_steps"]) <= 1e-6


def lambda_grad_inputs():
    g = torch.Generator().manual_seed(6)
    B, T, D = 2, 45, 300
    u = torch.randn(B, T, D, generator=g); lm = -torch.rand(B, T, D, generator=g) * 8; an = torch.randn(B, T, D, generator=g)
    h0 = (torch.randn(B, D, generator=g), torch.randn(B, D, generator=g))
    w, wl, wi = torch.randn(B, T, D, generator=g), torch.randn(B, D, generator=g), torch.randn(B, D, generator=g)
    return u, lm, an, h0, w, wl, wi


def test_lambda_scan_gradients_match_the_reference(golden):
    G = golden("grads")["lambda"]
    u, lm, an, h0, w, wl, wi = lambda_grad_inputs()
    assert abs(checksum(u, lm, an, *h0, w, wl, wi) - G["check"]) < 1e-6 * G["check"]
    mine = oracle.lambda_scan_grads(u, lm, an, h0, w, wl, wi)
    for a, b in zip(mine, G["grads"]):
        assert rel_err(a.float(), b) <= 1e-5


def prep_grad_inputs(Dk, Tp, gate, p0):
    g = torch.Generator().manual_seed(Dk + Tp)
    Hp = 3
    mk = lambda: (torch.randn(2, Tp, Hp, Dk, generator=g) * 3).to(torch.bfloat16)
    qp, kp, vp = mk(), mk(), mk()
    gl = (torch.randn(2, Tp, Hp, generator=g) * 2).to(torch.bfloat16) if gate else None
    th = (10000.0 ** (-torch.arange(0, Dk, 2).float() / Dk)).unsqueeze(0).repeat(Hp, 1)
    pos = p0 + torch.arange(Tp)
    ws = [torch.randn(2, Hp, Tp, Dk, generator=g) for _ in range(3)]
    return qp, kp, vp, gl, th, pos, ws


PREP = ((64, 2048, True, 0), (64, 333, False, 1000), (128, 512, True, 4096))


@pytest.mark.parametrize("Dk,Tp,gate,p0", PREP)
def test_prep_gradients_match_the_reference(golden, Dk, Tp, gate, p0):
    G = golden("grads")["prep"][(Dk, Tp, gate, p0)]
    qp, kp, vp, gl, th, pos, ws = prep_grad_inputs(Dk, Tp, gate, p0)
    assert abs(checksum(qp.float(), kp.float(), vp.float(), *ws) - G["check"]) < 1e-6 * G["check"]
    st = max(1, Tp // 64)
    with torch.enable_grad():
        ins = [t.clone().requires_grad_() for t in (qp, kp, vp, th)] + ([gl.clone().requires_grad_()] if gate else [])
        refs = oracle.prep_ref(ins[0], ins[1], ins[2], ins[4] if gate else None, ins[3], pos)
        gr = torch.autograd.grad(sum((r * w).sum() for r, w in zip(refs, ws)), ins)
    for r, g_ in zip(refs, G["outs"]):
        assert rel_err(r.detach()[:, :, ::st], g_.float()) <= 1e-2          # the fixture keeps bf16 outputs
    assert rel_err(gr[0][:, ::st].float(), G["dqp"]) <= 1e-5 and rel_err(gr[1][:, ::st].float(), G["dkp"]) <= 1e-5
    assert rel_err(gr[2][:, ::st].float(), G["dvp"]) <= 1e-5 and rel_err(gr[3].float(), G["dth"]) <= 1e-5
    if gate:
        assert rel_err(gr[4][:, ::st].float(), G["dgl"]) <= 1e-5
