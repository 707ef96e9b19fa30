"""The CPU oracle against outputs of the reference itself (fixtures made by tests/golden/make_golden.py)."""
import torch
import torch.nn.functional as F
import pytest

import oracle
from oracle import rel_err
from pragnosia_b200 import synth

torch.set_grad_enabled(False)


def checksum(*ts):
    return float(sum(t.double().abs().sum() for t in ts))


def close(a, b, tol):
    assert a.shape == b.shape
    e = rel_err(a, b)
    assert e <= tol, f"rel err {e:.3e} > {tol}"


def test_plain_and_delta_fp64_chunk_independent(golden):
    G = golden("plain_fp64")
    q, k, v, la, be, S0 = (G[n] for n in ("q", "k", "v", "la", "beta", "S0"))
    lit_o, lit_S = oracle.plain_literal(q, k, v, la, S0)
    dl_o, dl_S = oracle.delta_literal(q, k, v, la, be, S0)
    for c in (8, 45, 1):
        o, S = oracle.assoc_scan(q, k, v, la, S0, chunk=c)
        assert torch.allclose(o, G[f"plain_c{c}"][0], atol=1e-11) and torch.allclose(S, G[f"plain_c{c}"][1], atol=1e-11)
        assert torch.allclose(o, lit_o, atol=1e-11) and torch.allclose(S, lit_S, atol=1e-11)
        o, S = oracle.assoc_scan(q, k, v, la, S0, chunk=c, beta=be)
        assert torch.allclose(o, G[f"delta_c{c}"][0], atol=1e-10) and torch.allclose(S, G[f"delta_c{c}"][1], atol=1e-10)
        assert torch.allclose(o, dl_o, atol=1e-10) and torch.allclose(S, dl_S, atol=1e-10)
    o, S = oracle.assoc_scan(q, k, v, la, None, chunk=8)
    assert torch.allclose(o, G["plain_nostate"][0], atol=1e-11)
    a, st = oracle.assoc_scan(q[:, :, :20], k[:, :, :20], v[:, :, :20], la[:, :, :20], S0, chunk=8)
    b, st2 = oracle.assoc_scan(q[:, :, 20:], k[:, :, 20:], v[:, :, 20:], la[:, :, 20:], st, chunk=8)
    assert torch.allclose(torch.cat([a, b], 2), G["plain_two_windows"][0], atol=1e-11)
    assert torch.allclose(st2, G["plain_two_windows"][1], atol=1e-11)
    assert torch.allclose(oracle.rotate(q, G["theta"], torch.arange(1000, 1045)), G["rot_q"], atol=1e-12)


def test_rotation_is_relative():
    th = torch.rand(1, 4) * 0.3; qq = torch.randn(1, 1, 1, 8); kk = torch.randn(1, 1, 1, 8)
    s1 = (oracle.rotate(qq, th, torch.tensor([10])) * oracle.rotate(kk, th, torch.tensor([3]))).sum()
    s2 = (oracle.rotate(qq, th, torch.tensor([107])) * oracle.rotate(kk, th, torch.tensor([100]))).sum()
    assert abs(s1.item() - s2.item()) < 1e-4


def test_cfg0_full_size(golden):
    G = golden("cfg0")
    x = synth.assoc_op_inputs(2, 12, 512, 64, seed=0)
    assert abs(checksum(x["q"], x["k"], x["v"], x["la"]) - G["check"]) < 1e-6 * G["check"]
    qr, kr = oracle.rotate(x["q"], x["theta"], x["pos"]), oracle.rotate(x["k"], x["theta"], x["pos"])
    o, S = oracle.assoc_scan(qr, kr, x["v"], x["la"], None, chunk=64)
    close(o[:, :, ::8], G["o_sub"], 2e-6); close(S, G["S"], 2e-6)
    close(o[:, :, ::8], G["o_sub_literal"], 5e-6); close(S, G["S_literal"], 5e-6)
    assert o.transpose(1, 2).reshape(2, 512, 768).shape == (2, 512, 768)


@pytest.mark.parametrize("D", [64, 128])
def test_ragged_carried_both_rules(golden, D):
    G = golden("ragged")[D]
    x = synth.assoc_op_inputs(2, 3, 333, D, seed=10 + D, delta=True, with_state=True)
    assert abs(checksum(x["q"], x["k"], x["v"], x["la"], x["beta"], x["S0"]) - G["check"]) < 1e-6 * G["check"]
    qr, kr = oracle.rotate(x["q"], x["theta"], x["pos"]), oracle.rotate(x["k"], x["theta"], x["pos"])
    o, S = oracle.assoc_scan(qr, kr, x["v"], x["la"], x["S0"], chunk=64)
    close(o[:, :, ::4], G["o"], 2e-6); close(S, G["S"], 2e-6)
    o, S = oracle.assoc_scan(qr, kr, x["v"], x["la"], x["S0"], chunk=64, beta=x["beta"])
    close(o[:, :, ::4], G["od"], 1e-5); close(S, G["Sd"], 1e-5)
    # the literal delta recurrence on a slice, O(1) memory
    ol, Sl = oracle.delta_literal(qr[:1, :1].double(), kr[:1, :1].double(), x["v"][:1, :1].double(),
                                  x["la"][:1, :1].double(), x["beta"][:1, :1].double(), x["S0"][:1, :1].double())
    close(o[:1, :1], ol, 1e-5); close(S[:1, :1], Sl, 1e-5)


def test_delta_known_answers(golden):
    G = golden("delta_kat")
    K, V = G["overwrite"]["K"], G["overwrite"]["V"]
    z, one = torch.zeros(1, 1, 3, dtype=torch.float64), torch.ones(1, 1, 3, dtype=torch.float64)
    r1 = oracle.assoc_scan(K, K, V, z, None, chunk=1, beta=one)[0]
    r3 = oracle.assoc_scan(K, K, V, z, None, chunk=3, beta=one)[0]
    rp = oracle.assoc_scan(K, K, V, z, None, chunk=3)[0]
    assert torch.allclose(r1[0, 0, 1], V[0, 0, 1], atol=1e-9)                     # second write replaces the first
    assert torch.allclose(rp[0, 0, 1], V[0, 0, 0] + V[0, 0, 1], atol=1e-9)        # plain rule: the sum
    assert torch.allclose(r1, r3, atol=1e-10)
    for a, n in ((r1, "delta_c1"), (r3, "delta_c3"), (rp, "plain_c3")):
        assert torch.allclose(a, G["overwrite"][n], atol=1e-12)
    g = torch.Generator().manual_seed(1)
    Kr = F.normalize(torch.randn(2, 4, 256, 64, generator=g), dim=-1)
    Vr = F.normalize(torch.randn(2, 4, 256, 64, generator=g), dim=-1)
    assert abs(checksum(Kr, Vr) - G["correlated"]["check"]) < 1e-6 * G["correlated"]["check"]
    z, one = torch.zeros(2, 4, 256), torch.ones(2, 4, 256)
    y16, S16 = oracle.assoc_scan(Kr, Kr, Vr, z, None, chunk=16, beta=one)
    y256, _ = oracle.assoc_scan(Kr, Kr, Vr, z, None, chunk=256, beta=one)
    assert S16.abs().max().item() < 2.0
    assert (y16 - y256).abs().max().item() < 1e-5
    close(y16[:, :, ::8], G["correlated"]["y16"], 1e-5); close(S16, G["correlated"]["S16"], 1e-5)
    R = G["repeated"]
    k = R["k"].expand(1, 1, 128, 64).contiguous()
    be = torch.full((1, 1, 128), 0.99999, dtype=torch.float64); la = torch.full((1, 1, 128), -1e-4, dtype=torch.float64)
    o, S = oracle.assoc_scan(R["q"], k, R["v"], la, None, chunk=64, beta=be)
    assert torch.allclose(o, R["o"], atol=1e-9) and torch.allclose(S, R["S"], atol=1e-9)
    N = be.view(1, 1, 2, 64, 1) * (k.view(1, 1, 2, 64, 64) @ k.view(1, 1, 2, 64, 64).transpose(-1, -2)).tril(-1)
    X = oracle.unit_lower_inverse(N)
    assert abs(X.abs().max().item() - R["X_absmax"]) < 1e-9 and X.abs().max().item() <= 1.0 + 1e-9


def test_lambda_scan(golden):
    G = golden("lambda_scan")
    f = G["fp64"]
    u, lm, an, h0 = f["u"], f["lm"], f["an"], f["h0"]
    yl, (rl, il) = oracle.lambda_literal(u, lm, an, h0)
    for c, key in ((8, "c8"), (45, "c45")):
        y, (hr, hi) = oracle.lambda_scan(u, lm, an, h0, chunk=c)
        for a, b in ((y, f[key][0]), (hr, f[key][1][0]), (hi, f[key][1][1]), (y, yl), (hr, rl), (hi, il)):
            assert torch.allclose(a, b, atol=1e-12)
    y, _ = oracle.lambda_scan(u, lm, an, None, chunk=8)
    assert torch.allclose(y, f["nostate"][0], atol=1e-12)
    a, st = oracle.lambda_scan(u[:, :20], lm[:, :20], an[:, :20], h0, chunk=8)
    b, _ = oracle.lambda_scan(u[:, 20:], lm[:, 20:], an[:, 20:], st, chunk=8)
    assert torch.allclose(torch.cat([a, b], 1), yl, atol=1e-12)
    g = torch.Generator().manual_seed(6)
    u = torch.randn(2, 45, 300, generator=g); lm = -torch.rand(2, 45, 300, generator=g) * 8; an = torch.randn(2, 45, 300, generator=g)
    h0 = (torch.randn(2, 300, generator=g), torch.randn(2, 300, generator=g))
    d = G["d300"]
    assert abs(checksum(u, lm, an, *h0) - d["check"]) < 1e-6 * d["check"]
    y, (hr, hi) = oracle.lambda_literal(u.double(), lm.double(), an.double(), (h0[0].double(), h0[1].double()))
    assert torch.allclose(y, d["y"], atol=1e-11) and torch.allclose(hr, d["hr"], atol=1e-11) and torch.allclose(hi, d["hi"], atol=1e-11)
    y32, (r32, i32) = oracle.lambda_literal(u, lm, an, h0)
    assert (y32 - d["y"].float()).abs().max().item() < 1e-5 and (i32 - d["hi"].float()).abs().max().item() < 1e-5
    x = synth.lambda_scan_inputs(2, 2048, 96, seed=4, with_state=True)
    s = G["cfg4_slice"]
    assert abs(checksum(x["u"], x["logmag"], x["ang"]) - s["check"]) < 1e-6 * s["check"]
    y, (hr, hi) = oracle.lambda_literal(x["u"].double(), x["logmag"].double(), x["ang"].double(),
                                        (x["h0"][0].double(), x["h0"][1].double()))
    assert torch.allclose(y[:, ::16], s["y"], atol=1e-10) and torch.allclose(hi, s["hi"], atol=1e-10)
    uf = torch.randn(2, 512, 8); lmf = -torch.rand(2, 512, 8) * 30.0; anf = torch.randn(2, 512, 8)
    assert torch.isfinite(oracle.lambda_scan(uf, lmf, anf, None, chunk=16)[0]).all()


LAYERS = (("plain_d64", 64, 1, False), ("delta_d128_h2", 128, 2, True), ("plain_d128_hd128", 128, 1, False),
          ("delta_d256_hd128", 256, 2, True))


@pytest.mark.parametrize("name,d,heads,delta", LAYERS)
def test_assoc_layer(golden, name, d, heads, delta):
    G = golden("layers")[name]
    g = torch.Generator().manual_seed(len(name))
    P = oracle.init_assoc_params({}, "", d, heads, delta, g, jitter=0.3)
    x = torch.randn(2, 70, d, generator=g)
    assert abs(checksum(x, *P.values()) - G["check"]) < 1e-6 * G["check"]
    kw = dict(heads=heads, delta=delta)
    y, (S, p) = oracle.assoc_layer(P, "", x, None, **kw)
    assert p == G["p"] == 70 and tuple(S.shape) == (2, heads, d // heads, d // heads)
    close(y, G["y"], 2e-5); close(S, G["S"], 2e-5)
    ya, sa = oracle.assoc_layer(P, "", x[:, :30], None, **kw)
    yb, (Sb, pb) = oracle.assoc_layer(P, "", x[:, 30:], sa, **kw)
    close(torch.cat([ya, yb], 1), G["y_windows"], 2e-5); close(Sb, G["S_windows"], 2e-5); assert pb == G["p_windows"]
    close(torch.cat([ya, yb], 1), y, 1e-4)                                        # carried windows == one pass
    st = sa; steps = []
    for t in range(30, 40):
        yt, st = oracle.assoc_layer(P, "", x[:, t:t + 1], st, **kw); steps.append(yt)
    close(torch.cat(steps, 1), G["y_steps"], 2e-5); close(st[0], G["S_steps"], 2e-5); assert st[1] == G["p_steps"] == 1
    close(torch.cat(steps, 1), y[:, 30:40], 1e-4)                                 # decode steps == one pass
    # strict causality: editing token 50 changes nothing before it, bit for bit
    x2 = x.clone(); x2[:, 50] += 3.0
    y2, _ = oracle.assoc_layer(P, "", x2, None, **kw)
    assert torch.equal(y2[:, :50], y[:, :50])


def test_decode_step_algebra():
    """decode_step == the layer's T=1 path on prepared vectors (rebase, then the rank-1 update)."""
    x = synth.assoc_op_inputs(2, 3, 1, 64, seed=3, delta=True, with_state=True)
    q, k, v = x["q"][:, :, 0], x["k"][:, :, 0], x["v"][:, :, 0]
    for beta in (None, x["beta"][:, :, 0]):
        S0 = oracle.decode_rebase(x["S0"], x["theta"], 17.0)
        o_ref, S_ref = oracle.assoc_scan(x["q"], x["k"], x["v"], x["la"], S0, chunk=1,
                                         beta=None if beta is None else x["beta"])
        o, S = oracle.decode_step(x["S0"], 17.0, q, k, v, x["la"][:, :, 0], x["theta"], beta)
        close(o, o_ref[:, :, 0], 1e-6); close(S, S_ref, 1e-6)


def test_fspin_layer(golden):
    G = golden("layers")["fspin_d48"]
    g = torch.Generator().manual_seed(48)
    P = oracle.init_fspin_params({}, "", 48, g, jitter=0.3)
    x = torch.randn(2, 70, 48, generator=g)
    assert abs(checksum(x, *P.values()) - G["check"]) < 1e-6 * G["check"]
    y, h = oracle.fspin_layer(P, "", x)
    close(y, G["y"], 1e-5); close(h[0], G["h"][0], 1e-5); close(h[1], G["h"][1], 1e-5)
    ya, ha = oracle.fspin_layer(P, "", x[:, :30]); yb, hb = oracle.fspin_layer(P, "", x[:, 30:], ha)
    close(torch.cat([ya, yb], 1), G["y_windows"], 1e-5); close(hb[1], G["h_windows"][1], 1e-5)


@pytest.mark.parametrize("mixer,norm", [("aspin", "ln"), ("aspin", "rms"), ("dspin", "ln"), ("hspin", "rms"),
                                        ("hdspin", "ln"), ("fspin", "ln")])
def test_lm_windows_and_decode(golden, mixer, norm):
    G = golden("lm")[f"{mixer}_{norm}"]
    cfg = oracle.lm_config(vocab=256, d=128, layers=2, mlp_mult=2, ctx=32, mixer=mixer, norm=norm)
    P = oracle.init_lm_params(cfg, seed=7, jitter=0.2)
    assert abs(checksum(*P.values()) - G["check"]) < 1e-6 * G["check"]
    ids = synth.token_ids(2, 96, 256, seed=11)
    logits = oracle.lm_forward_carried(P, cfg, ids)
    assert tuple(logits.shape) == (2, 32, 256)
    close(logits, G["logits"], 5e-5)
    lg, states = oracle.lm_prefill(P, cfg, ids[:, :40])
    out = [lg[:, -1]]; pw = 40 % 32
    for t in range(40, 46):
        out.append(oracle.lm_decode_step(P, cfg, ids[:, t], pw, states)); pw = (pw + 1) % 32
    close(torch.stack(out, 1), G["decode_logits"], 5e-5)
    close(states[0][0], G["state0"], 5e-5)


def test_param_count_matches_reference_model():
    """LM(8192, 768, 12, 4, 512, 'aspin') has 91.93 M parameters (12 heads x 64)."""
    cfg = oracle.lm_config(norm="ln")
    n = sum(v.numel() for v in oracle.init_lm_params(cfg, 0).values())
    assert cfg["heads"] == 12 and abs(n / 1e6 - 91.93) < 0.01, n
