"""Generate the golden fixtures in this folder by running the REFERENCE ITSELF (imported read-only) on CPU.

Run where the reference checkout is available:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

It writes tests/golden/*.pt. Inputs come from seeds (pragnosia_b200.synth and oracle.init_*_params), so a fixture
holds only outputs (subsampled where large) plus a checksum of its inputs; tests/test_oracle_golden.py regenerates
the inputs from the same seeds, checks the checksum, and compares the oracle with the stored reference outputs.
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
if len(sys.argv) < 2:
    raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference repository>")
REF = sys.argv[1]
sys.path.insert(0, REF)

import oracle                                                    # noqa: E402
from pragnosia_b200 import synth                                 # noqa: E402
from src.assoc import AssocCarrier, assoc_scan, rotate, _unit_lower_inverse   # noqa: E402  (the reference)
from src.spin import SpinCarrier                                 # noqa: E402
from src.model import LM                                         # noqa: E402

torch.set_grad_enabled(False)


def checksum(*ts) -> float:
    return float(sum(t.double().abs().sum() for t in ts))


def save(name, obj):
    torch.save(obj, HERE / f"{name}.pt")
    print(f"  {name}.pt  {(HERE / f'{name}.pt').stat().st_size / 1024:.0f} KiB")


# ------------------------------------------------------------------ 1. fp64 small scan with a carried state
def plain_fp64():
    g = torch.Generator().manual_seed(100)
    B, H, T, D = 2, 3, 45, 8
    q, k, v = (torch.randn(B, H, T, D, generator=g, dtype=torch.float64) for _ in range(3))
    la = -torch.rand(B, H, T, generator=g, dtype=torch.float64) * 3.0
    be = torch.rand(B, H, T, generator=g, dtype=torch.float64)
    S0 = torch.randn(B, H, D, D, generator=g, dtype=torch.float64)
    out = dict(q=q, k=k, v=v, la=la, beta=be, S0=S0)
    for c in (8, 45, 1):
        out[f"plain_c{c}"] = assoc_scan(q, k, v, la, S0, chunk=c)
        out[f"delta_c{c}"] = assoc_scan(q, k, v, la, S0, chunk=c, beta=be)
    out["plain_nostate"] = assoc_scan(q, k, v, la, None, chunk=8)
    a, st = assoc_scan(q[:, :, :20], k[:, :, :20], v[:, :, :20], la[:, :, :20], S0, chunk=8)
    b, st2 = assoc_scan(q[:, :, 20:], k[:, :, 20:], v[:, :, 20:], la[:, :, 20:], st, chunk=8)
    out["plain_two_windows"] = (torch.cat([a, b], 2), st2)
    th = torch.rand(H, D // 2, generator=g, dtype=torch.float64) * 0.3
    pos = torch.arange(1000, 1000 + T)
    out["theta"] = th
    out["rot_q"] = rotate(q, th, pos)
    save("plain_fp64", out)


# ------------------------------------------------------------------ 2. configuration 0 at full size
def cfg0():
    x = synth.assoc_op_inputs(2, 12, 512, 64, seed=0)
    qr, kr = rotate(x["q"], x["theta"], x["pos"]), rotate(x["k"], x["theta"], x["pos"])
    o, S = assoc_scan(qr, kr, x["v"], x["la"], None, chunk=64)
    o1, S1 = assoc_scan(qr, kr, x["v"], x["la"], None, chunk=1)        # the literal recurrence
    save("cfg0", dict(check=checksum(x["q"], x["k"], x["v"], x["la"]), o_sub=o[:, :, ::8].clone(), S=S,
                      o_sub_literal=o1[:, :, ::8].clone(), S_literal=S1))


# ------------------------------------------------------------------ 3. ragged T, carried state, both rules, D 64 / 128
def ragged():
    out = {}
    for D in (64, 128):
        x = synth.assoc_op_inputs(2, 3, 333, D, seed=10 + D, delta=True, with_state=True)
        qr, kr = rotate(x["q"], x["theta"], x["pos"]), rotate(x["k"], x["theta"], x["pos"])
        o, S = assoc_scan(qr, kr, x["v"], x["la"], x["S0"], chunk=64)
        od, Sd = assoc_scan(qr, kr, x["v"], x["la"], x["S0"], chunk=64, beta=x["beta"])
        out[D] = dict(check=checksum(x["q"], x["k"], x["v"], x["la"], x["beta"], x["S0"]),
                      o=o[:, :, ::4].clone(), S=S, od=od[:, :, ::4].clone(), Sd=Sd)
    save("ragged", out)


# ------------------------------------------------------------------ 4. delta-rule known answers
def delta_kat():
    out = {}
    g = torch.Generator().manual_seed(4)
    kk = F.normalize(torch.randn(1, 1, 1, 4, generator=g, dtype=torch.float64), dim=-1)
    va = torch.tensor([[[[1., 0, 0, 0]]]], dtype=torch.float64)
    vb = torch.tensor([[[[0., 1., 0, 0]]]], dtype=torch.float64)
    Kd, Vd = torch.cat([kk, kk, kk], 2), torch.cat([va, vb, va], 2)
    lad, bed = torch.zeros(1, 1, 3, dtype=torch.float64), torch.ones(1, 1, 3, dtype=torch.float64)
    out["overwrite"] = dict(K=Kd, V=Vd, delta_c1=assoc_scan(Kd, Kd, Vd, lad, None, chunk=1, beta=bed)[0],
                            delta_c3=assoc_scan(Kd, Kd, Vd, lad, None, chunk=3, beta=bed)[0],
                            plain_c3=assoc_scan(Kd, Kd, Vd, lad, None, chunk=3)[0])
    # 256 correlated writes with beta = 1 and no decay (the case the Jacobi form diverged on)
    g = torch.Generator().manual_seed(1)
    Kr = F.normalize(torch.randn(2, 4, 256, 64, generator=g), dim=-1)
    Vr = F.normalize(torch.randn(2, 4, 256, 64, generator=g), dim=-1)
    z, one = torch.zeros(2, 4, 256), torch.ones(2, 4, 256)
    y16, S16 = assoc_scan(Kr, Kr, Vr, z, None, chunk=16, beta=one)
    y256, S256 = assoc_scan(Kr, Kr, Vr, z, None, chunk=256, beta=one)
    out["correlated"] = dict(check=checksum(Kr, Vr), y16=y16[:, :, ::8].clone(), S16=S16, y256=y256[:, :, ::8].clone())
    # one key repeated 128 times with beta -> 1: the true inverse has max |X| = 1 (the failure a reduced-precision
    # doubling produced is described at src/assoc_kernel.py:577-582)
    g = torch.Generator().manual_seed(2)
    k1 = F.normalize(torch.randn(1, 1, 1, 64, generator=g, dtype=torch.float64), dim=-1).expand(1, 1, 128, 64).contiguous()
    v1 = F.normalize(torch.randn(1, 1, 128, 64, generator=g, dtype=torch.float64), dim=-1)
    q1 = F.normalize(torch.randn(1, 1, 128, 64, generator=g, dtype=torch.float64), dim=-1)
    be = torch.full((1, 1, 128), 0.99999, dtype=torch.float64); la = torch.full((1, 1, 128), -1e-4, dtype=torch.float64)
    o, S = assoc_scan(q1, k1, v1, la, None, chunk=64, beta=be)
    N = be.view(1, 1, 2, 64, 1) * (k1.view(1, 1, 2, 64, 64) @ k1.view(1, 1, 2, 64, 64).transpose(-1, -2)).tril(-1)
    X = _unit_lower_inverse(N)
    out["repeated"] = dict(k=k1[:, :, :1].clone(), v=v1, q=q1, o=o, S=S, X_absmax=float(X.abs().max()))
    save("delta_kat", out)


# ------------------------------------------------------------------ 5. per-token lambda scan
def lam():
    out = {}
    g = torch.Generator().manual_seed(5)
    B, T, D = 2, 45, 6
    u = torch.randn(B, T, D, generator=g, dtype=torch.float64)
    lm = -torch.rand(B, T, D, generator=g, dtype=torch.float64) * 8.0
    lm[:, :, 0] = -1e-3
    an = torch.randn(B, T, D, generator=g, dtype=torch.float64)
    h0 = (torch.randn(B, D, generator=g, dtype=torch.float64), torch.randn(B, D, generator=g, dtype=torch.float64))
    out["fp64"] = dict(u=u, lm=lm, an=an, h0=h0, c8=SpinCarrier.scan_gated(u, lm, an, h0, chunk=8),
                       c45=SpinCarrier.scan_gated(u, lm, an, h0, chunk=45),
                       nostate=SpinCarrier.scan_gated(u, lm, an, None, chunk=8))
    g = torch.Generator().manual_seed(6)
    B, T, D = 2, 45, 300
    u = torch.randn(B, T, D, generator=g); lm = -torch.rand(B, T, D, generator=g) * 8; an = torch.randn(B, T, D, generator=g)
    h0 = (torch.randn(B, D, generator=g), torch.randn(B, D, generator=g))
    y, (hr, hi) = SpinCarrier.scan_gated(u.double(), lm.double(), an.double(), (h0[0].double(), h0[1].double()), chunk=8)
    out["d300"] = dict(check=checksum(u, lm, an, *h0), y=y, hr=hr, hi=hi)
    x = synth.lambda_scan_inputs(2, 2048, 96, seed=4, with_state=True)
    y, (hr, hi) = SpinCarrier.scan_gated(x["u"].double(), x["logmag"].double(), x["ang"].double(),
                                         (x["h0"][0].double(), x["h0"][1].double()), chunk=16)
    out["cfg4_slice"] = dict(check=checksum(x["u"], x["logmag"], x["ang"]), y=y[:, ::16].clone(), hr=hr, hi=hi)
    save("lambda_scan", out)


# ------------------------------------------------------------------ 6. the carrier layers as modules
def layers():
    out = {}
    for name, d, heads, delta, hd in (("plain_d64", 64, 1, False, None), ("delta_d128_h2", 128, 2, True, None),
                                      ("plain_d128_hd128", 128, 1, False, 128), ("delta_d256_hd128", 256, 2, True, 128)):
        g = torch.Generator().manual_seed(len(name))
        P = oracle.init_assoc_params({}, "", d, heads, delta, g, jitter=0.3)
        m = AssocCarrier(d, heads=heads, delta=delta, head_dim=hd)
        m.load_state_dict(P, strict=True)
        x = torch.randn(2, 70, d, generator=g)
        y, (S, p) = m(x)
        ya, sa = m(x[:, :30]); yb, (Sb, pb) = m(x[:, 30:], h0=sa)
        # decode: a 30-token pass, then 10 single-token steps with the carried state
        st = sa; steps = []
        for t in range(30, 40):
            yt, st = m(x[:, t:t + 1], h0=st); steps.append(yt)
        out[name] = dict(check=checksum(x, *P.values()), y=y, S=S, p=p, y_windows=torch.cat([ya, yb], 1), S_windows=Sb,
                         p_windows=pb, y_steps=torch.cat(steps, 1), S_steps=st[0], p_steps=st[1])
    g = torch.Generator().manual_seed(48)
    P = oracle.init_fspin_params({}, "", 48, g, jitter=0.3)
    m = SpinCarrier(48, gated="rf"); m.load_state_dict(P, strict=True)
    x = torch.randn(2, 70, 48, generator=g)
    y, h = m(x)
    ya, ha = m(x[:, :30]); yb, hb = m(x[:, 30:], h0=ha)
    out["fspin_d48"] = dict(check=checksum(x, *P.values()), y=y, h=h, y_windows=torch.cat([ya, yb], 1), h_windows=hb)
    save("layers", out)


# ------------------------------------------------------------------ 7. the language model: windows and decode steps
def lm():
    out = {}
    for mixer, norm in (("aspin", "ln"), ("aspin", "rms"), ("dspin", "ln"), ("hspin", "rms"), ("hdspin", "ln"), ("fspin", "ln")):
        cfg = oracle.lm_config(vocab=256, d=128, layers=2, mlp_mult=2, ctx=32, mixer=mixer, norm=norm)
        P = oracle.init_lm_params(cfg, seed=7, jitter=0.2)
        m = LM(vocab=256, d=128, layers=2, mlp_mult=2, ctx=32, mixer=mixer, norm=norm).eval()
        m.load_state_dict(P, strict=True)
        ids = synth.token_ids(2, 96, 256, seed=11)
        logits = m.forward_carried(ids)
        # the eager decode loop of src/bench.py:206-238 on a 40-token prompt, batch-generic, teacher-forced
        w = 32; states = [None] * 2; pw = 0; h = None
        for s in range(0, 40, w):
            xw = ids[:, s:min(s + w, 40)]; n = xw.shape[1]
            h = m.e(xw) + m.p(torch.arange(n))
            for i, (mx, mp) in enumerate(zip(m.mix, m.mlp)):
                h, states[i] = mx(h, states[i]); h = mp(h)
            pw = n % w
        lg = [F.linear(m.n(h[:, -1:]), m.e.weight)[:, -1]]
        for t in range(40, 46):
            h = m.e(ids[:, t:t + 1]) + m.p(torch.tensor([pw]))
            for i, (mx, mp) in enumerate(zip(m.mix, m.mlp)):
                h, states[i] = mx(h, states[i]); h = mp(h)
            lg.append(F.linear(m.n(h), m.e.weight)[:, -1]); pw = (pw + 1) % w
        out[f"{mixer}_{norm}"] = dict(check=checksum(*P.values()), logits=logits, decode_logits=torch.stack(lg, 1),
                                      state0=states[0][0])
    save("lm", out)


# ------------------------------------------------------------------ 8. the layer's options
def options():
    """AssocCarrier with each option of src/assoc.py on: one 70-token pass, two carried windows, ten T=1 steps."""
    out = {}
    cases = (("topk", dict(key_topk=8), False), ("floor", dict(hl_floor=True), False), ("write_all", dict(write_all=True), False),
             ("write_all_delta", dict(write_all=True), True), ("pos_wrap", {}, False), ("beta_scale", {}, True),
             ("sconv", {}, False), ("sconv_delta_topk", dict(key_topk=16), True))
    for name, kw, delta in cases:
        g = torch.Generator().manual_seed(1000 + len(name))
        d, heads = 128, 2
        P = oracle.init_assoc_params({}, "", d, heads, delta, g, jitter=0.3)
        m = AssocCarrier(d, heads=heads, delta=delta, **kw)
        if name.startswith("sconv"):
            m.add_short_conv(4)
            P["sconv"] = m.sconv.detach().clone() + 0.3 * torch.randn(3 * d, 4, generator=g)
        m.load_state_dict(P, strict=True)
        if name == "pos_wrap":
            m.pos_wrap = 16
        x = torch.randn(2, 70, d, generator=g)
        extra = {}
        if name == "beta_scale":
            extra["beta_scale"] = torch.rand(2, heads, 70, generator=g)
            m.beta_scale = extra["beta_scale"]
            y, st = m(x)
            out[name] = dict(check=checksum(x, *P.values()), y=y, S=st[0], **extra)
            continue
        y, st = m(x)
        ya, sa = m(x[:, :30]); yb, sb = m(x[:, 30:], h0=sa)
        cur = sa; steps = []
        for t in range(30, 40):
            yt, cur = m(x[:, t:t + 1], h0=cur); steps.append(yt)
        rec = dict(check=checksum(x, *P.values()), y=y, S=st[0], y_windows=torch.cat([ya, yb], 1), S_windows=sb[0],
                   y_steps=torch.cat(steps, 1), S_steps=cur[0])
        if name.startswith("sconv"):
            rec["cc"] = st[2]; rec["cc_steps"] = cur[2]
        out[name] = rec
    save("options", out)


# ------------------------------------------------------------------ 9. gradients of the two simplest operators
def grads():
    """The reference's gradients for the lambda scan (tests/test_spin.py:237-246: B2 T45 D300, carried h0, loss through
    Re h, the final Re and the final Im state; autograd through its fp64 scan_gated) and for the plumbing before the scan
    (tests/test_assoc.py:189-212: its torch form prep_ref, differentiated by autograd)."""
    out = {}
    torch.set_grad_enabled(True)
    g = torch.Generator().manual_seed(6)
    B, T, D = 2, 45, 300
    u = torch.randn(B, T, D, generator=g); lm = -torch.rand(B, T, D, generator=g) * 8; an = torch.randn(B, T, D, generator=g)
    h0 = (torch.randn(B, D, generator=g), torch.randn(B, D, generator=g))
    w, wl, wi = torch.randn(B, T, D, generator=g), torch.randn(B, D, generator=g), torch.randn(B, D, generator=g)
    a64 = [t.double().requires_grad_(True) for t in (u, lm, an, h0[0], h0[1])]
    y, (r, i) = SpinCarrier.scan_gated(a64[0], a64[1], a64[2], (a64[3], a64[4]), chunk=8)
    ((y * w).sum() + (r * wl).sum() + (i * wi).sum()).backward()
    out["lambda"] = dict(check=checksum(u, lm, an, *h0, w, wl, wi), grads=[t.grad.float() for t in a64])

    def prep_ref(qp, kp, vp, gl, theta, pos):                     # tests/test_assoc.py:189-193
        q_, k_, v_ = [F.normalize(t.transpose(1, 2).float(), dim=-1) for t in (qp, kp, vp)]
        if gl is not None:
            k_ = k_ * torch.sigmoid(gl.float()).transpose(1, 2).unsqueeze(-1)
        return rotate(q_, theta, pos), rotate(k_, theta, pos), v_
    out["prep"] = {}
    for Dk, Tp, gate, p0 in ((64, 2048, True, 0), (64, 333, False, 1000), (128, 512, True, 4096)):
        g = torch.Generator().manual_seed(Dk + Tp)
        Hp = 3
        mk = lambda: (torch.randn(2, Tp, Hp, Dk, generator=g) * 3).to(torch.bfloat16).requires_grad_()
        qp, kp, vp = mk(), mk(), mk()
        gl = (torch.randn(2, Tp, Hp, generator=g) * 2).to(torch.bfloat16).requires_grad_() if gate else None
        th = (10000.0 ** (-torch.arange(0, Dk, 2).float() / Dk)).unsqueeze(0).repeat(Hp, 1).requires_grad_()
        pos = p0 + torch.arange(Tp)
        refs = prep_ref(qp, kp, vp, gl, th, pos)
        ws = [torch.randn(r.shape, generator=g) for r in refs]
        ins = [qp, kp, vp, th] + ([gl] if gate else [])
        gr = torch.autograd.grad(sum((r * w_).sum() for r, w_ in zip(refs, ws)), ins)
        st = max(1, Tp // 64)                                     # keep every st-th token of the big tensors
        out["prep"][(Dk, Tp, gate, p0)] = dict(
            check=checksum(qp.detach().float(), kp.detach().float(), vp.detach().float(), *ws),
            outs=[r.detach()[:, :, ::st].to(torch.bfloat16).clone() for r in refs],
            dqp=gr[0][:, ::st].float().clone(), dkp=gr[1][:, ::st].float().clone(), dvp=gr[2][:, ::st].float().clone(),
            dth=gr[3].float().clone(), dgl=(gr[4][:, ::st].float().clone() if gate else None))
    torch.set_grad_enabled(False)
    save("grads", out)


ALL = (plain_fp64, cfg0, ragged, delta_kat, lam, layers, lm, options, grads)

if __name__ == "__main__":
    print(f"reference at {REF}, torch {torch.__version__}")
    want = set(sys.argv[2:])                                      # optional: names of the fixtures to (re)make
    for fn in ALL:
        if not want or fn.__name__ in want:
            print(fn.__name__); fn()
