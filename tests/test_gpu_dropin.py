"""The drop-in names and the torch custom operators on the GPU: the calls a maintainer of the reference makes after swapping
its imports (assoc_scan_kernel, delta_scan_kernel, prep_kernel, scan_triton, SpinCarrier.scan_gated, LM.trunk(carry=True)),
at the reference's own test shapes (tests/test_assoc.py:146-212, tests/test_spin.py:225-258), against the CPU oracle."""
import pytest
import torch
import torch.nn.functional as F

import oracle
from oracle import rel_err
from pragnosia_b200 import custom_ops, ops, synth  # noqa: F401
from pragnosia_b200.assoc import AssocCarrier
from pragnosia_b200.assoc_kernel import assoc_scan_kernel, delta_scan_kernel, prep_kernel
from pragnosia_b200.model import LM
from pragnosia_b200.scan_kernel import scan_triton
from pragnosia_b200.spin import SpinCarrier

pytestmark = pytest.mark.gpu
DEV = "cuda"
OPS = torch.ops.pragnosia_b200


@pytest.fixture(autouse=True)
def _grad_enabled():
    """Other test modules switch autograd off process-wide; the gradient checks here need it."""
    with torch.enable_grad():
        yield


def kernel_inputs(D, seed, delta):
    """tests/test_assoc.py:150-153 / :171-174: unit q, k, v, slow decays, a carried state; B2 H3 T333."""
    g = torch.Generator().manual_seed(seed)
    q, k, v = (F.normalize(torch.randn(2, 3, 333, D, generator=g), dim=-1) for _ in range(3))
    la = -F.softplus(torch.randn(2, 3, 333, generator=g)) * 0.05
    be = torch.sigmoid(torch.randn(2, 3, 333, generator=g)) if delta else None
    S0 = torch.randn(2, 3, D, D, generator=g) * 0.1
    return q, k, v, la, be, S0


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_assoc_and_delta_scan_kernel_names(D, dtype):
    with torch.no_grad():
        q, k, v, la, be, S0 = kernel_inputs(D, D, True)
        qd, kd, vd = (t.to(DEV).to(dtype) for t in (q, k, v))
        ref_in = [t.to(dtype).float() for t in (q, k, v)]
        tol_o, tol_S = (2e-5, 2e-5) if dtype == torch.float32 else (6e-3, 1e-4)      # bf16 OUTPUT rounding: 2^-9 of the largest
        o, sfin, sent = assoc_scan_kernel(qd, kd, vd, la.to(DEV), S0.to(DEV))
        ro, rS = oracle.assoc_scan(*ref_in, la, S0)
        assert o.dtype == dtype and tuple(o.shape) == (2, 3, 333, D)
        assert sfin.dtype == torch.float32 and tuple(sfin.shape) == (2, 3, D, D)
        assert sent.dtype == torch.bfloat16 and tuple(sent.shape) == (2, 3, 6, D, D)
        assert rel_err(o.float().cpu(), ro) <= tol_o and rel_err(sfin.cpu(), rS) <= tol_S
        assert rel_err(sent[:, :, 0].float().cpu(), S0) <= 4e-3                      # the first entering state is S0, in bf16
        o, sfin, sent = delta_scan_kernel(qd, kd, vd, la.to(DEV), be.to(DEV), S0.to(DEV), chunk=64, bv=32)
        ro, rS = oracle.assoc_scan(*ref_in, la, S0, beta=be)
        assert o.dtype == dtype and sent.dtype == torch.bfloat16 and tuple(sent.shape) == (2, 3, 6, D, D)
        assert rel_err(o.float().cpu(), ro) <= tol_o and rel_err(sfin.cpu(), rS) <= tol_S
        o2, s2, _ = assoc_scan_kernel(qd, kd, vd, la.to(DEV))                         # no carried state
        ro2, rS2 = oracle.assoc_scan(*ref_in, la, None)
        assert rel_err(o2.float().cpu(), ro2) <= tol_o and rel_err(s2.cpu(), rS2) <= tol_S


PREP = ((64, 2048, True, 0), (64, 333, False, 1000), (128, 512, True, 4096))


def prep_inputs(Dk, Tp, gate, p0):
    g = torch.Generator().manual_seed(Dk + Tp)
    mk = lambda: (torch.randn(2, Tp, 3, Dk, generator=g) * 3).to(torch.bfloat16)
    qp, kp, vp = mk(), mk(), mk()
    gl = (torch.randn(2, Tp, 3, generator=g) * 2).to(torch.bfloat16) if gate else None
    th = (10000.0 ** (-torch.arange(0, Dk, 2).float() / Dk)).unsqueeze(0).repeat(3, 1)
    ws = [torch.randn(2, 3, Tp, Dk, generator=g) for _ in range(3)]
    return qp, kp, vp, gl, th, p0 + torch.arange(Tp), ws


@pytest.mark.parametrize("Dk,Tp,gate,p0", PREP)
def test_prep_kernel_name_forward_and_gradients(golden, Dk, Tp, gate, p0):
    """tests/test_assoc.py:196-212: outputs and every gradient (projections, theta, gate) against the torch form; the
    gradients are also held to the reference's own (grads.pt)."""
    qp, kp, vp, gl, th, pos, ws = prep_inputs(Dk, Tp, gate, p0)
    dev = lambda t: None if t is None else t.to(DEV)
    ins = [dev(t).requires_grad_() for t in (qp, kp, vp, th)] + ([dev(gl).requires_grad_()] if gate else [])
    outs = prep_kernel(ins[0], ins[1], ins[2], ins[4] if gate else None, ins[3], dev(pos))
    refs = oracle.prep_ref(qp, kp, vp, gl, th, pos)
    for o, r in zip(outs, refs):
        assert o.dtype == torch.bfloat16 and tuple(o.shape) == (2, 3, Tp, Dk)
        assert rel_err(o.float().cpu(), r) <= 4e-3                                   # bf16 outputs
    gk = torch.autograd.grad(sum((o.float() * dev(w)).sum() for o, w in zip(outs, ws)), ins)
    with torch.enable_grad():
        rin = [t.clone().requires_grad_() for t in (qp, kp, vp, th)] + ([gl.clone().requires_grad_()] if gate else [])
        rr = oracle.prep_ref(rin[0], rin[1], rin[2], rin[4] if gate else None, rin[3], pos)
        gr = torch.autograd.grad(sum((r * w).sum() for r, w in zip(rr, ws)), rin)
    for a, b in zip(gk, gr):
        assert a.shape == b.shape and rel_err(a.float().cpu(), b.float()) <= 1e-2
    G = golden("grads")["prep"][(Dk, Tp, gate, p0)]
    st = max(1, Tp // 64)
    assert rel_err(gk[0][:, ::st].float().cpu(), G["dqp"]) <= 1e-2 and rel_err(gk[3].float().cpu(), G["dth"]) <= 1e-2
    # run twice: bit-identical (the theta partials are summed in a fixed order)
    outs2 = prep_kernel(ins[0], ins[1], ins[2], ins[4] if gate else None, ins[3], dev(pos))
    gk2 = torch.autograd.grad(sum((o.float() * dev(w)).sum() for o, w in zip(outs2, ws)), ins)
    assert all(torch.equal(a, b) for a, b in zip(gk, gk2))


def test_scan_triton_name_forward_and_gradients(golden):
    """tests/test_spin.py:225-258: B2 T45 D300 (not a multiple of anything), carried h0, forward < 1e-5 absolute and all five
    gradients < 1e-5 relative, the no-state case, exp(-40) decays finite."""
    g = torch.Generator().manual_seed(6)
    B, T, D = 2, 45, 300
    u = torch.randn(B, T, D, generator=g); lm = -torch.rand(B, T, D, generator=g) * 8; an = torch.randn(B, T, D, generator=g)
    h0 = (torch.randn(B, D, generator=g), torch.randn(B, D, generator=g))
    w, wl, wi = torch.randn(B, T, D, generator=g), torch.randn(B, D, generator=g), torch.randn(B, D, generator=g)
    G = golden("lambda_scan")["d300"]
    with torch.no_grad():
        y, (hr, hi) = scan_triton(u.to(DEV), lm.to(DEV), an.to(DEV), tuple(t.to(DEV) for t in h0))
        assert (y.cpu() - G["y"].float()).abs().max() < 1e-5 and (hr.cpu() - G["hr"].float()).abs().max() < 1e-5
        assert (hi.cpu() - G["hi"].float()).abs().max() < 1e-5
        y0, _ = SpinCarrier.scan_gated(u.to(DEV), lm.to(DEV), an.to(DEV), None, chunk=16)
        ry0, _ = oracle.lambda_literal(u.double(), lm.double(), an.double())
        assert (y0.cpu() - ry0.float()).abs().max() < 1e-5
        yx, _ = scan_triton(torch.randn(2, 512, 8, device=DEV), torch.full((2, 512, 8), -40.0, device=DEV), torch.randn(2, 512, 8, device=DEV))
        assert torch.isfinite(yx).all()
    a32 = [t.to(DEV).requires_grad_(True) for t in (u, lm, an, h0[0], h0[1])]
    y, (r, i) = scan_triton(a32[0], a32[1], a32[2], (a32[3], a32[4]))
    ((y * w.to(DEV)).sum() + (r * wl.to(DEV)).sum() + (i * wi.to(DEV)).sum()).backward()
    ref = golden("grads")["lambda"]["grads"]
    mine = oracle.lambda_scan_grads(u, lm, an, h0, w, wl, wi)
    for a, b, c in zip(a32, ref, mine):
        assert rel_err(a.grad.cpu(), b) < 1e-5 and rel_err(a.grad.cpu(), c.float()) < 1e-5
    # a long sequence with few channels takes the segmented adjoint; many channels the one-lane-per-channel walk
    for (B2, T2, D2) in ((1, 700, 24), (3, 130, 2048)):
        s = synth.lambda_scan_inputs(B2, T2, D2, seed=9, with_state=True)
        w2 = torch.randn(B2, T2, D2, generator=g)
        ins = [s["u"], s["logmag"], s["ang"], s["h0"][0], s["h0"][1]]
        a = [t.to(DEV).requires_grad_(True) for t in ins]
        y, (r, i) = scan_triton(a[0], a[1], a[2], (a[3], a[4]))
        ((y * w2.to(DEV)).sum() + r.sum() - i.sum()).backward()
        refg = oracle.lambda_scan_grads(*ins[:3], (ins[3], ins[4]), w2, torch.ones(B2, D2), -torch.ones(B2, D2))
        for x, b in zip(a, refg):
            assert rel_err(x.grad.cpu(), b.float()) < 2e-5


def test_fspin_layer_trains_through_the_kernel():
    """SpinCarrier(gated="rf") forward + backward on the GPU against autograd through the CPU oracle layer."""
    g = torch.Generator().manual_seed(48)
    P = oracle.init_fspin_params({}, "", 48, g, jitter=0.3)
    x = torch.randn(2, 70, 48, generator=g)
    m = SpinCarrier(48, gated="rf"); m.load_state_dict(P, strict=True); m = m.to(DEV)
    y, _ = m(x.to(DEV))
    y.square().sum().backward()
    with torch.enable_grad():
        Pr = {k: v.clone().requires_grad_() for k, v in P.items()}
        yr, _ = oracle.fspin_layer(Pr, "", x)
        yr.square().sum().backward()
    for name, p in m.named_parameters():
        assert p.grad is not None and rel_err(p.grad.cpu(), Pr[name].grad) < 2e-3, name


@pytest.mark.parametrize("D", [64, 128])
def test_split_operators_compose_to_the_fused_walk(D):
    """The reference's operator set (prefix_scan + assoc_out; delta_inv + delta_loop_fwd + assoc_out), called as
    src/assoc_kernel.py:302-323 and :512-546 call them, equals the oracle and the fused kernel's triple."""
    with torch.no_grad():
        q, k, v, la, be, S0 = kernel_inputs(D, 7 + D, True)
        B, H, T = 2, 3, 333
        NC, pad = 6, 6 * 64 - T
        d = lambda t: t.to(DEV)
        qb, kb, vb = (d(t).to(torch.bfloat16) for t in (q, k, v))
        rin = [t.float().cpu() for t in (qb, kb, vb)]
        # plain rule: the glue of assoc_scan_kernel
        lc = F.pad(d(la), (0, pad)).view(B, H, NC, 64)
        L = lc.cumsum(-1); a_log = lc.sum(-1)
        w = torch.exp(a_log.unsqueeze(-1) - L).unsqueeze(-1)
        kp, vp = F.pad(kb, (0, 0, 0, pad)), F.pad(vb, (0, 0, 0, pad))
        sent, sfin = OPS.prefix_scan(kp, vp, w, a_log, d(S0), True, 16)
        o = OPS.assoc_out(qb, kb, vb, d(la), sent, 64)
        ro, rS = oracle.assoc_scan(*rin, la, S0)
        assert rel_err(o.float().cpu(), ro) <= 6e-3 and rel_err(sfin.cpu(), rS) <= 1e-4   # sent is bf16, as the reference's
        fo, fS, fsent = ops.prefill(qb, kb, vb, d(la), None, d(S0), want_sent=True)
        assert rel_err(sent.float(), fsent.float()) <= 8e-3 and rel_err(sfin, fS) <= 1e-4
        s0, f0 = OPS.prefix_scan(kp, vp, w, a_log, None, False, 16)
        assert float(s0[:, :, 0].abs().max()) == 0.0
        # delta rule: the glue of delta_scan_kernel
        X = OPS.delta_inv(kb, d(la), d(be), NC)
        assert X.dtype == torch.bfloat16 and tuple(X.shape) == (B, H, NC, 64, 64)
        kc = F.pad(rin[1], (0, 0, 0, pad)).view(B, H, NC, 64, D)
        Lr = F.pad(la, (0, pad)).view(B, H, NC, 64).cumsum(-1)
        dec = (Lr[..., :, None] - Lr[..., None, :]).clamp(max=0).exp()
        N = F.pad(be, (0, pad)).view(B, H, NC, 64, 1) * ((kc @ kc.transpose(-1, -2)) * dec).tril(-1)
        assert rel_err(X.float().cpu(), oracle.unit_lower_inverse(N)) <= 4e-3
        W, sent, sfin = OPS.delta_loop_fwd(kb, vb, d(la), d(be), X, d(S0), True, 64, 32, 16)
        o = OPS.assoc_out(qb, kb, W, d(la), sent, 64)
        ro, rS = oracle.assoc_scan(*rin, la, S0, beta=be)
        assert W.dtype == torch.bfloat16 and tuple(W.shape) == (B, H, T, D)
        assert rel_err(o.float().cpu(), ro) <= 1e-2 and rel_err(sfin.cpu(), rS) <= 1e-2   # X, W, sent in bf16: the reference's own 1e-2


def test_trunk_with_carried_state():
    """LM.trunk(x, states, carry=True) (src/model.py:759-789): two carried windows equal forward_carried's."""
    with torch.no_grad():
        cfg = oracle.lm_config(vocab=256, d=128, layers=2, mlp_mult=2, ctx=32, mixer="aspin", norm="ln")
        P = oracle.init_lm_params(cfg, seed=7, jitter=0.2)
        m = LM(vocab=256, d=128, layers=2, mlp_mult=2, ctx=32, mixer="aspin", norm="ln")
        m.load_state_dict(P, strict=True); m = m.to(DEV).eval()
        ids = synth.token_ids(2, 64, 256, seed=3)
        h1, st = m.trunk(ids[:, :32].to(DEV), None, carry=True)
        h2, st = m.trunk(ids[:, 32:].to(DEV), st, carry=True)
        assert tuple(h2.shape) == (2, 32, 128) and len(st) == 2 and st[0][1] == 32
        lg = F.linear(h2, m.e.weight)
        ref, rst = oracle.lm_prefill(P, cfg, ids)
        assert rel_err(lg.cpu(), ref) <= 2e-4 and rel_err(st[1][0].cpu(), rst[1][0]) <= 2e-4
        assert rel_err(lg, m.forward_carried(ids.to(DEV))) <= 1e-5
        assert m.trunk(ids[:, :32].to(DEV)).shape == (2, 32, 128)


@pytest.mark.parametrize("delta", [False, True])
def test_compiled_layer_has_no_graph_break_and_matches_eager(delta):
    """torch.compile(fullgraph=True) of AssocCarrier.mix and of one LM layer: the custom operators keep the graph whole, and
    the compiled result equals the eager one bit for bit (same kernels, same order)."""
    torch._dynamo.reset()
    with torch.no_grad():
        g = torch.Generator().manual_seed(3)
        P = oracle.init_assoc_params({}, "", 128, 2, delta, g, jitter=0.3)
        m = AssocCarrier(128, heads=2, delta=delta); m.load_state_dict(P, strict=True)
        m = m.to(DEV).to(torch.bfloat16).eval()
        z = torch.randn(2, 96, 128, generator=g).to(DEV).to(torch.bfloat16)
        S0 = (torch.randn(2, 2, 64, 64, generator=g) * 0.1).to(DEV)
        eager, (Se, pe) = m.mix(z, (S0, 40))
        fn = torch.compile(lambda zz, ss: m.mix(zz, (ss, 40)), fullgraph=True)
        comp, (Sc, pc) = fn(z, S0)
        assert pc == pe == 96
        if delta:      # the gates' softplus / sigmoid run as compiled pointwise code there: last-bit differences in their inputs
            assert rel_err(comp.float(), eager.float()) <= 2e-3 and rel_err(Sc, Se) <= 1e-4
        else:
            assert torch.equal(comp, eager) and torch.equal(Sc, Se)
        # one whole layer of the language model (add + norm, mixer, add + norm, MLP with the fused up-projection)
        lm = LM(vocab=256, d=128, layers=1, mlp_mult=2, ctx=128, mixer="dspin" if delta else "aspin", norm="rms")
        lm = lm.to(DEV).to(torch.bfloat16).eval()
        h = torch.randn(2, 128, 128, generator=g).to(DEV).to(torch.bfloat16)

        def layer(hh):
            st = [None]
            x, dl = lm._layers(hh, st)
            return x, dl, st[0][0]
        e = layer(h)
        c = torch.compile(layer, fullgraph=True)(h)
        for a, b in zip(e, c):
            assert torch.equal(a, b) if not delta else rel_err(a.float(), b.float()) <= 4e-3


@pytest.mark.parametrize("delta", [False, True])
def test_scan_kernels_are_differentiable_by_their_drop_in_names(delta):
    """assoc_scan_kernel / delta_scan_kernel with requires_grad inputs compose the differentiable operators (the reference's
    own composition, src/assoc_kernel.py:302-323, 512-546) and give the gradients of the CPU oracle's chunked scan
    (tests/test_assoc.py:158-163, 174-185 check the same five / six gradients)."""
    from pragnosia_b200.assoc_kernel import assoc_scan_kernel, delta_scan_kernel
    B, H, T, D = 2, 2, 150, 64
    x = synth.assoc_op_inputs(B, H, T, D, seed=8, delta=delta, with_state=True)
    names = ("q", "k", "v", "la", "S0") + (("beta",) if delta else ())
    with torch.enable_grad():
        ref = {n: (x[n].to(torch.bfloat16).double() if n in "qkv" else x[n].double()).requires_grad_(True) for n in names}
        o_r, s_r = oracle.assoc_scan(ref["q"], ref["k"], ref["v"], ref["la"], ref["S0"], beta=ref.get("beta"))
        (o_r.square().sum() + s_r.square().sum()).backward()
        dev = {n: (x[n].to(torch.bfloat16) if n in "qkv" else x[n]).to(DEV).requires_grad_(True) for n in names}
        if delta:
            o, S, sent = delta_scan_kernel(dev["q"], dev["k"], dev["v"], dev["la"], dev["beta"], dev["S0"])
        else:
            o, S, sent = assoc_scan_kernel(dev["q"], dev["k"], dev["v"], dev["la"], dev["S0"])
        assert o.dtype == torch.bfloat16 and tuple(sent.shape) == (B, H, 3, D, D)
        (o.float().square().sum() + S.square().sum()).backward()
    for n in names:
        e = rel_err(dev[n].grad.float().cpu(), ref[n].grad.float())
        assert e <= 4e-2, (n, e)
