"""The layer's options on the GPU (short convolution, key_topk, hl_floor, write_all, pos_wrap, beta_scale: src/assoc.py
:361-382, :406-410, :435-439, :463-478) against the reference module's own CPU outputs (options.pt); housekeeping checks
that live beside them: weights changed after a captured graph, the one-row fused linear at long rows, min-p sampling."""
import pytest
import torch

import oracle
from oracle import rel_err
from pragnosia_b200 import ops, synth
from pragnosia_b200.assoc import AssocCarrier
from pragnosia_b200.generate import Decoder
from pragnosia_b200.model import LM
from test_oracle_options_grads import CASES, option_inputs

pytestmark = pytest.mark.gpu
torch.set_grad_enabled(False)
DEV = "cuda"


def build(name, kw, delta, dtype=torch.float32):
    P, x, bs = option_inputs(name, delta)
    ctor = {k: v for k, v in kw.items() if k != "pos_wrap"}
    m = AssocCarrier(128, heads=2, delta=delta, **ctor)
    if name.startswith("sconv"):
        m.add_short_conv(4)
    m.load_state_dict(P, strict=True)
    if "pos_wrap" in kw:
        m.pos_wrap = kw["pos_wrap"]
    return m.to(DEV).to(dtype).eval(), P, x, bs


@pytest.mark.parametrize("name,kw,delta", CASES)
def test_layer_options_match_the_reference_module(golden, name, kw, delta):
    G = golden("options")[name]
    m, P, x, bs = build(name, kw, delta)
    xd = x.to(DEV)
    if name == "beta_scale":
        m.beta_scale = bs.to(DEV)
        y, st = m(xd)
        assert rel_err(y.cpu(), G["y"]) <= 1e-4 and rel_err(st[0].cpu(), G["S"]) <= 1e-4
        return
    y, st = m(xd)
    assert rel_err(y.cpu(), G["y"]) <= 1e-4 and rel_err(st[0].cpu(), G["S"]) <= 1e-4
    ya, sa = m(xd[:, :30]); yb, sb = m(xd[:, 30:], h0=sa)
    assert rel_err(torch.cat([ya, yb], 1).cpu(), G["y_windows"]) <= 1e-4 and rel_err(sb[0].cpu(), G["S_windows"]) <= 1e-4
    cur, steps = sa, []
    for t in range(30, 40):
        yt, cur = m(xd[:, t:t + 1], h0=cur); steps.append(yt)
    assert rel_err(torch.cat(steps, 1).cpu(), G["y_steps"]) <= 1e-4 and rel_err(cur[0].cpu(), G["S_steps"]) <= 1e-4
    if name.startswith("sconv"):
        assert len(st) == 3 and rel_err(st[2].cpu(), G["cc"]) <= 1e-5 and rel_err(cur[2].cpu(), G["cc_steps"]) <= 1e-5


@pytest.mark.parametrize("name,kw,delta", [c for c in CASES if c[0] in ("write_all", "pos_wrap", "sconv", "floor")])
def test_layer_options_bf16_fused_path(name, kw, delta):
    """The same options with bf16 weights (the fused between-GEMMs kernel where the option allows it) against the oracle run
    on the bf16-rounded weights with the product's rounding points. (key_topk is left to the fp32 case above: which
    coordinates survive is a discontinuous choice, and bf16 keys tie.)"""
    m, P, x, _ = build(name, kw, delta, torch.bfloat16)
    Pb = {k: v.to(torch.bfloat16).float() for k, v in P.items()}
    xb = x.to(torch.bfloat16)
    y, st = m(xb.to(DEV))
    with oracle.rounding(torch.bfloat16):
        ry, rst = oracle.assoc_layer(Pb, "", xb.float(), None, heads=2, delta=delta, **kw)
    tol = 6e-2 if name == "sconv" else 2e-2                # random convolution taps of size 0.3 amplify the bf16 hand-overs
    assert rel_err(y.float().cpu(), ry) <= tol and rel_err(st[0].cpu(), rst[0]) <= tol


def test_key_topk_and_short_conv_kernels():
    g = torch.Generator().manual_seed(5)
    for dtype, D in ((torch.float32, 64), (torch.bfloat16, 128)):
        buf = torch.randn(2, 37, 3 * 2 * D + 8, generator=g).to(dtype)                # a view into a wider row, as in the layer
        # magnitudes 1/D .. 1 in a random order with random signs: all distinct and exact in bf16, so the choice has no ties
        mags = torch.stack([torch.randperm(D, generator=g) + 1 for _ in range(2 * 37 * 2)]).view(2, 37, 2 * D).float() / D
        buf[..., 2 * D:4 * D] = (mags * (torch.randint(0, 2, mags.shape, generator=g) * 2 - 1)).to(dtype)
        kp = buf[..., 2 * D:4 * D].unflatten(-1, (2, D))
        ref = kp.float() * torch.zeros_like(kp.float()).scatter_(-1, kp.float().abs().topk(9, dim=-1).indices, 1.0)
        bd = buf.to(DEV)
        ops.key_topk_mask_(bd[..., 2 * D:4 * D].unflatten(-1, (2, D)), 9)
        assert torch.equal(bd[..., 2 * D:4 * D].unflatten(-1, (2, D)).float().cpu(), ref)
        assert torch.equal(bd[..., :2 * D].cpu(), buf[..., :2 * D])                   # nothing else touched
    for T in (1, 2, 3, 50):
        x = torch.randn(2, T, 96, generator=g); w = torch.randn(96, 4, generator=g); cc = torch.randn(2, 96, 3, generator=g)
        for cache in (None, cc):
            P = {"sconv": w}
            q, k, v, new = oracle.short_conv(P, "", x[..., :32], x[..., 32:64], x[..., 64:], cache)
            y, nd = ops.short_conv(x.to(DEV), w.to(DEV), None if cache is None else cache.to(DEV))
            assert rel_err(y.cpu(), torch.cat([q, k, v], -1)) <= 1e-6 and torch.equal(nd.cpu(), new)


def test_weights_changed_after_a_captured_graph():
    """load_state_dict (and an in-place update) after the first graphed call: the next call computes with the NEW weights,
    as a fresh model does -- the captured graphs held the old derived constants."""
    cfg = oracle.lm_config(vocab=256, d=128, layers=2, mlp_mult=2, ctx=32, mixer="aspin", norm="rms")
    P1, P2 = oracle.init_lm_params(cfg, seed=1, jitter=0.2), oracle.init_lm_params(cfg, seed=2, jitter=0.2)
    mk = lambda: LM(vocab=256, d=128, layers=2, mlp_mult=2, ctx=32, mixer="aspin", norm="rms")
    ids = synth.token_ids(2, 96, 256, seed=5).to(DEV)
    for dtype in (torch.float32, torch.bfloat16):
        m = mk(); m.load_state_dict(P1); m = m.to(DEV).to(dtype).eval()
        first = m.forward_carried(ids).clone()
        dec = Decoder(m, batch=2); dec.prefill(ids[:, :40]); dec.step(ids[:, 40])
        m.load_state_dict(P2)
        fresh = mk(); fresh.load_state_dict(P2); fresh = fresh.to(DEV).to(dtype).eval()
        want = fresh.forward_carried(ids)
        got = m.forward_carried(ids)
        assert torch.equal(got, want) and not torch.equal(got, first)
        d2 = Decoder(fresh, batch=2); d2.prefill(ids[:, :40])
        dec.prefill(ids[:, :40])
        assert torch.equal(dec.step(ids[:, 40]), d2.step(ids[:, 40]))
        with torch.no_grad():
            m.mix[0].theta.mul_(1.5); fresh.mix[0].theta.mul_(1.5)                    # in place: same address, new version
        assert torch.equal(m.forward_carried(ids), fresh.forward_carried(ids))


def test_one_row_fused_linear_long_rows_is_deterministic():
    """One row with a norm and K beyond the per-lane register buffer (1024): every warp builds the row in its own slice of
    shared memory, so repeated launches are bit-identical and equal the two-row instantiation's first row."""
    g = torch.Generator().manual_seed(11)
    for K in (2048, 6144):
        for norm in (torch.nn.RMSNorm(K), torch.nn.LayerNorm(K)):
            norm = norm.to(DEV).to(torch.bfloat16)
            with torch.no_grad():
                norm.weight.copy_(torch.randn(K, generator=g)); 
                if hasattr(norm, "bias") and norm.bias is not None: norm.bias.copy_(torch.randn(K, generator=g) * 0.1)
            x = torch.randn(2, K, generator=g).to(torch.bfloat16).to(DEV); dl = torch.randn(2, K, generator=g).to(torch.bfloat16).to(DEV)
            W = (torch.randn(520, K, generator=g) * K ** -0.5).to(torch.bfloat16).to(DEV)
            two, _ = ops.skinny_linear(x, W, None, delta=dl, norm=norm, act="gelu", want_sum=True)
            outs = [ops.skinny_linear(x[:1], W, None, delta=dl[:1], norm=norm, act="gelu") for _ in range(40)]
            assert all(torch.equal(o, outs[0]) for o in outs) and torch.equal(outs[0], two[:1])
            ref = torch.nn.functional.gelu(torch.nn.functional.linear(norm((x[:1] + dl[:1])), W))
            assert rel_err(outs[0].float(), ref.float()) <= 2e-2


def test_min_p_sampling():
    """src/bench.py:79-86 with MIN_P: ids below min_p x the top probability are never drawn; min_p = 0 changes nothing."""
    g = torch.Generator().manual_seed(3)
    lg = (torch.randn(4, 512, generator=g) * 3).to(DEV)
    p = torch.softmax(lg, -1)
    allowed = p >= 0.2 * p.max(-1, keepdim=True).values
    tok = torch.zeros(4, dtype=torch.long, device=DEV); cnt = torch.zeros(1, dtype=torch.long, device=DEV)
    ticket = torch.zeros(1, dtype=torch.int32, device=DEV)
    seen = torch.zeros(4, 512, dtype=torch.bool, device=DEV)
    for _ in range(300):
        ops.decode_sample(lg, 1.0, 7, tok, cnt, ticket, min_p=0.2)
        seen[torch.arange(4), tok] = True
    assert not (seen & ~allowed).any() and (seen.sum(-1) >= 1).all() and int(seen.sum()) > 4
    assert (seen.sum(-1) <= allowed.sum(-1)).all() and int(allowed.sum()) < 4 * 512
    a, b = tok.clone(), tok.clone()
    c1, c2 = torch.zeros(1, dtype=torch.long, device=DEV), torch.zeros(1, dtype=torch.long, device=DEV)
    ops.decode_sample(lg, 1.0, 9, a, c1, ticket); ops.decode_sample(lg, 1.0, 9, b, c2, ticket, min_p=0.0)
    assert torch.equal(a, b)
    m = LM(vocab=256, d=128, layers=2, mlp_mult=2, ctx=32, mixer="aspin", norm="ln").to(DEV).eval()
    prompt = synth.token_ids(2, 40, 256, seed=2).to(DEV)
    out = Decoder(m, batch=2, min_p=0.3).generate(prompt, 10, temp=1.0, seed=1)
    assert tuple(out.shape) == (2, 10) and torch.equal(out, Decoder(m, batch=2, min_p=0.3, use_graph=False).generate(prompt, 10, temp=1.0, seed=1))


@pytest.mark.parametrize("D,T,io", [(64, 200, torch.float32), (128, 130, torch.float32), (64, 333, torch.bfloat16)])
def test_plain_rule_trains_through_the_split_operators(D, T, io):
    """assoc_out and prefix_scan carry the reference's backward kernels (src/assoc_kernel.py:75-126, 206-221): the
    gradients of the plain-rule scan composed from them, against autograd through the CPU oracle's chunked scan."""
    with torch.enable_grad():
        _split_operator_gradients(D, T, io)


def _split_operator_gradients(D, T, io):
    B, H = 2, 3
    x = synth.assoc_op_inputs(B, H, T, D, seed=5, with_state=True)
    w_o = torch.randn(B, H, T, D, generator=torch.Generator().manual_seed(1))
    w_s = torch.randn(B, H, D, D, generator=torch.Generator().manual_seed(2)) * 0.1
    names = ("q", "k", "v", "la", "S0")
    ref_in = {n: x[n].double().requires_grad_(True) for n in names}
    if io == torch.bfloat16:                                          # the kernels see bf16-rounded q, k, v
        ref_in = {n: (x[n].to(io).double() if n in "qkv" else x[n].double()).requires_grad_(True) for n in names}
    o_ref, s_ref = oracle.assoc_scan(ref_in["q"], ref_in["k"], ref_in["v"], ref_in["la"], ref_in["S0"])
    ((o_ref * w_o).sum() + (s_ref * w_s).sum()).backward()

    dev_in = {n: (x[n].to(io) if n in "qkv" else x[n]).to(DEV).requires_grad_(True) for n in names}
    q, k, v, la, S0 = (dev_in[n] for n in names)
    NC = (T + 63) // 64
    pad = NC * 64 - T
    kp, vp = (torch.nn.functional.pad(t, (0, 0, 0, pad)) for t in (k, v))
    Lc = torch.nn.functional.pad(la, (0, pad)).view(B, H, NC, 64).cumsum(-1)
    a_log = Lc[..., -1]
    w = torch.exp(a_log[..., None] - Lc)
    sent, sfin = ops.prefix_scan(kp, vp, w, a_log, S0)
    o = ops.assoc_out(q, k, v, la, sent)
    ((o.float() * w_o.to(DEV)).sum() + (sfin * w_s.to(DEV)).sum()).backward()
    tol = 2e-2 if io == torch.bfloat16 else 1e-2                      # the states between the two operators travel as bf16
    assert rel_err(o.detach().float().cpu(), o_ref.detach().float()) <= tol
    for n in names:
        e = rel_err(dev_in[n].grad.float().cpu(), ref_in[n].grad.float())
        assert e <= tol, (n, e)


@pytest.mark.parametrize("D,T,io", [(64, 200, torch.float32), (128, 130, torch.float32), (64, 333, torch.bfloat16)])
def test_delta_rule_trains_through_the_split_operators(D, T, io):
    """delta_inv and delta_loop_fwd carry the reference's backward kernels (src/assoc_kernel.py:390-459, 626-656): the
    gradients of the delta-rule scan composed as the reference composes it (inverse, walk, assoc_out on the residuals),
    against autograd through the CPU oracle's chunked scan."""
    with torch.enable_grad():
        B, H = 2, 2
        x = synth.assoc_op_inputs(B, H, T, D, seed=6, delta=True, with_state=True)
        w_o = torch.randn(B, H, T, D, generator=torch.Generator().manual_seed(1))
        w_s = torch.randn(B, H, D, D, generator=torch.Generator().manual_seed(2)) * 0.1
        names = ("q", "k", "v", "la", "beta", "S0")
        ref_in = {n: (x[n].to(torch.bfloat16).double() if n in "qkv" else x[n].double()).requires_grad_(True) for n in names}
        o_ref, s_ref = oracle.assoc_scan(ref_in["q"], ref_in["k"], ref_in["v"], ref_in["la"], ref_in["S0"], beta=ref_in["beta"])
        ((o_ref * w_o).sum() + (s_ref * w_s).sum()).backward()

        # q, k, v on the bf16 grid in both runs (delta_inv takes k in bf16); the op I/O dtype is io
        dev_in = {n: (x[n].to(torch.bfloat16).to(io) if n in "qkv" else x[n]).to(DEV).requires_grad_(True) for n in names}
        q, k, v, la, be, S0 = (dev_in[n] for n in names)
        NC = (T + 63) // 64
        X = ops.delta_inv(k, la, be, NC)
        W, sent, sfin = ops.delta_loop_fwd(k, v, la, be, X, S0)
        o = ops.assoc_out(q, k, W, la, sent)
        ((o.float() * w_o.to(DEV)).sum() + (sfin * w_s.to(DEV)).sum()).backward()
        assert rel_err(o.detach().float().cpu(), o_ref.detach().float()) <= 2e-2
        for n in names:                                               # X, W and the states between the operators travel as bf16
            e = rel_err(dev_in[n].grad.float().cpu(), ref_in[n].grad.float())
            assert e <= 3e-2, (n, e)


@pytest.mark.parametrize("delta", [False, True])
@pytest.mark.parametrize("jitter,scale", [(0.0, 0.04), (0.05, 0.2)])
def test_layer_trains_through_the_kernels(delta, jitter, scale):
    """AssocCarrier.forward with gradients wanted: parameter and input gradients of a small layer against autograd through
    the CPU oracle's layer (the reference trains through the same operators, src/assoc.py:440-505). Two parameter sets:
    the model's own initialisation (weights N(0, 0.02)) and a perturbed one with projections of order one."""
    d, heads, B, T = 128, 2, 2, 96
    cfgP = {}
    g = torch.Generator().manual_seed(11)
    oracle.init_assoc_params(cfgP, "m.", d, heads, delta, g, jitter=jitter)
    for n in ("q", "k", "v", "o", "wa", "wi", "wb"):
        if "m." + n + ".weight" in cfgP:
            cfgP["m." + n + ".weight"] = cfgP["m." + n + ".weight"] * scale     # init_assoc_params scales by 25 when it perturbs
    layer = AssocCarrier(d, heads=heads, delta=delta)
    layer.load_state_dict({k[2:]: v for k, v in cfgP.items()}, strict=True)
    layer = layer.to(DEV)
    x = torch.randn(B, T, d, generator=g)
    w_out = torch.randn(B, T, d, generator=g)
    # The oracle runs in fp32 like the layer: where a head's write gate is nearly shut the read is tiny and the per-head
    # norm's epsilon (the arithmetic type's) decides its size, so an fp64 oracle would normalise what fp32 leaves near zero.
    # The first token's read is rank one, o_0 = (q_0 . k_0) v_0, and the norm keeps little more than the SIGN of that dot
    # product, which bf16 operands (the operators' contract) can flip: the first 4 tokens stay out of loss and comparison.
    w_out[:, :4] = 0
    with torch.enable_grad():
        P = {k: v.clone().requires_grad_(True) for k, v in cfgP.items()}
        xr = x.clone().requires_grad_(True)
        out_r, (S_r, _) = oracle.assoc_layer(P, "m.", xr, None, heads=heads, delta=delta)
        ((out_r * w_out).sum() + S_r.square().sum()).backward()
        xd = x.detach().to(DEV).requires_grad_(True)
        out, (S, p) = layer(xd)
        ((out * w_out.to(DEV)).sum() + S.square().sum()).backward()
    assert p == T
    errs = {"out": rel_err(out.detach().cpu()[:, 4:], out_r.detach()[:, 4:]), "S": rel_err(S.detach().cpu(), S_r.detach()),
            "x": rel_err(xd.grad.cpu(), xr.grad)}
    for name, prm in layer.named_parameters():
        if prm.grad is None:
            assert P["m." + name].grad is None or P["m." + name].grad.abs().max() == 0, name
            continue
        errs[name] = rel_err(prm.grad.cpu(), P["m." + name].grad)
    # measured: every entry under 1.5e-2 except the decay's two per-head scalars (A, wa.bias), which are sums over all
    # tokens of terms of both signs and inherit the cancellation (up to 0.17 in the perturbed set)
    loose = ("A", "wa.bias")
    assert all(e <= (0.3 if k in loose else 3e-2) for k, e in errs.items()), errs
