"""CPU-only checks of the torch custom operators: every operator is registered, and its shape function (the fake kernel
torch.compile traces with) returns the documented shapes and dtypes. No kernel runs here."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

from pragnosia_b200 import custom_ops  # noqa: F401  (registers the operators)

OPS = torch.ops.pragnosia_b200
BF, F32 = torch.bfloat16, torch.float32
B, H, T, D = 2, 3, 333, 64
NC = 6


def sig(t):
    return tuple(t.shape), t.dtype


def test_every_operator_is_registered():
    for name in ("assoc_prep", "assoc_prep_bwd", "assoc_out", "prefix_scan", "delta_inv", "delta_loop_fwd", "aspin_prefill",
                 "aspin_prefill_fused", "aspin_layer_prefill", "aspin_decode_step", "lambda_scan", "lambda_scan_bwd", "rot_table",
                 "rotate", "add_norm", "linear_act"):
        assert hasattr(OPS, name), name


def test_shape_functions():
    with FakeTensorMode():
        e = lambda *s, dtype=BF: torch.empty(*s, dtype=dtype, device="cuda")
        q = e(B, H, T, D); la = e(B, H, T, dtype=F32); S0 = e(B, H, D, D, dtype=F32)
        # the reference's operator set (src/assoc_kernel.py:128, 231, 363, 658, 828)
        qp = e(B, T, H, D); gl = e(B, T, H); th = e(H, D // 2, dtype=F32); pos = e(T, dtype=torch.int64)
        for t in OPS.assoc_prep(qp, qp, qp, gl, th, pos):
            assert sig(t) == ((B, H, T, D), BF)
        dqp, dkp, dvp, dgl, dth = OPS.assoc_prep_bwd(qp, qp, qp, gl, th, pos, q, q, q)
        assert sig(dqp) == ((B, T, H, D), BF) and sig(dgl) == ((B, T, H), F32) and sig(dth) == ((H, D // 2), F32)
        assert OPS.assoc_prep_bwd(qp, qp, qp, None, th, pos, q, q, q)[3].numel() == 0
        sent = e(B, H, NC, D, D)
        assert sig(OPS.assoc_out(q, q, q, la, sent, 64)) == ((B, H, T, D), BF)
        kpad = e(B, H, NC * 64, D); w = e(B, H, NC, 64, 1, dtype=F32); al = e(B, H, NC, dtype=F32)
        s_ent, s_fin = OPS.prefix_scan(kpad, kpad, w, al, S0, True, 16)
        assert sig(s_ent) == ((B, H, NC, D, D), BF) and sig(s_fin) == ((B, H, D, D), F32)
        X = OPS.delta_inv(q, la, la, NC)
        assert sig(X) == ((B, H, NC, 64, 64), BF)
        W, s_ent, s_fin = OPS.delta_loop_fwd(q, q, la, la, X, S0, True, 64, 32, 16)
        assert sig(W) == ((B, H, T, D), BF) and sig(s_ent) == ((B, H, NC, D, D), BF) and sig(s_fin) == ((B, H, D, D), F32)
        # the fused operators
        o, S, s_ent = OPS.aspin_prefill(q, q, q, la, la, S0, th, None, 3.0, True, 0, True)
        assert sig(o) == ((B, H, T, D), F32) and sig(S) == ((B, H, D, D), F32) and sig(s_ent) == ((B, H, NC, D, D), BF)
        o, S, s_ent = OPS.aspin_prefill(q, q, q, la, None, None, None, None, 0.0, False, 0, False)
        assert sig(o) == ((B, H, T, D), BF) and s_ent.numel() == 0
        dl = e(B, T, H); A = e(H, dtype=F32); rw = e(D, dtype=F32)
        o, S, _ = OPS.aspin_prefill_fused(q, q, q, dl, A, S0, th, None, 0.0, rw, 1e-6, False, False)
        assert sig(o) == ((B, T, H * D), BF)
        table = OPS.rot_table(th, 384)
        assert sig(table) == ((H, 384, D // 2, 2), F32)
        o, S, _ = OPS.aspin_layer_prefill(qp, qp, qp, gl, dl, A, table, None, None, None, 0.0, rw, 1e-6, False, False)
        assert sig(o) == ((B, T, H * D), BF) and sig(S) == ((B, H, D, D), F32)
        q1 = e(B, H, D); g1 = e(B, H)
        o, S1 = OPS.aspin_decode_step(q1, q1, q1, g1, S0, th, g1, False, True, A, True, None, 1.0, rw, 1e-6, False)
        assert sig(o) == ((B, H, D), BF) and sig(S1) == ((B, H, D, D), F32)
        u = e(B, 45, 300, dtype=F32); h0 = e(B, 300, dtype=F32)
        y, hr, hi, hia = OPS.lambda_scan(u, u, u, h0, h0, 0, True)
        assert sig(y) == ((B, 45, 300), F32) and sig(hr) == ((B, 300), F32) and sig(hia) == ((B, 45, 300), F32)
        assert OPS.lambda_scan(u, u, u, None, None, 0, False)[3].numel() == 0
        du, dlm, dan, d0r, d0i = OPS.lambda_scan_bwd(u, u, u, u, u, u, h0, True)
        assert sig(du) == sig(dlm) == sig(dan) == ((B, 45, 300), F32) and sig(d0r) == sig(d0i) == ((B, 300), F32)
        assert sig(OPS.rotate(q, th, e(T, dtype=F32))) == ((B, H, T, D), BF)
        x = e(B * T, 768); wn = e(768)
        yy, z = OPS.add_norm(x, x, wn, None, 1e-6, 1)
        assert sig(yy) == sig(z) == ((B * T, 768), BF)
        assert OPS.add_norm(x, None, wn, wn, 1e-5, 2)[0].numel() == 0
        assert sig(OPS.linear_act(x, e(3072, 768), e(3072), 1)) == ((B * T, 3072), BF)


def test_operators_are_functional():
    """No operator declares a mutated argument: outputs are always new tensors (what lets a compiled graph reorder them)."""
    for name in ("assoc_prep", "assoc_out", "prefix_scan", "delta_inv", "delta_loop_fwd", "aspin_prefill", "aspin_layer_prefill",
                 "aspin_decode_step", "lambda_scan"):
        schema = getattr(OPS, name).default._schema
        assert not any(a.alias_info is not None and a.alias_info.is_write for a in schema.arguments), name


@pytest.mark.parametrize("delta", [False, True])
def test_layer_traces_whole(monkeypatch, delta):
    """torch._dynamo.export of AssocCarrier.mix and of one LM layer (trace only: shape functions, no kernel) finds no graph
    break and lands on the custom operators. CPU tensors stand in for the trace; the wrappers' CUDA check is lifted for it."""
    from pragnosia_b200 import ops
    from pragnosia_b200.assoc import AssocCarrier
    from pragnosia_b200.model import LM
    monkeypatch.setattr(ops, "need_cuda", lambda *a: None)
    torch._dynamo.reset()
    with torch.no_grad():
        m = AssocCarrier(128, heads=2, delta=delta).to(BF).eval()
        z, S0 = torch.randn(2, 96, 128).to(BF), torch.randn(2, 2, 64, 64)
        ep = torch._dynamo.export(lambda zz, ss: m.mix(zz, (ss, 40)))(z, S0)
        used = {str(n.target) for n in ep.graph_module.graph.nodes if n.op == "call_function"}
        want = {"pragnosia_b200.assoc_prep_ex", "pragnosia_b200.aspin_prefill"} if delta else {"pragnosia_b200.aspin_layer_prefill"}
        assert want <= used, used
        lm = LM(vocab=256, d=128, layers=1, mlp_mult=2, ctx=128, mixer="dspin" if delta else "aspin", norm="rms").to(BF).eval()

        def layer(hh):
            st = [None]
            x, dl = lm._layers(hh, st)
            return x, dl, st[0][0]
        ep = torch._dynamo.export(layer)(torch.randn(2, 128, 128).to(BF))
        used = [str(n.target) for n in ep.graph_module.graph.nodes if n.op == "call_function"]
        assert used.count("pragnosia_b200.add_norm") == 2
