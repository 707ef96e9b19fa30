"""torch custom operators over the C ABI (namespace pragnosia_b200::), each with a shape function, so callers under
torch.compile trace through the carrier without a graph break -- the role of the reference's membrae:: operators
(src/assoc_kernel.py:128, :231, :363, :658, :828, each with register_fake and register_autograd).

Two groups:
  * the reference's own operator set with its argument lists -- assoc_prep, assoc_out, prefix_scan, delta_inv,
    delta_loop_fwd -- for code written against those;
  * the fused operators this library adds -- aspin_prefill (one walk instead of three launches), aspin_prefill_fused,
    aspin_layer_prefill, aspin_decode_step, lambda_scan, rot_table, rotate, add_norm, linear_act.
Every operator is functional (mutates_args=()): outputs are new tensors; an absent optional output is an empty tensor.
Backward formulas are registered for lambda_scan (the adjoint scan), assoc_prep, assoc_out and prefix_scan (the plain
rule and the delta rule train through the split operators).

The operator bodies run eagerly and call pragnosia_b200.ops, which makes the one library call.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from . import ops

NS = "pragnosia_b200"
_BF16, _F32 = torch.bfloat16, torch.float32


def _e(t: Tensor, *shape, dtype=None) -> Tensor:
    return torch.empty(shape, device=t.device, dtype=dtype or t.dtype)


def _none(t: Tensor) -> Tensor:
    return torch.empty(0, device=t.device, dtype=t.dtype)


def _nc(T: int) -> int:
    return (T + ops.CHUNK - 1) // ops.CHUNK


# ------------------------------------------------------------------------------------------------ per-token lambda scan
@torch.library.custom_op(f"{NS}::lambda_scan", mutates_args=())
def lambda_scan(u: Tensor, logmag: Tensor, ang: Tensor, h0r: Optional[Tensor], h0i: Optional[Tensor], time_segments: int,
                keep_imag: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    h0 = None if h0r is None else (h0r, h0i)
    if keep_imag:
        y, (hr, hi), hia = ops.lambda_scan(u, logmag, ang, h0, time_segments, keep_imag=True)
        return y, hr, hi, hia
    y, (hr, hi) = ops.lambda_scan(u, logmag, ang, h0, time_segments)
    return y, hr, hi, _none(y)


@lambda_scan.register_fake
def _(u, logmag, ang, h0r, h0i, time_segments, keep_imag):
    B, T, D = u.shape
    return (_e(u, B, T, D, dtype=_F32), _e(u, B, D, dtype=_F32), _e(u, B, D, dtype=_F32),
            _e(u, B, T, D, dtype=_F32) if keep_imag else _e(u, 0, dtype=_F32))


@torch.library.custom_op(f"{NS}::lambda_scan_bwd", mutates_args=())
def lambda_scan_bwd(g: Tensor, u: Tensor, logmag: Tensor, ang: Tensor, hr_all: Tensor, hi_all: Tensor, g_last_i: Optional[Tensor],
                    want_dh0: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    du, dlm, dan, d0r, d0i = ops.lambda_scan_bwd(g, u, logmag, ang, hr_all, hi_all, g_last_i, want_dh0)
    return du, dlm, dan, (d0r if want_dh0 else _none(du)), (d0i if want_dh0 else _none(du))


@lambda_scan_bwd.register_fake
def _(g, u, logmag, ang, hr_all, hi_all, g_last_i, want_dh0):
    B, T, D = u.shape
    s = (B, D) if want_dh0 else (0,)
    return (_e(u, B, T, D, dtype=_F32), _e(u, B, T, D, dtype=_F32), _e(u, B, T, D, dtype=_F32), _e(u, *s, dtype=_F32),
            _e(u, *s, dtype=_F32))


class _LambdaScan(torch.autograd.Function):
    """Differentiable scan (the reference's _Scan, src/scan_kernel.py:105-140): the forward keeps Im h for the adjoint."""

    @staticmethod
    def forward(ctx, u, logmag, ang, h0r, h0i):
        h0 = None if h0r is None else (h0r, h0i)
        y, (hr, hi), hia = ops.lambda_scan(u, logmag, ang, h0, keep_imag=True)
        ctx.save_for_backward(u, logmag, ang, y, hia)
        ctx.has = h0r is not None
        return y, hr, hi

    @staticmethod
    def backward(ctx, g, g_last_r, g_last_i):
        u, logmag, ang, y, hia = ctx.saved_tensors
        g = torch.zeros_like(y) if g is None else g.to(torch.float32)
        if g_last_r is not None:
            g = g.clone()
            g[:, -1] += g_last_r.to(torch.float32)
        du, dlm, dan, d0r, d0i = ops.lambda_scan_bwd(g.contiguous(), u, logmag, ang, y, hia, g_last_i, want_dh0=ctx.has)
        return du, dlm, dan, d0r, d0i


def lambda_scan_autograd(u, logmag, ang, h0=None):
    """(y, (hr_last, hi_last)) with gradients to u, logmag, ang and h0."""
    h0r, h0i = (None, None) if h0 is None else (h0[0].float(), h0[1].float())
    y, hr, hi = _LambdaScan.apply(u.float(), logmag.float(), ang.float(), h0r, h0i)
    return y, (hr, hi)


# ------------------------------------------------------------------------------------------------ the reference's operator set
@torch.library.custom_op(f"{NS}::assoc_prep_ex", mutates_args=())
def assoc_prep_ex(qp: Tensor, kp: Tensor, vp: Tensor, gl: Optional[Tensor], theta: Tensor, pos: Tensor,
                  out_bf16: bool) -> Tuple[Tensor, Tensor, Tensor]:
    return ops.prep(qp, kp, vp, gl, theta, pos, out_dtype=_BF16 if out_bf16 else _F32)


@assoc_prep_ex.register_fake
def _(qp, kp, vp, gl, theta, pos, out_bf16):
    B, T, H, D = qp.shape
    dt = _BF16 if out_bf16 else _F32
    return _e(qp, B, H, T, D, dtype=dt), _e(qp, B, H, T, D, dtype=dt), _e(qp, B, H, T, D, dtype=dt)


@torch.library.custom_op(f"{NS}::assoc_prep", mutates_args=())
def assoc_prep(qp: Tensor, kp: Tensor, vp: Tensor, gl: Optional[Tensor], theta: Tensor, pos: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
    """The reference's signature (src/assoc_kernel.py:828-838): bf16 (B,H,T,D) outputs."""
    return ops.prep(qp, kp, vp, gl, theta, pos, out_dtype=_BF16)


@assoc_prep.register_fake
def _(qp, kp, vp, gl, theta, pos):
    B, T, H, D = qp.shape
    return _e(qp, B, H, T, D, dtype=_BF16), _e(qp, B, H, T, D, dtype=_BF16), _e(qp, B, H, T, D, dtype=_BF16)


@torch.library.custom_op(f"{NS}::assoc_prep_bwd", mutates_args=())
def assoc_prep_bwd(qp: Tensor, kp: Tensor, vp: Tensor, gl: Optional[Tensor], theta: Tensor, pos: Tensor, dq: Tensor, dk: Tensor,
                   dv: Tensor) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    dqp, dkp, dvp, dgl, dth = ops.prep_bwd(qp, kp, vp, gl, theta, pos, dq, dk, dv)
    return dqp, dkp, dvp, (dgl if dgl is not None else torch.empty(0, device=qp.device, dtype=_F32)), dth


@assoc_prep_bwd.register_fake
def _(qp, kp, vp, gl, theta, pos, dq, dk, dv):
    B, T, H, D = qp.shape
    dt = qp.dtype if qp.dtype in (_F32, _BF16) else _F32
    g = _e(qp, B, T, H, dtype=_F32) if gl is not None else _e(qp, 0, dtype=_F32)
    return _e(qp, B, T, H, D, dtype=dt), _e(qp, B, T, H, D, dtype=dt), _e(qp, B, T, H, D, dtype=dt), g, _e(qp, H, D // 2, dtype=_F32)


def _prep_setup(ctx, inputs, output):
    qp, kp, vp, gl, theta, pos = inputs
    ctx.has_gate = gl is not None
    ctx.save_for_backward(qp, kp, vp, theta, pos, *([gl] if ctx.has_gate else []))


def _prep_backward(ctx, dq, dk, dv):
    qp, kp, vp, theta, pos = ctx.saved_tensors[:5]
    gl = ctx.saved_tensors[5] if ctx.has_gate else None
    dqp, dkp, dvp, dgl, dth = assoc_prep_bwd(qp, kp, vp, gl, theta, pos, dq.contiguous(), dk.contiguous(), dv.contiguous())
    return (dqp.to(qp.dtype), dkp.to(kp.dtype), dvp.to(vp.dtype), (dgl.to(gl.dtype) if ctx.has_gate else None),
            dth.to(theta.dtype), None)


assoc_prep.register_autograd(_prep_backward, setup_context=_prep_setup)


@torch.library.custom_op(f"{NS}::assoc_out", mutates_args=())
def assoc_out(q: Tensor, k: Tensor, v: Tensor, la: Tensor, sent: Tensor, bc: int) -> Tensor:
    return ops.assoc_out(q, k, v, la, sent, bc)


@assoc_out.register_fake
def _(q, k, v, la, sent, bc):
    return torch.empty(q.shape, device=q.device, dtype=q.dtype if q.dtype in (_F32, _BF16) else _F32)


@torch.library.custom_op(f"{NS}::assoc_out_bwd", mutates_args=())
def assoc_out_bwd(q: Tensor, k: Tensor, v: Tensor, la: Tensor, sent: Tensor, dout: Tensor) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    return ops.assoc_out_bwd(q, k, v, la, sent, dout)


@assoc_out_bwd.register_fake
def _(q, k, v, la, sent, dout):
    B, H, T, D = q.shape
    return (_e(q, B, H, T, D, dtype=_F32), _e(q, B, H, T, D, dtype=_F32), _e(q, B, H, T, D, dtype=_F32), _e(q, B, H, T, dtype=_F32),
            _e(q, B, H, _nc(T), D, D, dtype=_F32))


def _out_setup(ctx, inputs, output):
    q, k, v, la, sent, bc = inputs
    ctx.save_for_backward(q, k, v, la, sent)


def _out_backward(ctx, dout):
    """The reference's _bwd_chunk (src/assoc_kernel.py:75-126, wired at :179)."""
    q, k, v, la, sent = ctx.saved_tensors
    dq, dk, dv, dla, dsent = assoc_out_bwd(q, k, v, la, sent, dout.contiguous())
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dla.to(la.dtype), dsent.to(sent.dtype), None


assoc_out.register_autograd(_out_backward, setup_context=_out_setup)


@torch.library.custom_op(f"{NS}::prefix_scan", mutates_args=())
def prefix_scan(k: Tensor, v: Tensor, w: Tensor, a_log: Tensor, S0: Optional[Tensor], has_s0: bool, bv: int) -> Tuple[Tensor, Tensor]:
    return ops.prefix_scan(k, v, w, a_log, S0, has_s0, bv)


@prefix_scan.register_fake
def _(k, v, w, a_log, S0, has_s0, bv):
    B, H, NC = w.shape[:3]
    D = k.shape[-1]
    return _e(k, B, H, NC, D, D, dtype=_BF16), _e(k, B, H, D, D, dtype=_F32)


@torch.library.custom_op(f"{NS}::prefix_scan_bwd", mutates_args=())
def prefix_scan_bwd(k: Tensor, v: Tensor, w: Tensor, a_log: Tensor, sent: Tensor, dsent: Optional[Tensor], dsfin: Optional[Tensor],
                    want_ds0: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    dk, dv, dw, da, ds0 = ops.prefix_scan_bwd(k, v, w, a_log, sent, dsent, dsfin, want_ds0)
    return dk, dv, dw, da, (ds0 if want_ds0 else _none(dk))


@prefix_scan_bwd.register_fake
def _(k, v, w, a_log, sent, dsent, dsfin, want_ds0):
    B, H, NC = a_log.shape
    D = k.shape[-1]
    return (_e(k, B, H, NC * ops.CHUNK, D, dtype=_F32), _e(k, B, H, NC * ops.CHUNK, D, dtype=_F32), _e(k, B, H, NC, ops.CHUNK, dtype=_F32),
            _e(k, B, H, NC, dtype=_F32), _e(k, *((B, H, D, D) if want_ds0 else (0,)), dtype=_F32))


def _prefix_setup(ctx, inputs, output):
    k, v, w, a_log, S0, has_s0, bv = inputs
    ctx.has_s0 = bool(has_s0 and S0 is not None)
    ctx.w_shape = w.shape
    ctx.save_for_backward(k, v, w, a_log, output[0], *([S0] if ctx.has_s0 else []))


def _prefix_backward(ctx, dsent, dsfin):
    """The reference's _prefix_bwd (src/assoc_kernel.py:206-221, wired at :299)."""
    k, v, w, a_log, sent = ctx.saved_tensors[:5]
    dk, dv, dw, da, ds0 = prefix_scan_bwd(k, v, w, a_log, sent, None if dsent is None else dsent.contiguous(),
                                          None if dsfin is None else dsfin.contiguous(), ctx.has_s0)
    return (dk.to(k.dtype), dv.to(v.dtype), dw.view(ctx.w_shape).to(w.dtype), da.to(a_log.dtype),
            (ds0.to(ctx.saved_tensors[5].dtype) if ctx.has_s0 else None), None, None)


prefix_scan.register_autograd(_prefix_backward, setup_context=_prefix_setup)


@torch.library.custom_op(f"{NS}::delta_inv", mutates_args=())
def delta_inv(k: Tensor, la: Tensor, be: Tensor, nc: int) -> Tensor:
    return ops.delta_inv(k, la, be, nc)


@delta_inv.register_fake
def _(k, la, be, nc):
    B, H = k.shape[:2]
    return _e(k, B, H, nc, ops.CHUNK, ops.CHUNK, dtype=_BF16)


@torch.library.custom_op(f"{NS}::delta_inv_bwd", mutates_args=())
def delta_inv_bwd(k: Tensor, la: Tensor, be: Tensor, X: Tensor, dX: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
    return ops.delta_inv_bwd(k, la, be, X, dX)


@delta_inv_bwd.register_fake
def _(k, la, be, X, dX):
    B, H, T, D = k.shape
    return _e(k, B, H, T, D, dtype=_F32), _e(k, B, H, T, dtype=_F32), _e(k, B, H, T, dtype=_F32)


def _inv_setup(ctx, inputs, output):
    k, la, be, nc = inputs
    ctx.save_for_backward(k, la, be, output)


def _inv_backward(ctx, dX):
    """The reference's _inv_bwd (src/assoc_kernel.py:626-656, wired at :704)."""
    k, la, be, X = ctx.saved_tensors
    dk, dla, dbe = delta_inv_bwd(k, la, be, X, dX.contiguous())
    return dk.to(k.dtype), dla.to(la.dtype), dbe.to(be.dtype), None


delta_inv.register_autograd(_inv_backward, setup_context=_inv_setup)


@torch.library.custom_op(f"{NS}::delta_loop_fwd", mutates_args=())
def delta_loop_fwd(k: Tensor, v: Tensor, la: Tensor, be: Tensor, X: Tensor, S0: Optional[Tensor], has_s0: bool, bc: int, bv: int,
                   bvb: int) -> Tuple[Tensor, Tensor, Tensor]:
    return ops.delta_loop_fwd(k, v, la, be, X, S0, has_s0, bc, bv, bvb)


@delta_loop_fwd.register_fake
def _(k, v, la, be, X, S0, has_s0, bc, bv, bvb):
    B, H, T, D = k.shape
    NC = X.shape[2]
    return _e(k, B, H, T, D, dtype=_BF16), _e(k, B, H, NC, D, D, dtype=_BF16), _e(k, B, H, D, D, dtype=_F32)


@torch.library.custom_op(f"{NS}::delta_loop_bwd", mutates_args=())
def delta_loop_bwd(k: Tensor, v: Tensor, la: Tensor, be: Tensor, X: Tensor, sent: Tensor, dW: Optional[Tensor], dsent: Optional[Tensor],
                   dsfin: Optional[Tensor], want_ds0: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    dk, dv, dla, dbe, dX, ds0 = ops.delta_loop_bwd(k, v, la, be, X, sent, dW, dsent, dsfin, want_ds0)
    return dk, dv, dla, dbe, dX, (ds0 if want_ds0 else _none(dk))


@delta_loop_bwd.register_fake
def _(k, v, la, be, X, sent, dW, dsent, dsfin, want_ds0):
    B, H, T, D = k.shape
    return (_e(k, B, H, T, D, dtype=_F32), _e(k, B, H, T, D, dtype=_F32), _e(k, B, H, T, dtype=_F32), _e(k, B, H, T, dtype=_F32),
            _e(k, *X.shape, dtype=_F32), _e(k, *((B, H, D, D) if want_ds0 else (0,)), dtype=_F32))


def _loop_setup(ctx, inputs, output):
    k, v, la, be, X, S0, has_s0, bc, bv, bvb = inputs
    ctx.has_s0 = bool(has_s0 and S0 is not None)
    ctx.save_for_backward(k, v, la, be, X, output[1], *([S0] if ctx.has_s0 else []))


def _loop_backward(ctx, dW, dsent, dsfin):
    """The reference's _delta_loop_bwd (src/assoc_kernel.py:390-459, wired at :509)."""
    k, v, la, be, X, sent = ctx.saved_tensors[:6]
    c = lambda t: None if t is None else t.contiguous()
    dk, dv, dla, dbe, dX, ds0 = delta_loop_bwd(k, v, la, be, X, sent, c(dW), c(dsent), c(dsfin), ctx.has_s0)
    return (dk.to(k.dtype), dv.to(v.dtype), dla.to(la.dtype), dbe.to(be.dtype), dX.to(X.dtype),
            (ds0.to(ctx.saved_tensors[6].dtype) if ctx.has_s0 else None), None, None, None, None)


delta_loop_fwd.register_autograd(_loop_backward, setup_context=_loop_setup)


# ------------------------------------------------------------------------------------------------ the fused operators
@torch.library.custom_op(f"{NS}::aspin_prefill", mutates_args=())
def aspin_prefill(q: Tensor, k: Tensor, v: Tensor, la: Tensor, beta: Optional[Tensor], S0: Optional[Tensor], theta: Optional[Tensor],
                  shift_dev: Optional[Tensor], shift: float, want_sent: bool, precision: int, out_f32: bool) -> Tuple[Tensor, Tensor, Tensor]:
    o, S, sent = ops.prefill(q, k, v, la, beta, S0, theta=theta, shift=shift_dev if shift_dev is not None else shift,
                             want_sent=want_sent, precision=precision, out_dtype=_F32 if out_f32 else q.dtype)
    return o, S, (sent if sent is not None else torch.empty(0, device=q.device, dtype=_BF16))


@aspin_prefill.register_fake
def _(q, k, v, la, beta, S0, theta, shift_dev, shift, want_sent, precision, out_f32):
    B, H, T, D = q.shape
    sent = _e(q, B, H, _nc(T), D, D, dtype=_BF16) if want_sent else _e(q, 0, dtype=_BF16)
    return _e(q, B, H, T, D, dtype=_F32 if out_f32 else q.dtype), _e(q, B, H, D, D, dtype=_F32), sent


@torch.library.custom_op(f"{NS}::aspin_prefill_fused", mutates_args=())
def aspin_prefill_fused(q: Tensor, k: Tensor, v: Tensor, decay_logits: Tensor, decay_A: Tensor, S0: Optional[Tensor],
                        theta: Optional[Tensor], shift_dev: Optional[Tensor], shift: float, rms_weight: Optional[Tensor], rms_eps: float,
                        want_sent: bool, out_f32: bool) -> Tuple[Tensor, Tensor, Tensor]:
    o, S, sent = ops.prefill_fused(q, k, v, decay_logits, decay_A, S0, theta=theta, shift=shift_dev if shift_dev is not None else shift,
                                   rms_weight=rms_weight, rms_eps=rms_eps, want_sent=want_sent, out_dtype=_F32 if out_f32 else q.dtype)
    return o, S, (sent if sent is not None else torch.empty(0, device=q.device, dtype=_BF16))


@aspin_prefill_fused.register_fake
def _(q, k, v, decay_logits, decay_A, S0, theta, shift_dev, shift, rms_weight, rms_eps, want_sent, out_f32):
    B, H, T, D = q.shape
    sent = _e(q, B, H, _nc(T), D, D, dtype=_BF16) if want_sent else _e(q, 0, dtype=_BF16)
    return _e(q, B, T, H * D, dtype=_F32 if out_f32 else q.dtype), _e(q, B, H, D, D, dtype=_F32), sent


@torch.library.custom_op(f"{NS}::aspin_layer_prefill", mutates_args=())
def aspin_layer_prefill(qp: Tensor, kp: Tensor, vp: Tensor, gate_logits: Optional[Tensor], decay_logits: Tensor, decay_A: Tensor,
                        table: Tensor, S0: Optional[Tensor], theta: Optional[Tensor], shift_dev: Optional[Tensor], shift: float,
                        rms_weight: Optional[Tensor], rms_eps: float, want_sent: bool, out_f32: bool) -> Tuple[Tensor, Tensor, Tensor]:
    o, S, sent = ops.layer_prefill(qp, kp, vp, gate_logits, decay_logits, decay_A, table, S0, theta=theta,
                                   shift=shift_dev if shift_dev is not None else shift, rms_weight=rms_weight, rms_eps=rms_eps,
                                   want_sent=want_sent, out_dtype=_F32 if out_f32 else qp.dtype)
    return o, S, (sent if sent is not None else torch.empty(0, device=qp.device, dtype=_BF16))


@aspin_layer_prefill.register_fake
def _(qp, kp, vp, gate_logits, decay_logits, decay_A, table, S0, theta, shift_dev, shift, rms_weight, rms_eps, want_sent, out_f32):
    B, T, H, D = qp.shape
    sent = _e(qp, B, H, _nc(T), D, D, dtype=_BF16) if want_sent else _e(qp, 0, dtype=_BF16)
    return _e(qp, B, T, H * D, dtype=_F32 if out_f32 else qp.dtype), _e(qp, B, H, D, D, dtype=_F32), sent


@torch.library.custom_op(f"{NS}::aspin_decode_step", mutates_args=())
def aspin_decode_step(qp: Tensor, kp: Tensor, vp: Tensor, decay: Tensor, S: Tensor, theta: Tensor, gate: Optional[Tensor], delta: bool,
                      gate_is_logit: bool, decay_A: Optional[Tensor], normalize: bool, shift_dev: Optional[Tensor], shift: float,
                      rms_weight: Optional[Tensor], rms_eps: float, out_f32: bool) -> Tuple[Tensor, Tensor]:
    o, S1 = ops.decode_step(qp, kp, vp, decay, S, theta, gate=gate, delta=delta, gate_is_logit=gate_is_logit, decay_A=decay_A,
                            normalize=normalize, shift=shift_dev if shift_dev is not None else shift, rms_weight=rms_weight,
                            rms_eps=rms_eps, out_dtype=_F32 if out_f32 else qp.dtype)
    return o, S1


@aspin_decode_step.register_fake
def _(qp, kp, vp, decay, S, theta, gate, delta, gate_is_logit, decay_A, normalize, shift_dev, shift, rms_weight, rms_eps, out_f32):
    B, H, D = qp.shape
    return _e(qp, B, H, D, dtype=_F32 if out_f32 else qp.dtype), torch.empty_like(S)


@torch.library.custom_op(f"{NS}::rot_table", mutates_args=())
def rot_table(theta: Tensor, T: int) -> Tensor:
    return ops.rot_table(theta, T)


@rot_table.register_fake
def _(theta, T):
    H, half = theta.shape
    return _e(theta, H, T, half, 2, dtype=_F32)


@torch.library.custom_op(f"{NS}::rotate", mutates_args=())
def rotate(x: Tensor, theta: Tensor, pos: Tensor) -> Tensor:
    return ops.rotate(x, theta, pos)


@rotate.register_fake
def _(x, theta, pos):
    return torch.empty(x.shape, device=x.device, dtype=x.dtype if x.dtype in (_F32, _BF16) else _F32)


@torch.library.custom_op(f"{NS}::add_norm", mutates_args=())
def add_norm(x: Tensor, delta: Optional[Tensor], weight: Tensor, bias: Optional[Tensor], eps: float, kind: int) -> Tuple[Tensor, Tensor]:
    y, z = ops.add_norm_raw(x, delta, weight, bias, eps, kind)
    return (y if delta is not None else torch.empty(0, device=x.device, dtype=x.dtype)), z


@add_norm.register_fake
def _(x, delta, weight, bias, eps, kind):
    return (torch.empty_like(x) if delta is not None else _e(x, 0)), torch.empty_like(x)


@torch.library.custom_op(f"{NS}::linear_act", mutates_args=())
def linear_act(x: Tensor, W: Tensor, bias: Optional[Tensor], act: int) -> Tensor:
    return ops.linear_act(x, W, bias, act="gelu" if act == 1 else None)


@linear_act.register_fake
def _(x, W, bias, act):
    return _e(x, *x.shape[:-1], W.shape[0])
