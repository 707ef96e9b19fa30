"""Tensor-level wrappers of the C ABI: shape checks, output allocation (by torch), one library call each.

All functions take CUDA tensors, launch on torch's current stream and never synchronise, so they can be captured in a
CUDA graph. They raise on CPU tensors: there is no fallback path.

Under torch.compile the wrappers hand over to the registered custom ops of the same name (pragnosia_b200/custom_ops.py,
namespace pragnosia_b200::), whose bodies call back into these functions eagerly: a compiled caller sees one opaque
operator with a shape function per kernel and no graph break.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ._lib import check, dtype_code, lib, need_cuda, on_device_of, ptr, stream_of

CHUNK = 64


def _f32c(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.to(torch.float32).contiguous()


def _compiling() -> bool:
    return torch.compiler.is_compiling()


def _cops():
    return torch.ops.pragnosia_b200                      # registered by custom_ops, imported at the end of this module


def _opt(t):
    """An operator returns an empty tensor where the wrapper returns None."""
    return None if t is None or t.numel() == 0 else t


def _shift_args(theta, S0, shift):
    """(theta or None, device shift or None, host shift): the rebase applies only with a state and a non-zero shift."""
    if theta is None or S0 is None:
        return None, None, 0.0
    if torch.is_tensor(shift):
        return _f32c(theta), shift.to(torch.float32).reshape(()), 0.0
    if float(shift) == 0.0:
        return None, None, 0.0
    return _f32c(theta), None, float(shift)


def _state_out(S_out, B, H, D, device):
    """The tensor the final state is written to: a new one, or the caller's (which may be the S0 it passed: every
    (sequence, head) reads its entering state before it writes its final one)."""
    if S_out is None:
        return torch.empty(B, H, D, D, device=device, dtype=torch.float32)
    if S_out.dtype != torch.float32 or not S_out.is_contiguous() or tuple(S_out.shape) != (B, H, D, D):
        raise ValueError("S_out must be a contiguous fp32 (B,H,D,D) tensor")
    return S_out


def _norm_args(norm: torch.nn.Module):
    """(kind 1 = RMS / 2 = layer norm, weight, bias or None, eps) of an nn.RMSNorm or nn.LayerNorm.
    nn.RMSNorm(eps=None) means the epsilon of the arithmetic type, which is fp32 for every dtype these kernels take."""
    if isinstance(norm, torch.nn.RMSNorm):
        return 1, norm.weight, None, (norm.eps if norm.eps is not None else torch.finfo(torch.float32).eps)
    return 2, norm.weight, norm.bias, norm.eps


# ----------------------------------------------------------------------------------------------------------
def _angle_view(ang, B, T, D):
    """The angle as fp32 with unit stride over D and either zero (batch, time) strides -- one angle per channel, read as
    such -- or the dense strides."""
    a32 = ang if ang.dtype == torch.float32 else ang.to(torch.float32)
    if a32.dim() == 1:
        a32 = a32.expand(B, T, D)
    if tuple(a32.shape) != (B, T, D):
        raise ValueError("lambda_scan: u, logmag, ang must share the shape (B,T,D)")
    if D > 1 and a32.stride(2) != 1:
        a32 = a32.contiguous()
    sb, st = (a32.stride(0) if B > 1 else 0), (a32.stride(1) if T > 1 else 0)
    if not (sb == 0 and st == 0) and not (st == D and sb == T * D):
        a32 = a32.contiguous(); sb, st = T * D, D
    return a32, sb, st


@on_device_of
def lambda_scan(u: torch.Tensor, logmag: torch.Tensor, ang: torch.Tensor, h0=None, time_segments: int = 0,
                keep_imag: bool = False):
    """h_t = lambda_t h_{t-1} + u_t with lambda_t = exp(logmag_t + i ang_t); returns (Re h (B,T,D) fp32,
    (Re h_T, Im h_T)).  `ang` may be an expanded view with zero batch/time strides (one angle per channel): it is
    read as such, not materialised.  keep_imag: also return Im h for every token as a third value (what the
    backward pass needs)."""
    need_cuda(u, logmag, ang)
    B, T, D = u.shape
    u32, lm32 = _f32c(u), _f32c(logmag)
    if tuple(lm32.shape) != (B, T, D):
        raise ValueError("lambda_scan: u, logmag, ang must share the shape (B,T,D)")
    h0r = h0i = None
    if h0 is not None:
        h0r, h0i = _f32c(h0[0]), _f32c(h0[1])
        need_cuda(h0r, h0i)
    if _compiling():
        y, hr, hi, hia = _cops().lambda_scan(u32, lm32, ang, h0r, h0i, int(time_segments), bool(keep_imag))
        return (y, (hr, hi), hia) if keep_imag else (y, (hr, hi))
    a32, sb, st = _angle_view(ang, B, T, D)
    y = torch.empty(B, T, D, device=u.device, dtype=torch.float32)
    hr = torch.empty(B, D, device=u.device, dtype=torch.float32)
    hi = torch.empty_like(hr)
    if keep_imag:
        hia = torch.empty_like(y)
        check(lib().pgb_lambda_scan_fwd_train(ptr(u32), ptr(lm32), ptr(a32), sb, st, ptr(h0r), ptr(h0i), ptr(y), ptr(hia), ptr(hr),
                                              ptr(hi), B, T, D, stream_of(u)), "pgb_lambda_scan_fwd_train")
        return y, (hr, hi), hia
    check(lib().pgb_lambda_scan_fwd_ex(ptr(u32), ptr(lm32), ptr(a32), sb, st, ptr(h0r), ptr(h0i), ptr(y), ptr(hr), ptr(hi),
                                       B, T, D, time_segments, stream_of(u)), "pgb_lambda_scan_fwd")
    return y, (hr, hi)


@on_device_of
def lambda_scan_bwd(g, u, logmag, ang, hr_all, hi_all, g_last_i=None, want_dh0: bool = False):
    """Adjoint of lambda_scan: g (B,T,D) is the gradient on Re h (the gradient on the final Re state already added to its
    last row), g_last_i (B,D) the gradient on the final Im state. Returns (du, dlogmag, dang, dh0r, dh0i); the last two
    are None unless want_dh0."""
    need_cuda(g, u, logmag, ang, hr_all, hi_all)
    B, T, D = u.shape
    g, u, logmag, hr_all, hi_all = (_f32c(t) for t in (g, u, logmag, hr_all, hi_all))
    gli = _f32c(g_last_i)
    if _compiling():
        du, dlm, dan, d0r, d0i = _cops().lambda_scan_bwd(g, u, logmag, ang, hr_all, hi_all, gli, bool(want_dh0))
        return du, dlm, dan, _opt(d0r), _opt(d0i)
    a32, sb, st = _angle_view(ang, B, T, D)
    du = torch.empty(B, T, D, device=u.device, dtype=torch.float32)
    dlm, dan = torch.empty_like(du), torch.empty_like(du)
    d0r = torch.empty(B, D, device=u.device, dtype=torch.float32) if want_dh0 else None
    d0i = torch.empty_like(d0r) if want_dh0 else None
    check(lib().pgb_lambda_scan_bwd(ptr(g), ptr(u), ptr(logmag), ptr(a32), sb, st, ptr(hr_all), ptr(hi_all), ptr(gli), ptr(du),
                                    ptr(dlm), ptr(dan), ptr(d0r), ptr(d0i), B, T, D, stream_of(u)), "pgb_lambda_scan_bwd")
    return du, dlm, dan, d0r, d0i


# ----------------------------------------------------------------------------------------------------------
def _prep_views(qp, kp, vp, gate_logits):
    B, T, H, D = qp.shape
    if kp.shape != qp.shape or vp.shape != qp.shape:
        raise ValueError("prep: qp, kp, vp must share the shape (B,T,H,D)")
    if qp.dtype not in (torch.float32, torch.bfloat16):
        qp, kp, vp = qp.float(), kp.float(), vp.float()
    kp, vp = kp.to(qp.dtype), vp.to(qp.dtype)

    def strided(t):
        per = D // 32                                   # channels a lane moves in one access: strides must keep it aligned
        ok = t.stride(3) == 1 and all(s % per == 0 for s in t.stride()[:3])
        return t if ok else t.contiguous()
    qp, kp, vp = strided(qp), strided(kp), strided(vp)
    if kp.stride() != qp.stride() or vp.stride() != qp.stride():
        qp, kp, vp = qp.contiguous(), kp.contiguous(), vp.contiguous()
    if gate_logits is not None:
        gate_logits = gate_logits.to(qp.dtype)
        if gate_logits.stride(2) != 1:
            gate_logits = gate_logits.contiguous()
    return qp, kp, vp, gate_logits


@on_device_of
def prep(qp, kp, vp, gate_logits, theta, pos, out_dtype=torch.bfloat16):
    """Normalise / gate / rotate / cast / transpose: (B,T,H,D) projections -> (B,H,T,D) scan operands."""
    need_cuda(qp, kp, vp, theta, pos)
    B, T, H, D = qp.shape
    qp, kp, vp, gate_logits = _prep_views(qp, kp, vp, gate_logits)
    theta = _f32c(theta)
    pos = pos.to(torch.int64).contiguous()
    if _compiling():
        return tuple(_cops().assoc_prep_ex(qp, kp, vp, gate_logits, theta, pos, out_dtype == torch.bfloat16))
    gsb, gst = (0, 0) if gate_logits is None else (gate_logits.stride(0), gate_logits.stride(1))
    q = torch.empty(B, H, T, D, device=qp.device, dtype=out_dtype)
    k, v = torch.empty_like(q), torch.empty_like(q)
    check(lib().pgb_aspin_prep_fwd(ptr(qp), ptr(kp), ptr(vp), dtype_code(qp), qp.stride(0), qp.stride(1), qp.stride(2),
                                   ptr(gate_logits), gsb, gst, ptr(theta), ptr(pos), ptr(q), ptr(k), ptr(v), dtype_code(q),
                                   B, T, H, D, stream_of(qp)), "pgb_aspin_prep_fwd")
    return q, k, v


@on_device_of
def prep_bwd(qp, kp, vp, gate_logits, theta, pos, dq, dk, dv):
    """Gradient of prep: returns (dqp, dkp, dvp in the projections' dtype, contiguous (B,T,H,D); dgate (B,T,H) fp32 or
    None; dtheta (H,D/2) fp32)."""
    need_cuda(qp, kp, vp, theta, pos, dq, dk, dv)
    B, T, H, D = qp.shape
    qp, kp, vp, gate_logits = _prep_views(qp, kp, vp, gate_logits)
    theta = _f32c(theta)
    pos = pos.to(torch.int64).contiguous()
    if dq.dtype not in (torch.float32, torch.bfloat16):
        dq = dq.float()
    dq, dk, dv = dq.contiguous(), dk.to(dq.dtype).contiguous(), dv.to(dq.dtype).contiguous()
    if _compiling():
        dqp, dkp, dvp, dgl, dth = _cops().assoc_prep_bwd(qp, kp, vp, gate_logits, theta, pos, dq, dk, dv)
        return dqp, dkp, dvp, _opt(dgl), dth
    gsb, gst = (0, 0) if gate_logits is None else (gate_logits.stride(0), gate_logits.stride(1))
    dqp = torch.empty(B, T, H, D, device=qp.device, dtype=qp.dtype)
    dkp, dvp = torch.empty_like(dqp), torch.empty_like(dqp)
    dgl = None if gate_logits is None else torch.empty(B, T, H, device=qp.device, dtype=torch.float32)
    nt = lib().pgb_aspin_prep_bwd_tiles(T)
    part = torch.empty(B * nt, H, D // 2, device=qp.device, dtype=torch.float32)
    check(lib().pgb_aspin_prep_bwd(ptr(qp), ptr(kp), ptr(vp), dtype_code(qp), qp.stride(0), qp.stride(1), qp.stride(2),
                                   ptr(gate_logits), gsb, gst, ptr(theta), ptr(pos), ptr(dq), ptr(dk), ptr(dv), dtype_code(dq),
                                   ptr(dqp), ptr(dkp), ptr(dvp), ptr(dgl), ptr(part), B, T, H, D, stream_of(qp)),
          "pgb_aspin_prep_bwd")
    return dqp, dkp, dvp, dgl, part.sum(0)


# ----------------------------------------------------------------------------------------------------------
@on_device_of
def prefill(q, k, v, la, beta=None, S0=None, theta=None, shift=0.0, want_sent: bool = False,
            precision: int = _lib.PREFILL_AUTO, out_dtype=None, S_out=None):
    """Chunked prefill. q,k,v (B,H,T,D) fp32 or bf16 (same dtype); la (B,H,T); beta (B,H,T) or None (plain rule);
    S0 (B,H,D,D) or None.  theta/shift: rebase S0's key axis by -shift*theta first (shift: number or 0-d CUDA tensor).
    Returns (o in out_dtype (default q's dtype), S fp32, sent bf16 (B,H,NC,D,D) or None)."""
    need_cuda(q, k, v, la)
    B, H, T, D = q.shape
    if q.dtype not in (torch.float32, torch.bfloat16):
        q = q.float()
    q, k, v = q.contiguous(), k.to(q.dtype).contiguous(), v.to(q.dtype).contiguous()
    la, beta, S0 = _f32c(la), _f32c(beta), _f32c(S0)
    theta, shift_dev, shift_host = _shift_args(theta, S0, shift)
    if shift_dev is not None:
        need_cuda(shift_dev)
    odt = out_dtype or q.dtype
    if _compiling():
        o, S, sent = _cops().aspin_prefill(q, k, v, la, beta, S0, theta, shift_dev, shift_host, bool(want_sent), int(precision),
                                           odt == torch.float32)
        return o, S, _opt(sent)
    o = torch.empty(B, H, T, D, device=q.device, dtype=odt)
    S = _state_out(S_out, B, H, D, q.device)
    NC = (T + CHUNK - 1) // CHUNK
    sent = torch.empty(B, H, NC, D, D, device=q.device, dtype=torch.bfloat16) if want_sent else None
    if beta is not None and q.dtype == torch.bfloat16 and precision != _lib.PREFILL_FP32 and B * H <= 65535:
        # delta rule on the tensor cores: the chunk inverses go through a scratch buffer (allocated here, by torch)
        nbytes = lib().pgb_aspin_delta_scratch_bytes(B, H, T)
        scratch = torch.empty(nbytes, device=q.device, dtype=torch.uint8)
        check(lib().pgb_aspin_delta_prefill_fwd(ptr(q), ptr(k), ptr(v), ptr(la), ptr(beta), ptr(S0), ptr(theta), ptr(shift_dev),
                                                shift_host, ptr(o), dtype_code(o), ptr(S), ptr(sent), ptr(scratch), nbytes,
                                                B, H, T, D, stream_of(q)), "pgb_aspin_delta_prefill_fwd")
        return o, S, sent
    check(lib().pgb_aspin_prefill_fwd(ptr(q), ptr(k), ptr(v), dtype_code(q), ptr(la), ptr(beta), ptr(S0), ptr(theta),
                                      ptr(shift_dev), shift_host, ptr(o), dtype_code(o), ptr(S), ptr(sent), B, H, T, D, precision,
                                      stream_of(q)), "pgb_aspin_prefill_fwd")
    return o, S, sent


# ----------------------------------------------------------------------------------------------------------
@on_device_of
def prefill_fused(q, k, v, decay_logits, decay_A, S0=None, theta=None, shift=0.0, rms_weight=None, rms_eps=0.0,
                  want_sent: bool = False, out_dtype=None, S_out=None):
    """Plain-rule prefill on the tensor cores with the decay gate, the per-head RMS norm and the transpose fused in.
    q,k,v (B,H,T,D) bf16 from prep(); decay_logits: bf16 (B,T,H) view with unit stride over H (the decay gate's linear
    output); decay_A (H,) fp32.  Returns (o (B,T,H*D) token-major, S fp32, sent or None)."""
    need_cuda(q, k, v, decay_logits)
    B, H, T, D = q.shape
    if q.dtype != torch.bfloat16 or decay_logits.dtype != torch.bfloat16:
        raise TypeError("prefill_fused takes bf16 operands")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if decay_logits.stride(2) != 1:
        decay_logits = decay_logits.contiguous()
    S0 = _f32c(S0)
    theta, shift_dev, shift_host = _shift_args(theta, S0, shift)
    decay_A, rms_weight = _f32c(decay_A), _f32c(rms_weight)
    odt = out_dtype or q.dtype
    if _compiling():
        o, S, sent = _cops().aspin_prefill_fused(q, k, v, decay_logits, decay_A, S0, theta, shift_dev, shift_host, rms_weight,
                                                 float(rms_eps), bool(want_sent), odt == torch.float32)
        return o, S, _opt(sent)
    o = torch.empty(B, T, H * D, device=q.device, dtype=odt)
    S = _state_out(S_out, B, H, D, q.device)
    NC = (T + CHUNK - 1) // CHUNK
    sent = torch.empty(B, H, NC, D, D, device=q.device, dtype=torch.bfloat16) if want_sent else None
    check(lib().pgb_aspin_prefill_fused_fwd(
        ptr(q), ptr(k), ptr(v), ptr(decay_logits), decay_logits.stride(0), decay_logits.stride(1), ptr(decay_A),
        ptr(S0), ptr(theta), ptr(shift_dev), shift_host, ptr(rms_weight), float(rms_eps), ptr(o), dtype_code(o),
        ptr(S), ptr(sent), B, H, T, D, stream_of(q)), "pgb_aspin_prefill_fused_fwd")
    return o, S, sent


# ----------------------------------------------------------------------------------------------------------
@on_device_of
def rot_table(theta, T: int):
    """(H, T, D/2, 2) fp32 table of (cos, sin)(t * theta[h, i]) for positions 0..T-1."""
    need_cuda(theta)
    theta = _f32c(theta)
    if _compiling():
        return _cops().rot_table(theta, int(T))
    H, half = theta.shape
    table = torch.empty(H, T, half, 2, device=theta.device, dtype=torch.float32)
    check(lib().pgb_rot_table_build(ptr(theta), ptr(table), H, T, 2 * half, stream_of(theta)), "pgb_rot_table_build")
    return table


@on_device_of
def layer_prefill(qp, kp, vp, gate_logits, decay_logits, decay_A, table, S0=None, theta=None, shift=0.0, rms_weight=None,
                  rms_eps=0.0, want_sent: bool = False, out_dtype=None, S_out=None):
    """The layer's prefill between its GEMMs in one kernel. qp,kp,vp: bf16 (B,T,H,D) views of the projection output
    sharing strides, unit stride over (H,D); gate_logits (or None) / decay_logits: bf16 (B,T,H) views sharing strides;
    table from rot_table(theta, >= T).  Returns (o (B,T,H*D), S fp32, sent or None)."""
    need_cuda(qp, kp, vp, decay_logits, table)
    B, T, H, D = qp.shape
    for t in (qp, kp, vp):
        if t.dtype != torch.bfloat16 or t.stride(3) != 1 or t.stride(2) != D or t.stride() != qp.stride():
            raise ValueError("layer_prefill: q,k,v must be bf16 (B,T,H,D) views with unit strides over (H,D) and common strides")
    if decay_logits.dtype != torch.bfloat16 or decay_logits.stride(2) != 1:
        raise ValueError("layer_prefill: decay_logits must be a bf16 (B,T,H) view with unit stride over H")
    if gate_logits is not None and (gate_logits.dtype != torch.bfloat16 or gate_logits.stride() != decay_logits.stride()):
        raise ValueError("layer_prefill: gate_logits must share decay_logits' dtype and strides")
    if table.shape[1] < (T + CHUNK - 1) // CHUNK * CHUNK:
        raise ValueError("layer_prefill: the rotation table must cover the window rounded up to whole 64-token chunks")
    S0 = _f32c(S0)
    theta, shift_dev, shift_host = _shift_args(theta, S0, shift)
    decay_A, rms_weight = _f32c(decay_A), _f32c(rms_weight)
    odt = out_dtype or qp.dtype
    if _compiling():
        o, S, sent = _cops().aspin_layer_prefill(qp, kp, vp, gate_logits, decay_logits, decay_A, table, S0, theta, shift_dev,
                                                 shift_host, rms_weight, float(rms_eps), bool(want_sent), odt == torch.float32)
        return o, S, _opt(sent)
    o = torch.empty(B, T, H * D, device=qp.device, dtype=odt)
    S = _state_out(S_out, B, H, D, qp.device)
    NC = (T + CHUNK - 1) // CHUNK
    sent = torch.empty(B, H, NC, D, D, device=qp.device, dtype=torch.bfloat16) if want_sent else None
    sbq = qp.stride(0) if B > 1 else T * qp.stride(1)
    sba = decay_logits.stride(0) if B > 1 else T * decay_logits.stride(1)
    check(lib().pgb_aspin_layer_prefill_fwd(
        ptr(qp), ptr(kp), ptr(vp), sbq, qp.stride(1), ptr(gate_logits), ptr(decay_logits), sba, decay_logits.stride(1),
        ptr(decay_A), ptr(table), table.shape[1], ptr(S0), ptr(theta), ptr(shift_dev), shift_host,
        ptr(rms_weight), float(rms_eps), ptr(o), dtype_code(o), ptr(S), ptr(sent), B, H, T, D, stream_of(qp)),
        "pgb_aspin_layer_prefill_fwd")
    return o, S, sent


# ----------------------------------------------------------------------------------------------------------
@on_device_of
def rotate(x, theta, pos):
    """Rotate channel pairs of x (B,H,T,D) by pos[t]*theta[h,i]."""
    need_cuda(x, theta, pos)
    B, H, T, D = x.shape
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.float()
    x, theta, pos = x.contiguous(), _f32c(theta), _f32c(pos)
    if _compiling():
        return _cops().rotate(x, theta, pos)
    out = torch.empty_like(x)
    check(lib().pgb_rotate_pairs(ptr(x), dtype_code(x), ptr(theta), ptr(pos), ptr(out), B, H, T, D,
                                 stream_of(x)), "pgb_rotate_pairs")
    return out


# ----------------------------------------------------------------------------------------------------------
@on_device_of
def decode_step(qp, kp, vp, decay, S, theta, *, gate=None, delta: bool = False, gate_is_logit: bool = True,
                decay_A=None, normalize: bool = True, shift=0.0, rms_weight=None, rms_eps: float = 0.0,
                out: Optional[torch.Tensor] = None, S_out: Optional[torch.Tensor] = None, out_dtype=None):
    """One fused recurrent step. qp,kp,vp: (B,H,D) views with unit strides over (H,D) and a common batch stride;
    decay, gate: (B,H) views with unit stride over H.  S (B,H,D,D) fp32; S_out defaults to a new tensor (pass S itself
    for an in-place update).  Returns (o (B,H,D), S_out)."""
    need_cuda(qp, kp, vp, decay, S, theta)
    B, H, D = qp.shape
    for t in (qp, kp, vp):
        if t.stride(2) != 1 or t.stride(1) != D or t.dtype != qp.dtype:
            raise ValueError("decode_step: q,k,v must be (B,H,D) with unit strides over (H,D) and one dtype")
    if kp.stride(0) != qp.stride(0) or vp.stride(0) != qp.stride(0):
        raise ValueError("decode_step: q,k,v must share the batch stride")
    if decay.dtype != qp.dtype or (gate is not None and gate.dtype != qp.dtype):
        raise ValueError("decode_step: decay and gate must have q's dtype")
    if S.dtype != torch.float32 or not S.is_contiguous():
        raise ValueError("decode_step: the state must be contiguous fp32")
    out_dtype = out_dtype or qp.dtype
    shift_dev, shift_host = (shift.to(torch.float32), 0.0) if torch.is_tensor(shift) else (None, float(shift))
    decay_A, theta, rms_weight = _f32c(decay_A), _f32c(theta), _f32c(rms_weight)
    if _compiling():
        o, S1 = _cops().aspin_decode_step(qp, kp, vp, decay, S, theta, gate, bool(delta), bool(gate_is_logit), decay_A,
                                          bool(normalize), shift_dev, shift_host, rms_weight, float(rms_eps),
                                          out_dtype == torch.float32)
        return o, S1
    S_out = torch.empty_like(S) if S_out is None else S_out
    if out is None:
        out = torch.empty(B, H, D, device=qp.device, dtype=out_dtype)
    sb = lambda t: t.stride(0) if B > 1 else max(t.stride(0), H * (t.shape[2] if t.dim() == 3 else 1))
    check(lib().pgb_aspin_decode_step(
        ptr(qp), ptr(kp), ptr(vp), dtype_code(qp), sb(qp), int(normalize), ptr(gate), 0 if gate is None else gate.stride(0),
        int(gate_is_logit), int(delta), ptr(decay), decay.stride(0), ptr(decay_A), ptr(theta),
        ptr(shift_dev), shift_host, ptr(S), ptr(S_out), ptr(rms_weight), float(rms_eps), ptr(out), dtype_code(out),
        sb(out), B, H, D, stream_of(qp)), "pgb_aspin_decode_step")
    return out, S_out


# ----------------------------------------------------------------------------------------------------------
@on_device_of
def add_norm_raw(x, delta, weight, bias, eps: float, kind: int):
    """y = x + delta (delta may be None); z = RMS norm (kind 1) or layer norm (kind 2) of y over the last dim with the given
    weight / bias / eps.  Returns (y, z); y is x itself when delta is None."""
    need_cuda(x)
    d = x.shape[-1]
    x = x.contiguous()
    if delta is not None:
        delta = delta.to(x.dtype).contiguous()
    w = weight.to(x.dtype)
    b = None if bias is None else bias.to(x.dtype)
    if _compiling():
        y, z = _cops().add_norm(x, delta, w, b, float(eps), int(kind))
        return (x if delta is None else y), z
    y = torch.empty_like(x) if delta is not None else None
    z = torch.empty_like(x)
    check(lib().pgb_add_norm(ptr(x), ptr(delta), ptr(w), ptr(b), float(eps), kind - 1, ptr(y), ptr(z),
                             x.numel() // d, d, dtype_code(x), stream_of(x)), "pgb_add_norm")
    return (x if delta is None else y), z


def add_norm(x, delta, norm: torch.nn.Module):
    """add_norm_raw with the parameters of an nn.RMSNorm or nn.LayerNorm."""
    kind, w, b, eps = _norm_args(norm)
    return add_norm_raw(x, delta, w, b, eps, kind)


def _cast_once(t, dtype):
    """(t in dtype and contiguous, whether a new tensor had to be made for it just now)."""
    if t is None:
        return None, False
    c = t.to(dtype).contiguous()
    return c, c.data_ptr() != t.data_ptr()


@on_device_of
def skinny_linear(x, W, bias=None, delta=None, norm: Optional[torch.nn.Module] = None, act: Optional[str] = None,
                  want_sum: bool = False):
    """y = act(norm(x + delta) W^T + bias) for a few rows in ONE launch (decode at batch <= 8; bf16).
    x, delta (B,K); W (N,K); norm an nn.RMSNorm / nn.LayerNorm or None; act None or "gelu" (erf).
    Returns y (B,N), or (y, x + delta) with want_sum (the new residual stream, rounded to bf16 like a separate add)."""
    need_cuda(x, W)
    B, K = x.shape
    N = W.shape[0]
    if x.dtype != torch.bfloat16 or W.dtype != torch.bfloat16:
        raise ValueError("skinny_linear: bf16 only")
    x = x.contiguous()
    W, fresh = _cast_once(W, x.dtype)
    if delta is not None:
        delta = delta.to(x.dtype).contiguous()
    kind, nw, nb, eps = 0, None, None, 0.0
    if norm is not None:
        kind, nw, nb, eps = _norm_args(norm)
        nw, f1 = _cast_once(nw, x.dtype)
        nb, f2 = _cast_once(nb, x.dtype)
        fresh = fresh or f1 or f2
    bias, f3 = _cast_once(bias, x.dtype)
    # The kernel requests its weights before it waits for the kernel ahead of it on the stream. A cast made just above is
    # that kernel: tell the launch to fetch the constants only after the wait.
    flags = 1 if (fresh or f3) else 0
    y = torch.empty(B, N, device=x.device, dtype=x.dtype)
    s = torch.empty_like(x) if (want_sum and delta is not None) else None
    check(lib().pgb_skinny_linear_ex(ptr(x), ptr(delta), ptr(nw), ptr(nb), kind, float(eps), ptr(W), ptr(bias),
                                     1 if act == "gelu" else 0, ptr(y), ptr(s), B, K, N, flags, stream_of(x)), "pgb_skinny_linear")
    if want_sum:
        return y, (x if delta is None else s)
    return y


@on_device_of
def batch_linear(x, W, bias=None, act: Optional[str] = None, folded=None, resid=None, want_sums: bool = False):
    """y = act(x W^T + bias) for up to 128 decode rows in ONE tensor-core launch (bf16); x (B,K), W (N,K), act None or
    "gelu" (erf). N and K multiples of 8.
    folded = (row_sums (P,B,2) fp32, c1 (N,) fp32, c2 (N,) fp32, kind, eps): x is the raw residual stream and W carries the
    norm's weight (fold_norm); the norm is applied on the accumulator. resid (B,N): returns resid + y, the new residual
    stream, and with want_sums also its partial row sums (parts,B,2) for the next folded norm."""
    need_cuda(x, W)
    if x.dtype != torch.bfloat16 or W.dtype != torch.bfloat16 or x.dim() != 2:
        raise ValueError("batch_linear: bf16, x (B,K)")
    B, K = x.shape
    N = W.shape[0]
    x = x.contiguous()
    W, fresh = _cast_once(W, x.dtype)
    b, f2 = _cast_once(bias, x.dtype)
    fresh = fresh or f2                                              # a constant made by a kernel just now: tell the launch
    y = torch.empty(B, N, device=x.device, dtype=x.dtype)
    sums_in, parts_in, c1, c2, kind, eps = None, 0, None, None, 0, 0.0
    if folded is not None:
        sums_in, c1, c2, kind, eps = folded
        parts_in = sums_in.shape[0]
        if sums_in.dtype != torch.float32 or tuple(sums_in.shape[1:]) != (B, 2) or not sums_in.is_contiguous() or b is not None:
            raise ValueError("batch_linear: row sums (parts,B,2) fp32, and no separate bias with a folded norm")
    sums_out = None
    if resid is not None:
        resid = resid.contiguous()
        if want_sums:
            sums_out = torch.empty(int(lib().pgb_batch_linear_parts(N)), B, 2, device=x.device, dtype=torch.float32)
    check(lib().pgb_batch_linear_ex(ptr(x), ptr(W), ptr(b), ptr(y), B, N, K, 1 if act == "gelu" else 0, ptr(sums_in), parts_in, ptr(c1),
                                    ptr(c2), int(kind), float(eps), ptr(resid), ptr(sums_out), 1 if fresh else 0, stream_of(x)),
          "pgb_batch_linear")
    return (y, sums_out) if want_sums else y


def fold_norm(norm: torch.nn.Module, W, bias=None):
    """The constants that let a linear layer take the norm in front of it (batch_linear's folded form): W' = W diag(w) in
    W's dtype, c1 = row sums of W' and c2 = W beta + bias in fp32. Returns (W', c1, c2, kind, eps)."""
    kind, w, beta, eps = _norm_args(norm)
    Wf = (W.float() * w.float()).to(W.dtype).contiguous()
    c1 = Wf.float().sum(1).contiguous()
    c2 = torch.zeros(W.shape[0], device=W.device, dtype=torch.float32)
    if beta is not None:
        c2 = c2 + W.float() @ beta.float()
    if bias is not None:
        c2 = c2 + bias.float()
    return Wf, c1, c2.contiguous(), kind, eps


@on_device_of
def decode_embed(tok, pos, E, P, want_sums: bool = False):
    """x (B,d) = E[tok] + P[pos] in one launch; tok (B,) / (B,1) int64 and pos (1,) int64 on the device, bf16 tables.
    want_sums: also the rows' (sum, sum of squares) as (1,B,2) fp32, for a norm folded into the next linear layer."""
    need_cuda(tok, pos, E, P)
    if E.dtype != torch.bfloat16 or P.dtype != torch.bfloat16 or tok.dtype != torch.long or pos.dtype != torch.long:
        raise ValueError("decode_embed: bf16 tables, int64 ids")
    B, d = tok.numel(), E.shape[1]
    x = torch.empty(B, d, device=E.device, dtype=E.dtype)
    sums = torch.empty(1, B, 2, device=E.device, dtype=torch.float32) if want_sums else None
    check(lib().pgb_decode_embed_ex(ptr(tok.contiguous()), ptr(pos), ptr(E.contiguous()), ptr(P.contiguous()), ptr(x), ptr(sums), B, d,
                                    E.shape[0], P.shape[0], stream_of(E)), "pgb_decode_embed")
    return (x, sums) if want_sums else x


@on_device_of
def decode_token(table, E, P, final_norm, tok, pos, shift, work, logits, sync, H, D, NP, dff, delta: bool):
    """One decode step of the whole model in ONE cooperative launch (decode_token.cu): embedding, every layer, final norm
    and tied head for 1..4 sequences. table (L,18) int64 on the device: the per-layer pointers and norm settings the C
    header documents (generate.Decoder builds it); work / sync: scratch from decode_token_work_bytes and two zeroed
    64-bit words; logits (B,V) fp32 out. The states the table points at are updated in place."""
    need_cuda(table, E, P, tok, pos, shift, work, logits, sync)
    if E.dtype != torch.bfloat16 or P.dtype != torch.bfloat16 or tok.dtype != torch.long or pos.dtype != torch.long:
        raise ValueError("decode_token: bf16 tables, int64 ids")
    if table.dtype != torch.int64 or table.dim() != 2 or table.shape[1] != 18 or not table.is_contiguous():
        raise ValueError("decode_token: table must be a contiguous (L,18) int64 tensor")
    if logits.dtype != torch.float32 or not logits.is_contiguous() or shift.dtype != torch.float32:
        raise ValueError("decode_token: fp32 logits and shift")
    kind, nw, nb, eps = _norm_args(final_norm)
    if nw.dtype != torch.bfloat16 or (nb is not None and nb.dtype != torch.bfloat16):
        raise ValueError("decode_token: bf16 norm parameters")
    B, V, d = logits.shape[0], E.shape[0], E.shape[1]
    check(lib().pgb_decode_token_fwd(ptr(table), table.shape[0], ptr(E), ptr(P), ptr(nw), ptr(nb), kind, float(eps), ptr(tok), ptr(pos),
                                     ptr(shift), ptr(work), work.numel() * work.element_size(), ptr(logits), ptr(sync), B, d, H, D, NP,
                                     dff, V, P.shape[0], 1 if delta else 0, stream_of(E)), "pgb_decode_token_fwd")
    return logits


def decode_token_work_bytes(B: int, d: int, NP: int, dff: int) -> int:
    return int(lib().pgb_decode_token_work_bytes(B, d, NP, dff))


@on_device_of
def decode_sample(logits, temp, seed, tok, count, ticket, hist=None, pos=None, shift=None, ctx: int = 1, min_p: float = 0.0):
    """Draw one id per row of logits (B,V) into tok (B,) / (B,1) int64, record it in hist[:, count] and advance the step
    counters (count, pos modulo ctx, shift) -- all on the device, one launch. ticket: a zeroed uint32/int32 scalar.
    min_p > 0 drops every id whose probability is below min_p times the largest one before the draw."""
    need_cuda(logits, tok, count, ticket)
    B, V = logits.shape
    if logits.dtype not in (torch.float32, torch.bfloat16):
        logits = logits.float()
    logits = logits.contiguous()
    cols = 0 if hist is None else hist.shape[1]
    check(lib().pgb_decode_sample_ex(ptr(logits), dtype_code(logits), float(temp), float(min_p), int(seed) & 0xFFFFFFFFFFFFFFFF,
                                     ptr(tok), ptr(hist), cols, ptr(count), ptr(pos), ptr(shift), ptr(ticket), B, V, int(ctx),
                                     stream_of(logits)), "pgb_decode_sample")
    return tok


@on_device_of
def linear_act(x, W, bias=None, act: Optional[str] = "gelu"):
    """act(x W^T + bias) as one tensor-core GEMM with the bias and the (erf) GELU in its epilogue; x (..., K) bf16, W (N, K)."""
    need_cuda(x, W)
    if x.dtype != torch.bfloat16 or W.dtype != torch.bfloat16:
        raise ValueError("linear_act: bf16 only")
    K, N = x.shape[-1], W.shape[0]
    x2 = x.reshape(-1, K).contiguous()
    W = W.contiguous()
    b = None if bias is None else bias.to(x.dtype).contiguous()
    if _compiling():
        return _cops().linear_act(x2, W, b, 1 if act == "gelu" else 0).view(*x.shape[:-1], N)
    y = torch.empty(x2.shape[0], N, device=x.device, dtype=x.dtype)
    check(lib().pgb_linear_act(ptr(x2), ptr(W), ptr(b), ptr(y), x2.shape[0], N, K, 1 if act == "gelu" else 0,
                               stream_of(x)), "pgb_linear_act")
    return y.view(*x.shape[:-1], N)


# ---------------------------------------------------------------------------------------------------------- split operators
def _needs_grad(*ts):
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in ts)


def _io(t):
    return t if t.dtype in (torch.float32, torch.bfloat16) else t.float()


@on_device_of
def assoc_out(q, k, v, la, sent, bc: int = CHUNK):
    """One chunk's output for every chunk, given the state entering each (the reference's membrae::assoc_out):
    o = ((q k^T) * dec) v + (q e^L) sent[c].  q,k,v (B,H,T,D); la (B,H,T); sent (B,H,NC,D,D)."""
    need_cuda(q, k, v, la, sent)
    if bc != CHUNK:
        raise ValueError("assoc_out: the kernels chunk by 64 tokens")
    B, H, T, D = q.shape
    q = _io(q).contiguous()
    k, v = k.to(q.dtype).contiguous(), v.to(q.dtype).contiguous()
    la, sent = _f32c(la), sent.to(torch.bfloat16).contiguous()
    if tuple(sent.shape) != (B, H, (T + CHUNK - 1) // CHUNK, D, D):
        raise ValueError("assoc_out: sent must be (B,H,ceil(T/64),D,D)")
    if _compiling() or _needs_grad(q, k, v, la, sent):
        return _cops().assoc_out(q, k, v, la, sent, int(bc))     # the operator carries the backward (assoc_out_bwd)
    o = torch.empty_like(q)
    check(lib().pgb_assoc_out_fwd(ptr(q), ptr(k), ptr(v), dtype_code(q), ptr(la), ptr(sent), ptr(o), B, H, T, D, stream_of(q)),
          "pgb_assoc_out_fwd")
    return o


@on_device_of
def prefix_scan(k, v, w, a_log, S0=None, has_s0: bool = True, bv: int = 16):
    """The state entering every chunk and the final state (membrae::prefix_scan): sent[c] = S; S = exp(a_log[c]) S + (k w)^T v.
    k, v (B,H,NC*64,D) whole chunks; w (B,H,NC,64,1) or (B,H,NC,64); a_log (B,H,NC)."""
    need_cuda(k, v, w, a_log)
    B, H, NC = w.shape[:3]
    D = k.shape[-1]
    k = _io(k).contiguous()
    v = v.to(k.dtype).contiguous()
    if k.shape[2] != NC * CHUNK:
        raise ValueError("prefix_scan: k and v must hold whole 64-token chunks")
    w, a_log = _f32c(w), _f32c(a_log)
    S0 = _f32c(S0) if (has_s0 and S0 is not None) else None
    if _compiling() or _needs_grad(k, v, w, a_log, S0):
        return tuple(_cops().prefix_scan(k, v, w, a_log, S0, S0 is not None, int(bv)))   # carries the backward (prefix_scan_bwd)
    sent = torch.empty(B, H, NC, D, D, device=k.device, dtype=torch.bfloat16)
    sfin = torch.empty(B, H, D, D, device=k.device, dtype=torch.float32)
    check(lib().pgb_prefix_scan_fwd(ptr(k), ptr(v), dtype_code(k), ptr(w), ptr(a_log), ptr(S0), ptr(sent), ptr(sfin), B, H, NC, D,
                                    stream_of(k)), "pgb_prefix_scan_fwd")
    return sent, sfin


@on_device_of
def assoc_out_bwd(q, k, v, la, sent, dout):
    """Gradients of assoc_out (the reference's _bwd_chunk): (dq, dk, dv (B,H,T,D), dla (B,H,T), dsent (B,H,NC,D,D)), fp32."""
    need_cuda(q, k, v, la, sent, dout)
    B, H, T, D = q.shape
    q = _io(q).contiguous()
    k, v, dout = k.to(q.dtype).contiguous(), v.to(q.dtype).contiguous(), dout.to(q.dtype).contiguous()
    la, sent = _f32c(la), sent.to(torch.bfloat16).contiguous()
    NC = (T + CHUNK - 1) // CHUNK
    f = dict(device=q.device, dtype=torch.float32)
    dq, dk, dv = (torch.empty(B, H, T, D, **f) for _ in range(3))
    dla, dsent = torch.empty(B, H, T, **f), torch.empty(B, H, NC, D, D, **f)
    check(lib().pgb_assoc_out_bwd(ptr(q), ptr(k), ptr(v), dtype_code(q), ptr(la), ptr(sent), ptr(dout), ptr(dq), ptr(dk), ptr(dv),
                                  ptr(dla), ptr(dsent), B, H, T, D, stream_of(q)), "pgb_assoc_out_bwd")
    return dq, dk, dv, dla, dsent


@on_device_of
def prefix_scan_bwd(k, v, w, a_log, sent, dsent, dsfin, want_ds0: bool = True):
    """Gradients of prefix_scan (the reference's _prefix_bwd): (dk, dv (B,H,NC*64,D), dw (B,H,NC,64), da_log (B,H,NC),
    dS0 (B,H,D,D) or None), fp32. dsent / dsfin may be None (no gradient arrived)."""
    need_cuda(k, v, w, a_log, sent)
    B, H, NC = a_log.shape
    D = k.shape[-1]
    k = _io(k).contiguous()
    v = v.to(k.dtype).contiguous()
    w, a_log, sent = _f32c(w), _f32c(a_log), sent.to(torch.bfloat16).contiguous()
    dsent = None if dsent is None else _f32c(dsent)
    dsfin = None if dsfin is None else _f32c(dsfin)
    f = dict(device=k.device, dtype=torch.float32)
    dk, dv = torch.empty(B, H, NC * CHUNK, D, **f), torch.empty(B, H, NC * CHUNK, D, **f)
    dw, da = torch.empty(B, H, NC, CHUNK, **f), torch.empty(B, H, NC, **f)
    ds0 = torch.empty(B, H, D, D, **f) if want_ds0 else None
    check(lib().pgb_prefix_scan_bwd(ptr(k), ptr(v), dtype_code(k), ptr(w), ptr(a_log), ptr(sent), ptr(dsent), ptr(dsfin), ptr(dk), ptr(dv),
                                    ptr(dw), ptr(da), ptr(ds0), B, H, NC, D, stream_of(k)), "pgb_prefix_scan_bwd")
    return dk, dv, dw, da, ds0


@on_device_of
def delta_inv(k, la, be, nc: int):
    """X = (I + beta strictly_lower((k k^T) dec))^-1 per 64-token chunk, bf16 (B,H,nc,64,64) (membrae::delta_inv)."""
    need_cuda(k, la, be)
    B, H, T, D = k.shape
    if nc != (T + CHUNK - 1) // CHUNK:
        raise ValueError("delta_inv: nc must be ceil(T/64)")
    k, la, be = k.to(torch.bfloat16).contiguous(), _f32c(la), _f32c(be)
    if _compiling() or _needs_grad(k, la, be):
        return _cops().delta_inv(k, la, be, int(nc))                 # the operator carries the backward (delta_inv_bwd)
    X = torch.empty(B, H, nc, CHUNK, CHUNK, device=k.device, dtype=torch.bfloat16)
    check(lib().pgb_delta_inv_fwd(ptr(k), ptr(la), ptr(be), ptr(X), B, H, T, D, stream_of(k)), "pgb_delta_inv_fwd")
    return X


@on_device_of
def delta_loop_fwd(k, v, la, be, X, S0=None, has_s0: bool = True, bc: int = CHUNK, bv: int = 32, bvb: int = 16):
    """The delta rule's walk over chunks with the inverses given (membrae::delta_loop_fwd): returns (W bf16 (B,H,T,D) --
    the residuals actually written --, sent bf16 (B,H,NC,D,D), sfin fp32)."""
    need_cuda(k, v, la, be, X)
    if bc != CHUNK:
        raise ValueError("delta_loop_fwd: the kernels chunk by 64 tokens")
    B, H, T, D = k.shape
    NC = X.shape[2]
    k = _io(k).contiguous()
    v = v.to(k.dtype).contiguous()
    la, be, X = _f32c(la), _f32c(be), X.to(torch.bfloat16).contiguous()
    S0 = _f32c(S0) if (has_s0 and S0 is not None) else None
    if _compiling() or _needs_grad(k, v, la, be, X, S0):
        return tuple(_cops().delta_loop_fwd(k, v, la, be, X, S0, S0 is not None, int(bc), int(bv), int(bvb)))   # carries delta_loop_bwd
    W = torch.empty(B, H, T, D, device=k.device, dtype=torch.bfloat16)
    sent = torch.empty(B, H, NC, D, D, device=k.device, dtype=torch.bfloat16)
    sfin = torch.empty(B, H, D, D, device=k.device, dtype=torch.float32)
    check(lib().pgb_delta_loop_fwd(ptr(k), ptr(v), dtype_code(k), ptr(la), ptr(be), ptr(X), ptr(S0), ptr(W), ptr(sent), ptr(sfin),
                                   B, H, T, D, stream_of(k)), "pgb_delta_loop_fwd")
    return W, sent, sfin


@on_device_of
def delta_inv_bwd(k, la, be, X, dX):
    """Gradients of delta_inv (the reference's _inv_bwd): (dk (B,H,T,D), dla, dbeta (B,H,T)), fp32."""
    need_cuda(k, la, be, X, dX)
    B, H, T, D = k.shape
    k = _io(k).contiguous()
    la, be, X, dX = _f32c(la), _f32c(be), X.to(torch.bfloat16).contiguous(), _f32c(dX)
    f = dict(device=k.device, dtype=torch.float32)
    dk, dla, dbe = torch.empty(B, H, T, D, **f), torch.empty(B, H, T, **f), torch.empty(B, H, T, **f)
    check(lib().pgb_delta_inv_bwd(ptr(k), dtype_code(k), ptr(la), ptr(be), ptr(X), ptr(dX), ptr(dk), ptr(dla), ptr(dbe), B, H, T, D,
                                  stream_of(k)), "pgb_delta_inv_bwd")
    return dk, dla, dbe


@on_device_of
def delta_loop_bwd(k, v, la, be, X, sent, dW, dsent, dsfin, want_ds0: bool = True):
    """Gradients of delta_loop_fwd (the reference's _delta_loop_bwd): (dk, dv (B,H,T,D), dla, dbeta (B,H,T),
    dX (B,H,NC,64,64), dS0 (B,H,D,D) or None), fp32. dW / dsent / dsfin may be None (no gradient arrived)."""
    need_cuda(k, v, la, be, X, sent)
    B, H, T, D = k.shape
    NC = X.shape[2]
    k = _io(k).contiguous()
    v = v.to(k.dtype).contiguous()
    la, be = _f32c(la), _f32c(be)
    X, sent = X.to(torch.bfloat16).contiguous(), sent.to(torch.bfloat16).contiguous()
    dW, dsent, dsfin = (None if t is None else _f32c(t) for t in (dW, dsent, dsfin))
    Pn = D // 64
    f = dict(device=k.device, dtype=torch.float32)
    dkp, dv = torch.empty(Pn, B, H, T, D, **f), torch.empty(B, H, T, D, **f)
    dlap, dbep = torch.empty(Pn, B, H, T, **f), torch.empty(Pn, B, H, T, **f)
    dXp = torch.empty(Pn, B, H, NC, CHUNK, CHUNK, **f)
    ds0 = torch.empty(B, H, D, D, **f) if want_ds0 else None
    check(lib().pgb_delta_loop_bwd(ptr(k), ptr(v), dtype_code(k), ptr(la), ptr(be), ptr(X), ptr(sent), ptr(dW), ptr(dsent), ptr(dsfin),
                                   ptr(dkp), ptr(dv), ptr(dlap), ptr(dbep), ptr(dXp), ptr(ds0), B, H, T, D, stream_of(k)),
          "pgb_delta_loop_bwd")
    return dkp.sum(0), dv, dlap.sum(0), dbep.sum(0), dXp.sum(0), ds0


# ---------------------------------------------------------------------------------------------------------- layer options
@on_device_of
def key_topk_mask_(kp, topk: int):
    """In place: keep the topk largest-magnitude coordinates of every key row of kp (B,T,H,D) (a view is fine), zero the rest."""
    need_cuda(kp)
    B, T, H, D = kp.shape
    if kp.stride(3) != 1 or kp.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("key_topk_mask_: fp32 or bf16 with unit stride over D")
    check(lib().pgb_key_topk_mask(ptr(kp), dtype_code(kp), kp.stride(0), kp.stride(1), kp.stride(2), B, T, H, D, int(topk),
                                  stream_of(kp)), "pgb_key_topk_mask")
    return kp


@on_device_of
def short_conv(x, w, cache=None):
    """Depthwise causal convolution over the last K tokens: x (B,T,C) (a view with unit stride over C), w (C,K), cache
    (B,C,K-1) = the previous call's last K-1 inputs or None.  Returns (y (B,T,C) contiguous, new cache (B,C,K-1))."""
    need_cuda(x, w)
    B, T, C = x.shape
    K = w.shape[1]
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.float()
    if x.stride(2) != 1:
        x = x.contiguous()
    w = w.to(x.dtype).contiguous()
    cache = None if cache is None else cache.to(x.dtype).contiguous()
    y = torch.empty(B, T, C, device=x.device, dtype=x.dtype)
    new = torch.empty(B, C, K - 1, device=x.device, dtype=x.dtype)
    check(lib().pgb_short_conv_fwd(ptr(x), dtype_code(x), x.stride(0) if B > 1 else T * x.stride(1), x.stride(1), ptr(w), ptr(cache),
                                   ptr(y), ptr(new), B, T, C, K, stream_of(x)), "pgb_short_conv_fwd")
    return y, new


from . import custom_ops  # noqa: E402,F401  (registers the pragnosia_b200:: operators the wrappers hand over to under torch.compile)
