"""Tensor-level wrappers of the C ABI: shape checks, output allocation (by torch), one library call each.

All functions take CUDA tensors, launch on torch's current stream and never synchronise, so they can be captured in a
CUDA graph. They raise on CPU tensors: there is no fallback path.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import check, dtype_code, lib, need_cuda, ptr, stream_of

CHUNK = 64


def _f32c(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.to(torch.float32).contiguous()


def _state_out(S_out, B, H, D, device):
    """The tensor the final state is written to: a new one, or the caller's (which may be the S0 it passed: every
    (sequence, head) reads its entering state before it writes its final one)."""
    if S_out is None:
        return torch.empty(B, H, D, D, device=device, dtype=torch.float32)
    if S_out.dtype != torch.float32 or not S_out.is_contiguous() or tuple(S_out.shape) != (B, H, D, D):
        raise ValueError("S_out must be a contiguous fp32 (B,H,D,D) tensor")
    return S_out


# ----------------------------------------------------------------------------------------------------------
def lambda_scan(u: torch.Tensor, logmag: torch.Tensor, ang: torch.Tensor, h0=None, time_segments: int = 0):
    """h_t = lambda_t h_{t-1} + u_t with lambda_t = exp(logmag_t + i ang_t); returns (Re h (B,T,D) fp32,
    (Re h_T, Im h_T)).  `ang` may be an expanded view with zero batch/time strides (one angle per channel): it is
    read as such, not materialised."""
    need_cuda(u, logmag, ang)
    B, T, D = u.shape
    u32, lm32 = _f32c(u), _f32c(logmag)
    a32 = ang if ang.dtype == torch.float32 else ang.to(torch.float32)
    if a32.dim() == 1:
        a32 = a32.expand(B, T, D)
    if tuple(a32.shape) != (B, T, D) or tuple(lm32.shape) != (B, T, D):
        raise ValueError("lambda_scan: u, logmag, ang must share the shape (B,T,D)")
    if D > 1 and a32.stride(2) != 1:
        a32 = a32.contiguous()
    sb, st = (a32.stride(0) if B > 1 else 0), (a32.stride(1) if T > 1 else 0)
    if not (sb == 0 and st == 0) and not (st == D and sb == T * D):
        a32 = a32.contiguous(); sb, st = T * D, D
    h0r = h0i = None
    if h0 is not None:
        h0r, h0i = _f32c(h0[0]), _f32c(h0[1])
        need_cuda(h0r, h0i)
    y = torch.empty(B, T, D, device=u.device, dtype=torch.float32)
    hr = torch.empty(B, D, device=u.device, dtype=torch.float32)
    hi = torch.empty_like(hr)
    check(lib().pgb_lambda_scan_fwd_ex(ptr(u32), ptr(lm32), ptr(a32), sb, st, ptr(h0r), ptr(h0i), ptr(y), ptr(hr), ptr(hi),
                                       B, T, D, time_segments, stream_of(u)), "pgb_lambda_scan_fwd")
    return y, (hr, hi)


# ----------------------------------------------------------------------------------------------------------
def prep(qp, kp, vp, gate_logits, theta, pos, out_dtype=torch.bfloat16):
    """Normalise / gate / rotate / cast / transpose: (B,T,H,D) projections -> (B,H,T,D) scan operands."""
    need_cuda(qp, kp, vp, theta, pos)
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
    gsb = gst = 0
    if gate_logits is not None:
        gate_logits = gate_logits.to(qp.dtype)
        if gate_logits.stride(2) != 1:
            gate_logits = gate_logits.contiguous()
        gsb, gst = gate_logits.stride(0), gate_logits.stride(1)
    theta = _f32c(theta)
    pos = pos.to(torch.int64).contiguous()
    q = torch.empty(B, H, T, D, device=qp.device, dtype=out_dtype)
    k, v = torch.empty_like(q), torch.empty_like(q)
    check(lib().pgb_aspin_prep_fwd(ptr(qp), ptr(kp), ptr(vp), dtype_code(qp), qp.stride(0), qp.stride(1), qp.stride(2),
                                   ptr(gate_logits), gsb, gst, ptr(theta), ptr(pos), ptr(q), ptr(k), ptr(v), dtype_code(q),
                                   B, T, H, D, stream_of(qp)), "pgb_aspin_prep_fwd")
    return q, k, v


# ----------------------------------------------------------------------------------------------------------
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
    shift_dev, shift_host = None, 0.0
    if theta is not None and S0 is not None:
        theta = _f32c(theta)
        if torch.is_tensor(shift):
            shift_dev = shift.to(torch.float32).reshape(())
            need_cuda(shift_dev)
        else:
            shift_host = float(shift)
            if shift_host == 0.0:
                theta = None
    else:
        theta = None
    o = torch.empty(B, H, T, D, device=q.device, dtype=out_dtype or q.dtype)
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
    shift_dev, shift_host = None, 0.0
    if theta is not None and S0 is not None:
        theta = _f32c(theta)
        if torch.is_tensor(shift):
            shift_dev = shift.to(torch.float32).reshape(())
        else:
            shift_host = float(shift)
            if shift_host == 0.0:
                theta = None
    else:
        theta = None
    o = torch.empty(B, T, H * D, device=q.device, dtype=out_dtype or q.dtype)
    S = _state_out(S_out, B, H, D, q.device)
    NC = (T + CHUNK - 1) // CHUNK
    sent = torch.empty(B, H, NC, D, D, device=q.device, dtype=torch.bfloat16) if want_sent else None
    check(lib().pgb_aspin_prefill_fused_fwd(
        ptr(q), ptr(k), ptr(v), ptr(decay_logits), decay_logits.stride(0), decay_logits.stride(1), ptr(_f32c(decay_A)),
        ptr(S0), ptr(theta), ptr(shift_dev), shift_host, ptr(_f32c(rms_weight)), float(rms_eps), ptr(o), dtype_code(o),
        ptr(S), ptr(sent), B, H, T, D, stream_of(q)), "pgb_aspin_prefill_fused_fwd")
    return o, S, sent


# ----------------------------------------------------------------------------------------------------------
def rot_table(theta, T: int):
    """(H, T, D/2, 2) fp32 table of (cos, sin)(t * theta[h, i]) for positions 0..T-1."""
    need_cuda(theta)
    theta = _f32c(theta)
    H, half = theta.shape
    table = torch.empty(H, T, half, 2, device=theta.device, dtype=torch.float32)
    check(lib().pgb_rot_table_build(ptr(theta), ptr(table), H, T, 2 * half, stream_of(theta)), "pgb_rot_table_build")
    return table


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
    shift_dev, shift_host = None, 0.0
    if theta is not None and S0 is not None:
        theta = _f32c(theta)
        if torch.is_tensor(shift):
            shift_dev = shift.to(torch.float32).reshape(())
        else:
            shift_host = float(shift)
            if shift_host == 0.0:
                theta = None
    else:
        theta = None
    o = torch.empty(B, T, H * D, device=qp.device, dtype=out_dtype or qp.dtype)
    S = _state_out(S_out, B, H, D, qp.device)
    NC = (T + CHUNK - 1) // CHUNK
    sent = torch.empty(B, H, NC, D, D, device=qp.device, dtype=torch.bfloat16) if want_sent else None
    sbq = qp.stride(0) if B > 1 else T * qp.stride(1)
    sba = decay_logits.stride(0) if B > 1 else T * decay_logits.stride(1)
    check(lib().pgb_aspin_layer_prefill_fwd(
        ptr(qp), ptr(kp), ptr(vp), sbq, qp.stride(1), ptr(gate_logits), ptr(decay_logits), sba, decay_logits.stride(1),
        ptr(_f32c(decay_A)), ptr(table), table.shape[1], ptr(S0), ptr(theta), ptr(shift_dev), shift_host,
        ptr(_f32c(rms_weight)), float(rms_eps), ptr(o), dtype_code(o), ptr(S), ptr(sent), B, H, T, D, stream_of(qp)),
        "pgb_aspin_layer_prefill_fwd")
    return o, S, sent


# ----------------------------------------------------------------------------------------------------------
def rotate(x, theta, pos):
    """Rotate channel pairs of x (B,H,T,D) by pos[t]*theta[h,i]."""
    need_cuda(x, theta, pos)
    B, H, T, D = x.shape
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.float()
    x = x.contiguous()
    out = torch.empty_like(x)
    check(lib().pgb_rotate_pairs(ptr(x), dtype_code(x), ptr(_f32c(theta)), ptr(_f32c(pos)), ptr(out), B, H, T, D,
                                 stream_of(x)), "pgb_rotate_pairs")
    return out


# ----------------------------------------------------------------------------------------------------------
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
    S_out = torch.empty_like(S) if S_out is None else S_out
    out_dtype = out_dtype or qp.dtype
    if out is None:
        out = torch.empty(B, H, D, device=qp.device, dtype=out_dtype)
    shift_dev, shift_host = (shift.to(torch.float32), 0.0) if torch.is_tensor(shift) else (None, float(shift))
    sb = lambda t: t.stride(0) if B > 1 else max(t.stride(0), H * (t.shape[2] if t.dim() == 3 else 1))
    check(lib().pgb_aspin_decode_step(
        ptr(qp), ptr(kp), ptr(vp), dtype_code(qp), sb(qp), int(normalize), ptr(gate), 0 if gate is None else gate.stride(0),
        int(gate_is_logit), int(delta), ptr(decay), decay.stride(0), ptr(_f32c(decay_A)), ptr(_f32c(theta)),
        ptr(shift_dev), shift_host, ptr(S), ptr(S_out), ptr(_f32c(rms_weight)), float(rms_eps), ptr(out), dtype_code(out),
        sb(out), B, H, D, stream_of(qp)), "pgb_aspin_decode_step")
    return out, S_out


# ----------------------------------------------------------------------------------------------------------
def add_norm(x, delta, norm: torch.nn.Module):
    """y = x + delta (delta may be None); z = norm(y) with norm an nn.RMSNorm or nn.LayerNorm over the last dim.
    Returns (y, z); y is x itself when delta is None."""
    need_cuda(x)
    d = x.shape[-1]
    x = x.contiguous()
    if delta is not None:
        delta = delta.to(x.dtype).contiguous()
    rms = isinstance(norm, torch.nn.RMSNorm)
    w = norm.weight.to(x.dtype)
    b = None if rms else norm.bias.to(x.dtype)
    # nn.RMSNorm(eps=None) means the epsilon of the arithmetic type, which is fp32 for every dtype these kernels take
    eps = (norm.eps if norm.eps is not None else torch.finfo(torch.float32).eps) if rms else norm.eps
    y = torch.empty_like(x) if delta is not None else None
    z = torch.empty_like(x)
    check(lib().pgb_add_norm(ptr(x), ptr(delta), ptr(w), ptr(b), float(eps), 0 if rms else 1, ptr(y), ptr(z),
                             x.numel() // d, d, dtype_code(x), stream_of(x)), "pgb_add_norm")
    return (x if delta is None else y), z


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
    x, W = x.contiguous(), W.contiguous()
    if delta is not None:
        delta = delta.to(x.dtype).contiguous()
    kind, nw, nb, eps = 0, None, None, 0.0
    if norm is not None:
        rms = isinstance(norm, torch.nn.RMSNorm)
        kind = 1 if rms else 2
        nw = norm.weight.to(x.dtype).contiguous()
        nb = None if rms else norm.bias.to(x.dtype).contiguous()
        eps = (norm.eps if norm.eps is not None else torch.finfo(torch.float32).eps) if rms else norm.eps
    if bias is not None:
        bias = bias.to(x.dtype).contiguous()
    y = torch.empty(B, N, device=x.device, dtype=x.dtype)
    s = torch.empty_like(x) if (want_sum and delta is not None) else None
    check(lib().pgb_skinny_linear(ptr(x), ptr(delta), ptr(nw), ptr(nb), kind, float(eps), ptr(W), ptr(bias),
                                  1 if act == "gelu" else 0, ptr(y), ptr(s), B, K, N, stream_of(x)), "pgb_skinny_linear")
    if want_sum:
        return y, (x if delta is None else s)
    return y


def decode_embed(tok, pos, E, P):
    """x (B,d) = E[tok] + P[pos] in one launch; tok (B,) / (B,1) int64 and pos (1,) int64 on the device, bf16 tables."""
    need_cuda(tok, pos, E, P)
    if E.dtype != torch.bfloat16 or P.dtype != torch.bfloat16 or tok.dtype != torch.long or pos.dtype != torch.long:
        raise ValueError("decode_embed: bf16 tables, int64 ids")
    B, d = tok.numel(), E.shape[1]
    x = torch.empty(B, d, device=E.device, dtype=E.dtype)
    check(lib().pgb_decode_embed(ptr(tok.contiguous()), ptr(pos), ptr(E.contiguous()), ptr(P.contiguous()), ptr(x), B, d,
                                 E.shape[0], P.shape[0], stream_of(E)), "pgb_decode_embed")
    return x


def decode_sample(logits, temp, seed, tok, count, ticket, hist=None, pos=None, shift=None, ctx: int = 1):
    """Draw one id per row of logits (B,V) into tok (B,) / (B,1) int64, record it in hist[:, count] and advance the step
    counters (count, pos modulo ctx, shift) -- all on the device, one launch. ticket: a zeroed uint32/int32 scalar."""
    need_cuda(logits, tok, count, ticket)
    B, V = logits.shape
    if logits.dtype not in (torch.float32, torch.bfloat16):
        logits = logits.float()
    logits = logits.contiguous()
    cols = 0 if hist is None else hist.shape[1]
    check(lib().pgb_decode_sample(ptr(logits), dtype_code(logits), float(temp), int(seed) & 0xFFFFFFFFFFFFFFFF, ptr(tok), ptr(hist),
                                  cols, ptr(count), ptr(pos), ptr(shift), ptr(ticket), B, V, int(ctx), stream_of(logits)),
          "pgb_decode_sample")
    return tok


def linear_act(x, W, bias=None, act: Optional[str] = "gelu"):
    """act(x W^T + bias) as one tensor-core GEMM with the bias and the (erf) GELU in its epilogue; x (..., K) bf16, W (N, K)."""
    need_cuda(x, W)
    if x.dtype != torch.bfloat16 or W.dtype != torch.bfloat16:
        raise ValueError("linear_act: bf16 only")
    K, N = x.shape[-1], W.shape[0]
    x2 = x.reshape(-1, K).contiguous()
    y = torch.empty(x2.shape[0], N, device=x.device, dtype=x.dtype)
    b = None if bias is None else bias.to(x.dtype).contiguous()
    check(lib().pgb_linear_act(ptr(x2), ptr(W.contiguous()), ptr(b), ptr(y), x2.shape[0], N, K, 1 if act == "gelu" else 0,
                               stream_of(x)), "pgb_linear_act")
    return y.view(*x.shape[:-1], N)
