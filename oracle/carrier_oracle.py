"""CPU restatement of the reference's carrier arithmetic. TEST INFRASTRUCTURE: see oracle/__init__.py.

Everything is plain PyTorch on CPU tensors, fp32 unless the inputs are fp64 (the reference's own rule,
src/assoc.py:260, src/spin.py:196). Each function cites the reference lines it restates. Parameters of the
layer / model functions are passed as a flat dict of tensors that uses the reference's state_dict names
("mix.0.q.weight", "mlp.3.a.bias", ...), so a reference checkpoint and a random-init dict are interchangeable.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

__all__ = [
    "rotate", "plain_literal", "delta_literal", "unit_lower_inverse", "assoc_scan", "lambda_literal",
    "lambda_scan", "decode_step", "assoc_layer", "fspin_layer", "mlp_block", "lm_layers", "lm_forward_carried",
    "lm_prefill", "lm_decode_step", "init_lm_params", "init_assoc_params", "init_fspin_params", "lm_config",
    "rel_err", "decode_rebase", "short_conv", "lambda_scan_grads", "prep_ref", "rounding",
]


def _work_dtype(t: torch.Tensor) -> torch.dtype:
    return torch.float64 if t.dtype == torch.float64 else torch.float32


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max|a-b| / max|b|: the reference's own agreement metric (tests/test_assoc.py:179)."""
    return ((a.double() - b.double()).abs().max() / (b.double().abs().max() + 1e-30)).item()


# ----------------------------------------------------------------------------------------------------------
# rotation of channel pairs (src/assoc.py:34-39)
# ----------------------------------------------------------------------------------------------------------
def rotate(x: torch.Tensor, theta: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """Rotate each channel pair (2i, 2i+1) of x (B,H,T,dk) by the angle pos[t] * theta[h,i]."""
    H, half = theta.shape
    ang = pos.to(theta.dtype).reshape(1, 1, -1, 1) * theta.reshape(1, H, 1, half)
    co, si = ang.cos(), ang.sin()
    ev, od = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x) if x.dtype == co.dtype else torch.empty(x.shape, dtype=torch.result_type(x, co))
    out[..., 0::2] = ev * co - od * si
    out[..., 1::2] = ev * si + od * co
    return out


# ----------------------------------------------------------------------------------------------------------
# the literal per-token recurrences: ground truth
# ----------------------------------------------------------------------------------------------------------
def plain_literal(q, k, v, la, S0=None):
    """S_t = exp(la_t) S_{t-1} + k_t v_t^T ; o_t = q_t S_t   (tests/test_assoc.py:22-27)."""
    B, H, T, D = q.shape
    S = torch.zeros(B, H, D, v.shape[-1], dtype=q.dtype) if S0 is None else S0.clone()
    outs = []
    for t in range(T):
        S = la[:, :, t].exp()[..., None, None] * S + k[:, :, t, :, None] * v[:, :, t, None, :]
        outs.append(torch.einsum("bhd,bhde->bhe", q[:, :, t], S))
    return torch.stack(outs, 2), S


def delta_literal(q, k, v, la, beta, S0=None):
    """Delta write rule, token by token: Sd = a_t S ; r = b_t (v_t - Sd^T k_t) ; S = Sd + k_t r^T ; o_t = S^T q_t.
    This is the recurrence src/assoc.py:207-215 states and its chunked form solves exactly."""
    B, H, T, D = q.shape
    S = torch.zeros(B, H, D, v.shape[-1], dtype=q.dtype) if S0 is None else S0.clone()
    outs = []
    for t in range(T):
        Sd = la[:, :, t].exp()[..., None, None] * S
        r = beta[:, :, t, None] * (v[:, :, t] - torch.einsum("bhde,bhd->bhe", Sd, k[:, :, t]))
        S = Sd + k[:, :, t, :, None] * r[:, :, None, :]
        outs.append(torch.einsum("bhd,bhde->bhe", q[:, :, t], S))
    return torch.stack(outs, 2), S


# ----------------------------------------------------------------------------------------------------------
# chunked two-pass scan (src/assoc.py:118-165 plain, :168-251 delta, :254-269 dispatcher)
# ----------------------------------------------------------------------------------------------------------
def unit_lower_inverse(N: torch.Tensor, block: int = 16) -> torch.Tensor:
    """(I + N)^-1 for strictly lower triangular N (..., C, C): diagonal blocks by Neumann doubling (exact, they
    are nilpotent), block rows by forward substitution (src/assoc.py:168-204)."""
    C = N.shape[-1]
    b = block if C % block == 0 else C
    nb = C // b
    eye_b = torch.eye(b, dtype=N.dtype)
    eye_c = torch.eye(C, dtype=N.dtype).expand(*N.shape[:-2], C, C)
    done = []
    for i in range(nb):
        r0, r1 = i * b, (i + 1) * b
        R = -N[..., r0:r1, r0:r1]
        Xi = eye_b.expand_as(R)
        span = 1
        while span < b:
            Xi = Xi + R @ Xi
            R = R @ R
            span *= 2
        rhs = eye_c[..., r0:r1, :]
        if i:
            rhs = rhs - N[..., r0:r1, :r0] @ torch.cat(done, dim=-2)
        done.append(Xi @ rhs)
    return torch.cat(done, dim=-2)


def _chunk_views(q, k, v, la, beta, chunk):
    B, H, T, D = q.shape
    C = min(chunk, T)
    pad = (-T) % C
    if pad:
        # zero tokens with log-decay 0 (alpha = 1) and beta = 0: they neither write nor decay
        q, k, v = (F.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
        la = F.pad(la, (0, pad))
        beta = None if beta is None else F.pad(beta, (0, pad))
    NC = q.shape[2] // C
    qc, kc, vc = (t.reshape(B, H, NC, C, t.shape[-1]) for t in (q, k, v))
    lc = la.reshape(B, H, NC, C)
    bc = None if beta is None else beta.reshape(B, H, NC, C)
    return qc, kc, vc, lc, bc, C, NC


def assoc_scan(q, k, v, logalpha, S0=None, chunk: int = 64, beta=None):
    """Chunked scan, plain rule (beta None) or delta rule. q,k,v (B,H,T,D); logalpha, beta (B,H,T); S0 (B,H,D,D).
    Returns (o in q's dtype, final state in fp32/fp64)."""
    B, H, T, D = q.shape
    wd = _work_dtype(q)
    out_dtype = q.dtype
    q, k, v, la = q.to(wd), k.to(wd), v.to(wd), logalpha.to(wd)
    beta = None if beta is None else beta.to(wd)
    S = torch.zeros(B, H, D, D, dtype=wd) if S0 is None else S0.to(wd)
    qc, kc, vc, lc, bc, C, NC = _chunk_views(q, k, v, la, beta, chunk)
    L = lc.cumsum(-1)                                                  # (B,H,NC,C): within-chunk cumulative log-decay
    causal = torch.ones(C, C, dtype=torch.bool).tril()
    dec = (L[..., :, None] - L[..., None, :]).clamp(max=0.0).exp() * causal   # exp(L_t - L_s), s <= t
    from_start = L.exp()[..., None]                                    # exp(L_t)
    to_end = (L[..., -1:] - L).clamp(max=0.0).exp()[..., None]         # exp(L_C - L_s)
    total = L[..., -1].exp()                                           # exp(L_C) per chunk
    kw_t = (kc * to_end).transpose(-1, -2)                             # (B,H,NC,D,C)
    entering = []
    if beta is None:
        A = (qc @ kc.transpose(-1, -2)) * dec
        intra = A @ vc
        KV = kw_t @ vc
        for c in range(NC):
            entering.append(S)
            S = total[:, :, c, None, None] * S + KV[:, :, c]
        Sent = torch.stack(entering, 2)
        o = intra + (qc * from_start) @ Sent
    else:
        KK = (kc @ kc.transpose(-1, -2)) * dec
        X = unit_lower_inverse(bc[..., None] * KK.tril(-1))
        A = (qc @ kc.transpose(-1, -2)) * dec
        written = []
        for c in range(NC):
            entering.append(S)
            rhs = bc[:, :, c, :, None] * (vc[:, :, c] - from_start[:, :, c] * (kc[:, :, c] @ S))
            Wc = X[:, :, c] @ rhs
            written.append(Wc)
            S = total[:, :, c, None, None] * S + kw_t[:, :, c] @ Wc
        Sent = torch.stack(entering, 2)
        W = torch.stack(written, 2)
        o = A @ W + (qc * from_start) @ Sent
    o = o.reshape(B, H, NC * C, D)[:, :, :T]
    return o.to(out_dtype), S


# ----------------------------------------------------------------------------------------------------------
# per-token complex recurrence h_t = lambda_t h_{t-1} + u_t   (src/scan_kernel.py:42-48, src/spin.py:182-215)
# ----------------------------------------------------------------------------------------------------------
def lambda_literal(u, logmag, ang, h0=None):
    """The definition, in the operation order of src/scan_kernel.py:42-48 / tests/test_spin.py:194-200."""
    Bn, T, D = u.shape
    hr = torch.zeros(Bn, D, dtype=u.dtype) if h0 is None else h0[0].clone()
    hi = torch.zeros(Bn, D, dtype=u.dtype) if h0 is None else h0[1].clone()
    ys = []
    for t in range(T):
        mag = logmag[:, t].exp()
        c, s = mag * ang[:, t].cos(), mag * ang[:, t].sin()
        hr, hi = c * hr - s * hi + u[:, t], s * hr + c * hi
        ys.append(hr)
    return torch.stack(ys, 1), (hr, hi)


def lambda_scan(u, logmag, ang, h0=None, chunk: int = 16):
    """Chunked closed form of the same recurrence (src/spin.py:182-215): inside a chunk
    h_t = sum_{s<=t} exp(L_t - L_s) u_s + exp(L_t) h_prev with L the complex cumulative log-lambda; only Re h is
    emitted, Im h is formed at each chunk's last position to carry."""
    Bn, T, D = u.shape
    wd = _work_dtype(u)
    out_dtype = u.dtype
    u, logmag, ang = u.to(wd), logmag.to(wd), ang.to(wd)
    hr = torch.zeros(Bn, D, dtype=wd) if h0 is None else h0[0].to(wd)
    hi = torch.zeros(Bn, D, dtype=wd) if h0 is None else h0[1].to(wd)
    pieces = []
    for t0 in range(0, T, chunk):
        uc, lr, li = u[:, t0:t0 + chunk], logmag[:, t0:t0 + chunk].cumsum(1), ang[:, t0:t0 + chunk].cumsum(1)
        C = uc.shape[1]
        causal = torch.ones(C, C, dtype=torch.bool).tril().reshape(1, C, C, 1)
        dmag = (lr[:, :, None] - lr[:, None, :]).clamp(max=0.0).exp() * causal        # (B,t,s,D)
        dphi = li[:, :, None] - li[:, None, :]
        re = (dmag * dphi.cos() * uc[:, None]).sum(2)
        grow = lr.exp()
        re = re + grow * (li.cos() * hr[:, None] - li.sin() * hi[:, None])
        im_last = (dmag[:, -1] * dphi[:, -1].sin() * uc).sum(1) \
            + grow[:, -1] * (li[:, -1].sin() * hr + li[:, -1].cos() * hi)
        hr, hi = re[:, -1], im_last
        pieces.append(re)
    return torch.cat(pieces, 1).to(out_dtype), (hr.to(out_dtype), hi.to(out_dtype))


def lambda_scan_grads(u, logmag, ang, h0, w_y, w_r, w_i):
    """Gradients of  (Re h * w_y).sum() + (Re h_T * w_r).sum() + (Im h_T * w_i).sum()  with respect to u, logmag, ang and
    the entering state, by autograd through the literal recurrence in fp64 (the check of tests/test_spin.py:237-246)."""
    with torch.enable_grad():
        a = [t.detach().double().requires_grad_(True) for t in (u, logmag, ang, h0[0], h0[1])]
        y, (hr, hi) = lambda_literal(a[0], a[1], a[2], (a[3], a[4]))
        loss = (y * w_y.double()).sum() + (hr * w_r.double()).sum() + (hi * w_i.double()).sum()
        return torch.autograd.grad(loss, a)


def prep_ref(qp, kp, vp, gl, theta, pos):
    """The plumbing before the scan in plain torch (tests/test_assoc.py:189-193): normalise q, k, v per head, scale k by
    the write gate, rotate q and k; (B,T,H,D) in, fp32 (B,H,T,D) out. Differentiable by autograd."""
    q_, k_, v_ = [F.normalize(t.transpose(1, 2).float(), dim=-1) for t in (qp, kp, vp)]
    if gl is not None:
        k_ = k_ * torch.sigmoid(gl.float()).transpose(1, 2).unsqueeze(-1)
    return rotate(q_, theta, pos), rotate(k_, theta, pos), v_


# ----------------------------------------------------------------------------------------------------------
# one recurrent decode step on already prepared vectors
# ----------------------------------------------------------------------------------------------------------
def decode_step(S, shift, q, k, v, la, theta, beta=None):
    """What AssocCarrier.forward does for T=1 with a carried state (src/assoc.py:399-405, 502 with chunk 1):
    the state's key axis is rotated back by `shift` positions (the rebase), then with the token at position 0
    (no rotation of q, k): S' = a S + k v^T (plain) or Sd = a S, r = b (v - Sd^T k), S' = Sd + k r^T (delta);
    o = S'^T q.  S (B,H,dk,dv) fp32; q,k,v (B,H,D); la, beta (B,H); theta (H,D/2); shift a number."""
    B, H, Dk, Dv = S.shape
    if shift != 0:
        pos = torch.full((Dv,), -float(shift), dtype=theta.dtype)
        S = rotate(S.transpose(2, 3), theta, pos).transpose(2, 3)
    a = la.exp()[..., None, None]
    Sd = a * S
    if beta is None:
        S1 = Sd + k[..., :, None] * v[..., None, :]
    else:
        r = beta[..., None] * (v - torch.einsum("bhde,bhd->bhe", Sd, k))
        S1 = Sd + k[..., :, None] * r[..., None, :]
    o = torch.einsum("bhd,bhde->bhe", q, S1)
    return o, S1


# ----------------------------------------------------------------------------------------------------------
# layers and the language model (functional, reference state_dict names)
# ----------------------------------------------------------------------------------------------------------
# Where a bf16 run of the model rounds. The reference under autocast, and the product with bf16 weights, keep activations in
# bf16: every linear layer, norm, activation and residual add hands on a value rounded to 8 bits of mantissa, while the
# scan's state and accumulations stay fp32. With `rounding(torch.bfloat16)` active the functions below round at exactly
# those hand-overs (and nowhere else), so a bf16 product run can be held to a tolerance that reflects its kernels rather
# than the accumulated rounding of twelve layers. Off by default: the oracle is then the plain fp32 / fp64 arithmetic.
_ROUND = [None]


class rounding:
    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        self.prev, _ROUND[0] = _ROUND[0], self.dtype

    def __exit__(self, *a):
        _ROUND[0] = self.prev


def _r(x):
    return x if _ROUND[0] is None else x.to(_ROUND[0]).to(x.dtype)


def _norm(P, name, x, kind):
    w = P[name + ".weight"]
    if kind == "rms":
        eps = torch.finfo(x.dtype).eps                                  # nn.RMSNorm(eps=None)
        return _r(x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w)
    return _r(F.layer_norm(x, (x.shape[-1],), w, P[name + ".bias"], 1e-5))


def _lin(P, name, x):
    return _r(F.linear(x, P[name + ".weight"], P.get(name + ".bias")))


def short_conv(P, pre, qo, ko, vo, cc):
    """The depthwise causal convolution over the last K tokens on q, k, v (B,T,d each) with the previous call's last K-1
    inputs as left context (src/assoc.py:375-382 _sconv). Returns q, k, v and the new context (B,3d,K-1)."""
    w = P[pre + "sconv"]
    d, K = qo.shape[-1], w.shape[1]
    x = torch.cat([qo, ko, vo], dim=-1).transpose(1, 2)                          # (B,3d,T)
    pad = cc.to(x.dtype) if cc is not None else x.new_zeros(x.shape[0], 3 * d, K - 1)
    xp = torch.cat([pad, x], dim=-1)
    y = _r(F.conv1d(xp, w.to(x.dtype).unsqueeze(1), groups=3 * d)).transpose(1, 2)
    return y[..., :d], y[..., d:2 * d], y[..., 2 * d:], xp[..., -(K - 1):]


def assoc_layer(P, pre, x, h0=None, *, heads: int, delta: bool = False, chunk: int = 64, norm: str = "ln", key_topk: int = 0,
                hl_floor: bool = False, write_all: bool = False, pos_wrap=None, beta_scale=None):
    """AssocCarrier.forward on its PyTorch path (src/assoc.py:384-512 with kernel off).  x (B,T,d); h0 = (S, p0[, conv
    cache]) or None.  Options as the reference's: key_topk (:435-439), hl_floor (:339-343, :357), write_all (:463, :472-478),
    pos_wrap (:406-410), beta_scale (:468-471); a short convolution is on when P holds pre + "sconv" (:361-382).
    Returns (out, (S, T[, conv cache]))."""
    B, T, d = x.shape
    dk = d // heads
    theta = P[pre + "theta"]
    z = _norm(P, pre + "ln", x, norm)
    S0, cc = None, None
    if h0 is not None:
        S0, p0 = h0[0], h0[1]
        cc = h0[2] if len(h0) == 3 else None
        if not (isinstance(p0, int) and p0 == 0):
            S0 = decode_rebase(S0, theta.float(), float(p0))
    pos = torch.arange(T)
    if pos_wrap:
        pos = pos % pos_wrap
    qo, ko, vo = (_lin(P, pre + n, z) for n in ("q", "k", "v"))
    sc = (pre + "sconv") in P
    if sc:
        qo, ko, vo, cc = short_conv(P, pre, qo, ko, vo, cc)
    split = lambda t: t.reshape(B, T, heads, dk).transpose(1, 2)
    kp = ko.reshape(B, T, heads, dk)
    if key_topk:
        m = torch.zeros_like(kp).scatter_(-1, kp.abs().topk(key_topk, dim=-1).indices, 1.0)
        kp = kp * m
    q, k, v = (F.normalize(t, dim=-1) for t in (split(qo), kp.transpose(1, 2), split(vo)))
    if not delta and not write_all:
        k = k * torch.sigmoid(_lin(P, pre + "wi", z)).transpose(1, 2).unsqueeze(-1)
    q, k, v = _r(rotate(q, theta, pos)), _r(rotate(k, theta, pos)), _r(v)      # the scan's operands (bf16 in a bf16 run)
    la = -F.softplus(_lin(P, pre + "wa", z)) * P[pre + "A"].exp()
    if hl_floor:
        hl = torch.logspace(math.log10(8.0), math.log10(131072.0), heads)
        la = la.clamp(min=(-math.log(2.0) / hl).to(la.dtype))
    la = la.transpose(1, 2)
    bt = torch.sigmoid(_lin(P, pre + "wb", z)).transpose(1, 2) if delta else None
    if beta_scale is not None and bt is not None:
        bt = bt * beta_scale.to(bt.dtype)
    if delta and write_all:
        bt = bt.clamp(min=0.75)
    o, S = assoc_scan(q, k, v, la, S0, chunk=chunk, beta=bt)
    eps = torch.finfo(o.dtype).eps
    o = _r(o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * P[pre + "on.weight"])
    o = o.transpose(1, 2).reshape(B, T, d)
    out = _r(x + _r(F.linear(o, _r(P[pre + "o.weight"] * torch.sigmoid(P[pre + "gate"])))))
    return out, ((S, T, cc) if sc else (S, T))


def decode_rebase(S0, theta, shift: float):
    """Rotate the key axis of a carried state back by `shift` positions, in fp32 (src/assoc.py:399-402)."""
    pos = torch.full((S0.shape[3],), -shift, dtype=theta.dtype)
    return rotate(S0.transpose(2, 3), theta, pos).transpose(2, 3).contiguous()


def fspin_layer(P, pre, x, h0=None, *, norm: str = "ln", chunk: int = 16):
    """SpinCarrier.forward with gated="rf" (src/spin.py:229-254): per-token |lambda_t| from a recurrence gate,
    gamma_t applied outside the scan."""
    z = _norm(P, pre + "ln", x, norm)
    nu = 1e-3 + F.softplus(P[pre + "nu_raw"])                                   # src/spin.py:105
    ang = P[pre + "theta"]
    logmag = -8.0 * torch.sigmoid(_lin(P, pre + "Wr", z)) * nu                  # -log(mag) == nu
    gam = torch.sqrt((1.0 - torch.exp(2.0 * logmag)).clamp_min(1e-6))
    u = _lin(P, pre + "B", z) * gam * torch.sigmoid(_lin(P, pre + "Wi", z))
    y, h = lambda_scan(u, logmag, ang.expand_as(logmag), h0, chunk=chunk)
    return x + torch.sigmoid(P[pre + "gate"]) * _lin(P, pre + "C", y), h


def mlp_block(P, pre, x, norm: str = "ln"):
    """norm -> Linear(4d) -> GELU (erf) -> Linear(d), residual (src/model.py:552-560)."""
    return _r(x + _lin(P, pre + "b", _r(F.gelu(_lin(P, pre + "a", _norm(P, pre + "n", x, norm))))))


_MIXERS = {  # mixer name -> (family, delta, head_dim)   (src/model.py:631-699, the pure-carrier entries)
    "aspin": ("assoc", False, 64), "dspin": ("assoc", True, 64),
    "hspin": ("assoc", False, 128), "hdspin": ("assoc", True, 128),
    "fspin": ("spin", False, 0),
}


def lm_config(vocab=8192, d=768, layers=12, mlp_mult=4, ctx=512, mixer="aspin", norm="ln"):
    fam, delta, hd = _MIXERS[mixer]
    heads = max(1, d // hd) if fam == "assoc" else 0
    return dict(vocab=vocab, d=d, layers=layers, mlp_mult=mlp_mult, ctx=ctx, mixer=mixer, norm=norm,
                family=fam, delta=delta, heads=heads)


def init_assoc_params(P, pre, d, heads, delta, g, jitter=0.0, norm="ln", dtype=torch.float32):
    """Parameters of one associative carrier layer under prefix `pre` (shapes and init of src/assoc.py:319-348 after
    the model-wide N(0, 0.02) re-init of src/model.py:730-738). jitter > 0 perturbs the constants (biases, norm
    weights, timescales, frequencies, gate) so parity cases exercise them."""
    dk = d // heads
    nrm = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(dtype)
    jit = lambda t: (t + jitter * torch.randn(t.shape, generator=g)).to(dtype) if jitter else t.to(dtype)
    P[pre + "ln.weight"] = jit(torch.ones(d))
    if norm != "rms":
        P[pre + "ln.bias"] = jit(torch.zeros(d))
    for n in ("q", "k", "v", "o"):
        P[pre + n + ".weight"] = nrm(d, d) * (25.0 if jitter else 1.0)
    for n in ("wa", "wi") + (("wb",) if delta else ()):
        P[pre + n + ".weight"] = nrm(heads, d) * (25.0 if jitter else 1.0)
        P[pre + n + ".bias"] = jit(torch.zeros(heads))
    P[pre + "A"] = jit(torch.linspace(math.log(0.1 / 0.69), math.log(1e-4 / 0.69), heads))
    base = 10000.0 ** (-torch.arange(0, dk, 2).float() / dk)
    P[pre + "theta"] = jit(base.unsqueeze(0).repeat(heads, 1))
    P[pre + "on.weight"] = jit(torch.ones(dk))
    P[pre + "gate"] = jit(torch.zeros(()))
    return P


def init_fspin_params(P, pre, d, g, jitter=0.0, norm="ln", dtype=torch.float32):
    """Parameters of one forget-gated diagonal carrier layer (src/spin.py:59-100 with gated="rf")."""
    nrm = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(dtype)
    jit = lambda t: (t + jitter * torch.randn(t.shape, generator=g)).to(dtype) if jitter else t.to(dtype)
    P[pre + "ln.weight"] = jit(torch.ones(d))
    if norm != "rms":
        P[pre + "ln.bias"] = jit(torch.zeros(d))
    P[pre + "nu_raw"] = jit(torch.linspace(math.log(math.expm1(1e-3)), math.log(math.expm1(0.3)), d))
    P[pre + "theta"] = jit(torch.linspace(0.0, math.pi, d))
    for n in ("B", "C"):
        P[pre + n + ".weight"] = nrm(d, d) * (25.0 if jitter else 1.0)
    for n in ("Wi", "Wr"):
        P[pre + n + ".weight"] = nrm(d, d) * (25.0 if jitter else 1.0)
        P[pre + n + ".bias"] = jit(torch.zeros(d))
    P[pre + "gate"] = jit(torch.zeros(()))
    return P


def init_lm_params(cfg, seed: int = 0, dtype=torch.float32, jitter: float = 0.0):
    """Random-init parameters with the reference's shapes, names and init rule (src/model.py:730-738: every
    Embedding and Linear weight N(0, 0.02), biases 0). Not bit-identical to a reference-constructed model (different
    draw order): parity runs load the SAME dict into both sides."""
    g = torch.Generator().manual_seed(seed)
    d, L, V = cfg["d"], cfg["layers"], cfg["vocab"]
    nrm = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(dtype)
    jit = lambda t: (t + jitter * torch.randn(t.shape, generator=g)).to(dtype) if jitter else t.to(dtype)
    P = {"e.weight": nrm(V, d), "p.weight": nrm(cfg["ctx"], d), "n.weight": jit(torch.ones(d))}
    if cfg["norm"] != "rms":
        P["n.bias"] = jit(torch.zeros(d))
    for i in range(L):
        m = f"mix.{i}."
        if cfg["family"] == "assoc":
            init_assoc_params(P, m, d, cfg["heads"], cfg["delta"], g, jitter, cfg["norm"], dtype)
        else:
            init_fspin_params(P, m, d, g, jitter, cfg["norm"], dtype)
        f = f"mlp.{i}."
        P[f + "n.weight"] = jit(torch.ones(d))
        if cfg["norm"] != "rms":
            P[f + "n.bias"] = jit(torch.zeros(d))
        P[f + "a.weight"] = nrm(cfg["mlp_mult"] * d, d); P[f + "a.bias"] = jit(torch.zeros(cfg["mlp_mult"] * d))
        P[f + "b.weight"] = nrm(d, cfg["mlp_mult"] * d); P[f + "b.bias"] = jit(torch.zeros(d))
    return P


def lm_layers(P, cfg, h, states):
    """One pass of every (mixer, MLP) pair over h (B,T,d) with per-layer carried states (updated in the list)."""
    for i in range(cfg["layers"]):
        if cfg["family"] == "assoc":
            h, states[i] = assoc_layer(P, f"mix.{i}.", h, states[i], heads=cfg["heads"], delta=cfg["delta"],
                                       norm=cfg["norm"])
        else:
            h, states[i] = fspin_layer(P, f"mix.{i}.", h, states[i], norm=cfg["norm"])
        h = mlp_block(P, f"mlp.{i}.", h, cfg["norm"])
    return h


def lm_prefill(P, cfg, x, window: Optional[int] = None, states: Optional[list] = None):
    """Windowed pass with carried state; returns (logits of the last window, states)
    (src/model.py:843-864; src/bench.py:206-213 is the same loop)."""
    window = window or cfg["ctx"]
    states = [None] * cfg["layers"] if states is None else states
    logits = None
    for s in range(0, x.shape[1], window):
        xw = x[:, s:s + window]
        h = _r(F.embedding(xw, P["e.weight"]) + P["p.weight"][: xw.shape[1]])
        h = lm_layers(P, cfg, h, states)
        logits = _r(F.linear(_norm(P, "n", h, cfg["norm"]), P["e.weight"]))
    return logits, states


def lm_forward_carried(P, cfg, x, window: Optional[int] = None):
    """LM.forward_carried (src/model.py:843-864): logits of the FINAL window only."""
    return lm_prefill(P, cfg, x, window)[0]


def lm_decode_step(P, cfg, tok, pos: int, states: list):
    """One eager decode step for a batch of sequences (src/bench.py:231-238 made batch-generic): tok (B,) ids at
    window position `pos`; returns logits (B,V); states are updated in the list."""
    h = _r(F.embedding(tok.reshape(-1, 1), P["e.weight"]) + P["p.weight"][pos])
    h = lm_layers(P, cfg, h, states)
    return _r(F.linear(_norm(P, "n", h, cfg["norm"]), P["e.weight"]))[:, -1]
