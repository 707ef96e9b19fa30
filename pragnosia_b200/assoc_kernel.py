"""Drop-in for the reference's src/assoc_kernel.py entry points, on the sm_100a kernels.

Same names, argument meaning and return triples as the reference (src/assoc_kernel.py:302, :512, :888). One
difference in favour of precision: fp32 inputs run the fp32 kernel instead of being rounded to bf16 first; bf16 inputs
run the tensor-core kernel. The tiling knobs bv / bv_bwd of the Triton kernels have no meaning here and are ignored.
The reference's individual operators (membrae::assoc_out, prefix_scan, delta_inv, delta_loop_fwd, assoc_prep) exist as
torch custom ops of the same argument lists in pragnosia_b200.custom_ops (torch.ops.pragnosia_b200.*).
"""
from __future__ import annotations

import torch

from . import ops


def _wants_grad(*ts) -> bool:
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in ts)


def prep_kernel(qp, kp, vp, gate_logits, theta, pos):
    """qp, kp, vp: the projections as (B,T,H,D) views; gate_logits (B,T,H) or None; theta (H,D/2); pos (T,) integer
    positions. Returns bf16 q, k, v as (B,H,T,D). Differentiable (the backward kernel of src/assoc_kernel.py:774-826)."""
    if _wants_grad(qp, kp, vp, gate_logits, theta):
        from . import custom_ops  # noqa: F401
        return tuple(torch.ops.pragnosia_b200.assoc_prep(qp, kp, vp, gate_logits, theta, pos))
    return ops.prep(qp, kp, vp, gate_logits, theta, pos)


def _chunk_decay(logalpha, T):
    """(a_log (B,H,NC), w (B,H,NC,64)) of whole 64-token chunks: the chunk's total log-decay and e^{total - cumulative}."""
    B, H = logalpha.shape[:2]
    NC = (T + ops.CHUNK - 1) // ops.CHUNK
    Lc = torch.nn.functional.pad(logalpha.float(), (0, NC * ops.CHUNK - T)).view(B, H, NC, ops.CHUNK).cumsum(-1)
    a_log = Lc[..., -1]
    return a_log, torch.exp(a_log[..., None] - Lc)


def assoc_scan_kernel(q, k, v, logalpha, S0=None, bv: int = 16):
    """Plain rule: (o in q's dtype, final state fp32, state entering each 64-token chunk bf16 (B,H,NC,D,D)).
    When a gradient is wanted the scan is composed from the differentiable operators, as the reference composes it
    (prefix_scan, then assoc_out: src/assoc_kernel.py:302-323); otherwise it is the one fused walk."""
    if _wants_grad(q, k, v, logalpha, S0):
        T = q.shape[2]
        pad = (-T) % ops.CHUNK
        a_log, w = _chunk_decay(logalpha, T)
        kp, vp = (torch.nn.functional.pad(t, (0, 0, 0, pad)) for t in (k, v))
        sent, S = ops.prefix_scan(kp, vp, w, a_log, S0)
        return ops.assoc_out(q, k, v, logalpha, sent).to(q.dtype), S, sent
    o, S, sent = ops.prefill(q, k, v, logalpha, None, S0, want_sent=True)
    return o, S, sent


def delta_scan_kernel(q, k, v, logalpha, beta, S0=None, chunk: int = 64, bv: int = 32, bv_bwd: int = 16):
    """Delta rule, same return triple. The kernels chunk by 64 tokens; the result does not depend on the chunk size.
    With a gradient wanted: delta_inv, delta_loop_fwd, then assoc_out on the residuals (src/assoc_kernel.py:512-546)."""
    if _wants_grad(q, k, v, logalpha, beta, S0):
        NC = (q.shape[2] + ops.CHUNK - 1) // ops.CHUNK
        X = ops.delta_inv(k, logalpha, beta, NC)
        W, sent, S = ops.delta_loop_fwd(k, v, logalpha, beta, X, S0)
        return ops.assoc_out(q, k, W, logalpha, sent).to(q.dtype), S, sent
    o, S, sent = ops.prefill(q, k, v, logalpha, beta, S0, want_sent=True)
    return o, S, sent
