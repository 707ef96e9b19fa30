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


def assoc_scan_kernel(q, k, v, logalpha, S0=None, bv: int = 16):
    """Plain rule: (o in q's dtype, final state fp32, state entering each 64-token chunk bf16 (B,H,NC,D,D))."""
    o, S, sent = ops.prefill(q, k, v, logalpha, None, S0, want_sent=True)
    return o, S, sent


def delta_scan_kernel(q, k, v, logalpha, beta, S0=None, chunk: int = 64, bv: int = 32, bv_bwd: int = 16):
    """Delta rule, same return triple. The kernels chunk by 64 tokens; the result does not depend on the chunk size."""
    o, S, sent = ops.prefill(q, k, v, logalpha, beta, S0, want_sent=True)
    return o, S, sent
