"""Drop-in for the reference's src/scan_kernel.py: the per-token-lambda complex scan on the sm_100a kernels."""
from __future__ import annotations

import torch

from . import ops


def scan_cuda(u, logmag, ang, h0=None):
    """Same contract as the reference's scan_triton (src/scan_kernel.py:144-148) and SpinCarrier.scan_gated:
    (Re h, (Re h_last, Im h_last)), fp32 inside, outputs in u's dtype. With gradients enabled and an input that requires
    them, the forward keeps Im h and the backward is the adjoint scan (src/scan_kernel.py:54-140)."""
    needs = torch.is_grad_enabled() and any(t is not None and t.requires_grad
                                            for t in (u, logmag, ang) + (tuple(h0) if h0 is not None else ()))
    if needs:
        from .custom_ops import lambda_scan_autograd
        y, (hr, hi) = lambda_scan_autograd(u, logmag, ang, h0)
    else:
        y, (hr, hi) = ops.lambda_scan(u, logmag, ang, h0)
    return y.to(u.dtype), (hr.to(u.dtype), hi.to(u.dtype))


scan_triton = scan_cuda          # the reference's name, so `from ...scan_kernel import scan_triton` keeps working
