"""Drop-in for the reference's src/scan_kernel.py: the per-token-lambda complex scan on the sm_100a kernel."""
from __future__ import annotations

from . import ops


def scan_cuda(u, logmag, ang, h0=None):
    """Same contract as the reference's scan_triton (src/scan_kernel.py:144-148) and SpinCarrier.scan_gated:
    (Re h, (Re h_last, Im h_last)), fp32 inside, outputs in u's dtype."""
    y, (hr, hi) = ops.lambda_scan(u, logmag, ang, h0)
    return y.to(u.dtype), (hr.to(u.dtype), hi.to(u.dtype))


scan_triton = scan_cuda          # the reference's name, so `from ...scan_kernel import scan_triton` keeps working
