"""The forget-gated diagonal carrier (the reference's SpinCarrier with gated="rf", src/spin.py:59-254) on the sm_100a
per-token-lambda scan. The time-invariant FFT variants are a different path and are not built here."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .scan_kernel import scan_cuda


class SpinCarrier(nn.Module):
    NU_MIN = 1e-3

    def __init__(self, d: int, chunk: int = 128, nu_min: float = 1e-3, nu_max: float = 0.3, gated: str | None = "rf"):
        super().__init__()
        if gated != "rf":
            raise NotImplementedError('only the forget-gated carrier (gated="rf") runs through the per-token scan')
        self.d, self.chunk, self.gated, self.gate_c = d, chunk, gated, 8.0
        self.nu_raw = nn.Parameter(torch.linspace(math.log(math.expm1(nu_min)), math.log(math.expm1(nu_max)), d))
        self.theta = nn.Parameter(torch.linspace(0.0, math.pi, d))
        self.B = nn.Linear(d, d, bias=False)
        self.C = nn.Linear(d, d, bias=False)
        self.ln = nn.LayerNorm(d)
        self.gate = nn.Parameter(torch.zeros(()))
        self.Wi = nn.Linear(d, d); self.Wr = nn.Linear(d, d)

    def lam(self):
        nu = self.NU_MIN + F.softplus(self.nu_raw)
        return torch.exp(-nu), self.theta

    def spectral_parameters(self):
        return [self.nu_raw, self.theta, self.gate]

    @staticmethod
    def scan_gated(u, logmag, ang, h0=None, chunk: int = 16):
        """(Re h, (Re h_last, Im h_last)) for h_t = lambda_t h_{t-1} + u_t; `chunk` is accepted and ignored."""
        return scan_cuda(u, logmag, ang, h0)

    def forward(self, x, h0=None):
        delta, h = self.mix(self.ln(x), h0)
        return x + delta, h

    def mix(self, z, h0=None):
        """The layer without its input norm and residual add (see AssocCarrier.mix)."""
        nu = (self.NU_MIN + F.softplus(self.nu_raw.float()))
        logmag = -self.gate_c * torch.sigmoid(self.Wr(z).float()) * nu
        gam = torch.sqrt((1.0 - torch.exp(2.0 * logmag)).clamp_min(1e-6))
        u = self.B(z).float() * gam * torch.sigmoid(self.Wi(z).float())
        y, h = scan_cuda(u, logmag, self.theta.float().expand_as(logmag), h0)
        return torch.sigmoid(self.gate) * self.C(y.to(z.dtype)), h
