"""Seeded synthetic workloads with the shapes and value distributions of the five benchmark configurations.

Everything is drawn on the CPU in fp32 from one torch.Generator per case, so a CPU checker and the GPU path see
the same numbers; callers cast / copy afterwards. Nothing here touches a GPU.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rope_theta(H: int, D: int, base: float = 10000.0) -> torch.Tensor:
    """theta[h, i] = base^(-2i/D), the same for every head (the carrier's init, reference src/assoc.py:345-346)."""
    return (base ** (-torch.arange(0, D, 2).float() / D)).unsqueeze(0).repeat(H, 1)


def assoc_op_inputs(B: int, H: int, T: int, D: int, seed: int, delta: bool = False, with_state: bool = False,
                    gate_mean: float = 2.0):
    """Op-level inputs of the chunked scan: q, v ~ N(0,1); k ~ N(0,1) L2-normalised per head; forget gate
    sigmoid(g), g ~ N(gate_mean, 1) given as log-decay; beta = sigmoid(N(0,1)) for the delta rule; theta as
    rope_theta; positions 0..T-1.  q and k are returned UNROTATED together with theta and pos."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, T, D, generator=g)
    k = F.normalize(torch.randn(B, H, T, D, generator=g), dim=-1)
    v = torch.randn(B, H, T, D, generator=g)
    la = F.logsigmoid(torch.randn(B, H, T, generator=g) + gate_mean)
    out = dict(q=q, k=k, v=v, la=la, theta=rope_theta(H, D), pos=torch.arange(T))
    if delta:
        out["beta"] = torch.sigmoid(torch.randn(B, H, T, generator=g))
    if with_state:
        out["S0"] = torch.randn(B, H, D, D, generator=g) * 0.1
    return out


def lambda_scan_inputs(B: int, T: int, D: int, seed: int, with_state: bool = False, per_channel_angle: bool = False):
    """|lambda_t| ~ U(0.9, 0.999) as logmag, phase ~ U(0, pi), gamma ~ N(0, 0.1) per channel, u ~ N(0,1); the scan's
    input is gamma * u (the reference applies gamma outside the scan, src/spin.py:240-241)."""
    g = torch.Generator().manual_seed(seed)
    mag = 0.9 + 0.099 * torch.rand(B, T, D, generator=g)
    if per_channel_angle:
        ang = (math.pi * torch.rand(D, generator=g)).expand(B, T, D)
    else:
        ang = math.pi * torch.rand(B, T, D, generator=g)
    gamma = 0.1 * torch.randn(D, generator=g)
    u = torch.randn(B, T, D, generator=g) * gamma
    out = dict(u=u, logmag=mag.log(), ang=ang)
    if with_state:
        out["h0"] = (torch.randn(B, D, generator=g), torch.randn(B, D, generator=g))
    return out


def token_ids(B: int, T: int, vocab: int, seed: int) -> torch.Tensor:
    """Token ids uniform over [0, vocab)."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (B, T), generator=g)
