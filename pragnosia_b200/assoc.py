"""The associative carrier layer on the sm_100a kernels: same module API and parameter names as the reference's
src/assoc.py (AssocCarrier :279-512, rotate :34, assoc_scan :254), so reference checkpoints load unchanged.

In scope: the plain and delta rules, head dims 64 and 128, carried state across windows, the T=1 decode step.
The reference's optional extras (short convolution, key_topk, hl_floor, write_all, pos_wrap, beta_scale) belong to its
hybrid / experimental mixers and raise NotImplementedError here.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops


def rotate(x, theta, pos):
    """RoPE-style rotation of channel pairs by theta_i * pos. x (B,H,T,dk); theta (H,dk/2); pos (T,)."""
    return ops.rotate(x, theta, pos)


def assoc_scan(q, k, v, logalpha, S0=None, chunk: int = 64, recompute: bool = False, mm=None, beta=None, kernel=False):
    """Chunked scan, (o, final state); plain rule or, with beta, the delta rule. The result does not depend on `chunk`;
    recompute / mm / kernel are accepted for signature compatibility and ignored."""
    o, S, _ = ops.prefill(q, k, v, logalpha, beta, S0)
    return o, S


class AssocCarrier(nn.Module):
    def __init__(self, d: int, heads: int | None = None, chunk: int = 64, recompute: bool = False, delta: bool = False,
                 head_dim: int | None = None, kernel: bool = True, key_topk: int = 0, hl_floor: bool = False,
                 write_all: bool = False):
        super().__init__()
        if key_topk or hl_floor or write_all:
            raise NotImplementedError("key_topk / hl_floor / write_all are outside the carrier hot path built here")
        self.d, self.delta, self.chunk, self.kernel = d, delta, chunk, kernel
        self.h = heads or max(1, d // (head_dim or 64))
        assert d % self.h == 0 and (d // self.h) % 2 == 0
        self.dk = d // self.h
        if self.dk not in (64, 128):
            raise NotImplementedError(f"head dim {self.dk}: the kernels are built for 64 and 128")
        self.need_sent = False          # True: keep the state entering every 64-token chunk in self.sent (bf16)
        self.inplace_state = False      # True: a T=1 step overwrites the state tensor it was given (graphed decode)
        self.ln = nn.LayerNorm(d)
        self.q = nn.Linear(d, d, bias=False); self.k = nn.Linear(d, d, bias=False)
        self.v = nn.Linear(d, d, bias=False); self.o = nn.Linear(d, d, bias=False)
        self.wa = nn.Linear(d, self.h)
        self.wi = nn.Linear(d, self.h)
        if delta:
            self.wb = nn.Linear(d, self.h)
        self.A = nn.Parameter(torch.linspace(math.log(0.1 / 0.69), math.log(1e-4 / 0.69), self.h))
        base = 10000.0 ** (-torch.arange(0, self.dk, 2).float() / self.dk)
        self.theta = nn.Parameter(base.unsqueeze(0).repeat(self.h, 1))
        self.on = nn.RMSNorm(self.dk)
        self.gate = nn.Parameter(torch.zeros(()))
        self.sent = None
        self._fused = None
        self._pos = None
        self._rot = None

    def spectral_parameters(self):
        return [self.A, self.theta, self.gate]

    def logalpha(self, z):
        return -F.softplus(self.wa(z)) * torch.exp(self.A)

    # One GEMM for q, k, v, the decay gate and the write gate / write strength: z is read once. Rows: [q | k | v | wa | wg],
    # padded to a multiple of 8 so every view into the product stays 16-byte aligned. Cached with the gated output
    # weight and fp32 copies of the small per-head constants; rebuilt when a parameter changes.
    def _consts(self):
        gatew = self.wb if self.delta else self.wi
        ps = (self.q.weight, self.k.weight, self.v.weight, self.wa.weight, self.wa.bias, gatew.weight, gatew.bias,
              self.o.weight, self.gate, self.theta, self.A, self.on.weight)
        key = tuple((p.data_ptr(), p._version, p.dtype) for p in ps)
        if self._fused is None or self._fused[0] != key:
            with torch.no_grad():
                W = torch.cat([self.q.weight, self.k.weight, self.v.weight, self.wa.weight, gatew.weight])
                b = torch.cat([torch.zeros(3 * self.d, device=W.device, dtype=W.dtype), self.wa.bias, gatew.bias])
                pad = (-W.shape[0]) % 8
                if pad:
                    W = torch.cat([W, W.new_zeros(pad, W.shape[1])]); b = torch.cat([b, b.new_zeros(pad)])
                c = dict(W=W.contiguous(), b=b.contiguous(), ow=(self.o.weight * torch.sigmoid(self.gate)).contiguous(),
                         theta=self.theta.detach().float().contiguous(), A=self.A.detach().float().contiguous(),
                         expA=torch.exp(self.A.detach().float()), onw=self.on.weight.detach().float().contiguous())
            self._fused = (key, c)
        return self._fused[1]

    def forward(self, x, h0=None, pos0: int = 0):
        """x (B,T,d) on CUDA; h0 = (S (B,H,dk,dk) fp32, p0) from the previous window or step, or None.
        Returns (out (B,T,d), (S, T)): positions restart at every call and the carried state is rotated back by the
        previous call's length instead (the reference's rebase, src/assoc.py:394-405)."""
        delta, st = self.mix(self.ln(x), h0)
        return x + delta, st

    def mix(self, z, h0=None):
        """The layer without its input norm and residual add: z = ln(x) in, (what is added to x, new state) out. The
        language model fuses the norm and the add of neighbouring blocks into one kernel and calls this directly."""
        B, T, D = z.shape
        H, dk = self.h, self.dk
        S0, p0 = (None, 0) if h0 is None else (h0[0], h0[1])
        if h0 is not None and len(h0) == 3:
            raise NotImplementedError("short-convolution state is outside the carrier hot path built here")
        c = self._consts()
        y = F.linear(z, c["W"], c["b"])                               # (B,T,3d+2h[+pad])
        d = self.d
        zero_shift = (not torch.is_tensor(p0)) and p0 == 0
        if T == 1:
            o, S = self.step_from_projection(y.view(B, -1), S0, 0.0 if zero_shift else p0)
            o = o.view(B, 1, d)
            self.sent = None
        else:
            qp, kp, vp = (y[..., i * d:(i + 1) * d].unflatten(-1, (H, dk)) for i in range(3))
            g = y[..., 3 * d + H:3 * d + 2 * H]
            bf16 = z.dtype == torch.bfloat16
            shift = 0.0 if zero_shift else p0
            S_out = S0 if (self.inplace_state and S0 is not None) else None
            if bf16 and not self.delta:
                # one kernel between the two GEMMs: plumbing (normalise, gate, rotate) on the TMA tiles, decay gate, scan on
                # the tensor cores, per-head RMS norm, token-major output
                o, S, sent = ops.layer_prefill(qp, kp, vp, g, y[..., 3 * d:3 * d + H], c["A"], self._rot_table(T, c), S0,
                                               theta=c["theta"], shift=shift, rms_weight=c["onw"],
                                               rms_eps=self._rms_eps(z.dtype), want_sent=self.need_sent, S_out=S_out)
            else:
                q, k, v = ops.prep(qp, kp, vp, None if self.delta else g, c["theta"], self._positions(T, z.device),
                                   out_dtype=torch.bfloat16 if bf16 else torch.float32)
                la = (-F.softplus(y[..., 3 * d:3 * d + H].float()) * c["expA"]).transpose(1, 2).contiguous()
                beta = torch.sigmoid(g.float()).transpose(1, 2).contiguous() if self.delta else None
                o, S, sent = ops.prefill(q, k, v, la, beta, S0, theta=c["theta"], shift=shift, want_sent=self.need_sent,
                                         S_out=S_out)
                o = self.on(o.to(z.dtype)).transpose(1, 2).reshape(B, T, D)
            self.sent = sent
        delta = F.linear(o, c["ow"])
        if torch.is_tensor(p0):
            # a device-side position (graphed decode): with inplace_state the caller owns and updates it
            return delta, (S, p0 if self.inplace_state else p0 * 0 + T)
        return delta, (S, T)

    def step_from_projection(self, y2, S0, shift):
        """The recurrent step of one token per sequence from the fused projection's output y2 (B, 3d+2h[+pad]) =
        [q | k | v | decay logits | gate logits]: one kernel (normalise, gates, rotate the state, write, read, per-head RMS
        norm). Returns (o (B,d), S); with inplace_state the state is updated where it lies."""
        c = self._consts()
        B, H, dk, d = y2.shape[0], self.h, self.dk, self.d
        if S0 is None:
            S0 = torch.zeros(B, H, dk, dk, device=y2.device, dtype=torch.float32)
        o = torch.empty(B, d, device=y2.device, dtype=y2.dtype)
        _, S = ops.decode_step(
            y2[:, 0:d].unflatten(1, (H, dk)), y2[:, d:2 * d].unflatten(1, (H, dk)), y2[:, 2 * d:3 * d].unflatten(1, (H, dk)),
            y2[:, 3 * d:3 * d + H], S0, c["theta"], gate=y2[:, 3 * d + H:3 * d + 2 * H], delta=self.delta,
            gate_is_logit=True, decay_A=c["A"], normalize=True, shift=shift,
            rms_weight=c["onw"], rms_eps=self._rms_eps(y2.dtype), out=o.view(B, H, dk),
            S_out=S0 if self.inplace_state else None)
        return o, S

    def _rot_table(self, T, c):
        """(cos, sin) of position * theta for this layer's window positions; rebuilt when theta changes or T grows."""
        key = c["theta"].data_ptr()
        need = (T + 63) // 64 * 64                                   # whole 64-token chunks
        if self._rot is None or self._rot[0] != key or self._rot[1].shape[1] < need:
            self._rot = (key, ops.rot_table(c["theta"], need))
        return self._rot[1]

    def _positions(self, T, device):
        if self._pos is None or self._pos.numel() < T or self._pos.device != device:
            self._pos = torch.arange(max(T, 512), device=device)
        return self._pos[:T]

    def _rms_eps(self, dtype):
        # nn.RMSNorm(eps=None) uses the epsilon of the ARITHMETIC type: fp32's for bf16 / fp16 / fp32 inputs
        return self.on.eps if self.on.eps is not None else torch.finfo(torch.float32).eps
