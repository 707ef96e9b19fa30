"""The associative carrier layer on the sm_100a kernels: same module API and parameter names as the reference's
src/assoc.py (AssocCarrier :279-512, rotate :34, assoc_scan :254), so reference checkpoints load unchanged.

Built: the plain and delta rules, head dims 64 and 128, carried state across windows, the T=1 decode step, and the
layer's options -- short convolution on q|k|v (add_short_conv), key_topk, hl_floor, write_all, and the attributes
pos_wrap / beta_scale a caller may set from outside (src/assoc.py:406-410, :471).
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
        self.d, self.delta, self.chunk, self.kernel, self.recompute = d, delta, chunk, kernel, recompute
        self.key_topk, self.hl_floor, self.write_all = key_topk, hl_floor, write_all
        self.h = heads or max(1, d // (head_dim or 64))
        assert d % self.h == 0 and (d // self.h) % 2 == 0
        self.dk = d // self.h
        if self.dk not in (64, 128):
            raise NotImplementedError(f"head dim {self.dk}: the kernels are built for 64 and 128")
        if key_topk and not 0 < key_topk <= self.dk:
            raise ValueError("key_topk must lie in 1..head_dim")
        self.need_sent = False          # True: keep the state entering every 64-token chunk in self.sent (bf16)
        self.inplace_state = False      # True: a T=1 step overwrites the state tensor it was given (graphed decode)
        self.bv = 32                    # the reference's tiling knob; no meaning for these kernels
        self.pos_wrap = None            # set from outside: rotation positions modulo this window (src/assoc.py:406-410)
        self.beta_scale = None          # set from outside for one call: (B,H,T) multiplier on the write strength (:471)
        self.ln = nn.LayerNorm(d)
        self.q = nn.Linear(d, d, bias=False); self.k = nn.Linear(d, d, bias=False)
        self.v = nn.Linear(d, d, bias=False); self.o = nn.Linear(d, d, bias=False)
        self.wa = nn.Linear(d, self.h)
        self.wi = nn.Linear(d, self.h)
        if delta:
            self.wb = nn.Linear(d, self.h)
        self.A = nn.Parameter(torch.linspace(math.log(0.1 / 0.69), math.log(1e-4 / 0.69), self.h))
        if hl_floor:
            # no head may forget faster than its floor: half-lives geometric from 8 to 131072 tokens (src/assoc.py:339-343)
            hl = torch.logspace(math.log10(8.0), math.log10(131072.0), self.h)
            self.register_buffer("la_floor", -math.log(2.0) / hl, persistent=False)
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
        la = -F.softplus(self.wa(z)) * torch.exp(self.A)
        return la.clamp(min=self.la_floor) if self.hl_floor else la

    def add_short_conv(self, K: int):
        """A depthwise causal convolution over the last K tokens on q, k and v, initialised as the identity
        (src/assoc.py:361-373). The carried state then has a third member: the last K-1 inputs."""
        w = torch.zeros(3 * self.d, K, device=self.q.weight.device, dtype=self.q.weight.dtype)
        w[:, -1] = 1.0
        self.sconv = nn.Parameter(w)
        return self

    @property
    def plain_step(self) -> bool:
        """True when a T=1 step is exactly step_from_projection on the fused projection's output (no option in the way)."""
        return not (getattr(self, "sconv", None) is not None or self.key_topk or self.hl_floor or self.write_all
                    or self.beta_scale is not None)

    # One GEMM for q, k, v, the decay gate and the write gate / write strength: z is read once. Rows: [q | k | v | wa | wg],
    # padded to a multiple of 8 so every view into the product stays 16-byte aligned. Cached with the gated output
    # weight and fp32 copies of the small per-head constants; rebuilt when a parameter changes.
    def consts_key(self):
        gatew = self.wb if self.delta else self.wi
        ps = (self.q.weight, self.k.weight, self.v.weight, self.wa.weight, self.wa.bias, gatew.weight, gatew.bias,
              self.o.weight, self.gate, self.theta, self.A, self.on.weight)
        return tuple((p.data_ptr(), p._version, p.dtype) for p in ps)

    def _build_consts(self):
        gatew = self.wb if self.delta else self.wi
        W = torch.cat([self.q.weight, self.k.weight, self.v.weight, self.wa.weight, gatew.weight])
        b = torch.cat([torch.zeros(3 * self.d, device=W.device, dtype=W.dtype), self.wa.bias, gatew.bias])
        pad = (-W.shape[0]) % 8
        if pad:
            W = torch.cat([W, W.new_zeros(pad, W.shape[1])]); b = torch.cat([b, b.new_zeros(pad)])
        # the gated output weight: formed in fp32 and rounded once (the reference multiplies its fp32 parameters and lets
        # autocast round the product)
        ow = (self.o.weight.float() * torch.sigmoid(self.gate.float())).to(self.o.weight.dtype)
        return dict(W=W.contiguous(), b=b.contiguous(), ow=ow.contiguous(),
                    theta=self.theta.detach().float().contiguous(), A=self.A.detach().float().contiguous(),
                    expA=torch.exp(self.A.detach().float()), onw=self.on.weight.detach().float().contiguous())

    def _consts(self):
        if torch.compiler.is_compiling():
            return self._build_consts()                 # traced into the caller's graph: nothing cached, nothing stale
        key = self.consts_key()
        if self._fused is None or self._fused[0] != key:
            with torch.no_grad():
                self._fused = (key, self._build_consts())
            self._rot = None                            # the rotation table follows theta
        return self._fused[1]

    def forward(self, x, h0=None, pos0: int = 0):
        """x (B,T,d) on CUDA; h0 = (S (B,H,dk,dk) fp32, p0[, conv cache]) from the previous window or step, or None.
        Returns (out (B,T,d), (S, T[, conv cache])): positions restart at every call and the carried state is rotated back
        by the previous call's length instead (the reference's rebase, src/assoc.py:394-405)."""
        delta, st = self.mix(self.ln(x), h0)
        return x + delta, st

    def mix(self, z, h0=None):
        """The layer without its input norm and residual add: z = ln(x) in, (what is added to x, new state) out. The
        language model fuses the norm and the add of neighbouring blocks into one kernel and calls this directly."""
        B, T, D = z.shape
        H, dk, d = self.h, self.dk, self.d
        sconv = getattr(self, "sconv", None)
        if T > 1 and torch.is_grad_enabled() and (z.requires_grad or any(p.requires_grad for p in self.parameters())):
            return self._mix_train(z, h0)
        S0, p0, cc = None, 0, None
        if h0 is not None:
            S0, p0 = h0[0], h0[1]
            cc = h0[2] if len(h0) == 3 else None
        c = self._consts()
        y = F.linear(z, c["W"], c["b"])                               # (B,T,3d+2h[+pad])
        zero_shift = (not torch.is_tensor(p0)) and p0 == 0
        shift = 0.0 if zero_shift else p0
        qkv = y
        if sconv is not None:
            qkv, cc = ops.short_conv(y[..., :3 * d], sconv, cc)       # (B,T,3d) contiguous; the gates stay in y
        qp, kp, vp = (qkv[..., i * d:(i + 1) * d].unflatten(-1, (H, dk)) for i in range(3))
        if self.key_topk:
            ops.key_topk_mask_(kp, self.key_topk)                     # in place, on this call's own projection buffer
        a_logit, g_logit = y[..., 3 * d:3 * d + H], y[..., 3 * d + H:3 * d + 2 * H]
        if T == 1:
            o, S = self._step(qp, kp, vp, a_logit, g_logit, c, S0, shift)
            o = o.view(B, 1, d)
            self.sent = None
        else:
            bf16 = z.dtype == torch.bfloat16
            S_out = S0 if (self.inplace_state and S0 is not None) else None
            if bf16 and not self.delta and not self.hl_floor:
                # one kernel between the two GEMMs: plumbing (normalise, gate, rotate) on the TMA tiles, decay gate, scan on
                # the tensor cores, per-head RMS norm, token-major output
                o, S, sent = ops.layer_prefill(qp, kp, vp, None if self.write_all else g_logit, a_logit, c["A"],
                                               self._rot_table(T, c), S0, theta=c["theta"], shift=shift, rms_weight=c["onw"],
                                               rms_eps=self._rms_eps(), want_sent=self.need_sent, S_out=S_out)
            else:
                gate = None if (self.delta or self.write_all) else g_logit
                q, k, v = ops.prep(qp, kp, vp, gate, c["theta"], self._positions(T, z.device),
                                   out_dtype=torch.bfloat16 if bf16 else torch.float32)
                la = self._la(a_logit, c).transpose(1, 2).contiguous()
                beta = self._beta(g_logit).transpose(1, 2).contiguous() if self.delta else None
                o, S, sent = ops.prefill(q, k, v, la, beta, S0, theta=c["theta"], shift=shift, want_sent=self.need_sent,
                                         S_out=S_out)
                o = self.on(o.to(z.dtype)).transpose(1, 2).reshape(B, T, D)
            self.sent = sent
        delta = F.linear(o, c["ow"])
        if torch.is_tensor(p0):
            # a device-side position (graphed decode): with inplace_state the caller owns and updates it
            p_new = p0 if self.inplace_state else p0 * 0 + T
        else:
            p_new = T
        return delta, ((S, p_new, cc) if sconv is not None else (S, p_new))

    def _mix_train(self, z, h0):
        """The layer with a gradient wanted (the reference's training path, src/assoc.py:384-512 with its kernels on):
        separate projections of the live parameters, the differentiable prep / scan operators (their backward kernels are
        the reference's six), torch for the rest. Plain rule and delta rule with hl_floor / write_all / beta_scale /
        pos_wrap; a carried state must come with position 0."""
        from .assoc_kernel import assoc_scan_kernel, delta_scan_kernel, prep_kernel
        if getattr(self, "sconv", None) is not None or self.key_topk:
            raise NotImplementedError("training path: short convolution and key_topk are inference-only here")
        B, T, D = z.shape
        H, dk = self.h, self.dk
        S0 = None
        if h0 is not None:
            S0, p0 = h0[0], h0[1]
            if torch.is_tensor(p0) or p0 != 0:
                raise NotImplementedError("training path: the carried state must be at position 0")
        qp, kp, vp = (lin(z).view(B, T, H, dk) for lin in (self.q, self.k, self.v))
        gl = None if (self.delta or self.write_all) else self.wi(z)
        q, k, v = prep_kernel(qp, kp, vp, gl, self.theta, self._positions(T, z.device))
        la = self.logalpha(z).float().transpose(1, 2)
        if self.delta:
            beta = self._beta(self.wb(z)).transpose(1, 2)
            o, S, sent = delta_scan_kernel(q, k, v, la, beta, S0)
        else:
            o, S, sent = assoc_scan_kernel(q, k, v, la, S0)
        self.sent = sent if self.need_sent else None
        o = self.on(o.to(z.dtype)).transpose(1, 2).reshape(B, T, D)
        return F.linear(o, (self.o.weight.float() * torch.sigmoid(self.gate.float())).to(z.dtype)), (S, T)

    def _la(self, a_logit, c):
        """log alpha (B,T,H) fp32 from the decay gate's logits, floored per head when hl_floor is set."""
        la = -F.softplus(a_logit.float()) * c["expA"]
        return la.clamp(min=self.la_floor.float()) if self.hl_floor else la

    def _beta(self, g_logit):
        """The delta rule's write strength (B,T,H) fp32 with the options applied (src/assoc.py:468-478)."""
        bt = torch.sigmoid(g_logit.float())
        if self.beta_scale is not None:
            bt = bt * self.beta_scale.to(bt.dtype).transpose(1, 2)   # given as (B,H,T)
        if self.write_all:
            bt = bt.clamp(min=0.75)                                   # beta = 1 makes the chunk inverse singular
        return bt

    def _step(self, qp, kp, vp, a_logit, g_logit, c, S0, shift):
        """One token per sequence: the fused recurrent step. With an option that changes the gates, the log-decay / write
        strength are formed here and handed over as values instead of logits."""
        B, H, dk, d = qp.shape[0], self.h, self.dk, self.d
        if S0 is None:
            S0 = torch.zeros(B, H, dk, dk, device=qp.device, dtype=torch.float32)
        q3, k3, v3 = qp[:, 0], kp[:, 0], vp[:, 0]                      # (B,H,dk) views, unit strides over (H,dk)
        decay, decay_A = a_logit[:, 0], c["A"]
        if self.hl_floor:
            decay, decay_A = self._la(a_logit, c)[:, 0].to(qp.dtype), None
        gate, is_logit = g_logit[:, 0], True
        if self.delta and (self.write_all or self.beta_scale is not None):
            gate, is_logit = self._beta(g_logit)[:, 0].to(qp.dtype), False
        elif not self.delta and self.write_all:
            gate = None
        o = torch.empty(B, d, device=qp.device, dtype=qp.dtype)
        _, S = ops.decode_step(q3, k3, v3, decay, S0, c["theta"], gate=gate, delta=self.delta, gate_is_logit=is_logit,
                               decay_A=decay_A, normalize=True, shift=shift, rms_weight=c["onw"], rms_eps=self._rms_eps(),
                               out=o.view(B, H, dk), S_out=S0 if self.inplace_state else None)
        return o, S

    def step_from_projection(self, y2, S0, shift):
        """The recurrent step of one token per sequence from the fused projection's output y2 (B, 3d+2h[+pad]) =
        [q | k | v | decay logits | gate logits]: one kernel (normalise, gates, rotate the state, write, read, per-head RMS
        norm). Returns (o (B,d), S); with inplace_state the state is updated where it lies. For a layer without options
        (plain_step)."""
        c = self._consts()
        H, dk, d = self.h, self.dk, self.d
        y3 = y2.unsqueeze(1)
        qp, kp, vp = (y3[..., i * d:(i + 1) * d].unflatten(-1, (H, dk)) for i in range(3))
        return self._step(qp, kp, vp, y3[..., 3 * d:3 * d + H], y3[..., 3 * d + H:3 * d + 2 * H], c, S0, shift)

    def _rot_table(self, T, c):
        """(cos, sin) of position * theta for this layer's window positions (wrapped by pos_wrap when set); rebuilt when
        theta changes or T grows."""
        need = (T + 63) // 64 * 64                                   # whole 64-token chunks
        if torch.compiler.is_compiling():
            return self._wrapped(ops.rot_table(c["theta"], need), need)
        if self._rot is None or self._rot[0] != self.pos_wrap or self._rot[1].shape[1] < need:
            self._rot = (self.pos_wrap, self._wrapped(ops.rot_table(c["theta"], need), need))
        return self._rot[1]

    def _wrapped(self, table, need):
        if not self.pos_wrap:
            return table
        return table.index_select(1, torch.arange(need, device=table.device) % self.pos_wrap).contiguous()

    def _positions(self, T, device):
        if torch.compiler.is_compiling():
            pos = torch.arange(T, device=device)
        else:
            if self._pos is None or self._pos.numel() < T or self._pos.device != device:
                self._pos = torch.arange(max(T, 512), device=device)
            pos = self._pos[:T]
        return pos % self.pos_wrap if self.pos_wrap else pos

    def _rms_eps(self):
        # nn.RMSNorm(eps=None) uses the epsilon of the ARITHMETIC type: fp32's for bf16 / fp16 / fp32 inputs
        return self.on.eps if self.on.eps is not None else torch.finfo(torch.float32).eps
