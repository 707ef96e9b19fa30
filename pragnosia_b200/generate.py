"""Windowed prefill and CUDA-graphed recurrent decode for a batch of sequences.

The reference's driver (src/bench.py Ours.generate :193-239 and _generate_graphed :242-317) decodes one sequence and
syncs with the host for every sampled token. Here the loop is batch-generic, each layer's T=1 step is one fused kernel
that updates its state in place, the whole step is one CUDA graph, and sampling stays on the device (no per-token
host round trip; tokens are read back once at the end).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
import torch.nn.functional as F

from . import ops
from ._lib import graph_capture
from .assoc import AssocCarrier


class Decoder:
    def __init__(self, model, batch: int, use_graph: bool = True, fused: bool = True, min_p: float = 0.0,
                 token_kernel: bool = True, folded: bool = False):
        self.m = model.eval()
        self.min_p = float(min_p)                            # drop ids below min_p x the most likely one's probability (src/bench.py:38)
        self.B = batch
        self.use_graph = use_graph
        self.fused = fused                                   # small-batch bf16 step through the fused linear kernel
        self.token_kernel = token_kernel                     # ... and, where it applies, the whole step as one launch
        self.folded = folded                                 # batches 5..128: this library's tensor-core linear with the norms folded in
        self._plan = None
        self.dev = next(model.parameters()).device
        self.w = model.ctx
        self.states = None
        self._graph = None
        self._stamp = None
        self.tok = torch.zeros(batch, 1, dtype=torch.long, device=self.dev)
        self.pos = torch.zeros(1, dtype=torch.long, device=self.dev)
        self.shift = torch.zeros((), dtype=torch.float32, device=self.dev)    # positions the states are rotated back by
        self.logits = None

    # ---- prompt
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor):
        """ids (B,Tp): consume the prompt window by window; returns the logits after its last token (B,V)."""
        m, w = self.m, self.w
        # the captured step holds parameter addresses and the mixers' derived constants: weights that changed since the
        # capture (load_state_dict, an in-place update, a dtype change) retire it
        stamp = m.weights_stamp()
        if stamp != self._stamp:
            self._graph, self._gen_key, self._stamp = None, None, stamp
        states = [None] * m.layers
        h = None; n = 0
        for s in range(0, ids.shape[1], w):
            xw = ids[:, s:s + w]; n = xw.shape[1]
            h = m._add_norm(*m._layers(m._embed(xw), states), m.n)[1]
        pw = n % w
        new = []
        for st in states:                                   # own, contiguous copies the graph can update in place
            new.append(tuple(t.clone().contiguous() if torch.is_tensor(t) else t for t in st))
        if self.states is None:
            self.states = new
        else:
            for old, cur in zip(self.states, new):
                for a, b in zip(old, cur):
                    if torch.is_tensor(a): a.copy_(b)
        if self._plan is not None:
            self._plan["sync"].zero_()                       # a fresh pair of barrier counters (a step that gave up leaves them uneven)
        self.pos.fill_(pw)
        self.shift.fill_(float(n))                           # the last window's length (src/assoc.py:512 returns p0 + T)
        return F.linear(h[:, -1:], m.e.weight)[:, -1].float()

    # ---- one token
    def _fused_ok(self):
        """The five-launches-per-layer step: bf16 weights, aspin-family mixers, at most four sequences (measured on B200:
        0.30 / 0.33 / 0.37 ms per token at batch 1 / 2 / 4 against 0.45-0.48 through the library GEMMs; from batch 8 on
        the library path wins)."""
        m = self.m
        return (self.fused and self.B <= 4 and m.e.weight.dtype == torch.bfloat16 and m.d % 8 == 0 and
                all(isinstance(mx, AssocCarrier) and mx.plain_step for mx in m.mix))

    def _token_ok(self):
        """The whole step as ONE cooperative launch (ops.decode_token): the fused path's conditions, one kind of mixer
        throughout, an MLP width the 128-bit loads divide."""
        m = self.m
        if not (self.token_kernel and self._fused_ok()):
            return False
        mx0 = m.mix[0]
        return (all(mx.delta == mx0.delta and mx.dk == mx0.dk and mx.h == mx0.h for mx in m.mix) and mx0.dk in (64, 128) and
                all(mp.a.weight.shape[0] % 8 == 0 and mp.a.weight.shape == m.mlp[0].a.weight.shape for mp in m.mlp))

    def _token_plan(self):
        """The device-side table of per-layer pointers and norm settings the one-launch step reads, its scratch, barrier
        counters and logits; rebuilt when the weights' stamp or a state's address changes."""
        m = self.m
        key = (self._stamp, tuple(st[0].data_ptr() for st in self.states))
        if self._plan is not None and self._plan["key"] == key:
            return self._plan
        rows = np.zeros((m.layers, 18), dtype=np.int64)
        i32, f32 = rows.view(np.int32), rows.view(np.float32)
        keep = []                                            # every tensor whose address the table holds

        def at(t):
            if t is None:
                return 0
            c = t.detach().to(torch.bfloat16).contiguous(); keep.append(c)
            return c.data_ptr()

        for i, (mx, mp) in enumerate(zip(m.mix, m.mlp)):
            c = mx._consts(); keep.append(c)
            k1, w1, b1, e1 = ops._norm_args(mx.ln)
            k2, w2, b2, e2 = ops._norm_args(mp.n)
            rows[i, :15] = [c["W"].data_ptr(), c["b"].data_ptr(), at(w1), at(b1), c["ow"].data_ptr(), at(w2), at(b2),
                            at(mp.a.weight), at(mp.a.bias), at(mp.b.weight), at(mp.b.bias), c["theta"].data_ptr(),
                            c["A"].data_ptr(), c["onw"].data_ptr(), self.states[i][0].data_ptr()]
            i32[i, 30], i32[i, 31] = k1, k2
            f32[i, 32], f32[i, 33], f32[i, 34] = e1, e2, mx._rms_eps()
        mx0, NP, dff = m.mix[0], m.mix[0]._consts()["W"].shape[0], m.mlp[0].a.weight.shape[0]
        work = torch.empty(ops.decode_token_work_bytes(self.B, m.d, NP, dff) // 2, dtype=torch.bfloat16, device=self.dev)
        self._plan = dict(key=key, keep=keep, table=torch.from_numpy(rows).to(self.dev), work=work, NP=NP, dff=dff,
                          sync=torch.zeros(2, dtype=torch.int64, device=self.dev), H=mx0.h, D=mx0.dk, delta=bool(mx0.delta),
                          logits=torch.empty(self.B, m.e.weight.shape[0], dtype=torch.float32, device=self.dev))
        return self._plan

    def _step_token(self, advance: bool = True, out: Optional[torch.Tensor] = None):
        m, p = self.m, self._token_plan()
        lg = ops.decode_token(p["table"], m.e.weight, m.p.weight, m.n, self.tok, self.pos, self.shift, p["work"],
                              p["logits"] if out is None else out, p["sync"], p["H"], p["D"], p["NP"], p["dff"], p["delta"])
        if advance:
            self.shift.fill_(1.0)
            self.pos.copy_((self.pos + 1) % self.w)
        return lg

    @property
    def launches_per_token(self):
        """Kernels in one token's graph: this library's on the one-launch path (draw, step) and on the fused path (draw,
        embedding, five per layer, head); on the library-GEMM path the count includes the GEMMs and the copies around them."""
        L = self.m.layers
        if self._token_ok():
            return 2
        if self._fused_ok():
            return 1 + 1 + 5 * L + 1
        if self._wide_ok():
            return 1 + 1 + 5 * L + 1 + 1                      # draw, embedding, five per layer, head, logits copy
        per_layer = 2 + 1 + 1 + 1 + 1 + 1 + 1            # two add+norm, projection, state step, output projection, MLP up (+GELU) and down
        return 1 + 3 + per_layer * L + 2 + 1               # draw; embedding gather x2 + add; layers; final add+norm, head; logits copy

    def _step_fused(self, advance: bool = True):
        """Every linear layer of the step as one launch that also does the residual add and norm before it and the
        activation after it (ops.skinny_linear): per layer projection, state step, output projection, MLP up, MLP down."""
        m, B = self.m, self.B
        x, delta = ops.decode_embed(self.tok, self.pos, m.e.weight, m.p.weight), None
        for i, (mx, mp) in enumerate(zip(m.mix, m.mlp)):
            c = mx._consts()
            y, x = ops.skinny_linear(x, c["W"], c["b"], delta=delta, norm=mx.ln, want_sum=True)
            mx.inplace_state = True
            o, _ = mx.step_from_projection(y, self.states[i][0], self.shift)
            mx.inplace_state = False
            d1 = ops.skinny_linear(o, c["ow"])
            hmid, x = ops.skinny_linear(x, mp.a.weight, mp.a.bias, delta=d1, norm=mp.n, act="gelu", want_sum=True)
            delta = ops.skinny_linear(hmid, mp.b.weight, mp.b.bias)
        if advance:
            self.shift.fill_(1.0)
            self.pos.copy_((self.pos + 1) % self.w)
        return ops.skinny_linear(x, m.e.weight, delta=delta, norm=m.n).float()

    def _wide_ok(self):
        """Batches past the few-row kernels and up to one 128-row tensor-core tile: every linear layer as one tcgen05
        launch (ops.batch_linear) with the norm in front and the residual add behind folded in. Opt-in (folded=True): it
        needs none of the library's GEMMs and 5 launches a layer instead of 8, measured 2-5 % faster than the library step
        (0.49 against 0.50 ms per token at batch 64), but the folded norm rounds at other places than the separate ops --
        the default keeps the roundings the oracle's bf16 mode models."""
        m = self.m
        return (self.fused and self.folded and 4 < self.B <= 128 and m.e.weight.dtype == torch.bfloat16 and m.d % 8 == 0 and
                m.e.weight.shape[0] % 8 == 0 and all(isinstance(mx, AssocCarrier) and mx.plain_step for mx in m.mix) and
                all(mp.a.weight.shape[0] % 8 == 0 for mp in m.mlp))

    def _wide_consts(self):
        """Per layer, the weights with the norm in front of them folded in (ops.fold_norm); rebuilt with the weights' stamp."""
        if getattr(self, "_wide", None) is None or self._wide[0] != self._stamp:
            m, per = self.m, []
            for mx, mp in zip(m.mix, m.mlp):
                c = mx._consts()
                per.append((ops.fold_norm(mx.ln, c["W"], c["b"]), ops.fold_norm(mp.n, mp.a.weight, mp.a.bias)))
            self._wide = (self._stamp, per, ops.fold_norm(m.n, m.e.weight))
        return self._wide[1], self._wide[2]

    def _step_wide(self, advance: bool = True):
        """Five launches a layer, every one this library's: each linear layer is one tcgen05 launch (ops.batch_linear) that
        also does what surrounds it -- the norm in front is folded into the weight and applied on the accumulator from row
        sums the producing launch left behind; the residual add behind is the producer's epilogue."""
        m = self.m
        per, head = self._wide_consts()
        x, sums = ops.decode_embed(self.tok, self.pos, m.e.weight, m.p.weight, want_sums=True)
        for i, (mx, mp) in enumerate(zip(m.mix, m.mlp)):
            c = mx._consts()
            (Wp, c1p, c2p, kp, ep), (Wa, c1a, c2a, ka, ea) = per[i]
            y = ops.batch_linear(x, Wp, folded=(sums, c1p, c2p, kp, ep))
            mx.inplace_state = True
            o, _ = mx.step_from_projection(y, self.states[i][0], self.shift)
            mx.inplace_state = False
            x, sums = ops.batch_linear(o, c["ow"], resid=x, want_sums=True)
            hmid = ops.batch_linear(x, Wa, act="gelu", folded=(sums, c1a, c2a, ka, ea))
            x, sums = ops.batch_linear(hmid, mp.b.weight, mp.b.bias, resid=x, want_sums=True)
        if advance:
            self.shift.fill_(1.0)
            self.pos.copy_((self.pos + 1) % self.w)
        We, c1e, c2e, ke, ee = head
        return ops.batch_linear(x, We, folded=(sums, c1e, c2e, ke, ee)).float()

    def _step(self, advance: bool = True):
        if self._token_ok():
            return self._step_token(advance)
        if self._fused_ok():
            return self._step_fused(advance)
        if self._wide_ok():
            return self._step_wide(advance)
        m = self.m
        x, delta = m.e(self.tok) + m.p(self.pos), None
        for i, (mx, mp) in enumerate(zip(m.mix, m.mlp)):
            st = self.states[i]
            x, z = m._add_norm(x, delta, mx.ln)
            if isinstance(mx, AssocCarrier):
                mx.inplace_state = True
                delta, new = mx.mix(z, (st[0], self.shift) + tuple(st[2:]))
                mx.inplace_state = False
                if len(st) == 3:                               # the short convolution's context comes back as a new tensor
                    st[2].copy_(new[2])
            else:
                delta, new = mx.mix(z, st)
                for a, b in zip(st, new): a.copy_(b)
            x, z = m._add_norm(x, delta, mp.n)
            delta = mp.ff(z)
        if advance:
            self.shift.fill_(1.0)
            self.pos.copy_((self.pos + 1) % self.w)
        z = m._add_norm(x, delta, m.n)[1]
        if self.B <= 128 and z.dtype == torch.bfloat16 and m.e.weight.dtype == torch.bfloat16 and m.d % 8 == 0 and m.e.weight.shape[0] % 8 == 0:
            # the tied head for up to 128 rows on this library's tensor-core kernel: for 64 rows by 8192 columns the
            # library's heuristic picked a kernel that took 78 us, a sixth of the whole step
            return ops.batch_linear(z.reshape(self.B, m.d), m.e.weight).float()
        return F.linear(z, m.e.weight)[:, -1].float()

    @torch.no_grad()
    def step(self, tok: torch.Tensor):
        """tok (B,) ids -> logits (B,V). The first call captures the graph."""
        self.tok.copy_(tok.reshape(self.B, 1))
        if not self.use_graph:
            return self._step()
        if self._graph is None:
            saved = [tuple(t.clone() if torch.is_tensor(t) else t for t in st) for st in self.states]
            pos, shift = self.pos.clone(), self.shift.clone()
            s = torch.cuda.Stream(); s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(2): self._step()
            torch.cuda.current_stream().wait_stream(s)
            self._graph = torch.cuda.CUDAGraph()
            with graph_capture(self._graph):
                self.logits = self._step()
            for st, sv in zip(self.states, saved):           # warm-up and capture advanced the state: restore it
                for a, b in zip(st, sv):
                    if torch.is_tensor(a): a.copy_(b)
            self.pos.copy_(pos); self.shift.copy_(shift)
        self._graph.replay()
        return self.logits

    @staticmethod
    def sample(lg: torch.Tensor, temp: float, g: Optional[torch.Generator]):
        """Greedy at temp 0, else one draw from softmax(lg / temp) per row (src/bench.py:79-86); on device."""
        if temp == 0:
            return lg.argmax(-1)
        return torch.multinomial(torch.softmax(lg.float() / temp, -1), 1, generator=g).squeeze(-1)

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, n: int, temp: float = 0.0, seed: int = 0):
        """prompt_ids (B,Tp) -> sampled ids (B,n). With use_graph the draw, the bookkeeping and the model step of one token
        are a single CUDA-graph replay (no per-token work on the host besides the replay itself)."""
        lg = self.prefill(prompt_ids)
        if self.use_graph:
            return self._generate_graphed(lg, n, temp, seed)
        out = torch.zeros(self.B, max(n, 1), dtype=torch.long, device=self.dev)
        cnt = torch.zeros(1, dtype=torch.long, device=self.dev)
        ticket = torch.zeros(1, dtype=torch.int32, device=self.dev)
        nxt = torch.empty(self.B, dtype=torch.long, device=self.dev)
        for _ in range(n):                                   # the same draws as the graphed loop, launched one by one
            ops.decode_sample(lg, temp, seed, nxt, cnt, ticket, hist=out, min_p=self.min_p)
            lg = self.step(nxt)
        return out[:, :n]

    def _token_body(self, temp: float, seed: int):
        """Draw from the waiting logits, record the token at the running index, run the model on the token, leave the next
        logits waiting: a fixed kernel sequence, nothing on the host. The position and the rebase shift belong to the token
        being fed, so the draw kernel advances them for the PREVIOUS token (from the second token on) before the step."""
        ops.decode_sample(self._lg_in, temp, seed, self.tok, self._cnt, self._ticket, hist=self._hist, pos=self.pos,
                          shift=self.shift, ctx=self.w, min_p=self.min_p)
        if self._token_ok():
            self._step_token(advance=False, out=self._lg_in)  # the step writes the waiting logits itself
        else:
            self._lg_in.copy_(self._step(advance=False))

    def _generate_graphed(self, lg, n: int, temp: float, seed: int):
        key = (n, float(temp), int(seed), self.min_p)
        if getattr(self, "_gen_key", None) != key:
            V = lg.shape[-1]
            self._lg_in = torch.empty(self.B, V, dtype=torch.float32, device=self.dev)
            self._hist = torch.zeros(self.B, max(n, 4), dtype=torch.long, device=self.dev)   # the warm-up passes write three columns
            self._cnt = torch.zeros(1, dtype=torch.long, device=self.dev)
            self._ticket = torch.zeros(1, dtype=torch.int32, device=self.dev)
            self._lg_in.copy_(lg)
            saved = [tuple(t.clone() if torch.is_tensor(t) else t for t in st) for st in self.states]
            pos, shift = self.pos.clone(), self.shift.clone()
            s = torch.cuda.Stream(); s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(2): self._token_body(temp, seed)
            torch.cuda.current_stream().wait_stream(s)
            self._gen_graph = torch.cuda.CUDAGraph()
            with graph_capture(self._gen_graph):
                self._token_body(temp, seed)
            for st, sv in zip(self.states, saved):           # warm-up and capture advanced the state: restore it
                for a, b in zip(st, sv):
                    if torch.is_tensor(a): a.copy_(b)
            self.pos.copy_(pos); self.shift.copy_(shift)
            self._gen_key = key
        self._lg_in.copy_(lg)
        self._cnt.zero_()
        for _ in range(n):
            self._gen_graph.replay()
        if n > 0:                                            # the last token's step has not been followed by a draw
            self.shift.fill_(1.0)
            self.pos.copy_((self.pos + 1) % self.w)
        return self._hist[:, :n].clone()
