"""The language model around the carrier layers: same constructor arguments, parameter names and carried-state
interface as the reference's src/model.py LM (:621-864), restricted to the pure-carrier mixers (aspin, dspin, hspin,
hdspin, fspin). Attention controls, hybrids, growth and the training loss are other subsystems and are not here."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from ._lib import graph_capture
from .assoc import AssocCarrier
from .spin import SpinCarrier


class MLP(nn.Module):
    """norm -> Linear(mult*d) -> GELU -> Linear(d), residual (src/model.py:552-560)."""

    def __init__(self, d: int, mult: int = 4):
        super().__init__()
        self.n = nn.LayerNorm(d)
        self.a = nn.Linear(d, mult * d)
        self.b = nn.Linear(mult * d, d)

    def forward(self, x):
        return x + self.ff(self.n(x))

    fused_up = True     # bf16 on CUDA: Linear(d, mult*d) + GELU as one tensor-core GEMM with the activation in its epilogue

    def ff(self, z):
        """The block without its norm and residual add."""
        if (self.fused_up and z.is_cuda and z.dtype == torch.bfloat16 and self.a.weight.dtype == torch.bfloat16
                and z.shape[-1] % 8 == 0 and self.a.weight.shape[0] % 8 == 0 and z.numel() // z.shape[-1] >= 128):
            return self.b(ops.linear_act(z, self.a.weight, self.a.bias, act="gelu"))
        return self.b(F.gelu(self.a(z)))


_MIXERS = {
    "aspin": lambda d: AssocCarrier(d), "dspin": lambda d: AssocCarrier(d, delta=True),
    "hspin": lambda d: AssocCarrier(d, head_dim=128), "hdspin": lambda d: AssocCarrier(d, delta=True, head_dim=128),
    "fspin": lambda d: SpinCarrier(d, gated="rf"),
}


class LM(nn.Module):
    def __init__(self, vocab=8192, d=768, layers=12, mlp_mult=4, ctx=512, mixer="aspin", norm="ln"):
        super().__init__()
        if mixer not in _MIXERS:
            raise NotImplementedError(f"mixer {mixer!r}: only the pure-carrier mixers {sorted(_MIXERS)} are built here")
        self.vocab, self.d, self.layers, self.ctx, self.mixer, self.norm = vocab, d, layers, ctx, mixer, norm
        self.wavefront = True                                # graphed forward_carried: consecutive windows a layer apart on separate streams
        self.wavefront_streams = 4
        self.e = nn.Embedding(vocab, d)
        self.p = nn.Embedding(ctx, d)
        self.mix = nn.ModuleList([_MIXERS[mixer](d) for _ in range(layers)])
        self.mlp = nn.ModuleList([MLP(d, mlp_mult) for _ in range(layers)])
        self.n = nn.LayerNorm(d)
        self.use_graphs = True          # CUDA: replay one captured graph per window in forward_carried
        self._graphs = {}
        self._graphs_stamp = None
        if norm == "rms":                      # every residual-stream LayerNorm becomes an RMSNorm of the same width
            for mod in list(self.modules()):
                for nm, child in list(mod.named_children()):
                    if isinstance(child, nn.LayerNorm):
                        setattr(mod, nm, nn.RMSNorm(child.normalized_shape[0]))
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Embedding, nn.Linear)):
            nn.init.normal_(m.weight, 0.0, 0.02)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)

    def weights_stamp(self):
        """Changes whenever a captured graph of this model would compute with something stale: a parameter that moved
        (another dtype or device) or a mixer whose derived constants must be rebuilt (an in-place update, load_state_dict)."""
        ptrs = tuple(p.data_ptr() for p in self.parameters())
        return ptrs, tuple(mx.consts_key() for mx in self.mix if isinstance(mx, AssocCarrier))

    def _embed(self, x):
        return self.e(x) + self.p(torch.arange(x.shape[1], device=x.device) % self.p.num_embeddings)

    @staticmethod
    def _add_norm(x, delta, norm):
        """y = x + delta, z = norm(y) in one kernel where the row length allows it; else the two torch ops."""
        d = x.shape[-1]
        lim = (2048, 8) if x.dtype == torch.bfloat16 else (1024, 4)
        if x.dtype in (torch.bfloat16, torch.float32) and d <= lim[0] and d % lim[1] == 0 and not torch.is_grad_enabled():
            return ops.add_norm(x, delta, norm)
        y = x if delta is None else x + delta
        return y, norm(y)

    def _layers(self, h, states):
        """Every (mixer, MLP) pair over h. Returns (x, delta): the residual stream and the last block's not-yet-added
        output, so the caller's final norm fuses that add as well. Each block's input norm is fused with the previous
        block's residual add."""
        x, delta = h, None
        for i, (mx, mp) in enumerate(zip(self.mix, self.mlp)):
            x, z = self._add_norm(x, delta, mx.ln)
            delta, states[i] = mx.mix(z, states[i])
            x, z = self._add_norm(x, delta, mp.n)
            delta = mp.ff(z)
        return x, delta

    def trunk(self, x, states=None, carry=False):
        """Everything but the output head; with carry=True also takes / returns the per-layer states."""
        new = list(states) if states is not None else [None] * self.layers
        h = self._add_norm(*self._layers(self._embed(x), new), self.n)[1]
        return (h, new) if carry else h

    def forward(self, x, return_hidden=False):
        h = self.trunk(x)
        logits = F.linear(h, self.e.weight)
        return (logits, h) if return_hidden else logits

    @torch.no_grad()
    def forward_carried(self, x, window=None, return_states=False):
        """A sequence longer than ctx, window by window with the carrier state carried; logits of the FINAL window only
        (src/model.py:843-864). The head runs once, on the last window (the reference computes and discards it for every
        window). On CUDA, with use_graphs set and whole windows, each window pass is one CUDA-graph replay."""
        window = window or self.ctx
        B, T = x.shape
        if self.use_graphs and x.is_cuda and T % window == 0 and T >= window:
            # A captured graph holds the addresses of the parameters and of the constants the mixers derive from them
            # (the concatenated projection weight, the gated output weight): any change of either retires every graph.
            stamp = self.weights_stamp()
            if stamp != self._graphs_stamp:
                self._graphs.clear()
                self._graphs_stamp = stamp
            nw = T // window
            if self.wavefront and nw >= 2 and all(isinstance(mx, AssocCarrier) for mx in self.mix):
                # every window of the call in ONE graph, consecutive windows on two streams a layer apart
                key = (B, window, nw, x.device, self.e.weight.dtype)
                run = self._graphs.get(key)
                if run is None:
                    run = self._graphs[key] = _StepGraph(self, B, window, nw, x.device)
                last = run(x)
            else:
                key = (B, window, x.device, self.e.weight.dtype)
                run = self._graphs.get(key)
                if run is None:
                    run = self._graphs[key] = _WindowGraphs(self, B, window, x.device)
                last = None
                for s in range(0, T, window):
                    last = run(x[:, s:s + window], first=(s == 0))
            states = run.states
        else:
            states = [None] * self.layers
            last = None
            for s in range(0, T, window):
                last = self._layers(self._embed(x[:, s:s + window]), states)
        logits = F.linear(self._add_norm(*last, self.n)[1], self.e.weight)
        return (logits, states) if return_states else logits


class _StepGraph:
    """ONE CUDA graph of a whole multi-window pass, with consecutive windows on separate streams. Window w + 1 needs from
    window w only each layer's carried state, so it can run one layer behind it instead of after it: layer l of window
    w + 1 waits for the event recorded after layer l of window w. The two windows' kernels then share the GPU -- the
    half-empty second wave of one window's prefill kernel (192 one-per-SM CTAs on 148 SMs) is filled by the other
    window's GEMM tiles. Same kernels in the same order along every dependency chain: results are those of the
    window-by-window pass to the bit. The reference runs the windows one after the other, eagerly (src/model.py:857-863)."""

    def __init__(self, model, B, Tw, NW, device):
        self.m, self.B, self.Tw, self.NW = model, B, Tw, NW
        self.ids = torch.zeros(B, Tw * NW, dtype=torch.long, device=device)
        self.sides = [torch.cuda.Stream(device=device) for _ in range(min(NW, model.wavefront_streams) - 1)]
        self.graph = None
        self.states = None
        self.out = None

    def _pass(self):
        m, main = self.m, torch.cuda.current_stream()
        streams = [main] + self.sides
        states = [None] * m.layers
        fork = torch.cuda.Event(); fork.record(main)
        for sd in self.sides:
            sd.wait_event(fork)
        prev, out = None, None
        try:
            for w in range(self.NW):
                st = streams[w % len(streams)]
                evs = [torch.cuda.Event() for _ in range(m.layers)]
                for mx in m.mix:
                    mx.inplace_state = w > 0                           # later windows update the first window's state tensors
                with torch.cuda.stream(st):
                    x, delta = m._embed(self.ids[:, w * self.Tw:(w + 1) * self.Tw]), None
                    for i, (mx, mp) in enumerate(zip(m.mix, m.mlp)):
                        x, z = m._add_norm(x, delta, mx.ln)
                        if prev is not None:
                            st.wait_event(prev[i])                     # the state this layer enters with
                        delta, states[i] = mx.mix(z, states[i])
                        evs[i].record(st)
                        x, z = m._add_norm(x, delta, mp.n)
                        delta = mp.ff(z)
                    out = (x, delta)
                prev = evs
            for sd in self.sides:
                join = torch.cuda.Event(); join.record(sd); main.wait_event(join)
        finally:
            for mx in m.mix:
                mx.inplace_state = False
        return out, states

    def __call__(self, ids):
        if self.graph is None:
            warm = torch.cuda.Stream()
            warm.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(warm):                              # warm-up: library workspaces, cached constants
                self._pass()
            torch.cuda.current_stream().wait_stream(warm)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with graph_capture(self.graph):
                self.out, self.states = self._pass()
        self.ids.copy_(ids)
        self.graph.replay()
        return self.out


class _WindowGraphs:
    """Two CUDA graphs of one window pass (embedding and every layer over a static (B,Tw) block of ids): one for a
    sequence's first window (no entering state) and one for every later window, which updates the per-layer state
    buffers in place. The reference runs this loop eagerly (src/model.py:857-863); at small batch it is launch-bound."""

    def __init__(self, model, B, Tw, device):
        self.m, self.B, self.Tw = model, B, Tw
        self.ids = torch.zeros(B, Tw, dtype=torch.long, device=device)
        self.states = None
        self.first = self.later = None
        self.out_first = self.out_later = None

    def _pass(self, states, inplace):
        m = self.m
        for mx in m.mix:
            if isinstance(mx, AssocCarrier):
                mx.inplace_state = inplace
        try:
            new = list(states)
            out = m._layers(m._embed(self.ids), new)
            if inplace:                        # states that came back as new tensors (the diagonal carrier) are copied home
                for old, cur in zip(states, new):
                    for a, b in zip(old, cur):
                        if torch.is_tensor(a) and a.data_ptr() != b.data_ptr():
                            a.copy_(b)
            return out, new
        finally:
            for mx in m.mix:
                if isinstance(mx, AssocCarrier):
                    mx.inplace_state = False

    def _capture(self):
        none = [None] * self.m.layers
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                                  # warm-up: library workspaces, cached constants
            _, st = self._pass(none, False)
            self._pass(st, True)
        torch.cuda.current_stream().wait_stream(side)
        self.first = torch.cuda.CUDAGraph()
        with graph_capture(self.first):
            self.out_first, self.states = self._pass(none, False)
        self.later = torch.cuda.CUDAGraph()
        with graph_capture(self.later, pool=self.first.pool()):
            self.out_later, _ = self._pass(self.states, True)

    def __call__(self, ids, first):
        if self.first is None:
            self._capture()
        self.ids.copy_(ids)
        if first:
            self.first.replay()
            return self.out_first
        self.later.replay()
        return self.out_later
