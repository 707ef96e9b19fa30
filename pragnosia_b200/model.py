"""The language model around the carrier layers: same constructor arguments, parameter names and carried-state
interface as the reference's src/model.py LM (:621-864), restricted to the pure-carrier mixers (aspin, dspin, hspin,
hdspin, fspin). Attention controls, hybrids, growth and the training loss are other subsystems and are not here."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

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
        return x + self.b(F.gelu(self.a(self.n(x))))


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
        self.e = nn.Embedding(vocab, d)
        self.p = nn.Embedding(ctx, d)
        self.mix = nn.ModuleList([_MIXERS[mixer](d) for _ in range(layers)])
        self.mlp = nn.ModuleList([MLP(d, mlp_mult) for _ in range(layers)])
        self.n = nn.LayerNorm(d)
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

    def _embed(self, x):
        return self.e(x) + self.p(torch.arange(x.shape[1], device=x.device) % self.p.num_embeddings)

    def _layers(self, h, states):
        for i, (mx, mp) in enumerate(zip(self.mix, self.mlp)):
            h, states[i] = mx(h, states[i])
            h = mp(h)
        return h

    def trunk(self, x, states=None, carry=False):
        """Everything but the output head; with carry=True also takes / returns the per-layer states."""
        new = list(states) if states is not None else [None] * self.layers
        h = self.n(self._layers(self._embed(x), new))
        return (h, new) if carry else h

    def forward(self, x, return_hidden=False):
        h = self.trunk(x)
        logits = F.linear(h, self.e.weight)
        return (logits, h) if return_hidden else logits

    @torch.no_grad()
    def forward_carried(self, x, window=None, return_states=False):
        """A sequence longer than ctx, window by window with the carrier state carried; logits of the FINAL window only
        (src/model.py:843-864). The head runs once, on the last window (the reference computes and discards it for every
        window)."""
        window = window or self.ctx
        states = [None] * self.layers
        h = None
        for s in range(0, x.shape[1], window):
            h = self._layers(self._embed(x[:, s:s + window]), states)
        logits = F.linear(self.n(h), self.e.weight)
        return (logits, states) if return_states else logits
