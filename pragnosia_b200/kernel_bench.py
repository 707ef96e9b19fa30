"""Each hand-written kernel alone on a fixed synthetic case: what bench.py times for its roofline entries and what the
ncu captures summarised under profiles/ run.

    python -m pragnosia_b200.kernel_bench NAME [--launches N] [--time]

NAME is one of CASES. Without --time it just launches the kernel N times (the form to put under ncu); with --time it
prints the CUDA-event time per launch (L2 flushed before each) and the achieved algorithmic GB/s.
"""
from __future__ import annotations

import argparse
import sys

import torch

from . import _lib, ops, synth


def _prefill(B, H, T, D, fused=False):
    dev = "cuda"
    x = synth.assoc_op_inputs(B, H, T, D, seed=1, with_state=True)
    q, k, v = (x[n].to(dev).to(torch.bfloat16) for n in "qkv")
    la, S0 = x["la"].to(dev), x["S0"].to(dev)
    alg = B * H * T * (4 * D * 2 + 4) + 2 * B * H * D * D * 4          # q,k,v,o bf16 + log-decay; state in and out
    return (lambda: ops.prefill(q, k, v, la, None, S0, precision=_lib.PREFILL_TENSOR)), alg


def _layer_prefill(B, H, T, D):
    """The fused between-GEMMs kernel on raw projection views (what LM.forward_carried launches per layer-window)."""
    dev = "cuda"
    d = H * D
    ld = (3 * d + 2 * H + 7) // 8 * 8
    proj = torch.randn(B, T, ld, device=dev, dtype=torch.bfloat16)
    qp, kp, vp = (proj[..., i * d:(i + 1) * d].unflatten(-1, (H, D)) for i in range(3))
    th = synth.rope_theta(H, D).to(dev)
    table = ops.rot_table(th, (T + 63) // 64 * 64)
    A, w = torch.zeros(H, device=dev) - 3, torch.ones(D, device=dev)
    S = torch.randn(B, H, D, D, device=dev) * 0.1
    alg = B * H * T * (4 * D * 2 + 4) + 2 * B * H * D * D * 4          # q,k,v,o bf16 + two bf16 gate logits; state in and out
    fn = lambda: ops.layer_prefill(qp, kp, vp, proj[..., 3 * d + H:3 * d + 2 * H], proj[..., 3 * d:3 * d + H], A, table, S,
                                   theta=th, shift=float(T), rms_weight=w, rms_eps=1e-6, S_out=S)
    return fn, alg


def _prefill_delta(B, H, T, D, on_device=False):
    dev = "cuda"
    if on_device:                                                     # the same distributions drawn on the GPU (a full-size case)
        g = torch.Generator(device=dev).manual_seed(1)
        r = lambda *shape: torch.randn(*shape, generator=g, device=dev)
        q, k, v = r(B, H, T, D).to(torch.bfloat16), torch.nn.functional.normalize(r(B, H, T, D), dim=-1).to(torch.bfloat16), r(B, H, T, D).to(torch.bfloat16)
        la, be, S0 = torch.nn.functional.logsigmoid(r(B, H, T) + 2.0), torch.sigmoid(r(B, H, T)), r(B, H, D, D) * 0.1
    else:
        x = synth.assoc_op_inputs(B, H, T, D, seed=1, delta=True, with_state=True)
        q, k, v = (x[n].to(dev).to(torch.bfloat16) for n in "qkv")
        la, be, S0 = x["la"].to(dev), x["beta"].to(dev), x["S0"].to(dev)
    alg = B * H * T * (4 * D * 2 + 8) + 2 * B * H * D * D * 4
    return (lambda: ops.prefill(q, k, v, la, be, S0)), alg


def _prep(B, T, H, D):
    dev = "cuda"
    d = H * D
    proj = torch.randn(B, T, 3 * d + 2 * H, device=dev, dtype=torch.bfloat16)
    views = [proj[..., i * d:(i + 1) * d].unflatten(-1, (H, D)) for i in range(3)]
    th, pos = synth.rope_theta(H, D).to(dev), torch.arange(T, device=dev)
    gate = proj[..., 3 * d + H:3 * d + 2 * H]
    return (lambda: ops.prep(*views, gate, th, pos)), B * T * H * D * 2 * 6


def _decode(B, H, D, delta=False):
    dev = "cuda"
    d = H * D
    S = torch.randn(B, H, D, D, device=dev) * 0.1
    row = torch.randn(B, 3 * d + 2 * H, device=dev, dtype=torch.bfloat16)
    vs = [row[:, i * d:(i + 1) * d].unflatten(1, (H, D)) for i in range(3)]
    A, th = torch.zeros(H, device=dev) - 5, synth.rope_theta(H, D).to(dev)
    fn = lambda: ops.decode_step(*vs, row[:, 3 * d:3 * d + H], S, th, gate=row[:, 3 * d + H:], decay_A=A, shift=1.0, S_out=S,
                                 delta=delta)
    return fn, 2 * B * H * D * D * 4 + B * H * D * 2 * 4               # state read + write, q,k,v in and o out (bf16)


def _lambda(B, T, D, bcast=False):
    dev = "cuda"
    xs = synth.lambda_scan_inputs(B, T, D, seed=4, per_channel_angle=bcast)
    u, lm = xs["u"].to(dev), xs["logmag"].to(dev)
    an = xs["ang"][0, 0].contiguous().to(dev).expand(B, T, D) if bcast else xs["ang"].to(dev)
    return (lambda: ops.lambda_scan(u, lm, an)), u.numel() * (12 if bcast else 16)


def _add_norm(rows, d):
    dev = "cuda"
    x = torch.randn(rows, d, device=dev, dtype=torch.bfloat16); dl = torch.randn_like(x)
    n = torch.nn.RMSNorm(d).to(dev).to(torch.bfloat16)
    return (lambda: ops.add_norm(x, dl, n)), rows * d * 2 * 4


CASES = {
    # name: (builder, what it is)
    "prefill": (lambda: _prefill(64, 12, 1024, 64), "aspin chunked prefill, plain rule, tensor cores: B64 H12 T1024 D64 bf16"),
    "prefill_cfg1": (lambda: _prefill(16, 12, 512, 64), "the same at one configuration-1 window: B16 H12 T512 D64"),
    "prefill_d128": (lambda: _prefill(8, 16, 2048, 128), "the same at head dim 128: B8 H16 T2048 D128"),
    "layer_prefill": (lambda: _layer_prefill(64, 12, 1024, 64), "fused layer prefill on raw projections (plumbing + scan + norm): B64 H12 T1024 D64"),
    "layer_prefill_cfg1": (lambda: _layer_prefill(16, 12, 512, 64), "the same at one configuration-1 window: B16 H12 T512 D64"),
    "prefill_delta": (lambda: _prefill_delta(8, 16, 1024, 128), "delta-rule chunked prefill, tensor cores: B8 H16 T1024 D128 bf16 I/O"),
    "prefill_delta_d64": (lambda: _prefill_delta(16, 12, 1024, 64), "the same at head dim 64: B16 H12 T1024 D64"),
    "prefill_delta_cfg3": (lambda: _prefill_delta(8, 16, 8192, 128, on_device=True), "configuration 3 at full size: B8 H16 T8192 D128 bf16 I/O"),
    "prep": (lambda: _prep(16, 512, 12, 64), "normalise / gate / rotate / transpose: B16 T512 H12 D64 bf16"),
    "decode": (lambda: _decode(64, 12, 64), "fused recurrent decode step, plain rule, in place: B64 H12 D64"),
    "decode_delta": (lambda: _decode(64, 12, 64, True), "fused recurrent decode step, delta rule, in place: B64 H12 D64"),
    "decode_b1024": (lambda: _decode(1024, 12, 64), "the plain-rule step at a batch whose state (403 MB) exceeds L2: B1024 H12 D64"),
    "lambda": (lambda: _lambda(64, 1024, 768), "per-token lambda scan, per-token angle: B64 T1024 D768 fp32"),
    "lambda_bcast": (lambda: _lambda(64, 1024, 768, True), "per-token lambda scan, one angle per channel: B64 T1024 D768 fp32"),
    "add_norm": (lambda: _add_norm(8192, 768), "residual add + RMS norm: 8192 rows of 768 bf16"),
    "mlp_up": (lambda: _linear_act(8192, 768, 3072), "MLP up-projection + bias + erf-GELU as one tensor-core GEMM: M8192 K768 N3072 bf16"),
    "mlp_up_pair": (lambda: _linear_act(8192, 768, 3072, variant=1), "the same GEMM with a 256 x 256 tile per pair of SMs (two-CTA cluster, cta_group::2)"),
    "skinny": (lambda: _skinny(1, 768, 3072), "decode-step linear (add + RMS norm + linear + GELU) at batch 1: K768 N3072 bf16"),
    "batch_linear": (lambda: _batch_linear(64, 768, 2328), "decode-step linear for 64 rows on the tensor cores (bias): K768 N2328 bf16"),
    "decode_token": (lambda: _decode_token(1), "the whole decode step of the configuration-2 model as one launch, batch 1 (12 layers, d768, vocabulary 8192)"),
    "decode_token_b4": (lambda: _decode_token(4), "the same at batch 4"),
}

# floating-point operations per launch of the cases that are bound by the tensor pipe rather than by HBM
FLOPS = {"mlp_up": 2 * 8192 * 768 * 3072, "mlp_up_pair": 2 * 8192 * 768 * 3072}


def _linear_act(M, K, N, variant=0):
    dev = "cuda"
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    W = (torch.randn(N, K, device=dev) * K ** -0.5).to(torch.bfloat16)
    b = torch.randn(N, device=dev).to(torch.bfloat16)

    def fn():
        if variant:                                                   # the process-wide switch, put back after the launch
            _lib.check(_lib.lib().pgb_linear_act_set_variant(variant), "pgb_linear_act_set_variant")
        try:
            return ops.linear_act(x, W, b, act="gelu")
        finally:
            if variant:
                _lib.check(_lib.lib().pgb_linear_act_set_variant(0), "pgb_linear_act_set_variant")
    return fn, (M * K + N * K + N + M * N) * 2


def _skinny(B, K, N):
    dev = "cuda"
    x, dl = (torch.randn(B, K, device=dev).to(torch.bfloat16) for _ in range(2))
    W = (torch.randn(N, K, device=dev) * K ** -0.5).to(torch.bfloat16)
    b = torch.randn(N, device=dev).to(torch.bfloat16)
    norm = torch.nn.RMSNorm(K).to(dev).to(torch.bfloat16)
    return (lambda: ops.skinny_linear(x, W, b, delta=dl, norm=norm, act="gelu")), (N * K + N + 3 * B * K + B * N) * 2


def _batch_linear(B, K, N):
    dev = "cuda"
    x = torch.randn(B, K, device=dev).to(torch.bfloat16)
    W = (torch.randn(N, K, device=dev) * K ** -0.5).to(torch.bfloat16)
    b = torch.randn(N, device=dev).to(torch.bfloat16)
    return (lambda: ops.batch_linear(x, W, b)), (N * K + N + B * K + B * N) * 2


def _decode_token(B):
    """One token through Decoder._step_token: the launch reads every weight once (the embedding table as the head) and
    reads and writes every layer's state."""
    from .generate import Decoder
    from .model import LM
    dev = "cuda"
    torch.manual_seed(0)
    m = LM(vocab=8192, d=768, layers=12, mlp_mult=4, ctx=512, mixer="aspin", norm="rms").to(dev).to(torch.bfloat16).eval()
    dec = Decoder(m, batch=B, use_graph=False)
    with torch.no_grad():
        dec.prefill(synth.token_ids(B, 64, 8192, seed=7).to(dev))
    tok = torch.zeros(B, dtype=torch.long, device=dev)
    assert dec._token_ok()
    weights = sum(p.numel() for n, p in m.named_parameters() if not n.startswith("p.")) * 2
    dec.tok.copy_(tok.view(B, 1))
    return (lambda: dec._step_token(advance=False)), weights + 2 * B * 12 * 12 * 64 * 64 * 4


def time_case(name: str, iters: int = 20, flush_mb: int = 256):
    """(microseconds per launch, algorithmic bytes) with the L2 flushed before every timed launch."""
    fn, alg = CASES[name][0]()
    flush = torch.empty(flush_mb << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    tot = 0.0
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record(); b.synchronize()
        tot += a.elapsed_time(b)
    return tot / iters * 1e3, alg


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("name", choices=sorted(CASES) + ["all"])
    ap.add_argument("--launches", type=int, default=2)
    ap.add_argument("--time", action="store_true")
    a = ap.parse_args(argv)
    names = sorted(CASES) if a.name == "all" else [a.name]
    with torch.no_grad():
        for n in names:
            if a.time:
                us, alg = time_case(n)
                print(f"{n:14s} {us:9.1f} us/launch  {alg / us / 1e3:8.0f} GB/s algorithmic   ({CASES[n][1]})")
            else:
                fn, _ = CASES[n][0]()
                for _ in range(a.launches):
                    fn()
                torch.cuda.synchronize()
                print(f"{n}: {a.launches} launches done")


if __name__ == "__main__":
    main()
