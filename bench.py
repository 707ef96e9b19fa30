#!/usr/bin/env python
"""Headline benchmark: aspin LM prefill tok/s (configuration 1) with decode ms/token and per-kernel roofline beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Product arm (default). One step = LM.forward_carried over B=16 sequences of 2048 synthetic token ids per GPU, as four
carried 512-token windows, on the random-init d768 / 12-layer / 12x64-head aspin LM with bf16 weights and fp32 state.
Sequences are independent, so N GPUs run N such batches (weak scaling, no collective on the data path). Prints ONE JSON
line on rank 0: `value` = tokens/s over all GPUs with inputs resident in HBM, timed per step with CUDA events on the
launching stream (L2 flushed between steps), max over ranks; `e2e` = the same call with token ids coming from pinned
host memory and the returned logits copied back, both copies inside the timed region; `roofline` = the chunked-prefill
kernel alone at the workload's shape; `cpu_baseline` = the CPU oracle's forward_carried on a bounded sample of the same
workload, timed on this host; `decode` = configuration 2 (ms/token at batch 1 and 64 and the state kernel's HBM GB/s).

Everything a reader of the line needs is nested under keys the line always carries: `roofline.kernels` (each hand-written
kernel alone on its kernel_bench case), `roofline.decode` (configuration 2: ms/token at batch 1 and 64, the state kernel's
GB/s), `roofline.cfg4` (configuration 4, the long-context scan + prefill split by batch over the ranks: compute only, with
every output gathered, and with only what a sharded consumer needs gathered).

Reference arm (--impl reference). The reference's CPU implementation of the path as restated in oracle/ (a Python
reference cannot travel with a prebuilt library), with all host threads; each step is the bounded sample named in
`cpu_baseline.sample`.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG = dict(vocab=8192, d=768, layers=12, mlp_mult=4, ctx=512, mixer="aspin", norm="rms")
B_PER_GPU, T_TOTAL, WINDOW = 16, 2048, 512
CPU_SAMPLE_B, CPU_SAMPLE_T = 2, 2048
WORKLOAD = "cfg1: aspin LM prefill d768 L12 H12x64 V8192, B=16 x T=2048 per GPU as four carried 512-token windows"


PROFILE_FOR_TRAFFIC = ROOT / "profiles" / "prefill_tc_layer_B64_H12_T1024_D64.md"


def profiled_traffic():
    """(DRAM bytes per launch of the fused layer prefill at B64 H12 T1024 D64, where that figure is kept): read + write as
    one ncu capture measured them, taken from the tracked summary of that capture rather than typed in here."""
    import re
    try:
        text = PROFILE_FOR_TRAFFIC.read_text()
        rd = re.search(r"\| DRAM read \| ([0-9.]+) ([KMG])byte", text)
        wr = re.search(r"\| DRAM write \| ([0-9.]+) ([KMG])byte", text)
        mult = {"K": 1e3, "M": 1e6, "G": 1e9}
        return float(rd.group(1)) * mult[rd.group(2)] + float(wr.group(1)) * mult[wr.group(2)], str(PROFILE_FOR_TRAFFIC.relative_to(ROOT))
    except Exception:
        return None, None


def tc_error_flag() -> int:
    """The device-side flag a bounded wait inside a tensor-core kernel sets when it runs out (0 = healthy)."""
    import ctypes
    from pragnosia_b200 import _lib
    out = ctypes.c_int(-1)
    _lib.check(_lib.lib().pgb_tc_error_flag(ctypes.byref(out)), "pgb_tc_error_flag")
    return out.value


def require_healthy(leg: str):
    code = tc_error_flag()
    if code != 0:
        raise SystemExit(f"bench.py: a bounded wait inside a tensor-core kernel ran out during the {leg} leg (code {code}); "
                         "its results are not to be trusted")


def bind_to_gpu_numa_node(index: int):
    """Best effort: run this rank on the CPUs of its GPU's NUMA node, so the pinned host buffers it allocates next are local
    to the GPU's PCIe root (eight ranks copying 134 MB of logits each otherwise share one socket's links)."""
    try:
        props = torch.cuda.get_device_properties(index)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        node = int(Path(f"/sys/bus/pci/devices/{bus}/numa_node").read_text())
        if node < 0:
            return None
        cpus = []
        for part in Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip().split(","):
            a, _, b = part.partition("-")
            cpus.extend(range(int(a), int(b or a) + 1))
        allowed = sorted(set(cpus) & os.sched_getaffinity(0))
        if allowed:
            os.sched_setaffinity(0, allowed)
            return node
    except Exception:
        pass
    return None


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), tflops=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    tflops_burst=float(d["bf16_tflops"]), src="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_burst=1590.0, src="fallback")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows = []; self.proc = None; self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.25)
        self.proc.terminate()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


# ------------------------------------------------------------------------------------------------------------------
def cpu_reference_time(steps: int, warmup: int):
    """The CPU oracle's forward_carried on the bounded sample; returns (tok/s, seconds per step, threads)."""
    import oracle
    from pragnosia_b200 import synth
    torch.set_num_threads(os.cpu_count() or 1)
    cfg = oracle.lm_config(**CFG)
    P = oracle.init_lm_params(cfg, seed=0)
    ids = synth.token_ids(CPU_SAMPLE_B, CPU_SAMPLE_T, CFG["vocab"], seed=1)
    times = []
    with torch.no_grad():
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            oracle.lm_forward_carried(P, cfg, ids, WINDOW)
            if i >= warmup:
                times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return CPU_SAMPLE_B * CPU_SAMPLE_T / sec, sec, torch.get_num_threads()


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    toks, sec, threads = cpu_reference_time(args.steps, args.warmup)
    sample = (f"B={CPU_SAMPLE_B} x T={CPU_SAMPLE_T} of the same LM and window (the path is linear in B*T), fp32, "
              f"torch CPU with {threads} threads")
    print(json.dumps({
        "impl": "reference", "metric": "aspin_lm_prefill_tokens_per_s", "value": toks, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": toks, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": toks, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------------------------------
def event_time_ms(fn, iters: int, flush=None):
    """Average CUDA-event time of fn() over iters calls on the current stream, L2 flushed before each."""
    tot = 0.0
    for _ in range(iters):
        if flush is not None:
            flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record(); b.synchronize()
        tot += a.elapsed_time(b)
    return tot / iters


def product_arm(args):
    import torch.distributed as dist
    from pragnosia_b200 import ops, synth
    from pragnosia_b200.model import LM

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product arm has no CPU path (use --impl reference for the CPU timing)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = bind_to_gpu_numa_node(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    model = LM(**CFG).to(dev).to(torch.bfloat16).eval()
    model.use_graphs = not args.eager
    ids_host = synth.token_ids(B_PER_GPU, T_TOTAL, CFG["vocab"], seed=1 + rank).pin_memory()
    ids = ids_host.to(dev)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flush = lambda: flush_buf.zero_()

    def step():
        return model.forward_carried(ids, WINDOW)

    copy_stream = torch.cuda.Stream(device=dev)

    def step_e2e(out_host):
        """ids from pinned host memory in, logits back to pinned host memory: the upload and the pass on the compute stream,
        the 134 MB read-back on a copy stream so that it overlaps the next step's compute (two host buffers alternate)."""
        x = ids_host.to(dev, non_blocking=True)
        lg = model.forward_carried(x, WINDOW)
        copy_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(copy_stream):
            out_host.copy_(lg, non_blocking=True)
        lg.record_stream(copy_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            step()
        sampler = ClockSampler(local); sampler.start()
        barrier()
        ms = []
        for _ in range(args.steps):
            flush()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); step(); b.record(); b.synchronize()
            ms.append(a.elapsed_time(b))
        barrier()
        clocks = sampler.stop()
        ms_step = sum(ms) / len(ms)
        # end to end: host ids in, logits out; wall clock from the first upload to the last byte of the last read-back
        outs = [torch.empty(B_PER_GPU, WINDOW, CFG["vocab"], dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        out_host = outs[0]
        for i in range(2):
            step_e2e(outs[i % 2])
        copy_stream.synchronize()
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            step_e2e(outs[i % 2])
        copy_stream.synchronize()
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    require_healthy("prefill step")
    t = torch.tensor([ms_step, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step, e2e_ms = t.tolist()
    tokens = world * B_PER_GPU * T_TOTAL
    result = {
        "metric": "aspin_lm_prefill_tokens_per_s", "value": tokens / (ms_step * 1e-3), "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "params_m": round(sum(p.numel() for p in model.parameters()) / 1e6, 2),
                   "state": "fp32", "l2": "flushed between timed steps (256 MiB write); weights 184 MB > L2",
                   "parallelism": f"batch-sharded x{world}, no data-path collective",
                   "host_numa_node": numa},
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": ids_host.numel() * 8,
                "d2h_bytes_per_step": out_host.numel() * 2},
        # this library's kernels per step: per window and layer one fused prefill, one fused up-projection GEMM and two
        # add+norm, plus the final norm before the head
        "gpu_launches": args.steps * ((T_TOTAL // WINDOW) * CFG["layers"] * 4 + 1),
        "clocks": clocks,
    }
    if args.step_only:
        if rank == 0:
            print(json.dumps(result))
    else:
        pk = peaks()
        roof = {}
        if rank == 0 and world == 1:
            with torch.no_grad():
                roof, kernels = kernel_rooflines(pk)
                roof["kernels"] = kernels
                require_healthy("per-kernel")
                roof["decode"] = decode_numbers(model, dev, pk, args)
                require_healthy("decode")
        # configuration 4 needs every rank (its gather is a collective): release the language model first
        del model, step, step_e2e, outs, out_host
        torch.cuda.empty_cache()
        with torch.no_grad():
            cfg4 = long_context_numbers(args, rank, world, local, dev, pk)
        require_healthy("configuration-4")
        if rank == 0:
            roof["cfg4"] = cfg4
            if "kernel" not in roof:
                roof.update({"kernel": "see the one-GPU line: per-kernel figures do not depend on the number of ranks", "bound": "hbm",
                             "achieved": None, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": None, "traffic": None,
                             "peak_source": pk["src"]})
            result["roofline"] = roof
            if world == 1:
                toks, sec, threads = cpu_reference_time(3, 1)
                result["cpu_baseline"] = {"value": toks, "unit": "tok/s", "cores": threads, "kind": "port",
                                          "sample": f"oracle forward_carried, B={CPU_SAMPLE_B} x T={CPU_SAMPLE_T}, fp32, "
                                                    f"{sec:.2f} s per pass, best-effort all {threads} threads"}
            print(json.dumps(result))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def kernel_rooflines(pk):
    """Each hand-written kernel alone on its kernel_bench case: algorithmic bytes / CUDA-event time against the measured
    HBM copy bandwidth. The first entry is the kernel the timed step spends its carrier time in."""
    from pragnosia_b200 import kernel_bench as kb
    out = []
    for name in ("layer_prefill_cfg1", "layer_prefill", "prefill", "prefill_d128", "prefill_delta", "prefill_delta_d64", "prefill_delta_cfg3", "decode", "decode_b1024",
                 "decode_delta", "decode_token", "decode_token_b4", "batch_linear", "lambda", "lambda_bcast", "prep", "add_norm"):
        us, alg = kb.time_case(name)
        out.append(dict(kernel=name, what=kb.CASES[name][1], bound="hbm", achieved=alg / us / 1e3, peak=pk["hbm_gbs"], unit="GB/s",
                        frac=alg / us / 1e3 / pk["hbm_gbs"], us_per_launch=us, algorithmic_bytes=alg))
    for name, flops in kb.FLOPS.items():                              # the tensor-bound kernels against the measured GEMM rate
        us, alg = kb.time_case(name)
        out.append(dict(kernel=name, what=kb.CASES[name][1], bound="tensor", achieved=flops / us / 1e6, peak=pk["tflops_burst"],
                        unit="TFLOP/s", frac=flops / us / 1e6 / pk["tflops_burst"], us_per_launch=us, algorithmic_bytes=alg,
                        flops=flops))
    roof = dict(out[0])
    big, src = profiled_traffic()
    # the capture is of the same kernel on the larger-than-L2 case (64 x 12 x 1024 head-tokens); traffic grows with the
    # head-tokens a launch processes, so it is scaled by that ratio to the bench window (16 x 12 x 512)
    roof["traffic"] = None if big is None else big * (16 * 12 * 512) / (64 * 12 * 1024)
    roof["traffic_source"] = src
    roof["traffic_scaling"] = "captured at B64 H12 T1024 (> L2), scaled by head-tokens (x 1/8) to the bench window B16 H12 T512"
    roof["peak_source"] = pk["src"]
    roof["kernel"] = "prefill_tc_ws_kernel<RAW> (fused layer prefill, B16 H12 T512 D64, bf16 I/O)"
    return roof, out


def decode_numbers(model, dev, pk, args):
    """Configuration 2: 512-token prompt, then sampled steps (temperature 1, seeded) at batch 1 and 64; the state kernel alone
    at batch 64 beside them."""
    from pragnosia_b200 import kernel_bench as kb
    from pragnosia_b200 import synth
    from pragnosia_b200.generate import Decoder
    n = args.decode_steps
    res = {"steps": n, "prompt": 512, "unit": "ms/token"}
    for B in (1, 64):
        dec = Decoder(model, batch=B)
        prompt = synth.token_ids(B, 512, CFG["vocab"], seed=7).to(dev)
        dec.generate(prompt, n, temp=1.0, seed=0)                       # captures the per-token graph for this length
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); dec.generate(prompt, n, temp=1.0, seed=0); b.record(); b.synchronize()
        # the prompt pass is inside generate(); time it alone and subtract
        c, d = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c.record(); dec.prefill(prompt); d.record(); d.synchronize()
        ms_tok = (a.elapsed_time(b) - c.elapsed_time(d)) / n
        state_bytes = 2 * B * CFG["layers"] * 12 * 64 * 64 * 4
        res[f"b{B}_ms_per_token"] = ms_tok
        res[f"b{B}_state_rw_gbs_over_whole_step"] = state_bytes / ms_tok / 1e6
        res[f"b{B}_launches_per_token"] = dec.launches_per_token
    us, alg = kb.time_case("decode")
    res["state_kernel_b64"] = dict(us_per_launch=us, achieved_gbs=alg / us / 1e3, frac=alg / us / 1e3 / pk["hbm_gbs"], peak_gbs=pk["hbm_gbs"])
    res["weight_stream_floor_ms"] = 184e6 / (pk["hbm_gbs"] * 1e9) * 1e3
    return res


CFG4 = dict(B=64, T=32768, H=12, D=64, DS=768, window=4096)


def long_context_numbers(args, rank, world, local, dev, pk, steps=None):
    """Configuration 4: the fspin per-token lambda scan (B=64, T=32768, D=768 complex channels, fp32) and the aspin prefill
    (B=64, T=32768, H=12, d=64, bf16), partitioned by batch over the ranks (STRONG scaling: the whole job is fixed), walked
    in 4096-token windows with the state carried. Timed three ways: compute only; with every window's output all-gathered
    over NVLink behind a side stream while the next window computes (the scan's output sent as bf16); and as a sharded
    consumer needs it -- outputs stay where they are, the final states and the last window's outputs are gathered."""
    import math
    import torch.distributed as dist
    import torch.nn.functional as F
    from pragnosia_b200 import ops, sharded, synth, _lib

    c = CFG4
    steps = steps or max(2, min(args.steps, 3))
    b0, b1 = sharded.shard_range(c["B"], rank, world)
    Bl = b1 - b0
    g = torch.Generator(device=dev).manual_seed(4 + rank)
    rn = lambda *sh: torch.randn(*sh, device=dev, generator=g)
    theta = synth.rope_theta(c["H"], c["D"]).to(dev)
    pos = torch.arange(c["T"], device=dev, dtype=torch.float32) % c["window"]
    q = ops.rotate(rn(Bl, c["H"], c["T"], c["D"]), theta, pos).to(torch.bfloat16)
    k = ops.rotate(F.normalize(rn(Bl, c["H"], c["T"], c["D"]), dim=-1), theta, pos).to(torch.bfloat16)
    v = rn(Bl, c["H"], c["T"], c["D"]).to(torch.bfloat16)
    la = F.logsigmoid(2.0 + rn(Bl, c["H"], c["T"]))
    logmag = (0.9 + 0.099 * torch.rand(Bl, c["T"], c["DS"], device=dev, generator=g)).log()
    ang = math.pi * torch.rand(Bl, c["T"], c["DS"], device=dev, generator=g)
    u = rn(Bl, c["T"], c["DS"]) * (0.1 * rn(c["DS"]))
    # a window of a (B, T, ...) tensor is not contiguous; the windows are laid out once, outside the timed region, as a
    # streaming caller would hand them over
    W = c["window"]
    nw = c["T"] // W
    split = lambda t, dim: [t.narrow(dim, w * W, W).contiguous() for w in range(nw)]
    qw, kw, vw, law = split(q, 2), split(k, 2), split(v, 2), split(la, 2)
    uw, lmw, anw = split(u, 1), split(logmag, 1), split(ang, 1)
    del q, k, v, la, u, logmag, ang

    def step(mode):
        full = mode == "gather"
        ga, gb = sharded.WindowGather(enabled=full), sharded.WindowGather(enabled=full)
        tail = sharded.WindowGather(enabled=(mode == "consumer"))
        a, b, e = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        st = {"h": None, "S": None}

        def scan_window(w):
            y, st["h"] = ops.lambda_scan(uw[w], lmw[w], anw[w], h0=st["h"])
            return y.to(torch.bfloat16) if full else y          # the gathered copy travels as bf16: half the NVLink bytes

        def prefill_window(w):
            o, st["S"], _ = ops.prefill(qw[w], kw[w], vw[w], law[w], None, st["S"], precision=_lib.PREFILL_TENSOR)
            return o

        a.record()
        ys = sharded.run_windows(scan_window, nw, ga)
        b.record()
        os_ = sharded.run_windows(prefill_window, nw, gb)
        if mode == "consumer":                                  # what the next stage of a sharded pipeline reads
            for t_ in (ys[-1], os_[-1], st["h"][0], st["h"][1], st["S"]):
                tail.submit(t_)
            tail.finish()
        e.record(); e.synchronize()
        nbytes = ga.bytes_received + gb.bytes_received + tail.bytes_received
        del ys, os_
        return a.elapsed_time(b), b.elapsed_time(e), nbytes

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    res = {}
    for mode in ("compute", "gather", "consumer"):
        if mode != "compute" and world == 1:
            continue
        for _ in range(2):
            step(mode)
        barrier()
        tl = tp = 0.0; nbytes = 0
        for _ in range(steps):
            x, y, nbytes = step(mode)
            tl += x; tp += y
        barrier()
        res[mode] = (tl / steps, tp / steps, nbytes)
    vals = []
    for mode in ("compute", "gather", "consumer"):
        vals += list(res.get(mode, (0.0, 0.0, 0))[:2])
    t = torch.tensor(vals, device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    l0, p0, l1, p1, l2, p2 = t.tolist()
    tokens = c["B"] * c["T"]
    lam_bytes, asp_bytes = Bl * c["T"] * c["DS"] * 16, Bl * c["H"] * c["T"] * (4 * c["D"] * 2 + 4)
    out = {
        "workload": "cfg4: lambda scan B64 T32768 D768 fp32 + aspin prefill B64 T32768 H12 D64 bf16, "
                    f"{c['window']}-token windows with carried state, batch split over {world} GPU(s) (strong scaling)",
        "steps": steps, "n_gpus": world,
        "compute_only": {"ms_per_step": l0 + p0, "tokens_per_s": tokens / ((l0 + p0) * 1e-3), "lambda_scan_ms": l0, "aspin_prefill_ms": p0,
                         "lambda_scan_gbs_per_gpu": lam_bytes / (l0 * 1e-3) / 1e9, "lambda_scan_frac": lam_bytes / (l0 * 1e-3) / 1e9 / pk["hbm_gbs"],
                         "aspin_prefill_gbs_per_gpu": asp_bytes / (p0 * 1e-3) / 1e9,
                         "aspin_prefill_frac": asp_bytes / (p0 * 1e-3) / 1e9 / pk["hbm_gbs"], "hbm_peak_gbs": pk["hbm_gbs"],
                         "peak_source": pk["src"]},
    }
    if world > 1:
        rx = res["gather"][2]
        out["with_full_gather"] = {"ms_per_step": l1 + p1, "tokens_per_s": tokens / ((l1 + p1) * 1e-3), "lambda_scan_ms": l1,
                                   "aspin_prefill_ms": p1, "bytes_received_per_rank": rx,
                                   "nvlink_rx_gbs_per_rank": rx / ((l1 + p1) * 1e-3) / 1e9, "nvlink_one_way_peak_gbs": 900.0,
                                   "nvlink_frac": rx / ((l1 + p1) * 1e-3) / 1e9 / 900.0,
                                   "note": "both outputs gathered per window with all_gather_into_tensor behind a side stream; "
                                           "the scan's output travels as bf16"}
        out["sharded_consumer"] = {"ms_per_step": l2 + p2, "tokens_per_s": tokens / ((l2 + p2) * 1e-3),
                                   "bytes_received_per_rank": res["consumer"][2],
                                   "note": "outputs stay sharded; final states and the last window's outputs are gathered"}
    return out


def long_context_arm(args):
    """`--workload cfg4`: configuration 4 alone, printed as its own line (the headline line nests the same numbers)."""
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product arm has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pk = peaks()
    sampler = ClockSampler(local); sampler.start()
    with torch.no_grad():
        r = long_context_numbers(args, rank, world, local, dev, pk, steps=args.steps)
    clocks = sampler.stop()
    require_healthy("configuration-4")
    if rank == 0:
        c = CFG4
        print(json.dumps({
            "metric": "long_context_tokens_per_s", "value": r["compute_only"]["tokens_per_s"], "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": 2, "ms_per_step": r["compute_only"]["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp32 scan / bf16 prefill, fp32 state", "data": "synthetic",
            "config": {"workload": r["workload"], "l2": "inputs of 3-6 GB per tensor per GPU: far larger than L2"},
            "roofline": {"cfg4": r}, "gpu_launches": args.steps * 2 * (c["T"] // c["window"]), "clocks": clocks}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="product", choices=["product", "reference"])
    ap.add_argument("--decode-steps", type=int, default=4096)
    ap.add_argument("--eager", action="store_true", help="no CUDA graphs in the timed step (for a per-kernel launch list)")
    ap.add_argument("--step-only", action="store_true", help="only the timed step: no kernel roofline, decode or CPU legs")
    ap.add_argument("--workload", default="cfg1", choices=["cfg1", "cfg4"],
                    help="cfg1 (default): the headline LM prefill; cfg4: the long-context scan + prefill, batch split over the ranks")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
    elif args.workload == "cfg4":
        long_context_arm(args)
    else:
        product_arm(args)


if __name__ == "__main__":
    main()
