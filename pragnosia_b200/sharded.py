"""Long-context runs sharded by batch over the GPUs of one node (the reference has no multi-GPU carrier path: sequences
and heads are independent everywhere, the only serial dependency is along T inside one (sequence, head); src/model.py:843-864
carries the state window to window on one device).

One process per GPU holds B/G whole sequences and walks them window by window with the carried state. No collective is
needed inside the path. Where a caller wants the full output tensor, each window's output is all-gathered along the
batch axis on a side stream while the next window computes, so the transfer over NVLink overlaps the kernels; NCCL is
used as the plain library call it is (no peer memory inside the kernels, no multicast loads).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib, ops


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of `total` sequences on `rank` of `world`: contiguous, sizes differ by at most one, low ranks first."""
    if not (0 <= rank < world) or total < 0:
        raise ValueError("shard_range: rank outside the world, or a negative total")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


class WindowGather:
    """All-gather of per-window outputs along dim 0, overlapped with the following windows' compute.

    submit(local) starts the gather of one window's local output (every rank must submit the same shapes in the same
    order) and returns at once; finish() waits for all of them and returns the gathered tensors in submission order.
    With CUDA tensors the collective runs behind a side stream; with CPU tensors (gloo) it is synchronous. Disabled
    (`enabled=False`, or a world of one) it hands the local tensors back untouched: the compute-only arm of a measurement.
    """

    def __init__(self, group=None, enabled: bool = True):
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.enabled = enabled and self.world > 1
        self._side: Optional[torch.cuda.Stream] = None
        self._out: List[torch.Tensor] = []
        self.bytes_received = 0

    def submit(self, local: torch.Tensor) -> None:
        if not self.enabled:
            self._out.append(local)
            return
        local = local.contiguous()
        full = torch.empty((self.world * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        self.bytes_received += (self.world - 1) * local.numel() * local.element_size()
        if local.is_cuda:
            if self._side is None:
                self._side = torch.cuda.Stream(device=local.device)
            cur = torch.cuda.current_stream(local.device)
            self._side.wait_stream(cur)                          # the window's kernels come first
            with torch.cuda.stream(self._side):
                dist.all_gather_into_tensor(full, local, group=self.group)
            local.record_stream(self._side)
            full.record_stream(self._side)
        else:
            dist.all_gather_into_tensor(full, local, group=self.group)
        self._out.append(full)

    def finish(self) -> List[torch.Tensor]:
        if self._side is not None:
            torch.cuda.current_stream().wait_stream(self._side)
        out, self._out = self._out, []
        return out


def windows_of(T: int, window: int):
    for s in range(0, T, window):
        yield slice(s, min(s + window, T))


def prefill_windows(q, k, v, la, window: int, beta=None, S0=None, gather: Optional[WindowGather] = None,
                    precision: int = _lib.PREFILL_AUTO):
    """Chunked prefill of this rank's sequences, `window` tokens at a time with the state carried (q, k, v (B,H,T,D),
    la (B,H,T)). Returns (list of per-window outputs -- gathered over ranks along B when `gather` is enabled --, S)."""
    gather = gather or WindowGather(enabled=False)
    S = S0
    for sl in windows_of(q.shape[2], window):
        o, S, _ = ops.prefill(q[:, :, sl], k[:, :, sl], v[:, :, sl], la[:, :, sl], None if beta is None else beta[:, :, sl], S,
                              precision=precision)
        gather.submit(o)
    return gather.finish(), S


def lambda_scan_windows(u, logmag, ang, window: int, h0=None, gather: Optional[WindowGather] = None):
    """The per-token lambda scan of this rank's sequences (B,T,D), `window` steps at a time with (Re h, Im h) carried.
    Returns (list of per-window Re h -- gathered along B when `gather` is enabled --, (Re h_T, Im h_T))."""
    gather = gather or WindowGather(enabled=False)
    h = h0
    for sl in windows_of(u.shape[1], window):
        y, h = ops.lambda_scan(u[:, sl], logmag[:, sl], ang[:, sl], h0=h)
        gather.submit(y)
    return gather.finish(), h


def run_windows(fn: Callable[[int], torch.Tensor], n: int, gather: Optional[WindowGather] = None) -> List[torch.Tensor]:
    """fn(w) computes window w's local output (carrying whatever state it needs); the outputs go through `gather`."""
    gather = gather or WindowGather(enabled=False)
    for w in range(n):
        gather.submit(fn(w))
    return gather.finish()
