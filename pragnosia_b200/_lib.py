"""ctypes binding of the C ABI declared in include/pragnosia_b200.h.

There is no fallback: if the shared library is missing, or a call returns a non-zero status, a RuntimeError is raised.
"""
from __future__ import annotations

import contextlib
import ctypes as C
from pathlib import Path

import torch

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libpragnosia_b200.so"

F32, BF16 = 0, 1
PREFILL_AUTO, PREFILL_FP32, PREFILL_TENSOR = 0, 1, 2

_vp, _ll, _i, _f = C.c_void_p, C.c_longlong, C.c_int, C.c_float

# name -> argument types (every entry point returns int except the two string getters)
SIGNATURES = {
    "pgb_abi_version": [],
    "pgb_lambda_scan_fwd": [_vp, _vp, _vp, _ll, _ll, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "pgb_lambda_scan_fwd_ex": [_vp, _vp, _vp, _ll, _ll, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_aspin_prep_fwd": [_vp, _vp, _vp, _i, _ll, _ll, _ll, _vp, _ll, _ll, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "pgb_aspin_prefill_fwd": [_vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _f, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "pgb_aspin_delta_prefill_fwd": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _vp, _i, _vp, _vp, _vp, _ll, _i, _i, _i, _i, _vp],
    "pgb_aspin_delta_scratch_bytes": [_i, _i, _i],
    "pgb_aspin_delta_prefill_noscratch_fwd": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_aspin_prefill_fused_fwd": [_vp, _vp, _vp, _vp, _ll, _ll, _vp, _vp, _vp, _vp, _f, _vp, _f, _vp, _i, _vp, _vp,
                                    _i, _i, _i, _i, _vp],
    "pgb_aspin_layer_prefill_fwd": [_vp, _vp, _vp, _ll, _ll, _vp, _vp, _ll, _ll, _vp, _vp, _i, _vp, _vp, _vp, _f, _vp, _f,
                                    _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_rot_table_build": [_vp, _vp, _i, _i, _i, _vp],
    "pgb_add_norm": [_vp, _vp, _vp, _vp, _f, _i, _vp, _vp, _ll, _i, _i, _vp],
    "pgb_decode_embed": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_decode_sample": [_vp, _i, _f, C.c_ulonglong, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "pgb_decode_sample_ex": [_vp, _i, _f, _f, C.c_ulonglong, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "pgb_batch_linear": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_batch_linear_ex": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp, _vp, _i, _f, _vp, _vp, _i, _vp],
    "pgb_batch_linear_parts": [_i],
    "pgb_decode_embed_ex": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_decode_token_work_bytes": [_i, _i, _i, _i],
    "pgb_decode_token_wait_selftest": [_vp, _ll, _vp],
    "pgb_decode_token_fwd": [_vp, _i, _vp, _vp, _vp, _vp, _i, _f, _vp, _vp, _vp, _vp, _ll, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i,
                             _i, _vp],
    "pgb_tc_wait_selftest": [_ll, _vp],
    "pgb_linear_act": [_vp, _vp, _vp, _vp, _ll, _i, _i, _i, _vp],
    "pgb_skinny_linear": [_vp, _vp, _vp, _vp, _i, _f, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _vp],
    "pgb_tc_error_flag": [_vp],
    "pgb_tc_set_variant": [_i],
    "pgb_linear_act_set_variant": [_i],
    "pgb_decode_set_variant": [_i],
    "pgb_rotate_pairs": [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_skinny_linear_ex": [_vp, _vp, _vp, _vp, _i, _f, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_lambda_scan_time_segments": [_i, _i, _i, _i],
    "pgb_lambda_scan_fwd_train": [_vp, _vp, _vp, _ll, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "pgb_lambda_scan_bwd": [_vp, _vp, _vp, _vp, _ll, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "pgb_aspin_prep_bwd": [_vp, _vp, _vp, _i, _ll, _ll, _ll, _vp, _ll, _ll, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp,
                           _i, _i, _i, _i, _vp],
    "pgb_aspin_prep_bwd_tiles": [_i],
    "pgb_assoc_out_fwd": [_vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_prefix_scan_fwd": [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_assoc_out_bwd": [_vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_prefix_scan_bwd": [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_delta_inv_bwd": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_delta_loop_bwd": [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_delta_inv_fwd": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_delta_loop_fwd": [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_key_topk_mask": [_vp, _i, _ll, _ll, _ll, _i, _i, _i, _i, _i, _vp],
    "pgb_short_conv_fwd": [_vp, _i, _ll, _ll, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "pgb_aspin_decode_step": [_vp, _vp, _vp, _i, _ll, _i, _vp, _ll, _i, _i, _vp, _ll, _vp, _vp, _vp, _f, _vp, _vp, _vp,
                              _f, _vp, _i, _ll, _i, _i, _i, _vp],
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built (python -m pragnosia_b200.build)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m pragnosia_b200.build`. "
                               "pragnosia_b200 has no CPU or PyTorch fallback.")
        L = C.CDLL(str(LIB_PATH))
        for name, args in SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = _ll if name.endswith("_bytes") else _i
        L.pgb_status_string.argtypes = [_i]; L.pgb_status_string.restype = C.c_char_p
        L.pgb_last_cuda_error.argtypes = []; L.pgb_last_cuda_error.restype = C.c_char_p
        _lib = L
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        L = lib()
        msg = L.pgb_status_string(status).decode()
        extra = L.pgb_last_cuda_error().decode() if status == 6 else ""
        raise RuntimeError(f"{what}: {msg}" + (f" [{extra}]" if extra else ""))


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"pragnosia_b200 kernels take float32 or bfloat16 tensors, got {t.dtype}")


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_of(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def on_device_of(fn):
    """Decorator for the tensor-level wrappers: the library reads CUDA's CURRENT device (SM count, kernel attributes, its
    per-device scratch array and error flags), so a call whose first tensor lives on another GPU runs with that GPU made
    current for its duration. Same device (the usual case): no context switch, no cost."""
    import functools

    @functools.wraps(fn)
    def run(*args, **kw):
        if torch.compiler.is_compiling():
            return fn(*args, **kw)
        for a in args:
            if torch.is_tensor(a):
                if a.is_cuda and a.device.index != torch.cuda.current_device():
                    with torch.cuda.device(a.device):
                        return fn(*args, **kw)
                break
        return fn(*args, **kw)
    return run


def need_cuda(*ts) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("pragnosia_b200 ops run on CUDA tensors only (there is no CPU path)")


@contextlib.contextmanager
def graph_capture(graph, **kw):
    """torch.cuda.graph(graph, **kw) with the cyclic garbage collector out of the way. A CUDAGraph of an earlier model
    that the collector frees in the middle of a capture destroys its executable graph; CUDA refuses that call while the
    thread is capturing and the capture is invalidated. So: collect first, then no collections until the capture ends."""
    import gc
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph, **kw):
            yield
    finally:
        if was_enabled:
            gc.enable()
